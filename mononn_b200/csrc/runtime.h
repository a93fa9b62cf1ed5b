// Device-side life of a module: constant arena, scratch, bound stage table, launch.
//
// Stands where the (absent) TF side of the reference stood: it loads the kernel, sets the
// dynamic shared-memory attribute and launches (grid, block, smem) with the argument list
// (params.., live-outs.., temp) -- the sequence mirrored in
// mononn_engine/module/mononn_module_tuner.cc:99-150 -- except that the "kernel" is the
// pre-compiled table interpreter and the per-graph artefact is the table.
#pragma once
#include <map>
#include <set>
#include <string>
#include <vector>

#include <cuda_runtime.h>

#include "plan.h"

namespace mononn {

void set_last_error(const std::string& msg);
const char* get_last_error();

struct PerfRow {
  std::string context;  // "<grid>_1_1__<block>_1_1"
  std::string node;
  double us;
};

class Runtime {
 public:
  Runtime() = default;
  ~Runtime();
  Runtime(const Runtime&) = delete;
  Runtime& operator=(const Runtime&) = delete;

  int init(int device);           // selects the device, checks sm_100, queries SM count
  uint32_t sm_count() const { return sm_count_; }
  int max_coresident_ctas();      // occupancy query for the cooperative launch

  // (Re)builds device state for a plan. Constants already given are re-packed.
  int load_plan(const Plan& plan);
  const Plan& plan() const { return plan_; }

  int set_constant(const std::string& name, const void* host, size_t bytes);
  bool constants_ready(std::string* missing) const;

  // One cooperative launch over stages [begin, end). stamps: record per-stage timers.
  int launch(void* const* args, int n, void* stream, uint32_t stage_begin, uint32_t stage_end,
             bool stamps);
  int launch_all(void* const* args, int n, void* stream) {
    return launch(args, n, stream, 0, static_cast<uint32_t>(plan_.stages.size()), false);
  }
  // Host buffers in, one launch, host buffers out, status word checked, stream synchronised.
  int infer_host(const void* const* host_in, int n_in, void* const* host_out, int n_out,
                 void* const* args, int n, void* stream);
  // cudaDeviceSynchronize + status word; resets barrier and accumulators after a failure.
  int check_status(int* stage, int* cta);
  int read_stamps(std::vector<double>* us);  // after a stamps launch + sync
  // One launch of all stages with the per-CTA event trace on; out = [grid][stages][kTraceEvents]
  // nanoseconds relative to the earliest event (0 where an event did not occur).
  int trace_launch(void* const* args, int n, void* stream, std::vector<double>* out);
  // Mean device time (microseconds) of `iters` launches of stages [begin, end) after `warmup`.
  int time_stages(void* const* args, int n, void* stream, uint32_t begin, uint32_t end, int warmup,
                  int iters, double* us);

  // Host-side fault injection for tests: the next launch expects `n` arrivals that never come,
  // so its first grid-barrier wait runs into the timeout and the kernel reports it.
  void skew_epoch(uint32_t n) { epoch_ += n; }

  // Per-warp barrier arrival is the default; a cluster launch arrives per CTA through the cluster.
  // 0: one arrival per CTA after a CTA-wide sync (always with clusters), 1: one per epilogue warp,
  // 2: one per CTA by the warp that finishes last
  uint32_t arrive_mode() const {
    if (plan_.cluster > 1 || plan_.spec.barrier_arrive == 1) return 0;
    return plan_.spec.barrier_arrive == 2 ? 1u : 2u;
  }
  unsigned timeout_us = 2000000;
  int pack_threads = 0;  // host threads that re-pack weights when a plan is (re)loaded; 0 = all cores
  const std::map<std::string, std::vector<uint8_t>>& host_constants() const { return host_consts_; }

 private:
  int bind(void* const* args, int n, void* stream);
  int upload_constant(const ConstBinding& b, const std::vector<uint8_t>& src);
  int upload_all_constants();
  void fill_cluster_launch(cudaLaunchConfig_t* cfg, cudaLaunchAttribute* attrs, cudaStream_t stream) const;
  void release();

  int device_ = 0;
  uint32_t sm_count_ = 0;
  Plan plan_;
  void* d_const_ = nullptr;
  void* d_scratch_ = nullptr;
  void* d_table_ = nullptr;
  void* d_trace_ = nullptr;
  void* h_status_ = nullptr;  // pinned copy of the status word for infer_host
  bool trace_on_ = false;
  size_t table_bytes_ = 0, off_ops_ = 0, off_tmaps_ = 0;
  std::vector<uint8_t> h_table_;
  std::vector<void*> bound_args_;
  bool bound_ = false;
  uint32_t epoch_ = 0;
  uint32_t flag_epoch_ = 0;    // launches since the row ops' arrival counters were cleared
  bool flags_uneven_ = false;  // the last launch ran a stage sub-range
  uint32_t n_stamp_stages_ = 0;
  std::map<std::string, std::vector<uint8_t>> host_consts_;
  void* encode_fn_ = nullptr;
  bool attr_set_ = false;
};

}  // namespace mononn
