// Device-side life of a module (see runtime.h).
#include "runtime.h"

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>
#include <cstdio>
#include <cstring>
#include <thread>

#include "../../include/mononn.h"

namespace mononn {

extern "C" __global__ void mononn_megakernel(const __grid_constant__ KernelParams P);

static thread_local std::string g_last_error;
void set_last_error(const std::string& msg) { g_last_error = msg; }
const char* get_last_error() { return g_last_error.c_str(); }

#define CUDA_TRY(expr)                                                                   \
  do {                                                                                   \
    cudaError_t e__ = (expr);                                                            \
    if (e__ != cudaSuccess) {                                                            \
      set_last_error(std::string(#expr) + ": " + cudaGetErrorString(e__));               \
      return MONONN_ERR_CUDA;                                                            \
    }                                                                                    \
  } while (0)

// Every entry point runs on the module's device and puts the caller's current device back
// when it returns (the reference hard-codes device 0 and never switches).
namespace {
struct DeviceGuard {
  int prev = -1;
  bool ok = false;
  explicit DeviceGuard(int device) {
    if (cudaGetDevice(&prev) != cudaSuccess) prev = -1;
    ok = (prev == device) || cudaSetDevice(device) == cudaSuccess;
    if (prev == device) prev = -1;  // nothing to restore
  }
  ~DeviceGuard() {
    if (prev >= 0) cudaSetDevice(prev);
  }
};
}  // namespace
#define ON_DEVICE()                                             \
  DeviceGuard guard__(device_);                                  \
  if (!guard__.ok) {                                            \
    set_last_error("cannot select the module's CUDA device");   \
    return MONONN_ERR_CUDA;                                     \
  }

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

Runtime::~Runtime() { release(); }

void Runtime::release() {
  if (d_const_) cudaFree(d_const_);
  if (d_scratch_) cudaFree(d_scratch_);
  if (d_table_) cudaFree(d_table_);
  if (d_trace_) cudaFree(d_trace_);
  if (h_status_) cudaFreeHost(h_status_);
  d_const_ = d_scratch_ = d_table_ = d_trace_ = h_status_ = nullptr;
}

int Runtime::init(int device) {
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess || count <= 0) {
    set_last_error("no CUDA device is visible; this backend has no CPU path");
    return MONONN_ERR_NO_DEVICE;
  }
  if (device < 0 || device >= count) {
    set_last_error("device ordinal out of range");
    return MONONN_ERR_INVALID_ARGUMENT;
  }
  device_ = device;
  ON_DEVICE();
  cudaDeviceProp prop;
  CUDA_TRY(cudaGetDeviceProperties(&prop, device));
  if (prop.major != 10) {
    set_last_error("device is sm_" + std::to_string(prop.major * 10 + prop.minor) +
                   "; the kernel is built for sm_100a only");
    return MONONN_ERR_NO_DEVICE;
  }
  int coop = 0;
  CUDA_TRY(cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, device));
  if (!coop) {
    set_last_error("device does not support cooperative launches");
    return MONONN_ERR_NO_DEVICE;
  }
  device_ = device;
  sm_count_ = static_cast<uint32_t>(prop.multiProcessorCount);
  cudaDriverEntryPointQueryResult qres;
  CUDA_TRY(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &encode_fn_, cudaEnableDefault, &qres));
  if (qres != cudaDriverEntryPointSuccess || encode_fn_ == nullptr) {
    set_last_error("cuTensorMapEncodeTiled is not available from the driver");
    return MONONN_ERR_CUDA;
  }
  CUDA_TRY(cudaFuncSetAttribute(mononn_megakernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                static_cast<int>(kSmemBytes)));
  attr_set_ = true;
  return MONONN_OK;
}

// Cooperative launch of clusters: both attributes on one launch (the grid barrier needs every
// CTA resident, the cluster-scoped arrival needs the cluster shape).
void Runtime::fill_cluster_launch(cudaLaunchConfig_t* cfg, cudaLaunchAttribute* attrs, cudaStream_t stream) const {
  cfg->gridDim = dim3(plan_.grid);
  cfg->blockDim = dim3(plan_.block);
  cfg->dynamicSmemBytes = plan_.smem_bytes;
  cfg->stream = stream;
  attrs[0].id = cudaLaunchAttributeCooperative;
  attrs[0].val.cooperative = 1;
  attrs[1].id = cudaLaunchAttributeClusterDimension;
  attrs[1].val.clusterDim.x = plan_.cluster;
  attrs[1].val.clusterDim.y = 1;
  attrs[1].val.clusterDim.z = 1;
  cfg->attrs = attrs;
  cfg->numAttrs = 2;
}

int Runtime::max_coresident_ctas() {
  int per_sm = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, mononn_megakernel, kThreads,
                                                    kSmemBytes) != cudaSuccess)
    return 0;
  return per_sm * static_cast<int>(sm_count_);
}

int Runtime::load_plan(const Plan& plan) {
  ON_DEVICE();
  const int cap = max_coresident_ctas();
  if (static_cast<int>(plan.grid) > cap) {
    set_last_error("grid of " + std::to_string(plan.grid) + " CTAs exceeds the " +
                   std::to_string(cap) + " that can be co-resident; the grid barrier would hang");
    return MONONN_ERR_INVALID_ARGUMENT;
  }
  {
    std::string verr;
    int vrc = validate_plan(plan, &verr);
    if (vrc) {
      set_last_error(verr);
      return vrc;
    }
  }
  CUDA_TRY(cudaDeviceSynchronize());
  release();
  plan_ = plan;
  if (plan_.cluster > 1) {
    // every cluster of the grid must be resident at once, or the grid barrier cannot complete
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attrs[2];
    fill_cluster_launch(&cfg, attrs, nullptr);
    cfg.numAttrs = 2;
    int clusters = 0;
    cudaError_t e = cudaOccupancyMaxActiveClusters(&clusters, reinterpret_cast<const void*>(mononn_megakernel), &cfg);
    if (e != cudaSuccess || clusters * static_cast<int>(plan_.cluster) < static_cast<int>(plan_.grid)) {
      cudaGetLastError();
      set_last_error("clusters of " + std::to_string(plan_.cluster) + " CTAs: only " + std::to_string(clusters) +
                     " can be co-resident, the grid needs " + std::to_string(plan_.grid / plan_.cluster));
      return MONONN_ERR_INVALID_ARGUMENT;
    }
  }
  CUDA_TRY(cudaMalloc(&d_const_, plan_.const_bytes));
  CUDA_TRY(cudaMemset(d_const_, 0, plan_.const_bytes));
  CUDA_TRY(cudaMalloc(&d_scratch_, plan_.scratch_bytes));
  CUDA_TRY(cudaMemset(d_scratch_, 0, plan_.scratch_bytes));
  off_ops_ = plan_.stages.size() * sizeof(StageDesc);
  off_ops_ = (off_ops_ + 127) / 128 * 128;
  off_tmaps_ = off_ops_ + plan_.ops.size() * sizeof(OpDesc);
  off_tmaps_ = (off_tmaps_ + 127) / 128 * 128;
  table_bytes_ = off_tmaps_ + plan_.tmaps.size() * 128;
  CUDA_TRY(cudaMalloc(&d_table_, table_bytes_ + 128));
  h_table_.assign(table_bytes_, 0);
  bound_ = false;
  bound_args_.clear();
  epoch_ = 0;
  flag_epoch_ = 0;
  flags_uneven_ = false;
  return upload_all_constants();
}

// PACK_B: [n_tiles][K/64][n_tile][64], zero padded in N (host side of a weight's tiled copy)
static void pack_weight(const ConstBinding& b, const std::vector<uint8_t>& src, std::vector<uint16_t>* packed) {
  const uint32_t K = b.K, N = b.N, nt = b.n_tile, kb = K / 64, Ks = b.K_src ? b.K_src : b.K;
  const uint32_t n_tiles = (N + nt - 1) / nt;
  packed->assign(static_cast<size_t>(n_tiles) * nt * K, 0);
  const uint16_t* w = reinterpret_cast<const uint16_t*>(src.data());
  for (uint32_t t = 0; t < n_tiles; ++t)
    for (uint32_t k = 0; k < kb; ++k)
      for (uint32_t r = 0; r < nt; ++r) {
        const uint32_t n = t * nt + r;
        if (n >= N) continue;
        uint16_t* d = &(*packed)[((static_cast<size_t>(t) * kb + k) * nt + r) * 64];
        if (k * 64 >= Ks) continue;
        const uint32_t take = std::min(64u, Ks - k * 64);  // source rows past Ks pack as zeros
        if (b.transposed) {
          std::memcpy(d, w + static_cast<size_t>(n) * Ks + k * 64, take * 2);
        } else {
          const uint16_t* s = w + static_cast<size_t>(k) * 64 * N + n;
          for (uint32_t c = 0; c < take; ++c) d[c] = s[static_cast<size_t>(c) * N];
        }
      }
}

int Runtime::upload_constant(const ConstBinding& b, const std::vector<uint8_t>& src) {
  uint8_t* dst = static_cast<uint8_t*>(d_const_) + b.offset;
  if (b.kind == ConstBinding::RAW) {
    CUDA_TRY(cudaMemcpy(dst, src.data(), b.bytes, cudaMemcpyHostToDevice));
    return MONONN_OK;
  }
  std::vector<uint16_t> packed;
  pack_weight(b, src, &packed);
  CUDA_TRY(cudaMemcpy(dst, packed.data(), packed.size() * 2, cudaMemcpyHostToDevice));
  return MONONN_OK;
}

// Re-packs every constant already given for the current plan. The tiled copies are made by a
// pool of host threads (the reference's CompilationThreadpool compiles candidates in parallel,
// mononn_engine/codegen/compilation_threadpool.cc:41-125; here a candidate costs a re-pack of
// the weights whose tile changed, and that is what the pool shares out); uploads stay on the
// calling thread.
int Runtime::upload_all_constants() {
  std::vector<const ConstBinding*> jobs;
  for (const ConstBinding& b : plan_.consts)
    if (host_consts_.count(b.const_name)) jobs.push_back(&b);
  unsigned workers = pack_threads > 0 ? static_cast<unsigned>(pack_threads) : std::thread::hardware_concurrency();
  workers = std::max(1u, std::min<unsigned>(workers, 64u));
  const size_t kBatch = 32;  // bounds the host memory held by packed copies
  for (size_t base = 0; base < jobs.size(); base += kBatch) {
    const size_t end = std::min(jobs.size(), base + kBatch);
    std::vector<std::vector<uint16_t>> packed(end - base);
    std::atomic<size_t> next{base};
    auto work = [&]() {
      for (size_t i = next.fetch_add(1); i < end; i = next.fetch_add(1))
        if (jobs[i]->kind == ConstBinding::PACK_B)
          pack_weight(*jobs[i], host_consts_.at(jobs[i]->const_name), &packed[i - base]);
    };
    std::vector<std::thread> pool;
    for (unsigned t = 1; t < workers && t < end - base; ++t) pool.emplace_back(work);
    work();
    for (std::thread& t : pool) t.join();
    for (size_t i = base; i < end; ++i) {
      const ConstBinding& b = *jobs[i];
      uint8_t* dst = static_cast<uint8_t*>(d_const_) + b.offset;
      if (b.kind == ConstBinding::RAW) {
        CUDA_TRY(cudaMemcpy(dst, host_consts_.at(b.const_name).data(), b.bytes, cudaMemcpyHostToDevice));
      } else {
        CUDA_TRY(cudaMemcpy(dst, packed[i - base].data(), packed[i - base].size() * 2, cudaMemcpyHostToDevice));
      }
    }
  }
  return MONONN_OK;
}

// '.' and '-' are interchangeable with '_' in constant names, as in the reference's
// canonical node names (mononn_engine/helpers/string_helpers.cc:22-32).
static std::string canon(const std::string& n) {
  std::string v = n;
  for (char& c : v)
    if (c == '.' || c == '-') c = '_';
  return v;
}

int Runtime::set_constant(const std::string& given, const void* host, size_t bytes) {
  ON_DEVICE();
  std::string name = given;
  for (const ConstBinding& b : plan_.consts)
    if (b.const_name != given && canon(b.const_name) == canon(given)) name = b.const_name;
  bool found = false;
  for (const ConstBinding& b : plan_.consts)
    if (b.const_name == name) {
      found = true;
      if (b.src_bytes != bytes) {
        set_last_error("constant " + name + ": expected " + std::to_string(b.src_bytes) +
                       " bytes, got " + std::to_string(bytes));
        return MONONN_ERR_CONSTANT;
      }
    }
  if (!found) {
    set_last_error("unknown constant " + name);
    return MONONN_ERR_CONSTANT;
  }
  std::vector<uint8_t>& copy = host_consts_[name];
  copy.assign(static_cast<const uint8_t*>(host), static_cast<const uint8_t*>(host) + bytes);
  for (const ConstBinding& b : plan_.consts)
    if (b.const_name == name) {
      int rc = upload_constant(b, copy);
      if (rc) return rc;
    }
  return MONONN_OK;
}

bool Runtime::constants_ready(std::string* missing) const {
  for (const ConstBinding& b : plan_.consts)
    if (!host_consts_.count(b.const_name)) {
      if (missing) *missing = b.const_name;
      return false;
    }
  return true;
}

int Runtime::bind(void* const* args, int n, void* stream) {
  if (n != static_cast<int>(plan_.args.size())) {
    set_last_error("expected " + std::to_string(plan_.args.size()) + " kernel arguments, got " +
                   std::to_string(n));
    return MONONN_ERR_INVALID_ARGUMENT;
  }
  if (bound_ && bound_args_.size() == static_cast<size_t>(n) &&
      std::memcmp(bound_args_.data(), args, sizeof(void*) * n) == 0)
    return MONONN_OK;
  auto resolve = [&](const BufRef& r) -> uint64_t {
    switch (r.space) {
      case SPACE_ARG:
        return reinterpret_cast<uint64_t>(args[r.index]) + r.offset;
      case SPACE_CONST:
        return reinterpret_cast<uint64_t>(d_const_) + r.offset;
      case SPACE_SCRATCH:
        return reinterpret_cast<uint64_t>(d_scratch_) + r.offset;
      default:
        return 0;
    }
  };
  std::memcpy(h_table_.data(), plan_.stages.data(), plan_.stages.size() * sizeof(StageDesc));
  OpDesc* ops = reinterpret_cast<OpDesc*>(h_table_.data() + off_ops_);
  for (size_t i = 0; i < plan_.ops.size(); ++i) {
    ops[i] = plan_.ops[i].d;
    for (int k = 0; k < 8; ++k) ops[i].p[k] = resolve(plan_.ops[i].p[k]);
    for (int k = 0; k < 4; ++k) ops[i].q[k] = resolve(plan_.ops[i].q[k]);
    ops[i].flag = resolve(plan_.ops[i].flag);
    ops[i].wait_flag = resolve(plan_.ops[i].wflag);
  }
  EncodeTiledFn encode = reinterpret_cast<EncodeTiledFn>(encode_fn_);
  for (size_t i = 0; i < plan_.tmaps.size(); ++i) {
    const TmapSpec& t = plan_.tmaps[i];
    CUtensorMap tm;
    const cuuint64_t dims[2] = {t.dim0, t.dim1};
    const cuuint64_t strides[1] = {t.stride1_bytes};
    const cuuint32_t box[2] = {t.box0, t.box1};
    const cuuint32_t estr[2] = {1, 1};
    const uint64_t base = resolve(t.base);
    if ((base & 15u) || (t.stride1_bytes & 15u)) {
      set_last_error("tensor map " + std::to_string(i) + ": base or stride is not 16-byte aligned");
      return MONONN_ERR_INVALID_ARGUMENT;
    }
    CUresult r = encode(&tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, reinterpret_cast<void*>(base), dims,
                        strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
      set_last_error("cuTensorMapEncodeTiled failed for tensor map " + std::to_string(i) +
                     " (CUresult " + std::to_string(static_cast<int>(r)) + ")");
      return MONONN_ERR_CUDA;
    }
    std::memcpy(h_table_.data() + off_tmaps_ + i * 128, &tm, 128);
  }
  // the table base must be 128-byte aligned for the tensor maps (cudaMalloc gives 256)
  CUDA_TRY(cudaMemcpyAsync(d_table_, h_table_.data(), table_bytes_, cudaMemcpyHostToDevice,
                           static_cast<cudaStream_t>(stream)));
  bound_args_.assign(args, args + n);
  bound_ = true;
  return MONONN_OK;
}

int Runtime::launch(void* const* args, int n, void* stream, uint32_t stage_begin,
                    uint32_t stage_end, bool stamps) {
  ON_DEVICE();
  if (stage_end > plan_.stages.size() || stage_begin >= stage_end) {
    set_last_error("stage range out of bounds");
    return MONONN_ERR_INVALID_ARGUMENT;
  }
  std::string missing;
  if (!constants_ready(&missing)) {
    set_last_error("constant " + missing + " has not been set");
    return MONONN_ERR_NOT_READY;
  }
  int rc = bind(args, n, stream);
  if (rc) return rc;
  KernelParams kp;
  std::memset(&kp, 0, sizeof(kp));
  uint8_t* tab = static_cast<uint8_t*>(d_table_);
  uint8_t* scr = static_cast<uint8_t*>(d_scratch_);
  kp.stages = reinterpret_cast<const StageDesc*>(tab);
  kp.ops = reinterpret_cast<const OpDesc*>(tab + off_ops_);
  kp.tmaps = tab + off_tmaps_;
  kp.barrier = reinterpret_cast<uint32_t*>(scr + kScratchBarrierOff);
  kp.status = reinterpret_cast<KernelStatus*>(scr + kScratchStatusOff);
  kp.stamps = stamps ? reinterpret_cast<uint64_t*>(scr + kScratchStampsOff) : nullptr;
  kp.trace = trace_on_ ? static_cast<uint64_t*>(d_trace_) : nullptr;
  kp.hot_consts = static_cast<const uint8_t*>(d_const_);
  kp.hot_const_bytes = plan_.hot_const_bytes;
  kp.n_stages = static_cast<uint32_t>(plan_.stages.size());
  kp.epoch_base = epoch_;
  kp.timeout_us = timeout_us ? timeout_us : 2000000u;
  kp.stage_begin = stage_begin;
  kp.stage_end = stage_end;
  // Arrival counters of row ops that share a stage with their GEMMs grow by the same amount on
  // every launch of all stages. A launch of a stage sub-range (tuning, profiling) would leave
  // them uneven, so it starts from cleared counters and the launch after it clears them again.
  const bool full = (stage_begin == 0 && stage_end == plan_.stages.size());
  if (plan_.flag_bytes != 0 && (!full || flags_uneven_)) {
    CUDA_TRY(cudaMemsetAsync(scr + plan_.flag_offset, 0, plan_.flag_bytes, static_cast<cudaStream_t>(stream)));
    flag_epoch_ = 0;
  }
  flags_uneven_ = !full;
  kp.flag_epoch = ++flag_epoch_;
  kp.cluster = plan_.cluster;
  kp.l2_hints = plan_.spec.l2_hints == 1 ? 0u : 1u;
  kp.warp_arrive = arrive_mode();
  kp.table_bytes = static_cast<uint32_t>(table_bytes_);
  kp.host_flag = static_cast<uint32_t*>(h_status_);  // null until infer_host has been used
  void* kargs[1] = {&kp};
  if (plan_.cluster <= 1) {
    CUDA_TRY(cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(mononn_megakernel),
                                         dim3(plan_.grid), dim3(plan_.block), kargs, plan_.smem_bytes,
                                         static_cast<cudaStream_t>(stream)));
  } else {
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attrs[2];
    fill_cluster_launch(&cfg, attrs, static_cast<cudaStream_t>(stream));
    CUDA_TRY(cudaLaunchKernelExC(&cfg, reinterpret_cast<const void*>(mononn_megakernel), kargs));
  }
  epoch_ += (stage_end - stage_begin) * (plan_.grid / plan_.cluster) * (arrive_mode() == 1u ? kSimtWarps : 1u);
  if (stamps) n_stamp_stages_ = stage_end - stage_begin;
  return MONONN_OK;
}

int Runtime::infer_host(const void* const* host_in, int n_in, void* const* host_out, int n_out,
                        void* const* args, int n, void* stream) {
  ON_DEVICE();
  if (n != static_cast<int>(plan_.args.size())) {
    set_last_error("argument count does not match the module");
    return MONONN_ERR_INVALID_ARGUMENT;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int seen_in = 0, seen_out = 0;
  for (const ArgDesc& a : plan_.args) seen_in += (a.kind == 0), seen_out += (a.kind == 1);
  if (seen_in != n_in || seen_out != n_out) {
    set_last_error("host buffer counts do not match the module's parameters / live-outs");
    return MONONN_ERR_INVALID_ARGUMENT;
  }
  // One copy per parameter: two host buffers that happen to be neighbours in the address space
  // may still be separate pinned allocations, and a copy across their boundary is refused.
  for (int i = 0; i < n; ++i) {
    const ArgDesc& a = plan_.args[i];
    // (a parameter bound to the host buffer itself -- mapped pinned memory -- is read in place)
    if (a.kind == 0 && args[i] != host_in[a.param_number])
      CUDA_TRY(cudaMemcpyAsync(args[i], host_in[a.param_number], a.bytes, cudaMemcpyHostToDevice, st));
  }
  // A word in pinned host memory (device-accessible under unified addressing) that the kernel
  // sets when a bounded wait expires: no status copy sits behind the outputs' copies.
  if (!h_status_) CUDA_TRY(cudaHostAlloc(&h_status_, sizeof(KernelStatus), cudaHostAllocMapped));
  *static_cast<volatile uint32_t*>(h_status_) = ST_OK;
  int rc = launch_all(args, n, stream);
  if (rc) return rc;
  for (int i = 0; i < n; ++i) {
    const ArgDesc& a = plan_.args[i];
    if (a.kind == 1 && args[i] != host_out[a.param_number])
      CUDA_TRY(cudaMemcpyAsync(host_out[a.param_number], args[i], a.bytes, cudaMemcpyDeviceToHost, st));
  }
  cudaError_t e = cudaStreamSynchronize(st);
  if (e != cudaSuccess) {
    set_last_error(std::string("kernel failed: ") + cudaGetErrorString(e));
    return MONONN_ERR_CUDA;
  }
  if (*static_cast<volatile uint32_t*>(h_status_) == ST_OK) return MONONN_OK;
  int stage = 0, cta = 0;
  return check_status(&stage, &cta);  // formats the message and restores the module
}

int Runtime::check_status(int* stage, int* cta) {
  ON_DEVICE();
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) {
    set_last_error(std::string("kernel failed: ") + cudaGetErrorString(e));
    return MONONN_ERR_CUDA;
  }
  KernelStatus st;
  CUDA_TRY(cudaMemcpy(&st, static_cast<uint8_t*>(d_scratch_) + kScratchStatusOff, sizeof(st),
                      cudaMemcpyDeviceToHost));
  if (st.code == ST_OK) return MONONN_OK;
  if (stage) *stage = static_cast<int>(st.stage);
  if (cta) *cta = static_cast<int>(st.cta);
  char buf[160];
  std::snprintf(buf, sizeof(buf),
                "bounded wait expired in the kernel: code %u, stage %u, CTA %u, wait site 0x%x",
                st.code, st.stage, st.cta, st.where);
  set_last_error(buf);
  // restore the invariants the next launch relies on: counter, status, zeroed accumulators
  CUDA_TRY(cudaMemset(d_scratch_, 0, plan_.scratch_bytes));
  epoch_ = 0;
  flag_epoch_ = 0;
  flags_uneven_ = false;
  return MONONN_ERR_BARRIER_TIMEOUT;
}

int Runtime::read_stamps(std::vector<double>* us) {
  ON_DEVICE();
  std::vector<uint64_t> t(n_stamp_stages_ + 1);
  CUDA_TRY(cudaMemcpy(t.data(), static_cast<uint8_t*>(d_scratch_) + kScratchStampsOff,
                      t.size() * 8, cudaMemcpyDeviceToHost));
  us->clear();
  for (uint32_t i = 0; i < n_stamp_stages_; ++i)
    us->push_back(static_cast<double>(t[i + 1] - t[i]) * 1e-3);
  return MONONN_OK;
}

int Runtime::trace_launch(void* const* args, int n, void* stream, std::vector<double>* out) {
  ON_DEVICE();
  const size_t ns = plan_.stages.size();
  const size_t words = static_cast<size_t>(plan_.grid) * ns * kTraceEvents;
  if (!d_trace_) CUDA_TRY(cudaMalloc(&d_trace_, words * 8));
  CUDA_TRY(cudaMemsetAsync(d_trace_, 0, words * 8, static_cast<cudaStream_t>(stream)));
  trace_on_ = true;
  int rc = launch(args, n, stream, 0, static_cast<uint32_t>(ns), false);
  trace_on_ = false;
  if (rc) return rc;
  int st = 0, cta = 0;
  rc = check_status(&st, &cta);
  if (rc) return rc;
  std::vector<uint64_t> raw(words);
  CUDA_TRY(cudaMemcpy(raw.data(), d_trace_, words * 8, cudaMemcpyDeviceToHost));
  uint64_t t0 = ~0ull;
  for (uint64_t v : raw)
    if (v && v < t0) t0 = v;
  out->assign(words, 0.0);
  for (size_t i = 0; i < words; ++i)
    if (raw[i]) (*out)[i] = static_cast<double>(raw[i] - t0) + 1.0;
  return MONONN_OK;
}

int Runtime::time_stages(void* const* args, int n, void* stream, uint32_t begin, uint32_t end,
                         int warmup, int iters, double* us) {
  ON_DEVICE();
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  for (int i = 0; i < warmup; ++i) {
    int rc = launch(args, n, stream, begin, end, false);
    if (rc) return rc;
  }
  cudaEvent_t e0, e1;
  CUDA_TRY(cudaEventCreate(&e0));
  CUDA_TRY(cudaEventCreate(&e1));
  CUDA_TRY(cudaEventRecord(e0, s));
  for (int i = 0; i < iters; ++i) {
    int rc = launch(args, n, stream, begin, end, false);
    if (rc) return rc;
  }
  CUDA_TRY(cudaEventRecord(e1, s));
  CUDA_TRY(cudaEventSynchronize(e1));
  float ms = 0;
  CUDA_TRY(cudaEventElapsedTime(&ms, e0, e1));
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  *us = static_cast<double>(ms) * 1000.0 / iters;
  int st = 0, cta = 0;
  return check_status(&st, &cta);
}

}  // namespace mononn
