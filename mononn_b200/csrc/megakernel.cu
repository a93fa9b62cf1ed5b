// One persistent, table-driven kernel for the whole inference graph (sm_100a).
//
// Replaces the per-graph generated kernel of the reference
// (mononn_engine/codegen/graph_codegen.cc:734-803): instead of emitting CUDA
// text per HLO module, the host fills a stage table (stage_table.h) and this
// kernel interprets it in a single cooperative launch.
//
// Warp roles inside each 384-thread CTA (one CTA per SM):
//   warp 0  weight producer : streams packed weight tiles HBM -> smem ring via TMA.
//                             It never waits for the grid barrier (weights do not
//                             depend on activations), so HBM stays busy across stages.
//   warp 1  activation producer : after the previous stage's grid barrier, TMA-loads
//                             128x64 activation tiles (L2 resident) into the A ring.
//   warp 2  MMA issuer      : tcgen05.mma (kind::f16, fp32 accumulate in TMEM).
//   warps 4-11 epilogue/SIMT: tcgen05.ld -> bias/activation/residual -> global;
//                             softmax of the attention stage; LayerNorm / embedding rows;
//                             grid-barrier arrive. Two warps share each 32-lane quarter of
//                             TMEM (warp w reads lanes 32*(w%4)..) and split its columns.
//
// Grid barrier (replaces mononn_engine/core/gpu/synchronization.cc:45-97): one
// monotonically increasing counter; each CTA adds 1 with release semantics after
// its stores of a stage and polls with acquire until (stage+1)*gridDim arrivals.
// Every wait in this file is bounded; on expiry the kernel records where it gave
// up in KernelStatus and all roles drain and return.
#include <cuda.h>
#include <cuda_fp16.h>
#include <stddef.h>
#include <stdint.h>

#include "stage_table.h"

namespace mononn {

// ----------------------------------------------------------------------------
// PTX wrappers
// ----------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void* tmap, int32_t x, int32_t y,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
      "l"(tmap), "r"(x), "r"(y), "r"(bar)
      : "memory");
}
// The same copy with an L2 eviction-priority hint (replaces the evict-last / streaming loads the
// reference selects per access pattern, mononn_engine/core/gpu/memory.cc:172-235): weights are
// read once per inference (evict first), activation tiles are re-read by every CTA of a stage
// (evict last).
__device__ __forceinline__ void tma_load_2d_hint(uint32_t dst, const void* tmap, int32_t x, int32_t y,
                                                 uint32_t bar, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint "
      "[%0], [%1, {%2, %3}], [%4], %5;" ::"r"(dst),
      "l"(tmap), "r"(x), "r"(y), "r"(bar), "l"(policy)
      : "memory");
}
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
  return p;
}
// Orders the generic-proxy stores of other CTAs (acquired through the grid barrier) before this
// thread's TMA loads of the same global memory. Only the global state space is involved; the
// fence over all state spaces measured 13 us slower per inference.
__device__ __forceinline__ void fence_proxy_async_global() {
  asm volatile("fence.proxy.async.global;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}
__device__ __forceinline__ void tc_mma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                           uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
      : "memory");
}
// One lane of a converged warp (the same one every time for a full mask).
__device__ __forceinline__ bool elect_one_sync() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred)::"memory");
  return pred != 0u;
}
__device__ __forceinline__ void tc_ld16(uint32_t taddr, float (&v)[16]) {
  uint32_t r[16];
  __syncwarp();
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n\t"
      "tcgen05.wait::ld.sync.aligned;"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}
// Issue only: the registers are valid after the next tc_wait_ld(). Lets the following load be in
// flight while the previous one is processed.
__device__ __forceinline__ void tc_ld32_issue(uint32_t taddr, uint32_t (&r)[32]) {
  __syncwarp();
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tc_wait_ld() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, float (&v)[32]) {
  uint32_t r[32];
  __syncwarp();
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n\t"
      "tcgen05.wait::ld.sync.aligned;"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
// Polling uses relaxed loads: an acquire load in a spin loop would invalidate the SM's L1 on
// every iteration, under the feet of the warps that are doing the stage's work. One acquire
// load after the poll succeeds gives the ordering.
__device__ __forceinline__ uint32_t ld_relaxed_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Thread-block cluster helpers: rank of this CTA, the shared::cluster address of a peer's copy of
// a shared-memory object, a remote mbarrier arrival with release at cluster scope, the matching
// acquire-side test, and the whole-cluster barrier used around set-up and teardown.
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t mapa_smem(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_remote_release_cluster(uint32_t remote_bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(remote_bar) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait_acquire_cluster(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release;\n\tbarrier.cluster.wait.acquire;" ::: "memory");
}
__device__ __forceinline__ void st_release_cta_smem(uint32_t* p, uint32_t v) {
  asm volatile("st.release.cta.shared::cta.u32 [%0], %1;" ::"r"(smem_u32(p)), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_cta_smem(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.cta.shared::cta.u32 %0, [%1];" : "=r"(v) : "r"(smem_u32(p)) : "memory");
  return v;
}
__device__ __forceinline__ void fence_acq_rel_gpu() {
  asm volatile("fence.acq_rel.gpu;" ::: "memory");
}
__device__ __forceinline__ uint32_t atom_add_acq_rel_cta_smem(uint32_t* p, uint32_t v) {
  uint32_t old;
  asm volatile("atom.acq_rel.cta.shared::cta.add.u32 %0, [%1], %2;" : "=r"(old) : "r"(smem_u32(p)), "r"(v) : "memory");
  return old;
}
// Counts the calling warp on a shared-memory counter (acquire + release at CTA scope, after a warp
// barrier that orders the other lanes' accesses) and tells lane 0 of the warp that counted
// eighth: whatever that lane releases next is cumulative over the eight warps' earlier stores.
__device__ __forceinline__ bool last_warp_of(uint32_t* counter, uint32_t lane) {
  __syncwarp();
  if (lane != 0u) return false;
  return (atom_add_acq_rel_cta_smem(counter, 1u) & (kSimtWarps - 1u)) == kSimtWarps - 1u;
}
__device__ __forceinline__ void red_release_gpu_add(uint32_t* p, uint32_t v) {
  asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void red_add_f32x4(float* p, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(a), "f"(b), "f"(c),
               "f"(d)
               : "memory");
}

// K-major, 128-byte-swizzled operand tile: rows of 64 f16 (128 B), 8-row groups 1024 B apart.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t saddr) {
  return static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4) | (1ull << 16) | (64ull << 32) |
         (1ull << 46) | (2ull << 61);
}
// f16 x f16 -> f32, both operands K-major, M = 128.
__device__ __forceinline__ uint32_t umma_idesc_m128(uint32_t n) {
  return (1u << 4) | ((n >> 3) << 17) | ((128u >> 4) << 24);
}

// ----------------------------------------------------------------------------
// Shared-memory control block and per-thread context
// ----------------------------------------------------------------------------
struct Ctrl {
  uint64_t a_full[kASlots];
  uint64_t a_empty[kASlots];
  uint64_t b_full[kBSlots];
  uint64_t b_empty[kBSlots];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint64_t group_bar;  // the eight epilogue warps (one arrival per warp and phase)
  uint64_t cl_bar;     // first CTA of a cluster: one arrival per CTA of the cluster per stage
  uint32_t tmem_base;
  uint32_t abort_flag;
  uint32_t barriers_seen;  // grid barriers of this launch the CTA's poller has observed (monotonic)
  uint32_t warps_done;     // epilogue warps that finished a stage (monotonic; every eighth arrives for the CTA)
  uint32_t items_done[2];  // per accumulator buffer: epilogue warps that finished a GEMM item a row op waits for
  uint32_t tiles_done[5];  // attention: epilogue warps that finished writing the Q/K/V tiles ([0]) or the P
                           // tiles of key chunk j ([1 + j]); every eighth count hands the tiles to the MMA issuer;
                           // [4]: warps that stored their part of an item's output (every eighth counts the item)
  uint32_t pad_;
  alignas(16) float bias_tile[2][256];  // bias of the current GEMM tile, double buffered across items
  float mask_row[384];      // additive key mask of the current attention tile (log2 units)
  float row_max[2][128];    // attention: row maximum / row sum over each warp half's columns,
  float row_sum[2][128];    // exchanged between the two threads that share a query row
  float ln_part[2][kSplitRowsPerItem][4];  // split LayerNorm: per-warp partial sum / squared deviation
  float red_val[kSimtWarps];  // arg-max: per-warp partial results of the current row
  uint32_t red_idx[kSimtWarps];
  // Shared-memory copies of the operator descriptor each role is working on: slot 0 weight
  // producer, 1 activation producer, 2 MMA issuer, 3.. the eight epilogue warps.
  uint4 desc[3 + kSimtWarps][16];
};

static_assert(sizeof(Ctrl) <= kCtrlBytes, "control block exceeds its shared-memory reserve");
// these members are read with 16-byte vector loads
static_assert(offsetof(Ctrl, bias_tile) % 16 == 0 && offsetof(Ctrl, mask_row) % 16 == 0 &&
                  offsetof(Ctrl, desc) % 16 == 0,
              "vector-loaded members of the control block must be 16-byte aligned");
static_assert(sizeof(OpDesc) % 16 == 0 && sizeof(OpDesc) <= 256, "descriptor slot size");
static_assert(sizeof(StageDesc) == 48, "stage descriptor is read as three 16-byte words");

struct Ctx {
  const KernelParams* P;
  Ctrl* ctrl;
  uint32_t a_ring;  // shared addresses
  uint32_t b_ring;
  uint8_t* a_ring_ptr;
  uint8_t* store_stage;  // kStoreStageBytes after the control block: 2 KB per epilogue warp
  uint32_t stage;   // current stage (for status)
  uint32_t group_phase;  // parity of the next group_bar phase (epilogue warps only)
  uint64_t timeout_ns;
};

__device__ __noinline__ void report_failure(const KernelParams* P, Ctrl* ctrl, uint32_t stage,
                                            uint32_t code, uint32_t where) {
  volatile uint32_t* af = &ctrl->abort_flag;
  *af = 1;
  KernelStatus* st = P->status;
  if (atomicCAS(&st->code, 0u, code) == 0u) {
    st->stage = stage;
    st->cta = blockIdx.x;
    st->where = where;
    __threadfence();
    if (P->host_flag != nullptr) {
      *reinterpret_cast<volatile uint32_t*>(P->host_flag) = code;
      __threadfence_system();
    }
  }
}

// Optional per-CTA event trace: trace[(cta * n_stages + stage) * 8 + event] = %globaltimer.
enum TraceEvent : uint32_t {
  TR_SIMT_READY = 0,   // epilogue warps passed the previous stage's grid barrier
  TR_SIMT_DONE = 1,    // ... finished this stage's items
  TR_SIMT_ARRIVED = 2, // ... arrived at this stage's grid barrier
  TR_ACT_READY = 3,    // activation producer passed the grid barrier
  TR_ACT_ISSUED = 4,   // ... issued its last activation tile load of the stage
  TR_MMA_FIRST = 5,    // MMA issuer saw its first operands of the stage
  TR_MMA_LAST = 6,     // ... committed its last MMA of the stage
  TR_W_ISSUED = 7,     // weight producer issued its last tile load of the stage
  TR_MARK0 = 8,        // 8..15: free marks inside the epilogue / row-wise code (thread 0 of the group)
};
__device__ __forceinline__ void trace(const KernelParams& P, uint32_t stage, uint32_t ev) {
  if (P.trace != nullptr)
    P.trace[(static_cast<size_t>(blockIdx.x) * (P.stage_end - P.stage_begin) +
             (stage - P.stage_begin)) * kTraceEvents + ev] = globaltimer_ns();
}
// Bounded wait on an mbarrier phase. Returns false when the kernel is aborting. The slow
// path is out of line so that the many wait sites stay a few instructions each.
__device__ __noinline__ bool mbar_wait_slow(const KernelParams* P, Ctrl* ctrl, uint32_t b,
                                            uint32_t parity, uint32_t stage, uint32_t where) {
  const uint64_t t0 = globaltimer_ns();
  const uint64_t limit = static_cast<uint64_t>(P->timeout_us) * 1000ull;
  uint32_t it = 0;
  for (;;) {
    if (mbar_try_wait(b, parity)) return true;
    if ((++it & 63u) == 0u) {
      if (*reinterpret_cast<volatile uint32_t*>(&ctrl->abort_flag)) return false;
      if (globaltimer_ns() - t0 > limit) {
        report_failure(P, ctrl, stage, ST_MBARRIER_TIMEOUT, where);
        return false;
      }
    }
  }
}
__device__ __forceinline__ bool mbar_wait(const Ctx& c, uint64_t* bar, uint32_t parity,
                                          uint32_t where) {
  const uint32_t b = smem_u32(bar);
  if (mbar_try_wait(b, parity)) return true;
  return mbar_wait_slow(c.P, c.ctrl, b, parity, c.stage, where);
}

// The counters are polled with acquire loads: the load that sees the count observes the last
// arrival (a release atomic) and through the chain of atomics all earlier ones, so nothing else
// is needed before the data is read. Measured per inference against this: relaxed polls plus one
// acquire load at the end +7 us (one more L2 round trip per wait), a fence.acq_rel.gpu after a
// relaxed poll +39 us (it also waits for this thread's own outstanding stores). A pause between
// polls (__nanosleep) only delays the detection (+2 us at 32 ns).
#ifndef MONONN_POLL_ACQUIRE
#define MONONN_POLL_ACQUIRE 1  // 0: relaxed polls, then one acquire load
#endif
__device__ __forceinline__ uint32_t poll_load(const uint32_t* p) {
#if MONONN_POLL_ACQUIRE
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
#else
  return ld_relaxed_gpu(p);
#endif
}
__device__ __forceinline__ void acquire_after_poll(const uint32_t* p) {
#if MONONN_POLL_ACQUIRE
  (void)p;
#else
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  (void)v;
#endif
}
#ifndef MONONN_ALL_POLL
#define MONONN_ALL_POLL 0  // 1: every epilogue warp polls the global counter itself
#endif
#ifndef MONONN_POLL_SLEEP
#define MONONN_POLL_SLEEP 0
#endif
// Bounded wait until every CTA has arrived for all stages before `stage`. Two threads per CTA
// poll the global counter: the activation producer (its first tile load is the critical path of
// a GEMM stage; routing it through a second hop measured 20 us slower over a whole inference)
// and the first epilogue warp's lane 0, which then publishes the number of barriers seen in
// shared memory for the other seven epilogue warps: some 300 pollers on the counter's L2 line
// instead of 1300.
__device__ __noinline__ bool grid_wait_slow(const KernelParams* P, Ctrl* ctrl, uint32_t target,
                                            uint32_t stage, uint32_t where) {
  const uint64_t t0 = globaltimer_ns();
  const uint64_t limit = static_cast<uint64_t>(P->timeout_us) * 1000ull;
  uint32_t it = 0;
  for (;;) {
    if (static_cast<int32_t>(poll_load(P->barrier) - target) >= 0) {
      acquire_after_poll(P->barrier);
      return true;
    }
#if MONONN_POLL_SLEEP > 0
    __nanosleep(MONONN_POLL_SLEEP);
#endif
    if ((++it & 31u) == 0u) {
      if (*reinterpret_cast<volatile uint32_t*>(&ctrl->abort_flag)) return false;
      if (*reinterpret_cast<volatile uint32_t*>(&P->status->code) != 0u) {
        *reinterpret_cast<volatile uint32_t*>(&ctrl->abort_flag) = 1;
        return false;
      }
      if (globaltimer_ns() - t0 > limit) {
        report_failure(P, ctrl, stage, ST_GRID_BARRIER_TIMEOUT, where);
        return false;
      }
    }
  }
}
// A global poller; with `announce` it also makes the shared-memory announcement.
__device__ __forceinline__ bool grid_wait(const Ctx& c, uint32_t stage, uint32_t where, bool announce) {
  const KernelParams& P = *c.P;
  if (stage == P.stage_begin) return true;
  const uint32_t target =
      P.epoch_base + (stage - P.stage_begin) * (gridDim.x / P.cluster) * (P.warp_arrive == 1u ? kSimtWarps : 1u);
  bool ok = true;
  if (static_cast<int32_t>(poll_load(P.barrier) - target) >= 0) {
    acquire_after_poll(P.barrier);
  } else {
    ok = grid_wait_slow(c.P, c.ctrl, target, stage, where);
  }
  if (ok && announce) st_release_cta_smem(&c.ctrl->barriers_seen, stage - P.stage_begin);
  return ok;
}
// Everybody else in the CTA: wait for the poller's announcement (acquire at CTA scope after the
// poller's acquire at GPU scope orders the other CTAs' stores before this thread's loads).
__device__ __noinline__ bool local_wait_slow(const KernelParams* P, Ctrl* ctrl, uint32_t need,
                                             uint32_t stage, uint32_t where) {
  const uint64_t t0 = globaltimer_ns();
  const uint64_t limit = static_cast<uint64_t>(P->timeout_us) * 1000ull;
  uint32_t it = 0;
  for (;;) {
    if (ld_acquire_cta_smem(&ctrl->barriers_seen) >= need) return true;
    if ((++it & 63u) == 0u) {
      if (*reinterpret_cast<volatile uint32_t*>(&ctrl->abort_flag)) return false;
      if (globaltimer_ns() - t0 > limit) {
        report_failure(P, ctrl, stage, ST_GRID_BARRIER_TIMEOUT, where);
        return false;
      }
    }
  }
}
__device__ __forceinline__ bool grid_wait_local(const Ctx& c, uint32_t stage, uint32_t where) {
  const KernelParams& P = *c.P;
  if (stage == P.stage_begin) return true;
  const uint32_t need = stage - P.stage_begin;
  if (ld_acquire_cta_smem(&c.ctrl->barriers_seen) >= need) return true;
  return local_wait_slow(c.P, c.ctrl, need, stage, where);
}

// Warp-collective variants for the epilogue warps: every lane gets the same answer, so a
// warp never splits around the warp-wide tcgen05.ld that follows.
__device__ __forceinline__ bool mbar_wait_warp(const Ctx& c, uint64_t* bar, uint32_t parity,
                                               uint32_t where) {
  const bool ok = mbar_wait(c, bar, parity, where);
  return __all_sync(0xffffffffu, ok);
}
__device__ __forceinline__ bool grid_wait_warp(const Ctx& c, uint32_t stage, uint32_t where) {
  bool ok = true;
  if ((threadIdx.x & 31u) == 0u)
#if MONONN_ALL_POLL
    ok = grid_wait(c, stage, where, threadIdx.x == kRoleThreads);
#else
    ok = (threadIdx.x == kRoleThreads) ? grid_wait(c, stage, where, true) : grid_wait_local(c, stage, where);
#endif
  return __all_sync(0xffffffffu, ok);
}
// A row op that shares a stage with the split-K GEMMs feeding it waits until all of their work
// items of this launch have added themselves to the arrival counter (each after its reductions,
// with release).
// Bounded like every wait; the waiting CTAs have no GEMM item left to do, so the GEMM items
// never depend on a waiter.
__device__ __noinline__ bool flag_wait_slow(const KernelParams* P, Ctrl* ctrl, const uint32_t* flag,
                                            uint32_t target, uint32_t stage, uint32_t where) {
  const uint64_t t0 = globaltimer_ns();
  const uint64_t limit = static_cast<uint64_t>(P->timeout_us) * 1000ull;
  uint32_t it = 0;
  for (;;) {
    if (static_cast<int32_t>(poll_load(flag) - target) >= 0) {
      acquire_after_poll(flag);
      return true;
    }
    if ((++it & 31u) == 0u) {
      if (*reinterpret_cast<volatile uint32_t*>(&ctrl->abort_flag)) return false;
      if (*reinterpret_cast<volatile uint32_t*>(&P->status->code) != 0u) {
        *reinterpret_cast<volatile uint32_t*>(&ctrl->abort_flag) = 1;
        return false;
      }
      if (globaltimer_ns() - t0 > limit) {
        report_failure(P, ctrl, stage, ST_GRID_BARRIER_TIMEOUT, where);
        return false;
      }
    }
  }
}
// The counter is never reset inside the kernel: like the grid-barrier counter it grows by the
// same amount every launch, and the host passes the number of launches since it was last
// cleared (flag_epoch), so the target is flag_epoch * arrivals-per-launch. No atomic with a
// return value, and so no extra L2 round trip, sits in the row op's critical path.
__device__ __forceinline__ bool flag_wait_warp(const Ctx& c, uint64_t counter, uint32_t per_launch, uint32_t where) {
  bool ok = true;
  if ((threadIdx.x & 31u) == 0u) {
    const uint32_t* flag = reinterpret_cast<const uint32_t*>(counter);
    const uint32_t target = c.P->flag_epoch * per_launch;
    if (static_cast<int32_t>(poll_load(flag) - target) >= 0) {
      acquire_after_poll(flag);
    } else {
      ok = flag_wait_slow(c.P, c.ctrl, flag, target, c.stage, where);
    }
  }
  return __all_sync(0xffffffffu, ok);
}
// One arrival for the whole warp on an mbarrier that counts the eight epilogue warps.
__device__ __forceinline__ void warp_arrive(uint64_t* bar) {
  __syncwarp();
  if ((threadIdx.x & 31u) == 0u) mbar_arrive(smem_u32(bar));
}
// Barrier across the 256 epilogue threads built on an mbarrier so that, unlike bar.sync,
// the wait is bounded when a warp has already left on the abort path.
__device__ __forceinline__ bool group_sync(Ctx& c, uint32_t where) {
  // one arrival per warp (the warp barrier orders the other lanes' accesses before it): 256
  // arrivals on one shared-memory word would serialise for a quarter of a microsecond
  __syncwarp();
  if ((threadIdx.x & 31u) == 0u) mbar_arrive(smem_u32(&c.ctrl->group_bar));
  const bool ok = mbar_wait(c, &c.ctrl->group_bar, c.group_phase, where);
  c.group_phase ^= 1u;
  return __all_sync(0xffffffffu, ok);
}

#define WAIT_OR_RETURN(expr) \
  do {                       \
    if (!(expr)) return;     \
  } while (0)

struct Item {
  const OpDesc* op;
  uint32_t local;  // item index inside the op
};

// Descriptors are read with straight-line code (no branch between two loads, which would
// serialise them) into registers / shared memory, and the first item's descriptor of a stage
// is fetched before the role waits for the previous stage's barrier.
__device__ __forceinline__ StageDesc load_stage(const KernelParams& P, uint32_t s) {
  StageDesc st;
  const uint4* g = reinterpret_cast<const uint4*>(P.stages + s);
  uint4* d = reinterpret_cast<uint4*>(&st);
  d[0] = __ldg(g);
  d[1] = __ldg(g + 1);
  d[2] = __ldg(g + 2);
  return st;
}

// Copies the descriptor of the operator that owns work item `item` of the stage into `slot`
// and returns it with the item's index inside that operator. WARP: all 32 lanes call it and
// share the slot; otherwise one thread does the copy.
template <bool WARP>
__device__ __forceinline__ Item fetch_item(const KernelParams& P, const StageDesc& st, uint32_t item,
                                           uint4* slot, uint32_t lane) {
  uint32_t k = 0, base = 0;
#pragma unroll
  for (int j = 0; j < 7; ++j) {  // unused entries of item_end are 0xffffffff
    const bool past = item >= st.item_end[j];
    k += past ? 1u : 0u;
    base = past ? st.item_end[j] : base;
  }
  const uint4* g = reinterpret_cast<const uint4*>(P.ops + st.op_begin + k);
  constexpr int kWords = sizeof(OpDesc) / 16;
  if (WARP) {
    __syncwarp();
    if (lane < kWords) slot[lane] = __ldg(g + lane);
    __syncwarp();
  } else {
    uint4 r[kWords];
#pragma unroll
    for (int i = 0; i < kWords; ++i) r[i] = __ldg(g + i);
#pragma unroll
    for (int i = 0; i < kWords; ++i) slot[i] = r[i];
  }
  return Item{reinterpret_cast<const OpDesc*>(slot), item - base};
}

struct GemmTile {
  uint32_t mt, nt, ks;
};
__device__ __forceinline__ GemmTile gemm_tile(const OpDesc& op, uint32_t local) {
  GemmTile t;
  t.ks = local % op.k_split;
  const uint32_t r = local / op.k_split;
  t.nt = r % op.n_tiles;
  t.mt = r / op.n_tiles;
  return t;
}

struct AttnTile {
  uint32_t b, h, mt;
};
__device__ __forceinline__ AttnTile attn_tile(const OpDesc& op, uint32_t local) {
  AttnTile t;
  const uint32_t mts = (op.seq + 127u) / 128u;
  t.mt = local % mts;
  const uint32_t r = local / mts;
  t.h = r % op.heads;
  t.b = r / op.heads;
  return t;
}

// Attention work item: 128 query rows of one (batch, head) against all keys, in chunks of
// 128 keys. All score chunks stay in TMEM (columns 0 .. 128*chunks) next to the output
// (columns kAttnOutCol..+63), so sequences up to 384 need no rescaling pass. Activation-ring
// slots of an item, in allocation order: Q, K_0..K_{n-1}, then per chunk V^T_j, P_j (two
// slots, written by the softmax warps).
constexpr uint32_t kAttnOutCol = 448;
// With F_FUSED_QKV (sequences up to 128) the item first computes [Q_h | K_h | V_h] = x_b W_h: the
// K/64 k-block tiles of x come through the activation ring before the five attention slots, the
// 192-column accumulator sits at columns kAttnQkvCol.., and the softmax warps turn it into the
// Q, K and V^T operand tiles in the slots that the activation producer would have loaded.
constexpr uint32_t kAttnQkvCol = 192;
__device__ __forceinline__ bool attn_fused(const OpDesc& op) { return (op.flags & F_FUSED_QKV) != 0u; }
__device__ __forceinline__ uint32_t attn_chunks(const OpDesc& op) { return (op.seq + 127u) / 128u; }
__device__ __forceinline__ uint32_t attn_slots(const OpDesc& op) {
  return 1u + 4u * attn_chunks(op) + (attn_fused(op) ? op.kb_per_split : 0u);
}

// The CTAs of a GEMM stage all walk the same K range of the A operand. Starting each CTA at
// a different k-block group (and wrapping around) spreads their simultaneous tile requests
// over the whole operand instead of hammering the L2 lines of one tile in lock-step. The
// rotation is in units of weight-ring groups and only used when the groups are all full, so
// that the MMA issuer's pairing of A slots with weight sub-tiles is unchanged.
__device__ __forceinline__ uint32_t k_rotation(uint32_t nkb, uint32_t kbps) {
  return (nkb % kbps == 0u) ? blockIdx.x % (nkb / kbps) : 0u;
}

// One elected lane of a converged producer warp issues the copy (with or without an L2 hint).
__device__ __forceinline__ void tma_issue(bool issuer, bool hint, uint32_t dst, const void* tmap, int32_t x,
                                          int32_t y, uint32_t bar, uint64_t policy) {
  if (!issuer) return;
  if (hint)
    tma_load_2d_hint(dst, tmap, x, y, bar, policy);
  else
    tma_load_2d(dst, tmap, x, y, bar);
}

// ----------------------------------------------------------------------------
// Role: weight producer (warp 0). Like the MMA role, the producers run all 32 lanes converged
// and one elected lane issues the copies and the barrier arrivals.
// ----------------------------------------------------------------------------
__device__ void role_weight_producer(Ctx c, uint32_t lane) {
  const KernelParams& P = *c.P;
  const bool issuer = elect_one_sync();
  const uint8_t* tmaps = static_cast<const uint8_t*>(P.tmaps);
  const bool hint = P.l2_hints != 0u;
  const uint64_t pol = l2_policy_evict_first();
  uint32_t b_cnt = 0;
  for (uint32_t s = P.stage_begin; s < P.stage_end; ++s) {
    c.stage = s;
    const StageDesc st = load_stage(P, s);
    {
      // If the stage holds attention items that compute their own projections, only a few SMs will
      // pull those weights, each through a three-slot ring. The CTAs that got none of those items
      // (idle in this stage, or holding items of operators that wait for the attention) bring the
      // weights into L2 now (this role runs ahead of the barriers), shared out among them, so that
      // the few stream them from L2 instead of HBM.
      const uint32_t busy = st.attn_prefetch_from;  // (found by the scheduler: no descriptor is read to learn it)
      if (busy != 0u && blockIdx.x >= busy) {
        const uint32_t n_idle = gridDim.x - busy, me = blockIdx.x - busy;
        for (uint32_t k = 0; k < st.op_count; ++k) {
          const OpDesc* gop = P.ops + st.op_begin + k;
          if (__ldg(&gop->kind) != OP_ATTENTION || !(__ldg(&gop->flags) & F_FUSED_QKV)) continue;
          const uint32_t chunks = (__ldg(&gop->heads) * __ldg(&gop->K) * 128u) >> 14;  // 16 KB units per weight
          for (uint32_t j = 0; j < 3; ++j) {
            const uint8_t* wbase = reinterpret_cast<const uint8_t*>(__ldg(&gop->p[5 + j]));
            for (uint32_t ch = me + lane * n_idle; ch < chunks; ch += 32u * n_idle)  // shared out over the lanes too
              asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(wbase + (static_cast<size_t>(ch) << 14)),
                           "r"(16384u)
                           : "memory");
          }
        }
      }
    }
    for (uint32_t item = blockIdx.x; item < st.n_items; item += gridDim.x) {
      const Item it = fetch_item<true>(P, st, item, c.ctrl->desc[0], lane);
      const OpDesc& op = *it.op;
      if (op.kind == OP_ATTENTION && attn_fused(op)) {
        // per k-block one slot: the 64-row tiles of head h of the Q, K and V weights, stacked
        const AttnTile t = attn_tile(op, it.local);
        const uint32_t nkb = op.kb_per_split;
        const void* tmw[3] = {tmaps + static_cast<size_t>(op.tmap_b) * 128u,
                              tmaps + static_cast<size_t>(op.tmap_vt) * 128u,
                              tmaps + static_cast<size_t>(op.vocab) * 128u};
        for (uint32_t kb = 0; kb < nkb; ++kb) {
          const uint32_t slot = b_cnt % kBSlots, use = b_cnt / kBSlots;
          WAIT_OR_RETURN(mbar_wait(c, &c.ctrl->b_empty[slot], (use & 1u) ^ 1u, 0x101));
          const uint32_t full = smem_u32(&c.ctrl->b_full[slot]);
          if (issuer) mbar_arrive_expect_tx(full, 3u * 8192u);
#pragma unroll
          for (uint32_t j = 0; j < 3; ++j) {
            tma_issue(issuer, hint, c.b_ring + slot * kBSlotBytes + j * 8192u, tmw[j], 0,
                               static_cast<int32_t>((t.h * nkb + kb) * 64u), full, pol);
          }
          ++b_cnt;
        }
        if (issuer) trace(P, s, TR_W_ISSUED);
        continue;
      }
      if (op.kind != OP_GEMM) continue;
      const GemmTile t = gemm_tile(op, it.local);
      const uint32_t nkb = op.kb_per_split, kbps = op.kb_per_bslot;
      const uint32_t kb_total = op.k_split * nkb;
      const uint32_t row0 = (t.nt * kb_total + t.ks * nkb) * op.n_tile;
      const uint32_t bytes = op.n_tile * kbps * 128u;
      const void* tm = tmaps + static_cast<size_t>(op.tmap_b) * 128u;
      const uint32_t groups = (nkb + kbps - 1) / kbps, rot = k_rotation(nkb, kbps);
      for (uint32_t gi = 0, grp = rot; gi < groups; ++gi) {
        const uint32_t kb = grp * kbps;  // ((gi + rot) % groups) * kbps
        if (++grp == groups) grp = 0;
        const uint32_t slot = b_cnt % kBSlots, use = b_cnt / kBSlots;
        WAIT_OR_RETURN(mbar_wait(c, &c.ctrl->b_empty[slot], (use & 1u) ^ 1u, 0x100));
        const uint32_t full = smem_u32(&c.ctrl->b_full[slot]);
        if (issuer) mbar_arrive_expect_tx(full, bytes);
        tma_issue(issuer, hint, c.b_ring + slot * kBSlotBytes, tm, 0, static_cast<int32_t>(row0 + kb * op.n_tile),
                           full, pol);
        ++b_cnt;
      }
      if (issuer) trace(P, s, TR_W_ISSUED);
    }
  }
}

// ----------------------------------------------------------------------------
// Role: activation producer (warp 1)
// ----------------------------------------------------------------------------
__device__ void role_act_producer(Ctx c, uint32_t lane) {
  const KernelParams& P = *c.P;
  const bool issuer = elect_one_sync();
  const uint8_t* tmaps = static_cast<const uint8_t*>(P.tmaps);
  const bool hint = P.l2_hints != 0u;
  const uint64_t pol = l2_policy_evict_last();
  uint32_t a_cnt = 0;
  for (uint32_t s = P.stage_begin; s < P.stage_end; ++s) {
    c.stage = s;
    const StageDesc st = load_stage(P, s);
    Item first{nullptr, 0};
    if (blockIdx.x < st.n_items) {
      first = fetch_item<true>(P, st, blockIdx.x, c.ctrl->desc[1], lane);
      const OpDesc& op0 = *first.op;
      if (issuer && (op0.kind == OP_GEMM || op0.kind == OP_ATTENTION)) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(tmaps + static_cast<size_t>(op0.tmap_a) * 128u));
        if (op0.kind == OP_ATTENTION) {
          asm volatile("prefetch.tensormap [%0];" ::"l"(tmaps + static_cast<size_t>(op0.tmap_b) * 128u));
          asm volatile("prefetch.tensormap [%0];" ::"l"(tmaps + static_cast<size_t>(op0.tmap_vt) * 128u));
        }
      }
    }
    bool waited = false;
    for (uint32_t item = blockIdx.x; item < st.n_items; item += gridDim.x) {
      const Item it = (item == blockIdx.x) ? first : fetch_item<true>(P, st, item, c.ctrl->desc[1], lane);
      const OpDesc& op = *it.op;
      if (op.kind != OP_GEMM && op.kind != OP_ATTENTION) continue;
      // everything the first copy needs is worked out before the wait (descriptor fields, tile
      // coordinates with their divisions), so that the copy is issued as soon as the barrier opens
      const bool is_gemm = op.kind == OP_GEMM;
      const GemmTile gt = is_gemm ? gemm_tile(op, it.local) : GemmTile{0u, 0u, 0u};
      const void* tm_a = tmaps + static_cast<size_t>(op.tmap_a) * 128u;
      const uint32_t g_nkb = op.kb_per_split, g_kbps = is_gemm ? op.kb_per_bslot : 1u;
      const uint32_t g_groups = (g_nkb + g_kbps - 1) / g_kbps, g_rot = is_gemm ? k_rotation(g_nkb, g_kbps) : 0u;
      const AttnTile at = is_gemm ? AttnTile{0u, 0u, 0u} : attn_tile(op, it.local);
      if (!waited) {
        bool ok = true;  // one lane polls the global counter; the acquire, the proxy fence and the copies are its
        if (issuer) ok = grid_wait(c, s, 0x200, false);
        WAIT_OR_RETURN(__all_sync(0xffffffffu, ok));
        fence_proxy_async_global();
        waited = true;
        if (issuer) trace(P, s, TR_ACT_READY);
      }
      if (op.kind == OP_GEMM) {
        if (op.wait_target != 0u) {
          // the A operand is the output of an attention operator of this stage: wait until all of
          // its items have counted themselves (each after its stores, with release), then make
          // those stores visible to the copies as after a grid barrier
          WAIT_OR_RETURN(flag_wait_warp(c, op.wait_flag, op.wait_target, 0x204));
          fence_proxy_async_global();
          if (issuer) trace(P, s, TR_MARK0 + 7);
        }
        const GemmTile t = gt;
        const void* tm = tm_a;
        const uint32_t nkb = g_nkb, kbps = g_kbps, groups = g_groups, rot = g_rot;
        // k block of step j: ((j / kbps + rot) % groups) * kbps + j % kbps, kept in two counters
        uint32_t grp = rot, in_grp = 0;
        for (uint32_t j = 0; j < nkb; ++j) {
          const uint32_t kb = grp * kbps + in_grp;
          if (++in_grp == kbps) {
            in_grp = 0;
            if (++grp == groups) grp = 0;
          }
          const uint32_t slot = a_cnt % kASlots, use = a_cnt / kASlots;
          WAIT_OR_RETURN(mbar_wait(c, &c.ctrl->a_empty[slot], (use & 1u) ^ 1u, 0x201));
          const uint32_t full = smem_u32(&c.ctrl->a_full[slot]);
          if (issuer) mbar_arrive_expect_tx(full, kSlotBytes);
          tma_issue(issuer, hint, c.a_ring + slot * kSlotBytes, tm, static_cast<int32_t>((t.ks * nkb + kb) * 64u),
                             static_cast<int32_t>(t.mt * 128u), full, pol);
          ++a_cnt;
        }
      } else {
        const AttnTile t = at;
        const void* tm = tm_a;
        const void* tmk = tmaps + static_cast<size_t>(op.tmap_b) * 128u;
        const void* tmv = tmaps + static_cast<size_t>(op.tmap_vt) * 128u;
        const uint32_t nc = attn_chunks(op);
        if (attn_fused(op)) {
          // the k-block tiles of this batch's rows of x; Q, K, V^T and P are written on chip
          for (uint32_t kb = 0; kb < op.kb_per_split; ++kb) {
            const uint32_t slot = a_cnt % kASlots, use = a_cnt / kASlots;
            WAIT_OR_RETURN(mbar_wait(c, &c.ctrl->a_empty[slot], (use & 1u) ^ 1u, 0x203));
            const uint32_t full = smem_u32(&c.ctrl->a_full[slot]);
            if (issuer) mbar_arrive_expect_tx(full, kSlotBytes);
            tma_issue(issuer, false, c.a_ring + slot * kSlotBytes, tm, static_cast<int32_t>(kb * 64u),
                        static_cast<int32_t>(t.b * op.seq), full, 0ull);
            ++a_cnt;
          }
          a_cnt += 5;
          if (issuer) trace(P, s, TR_ACT_ISSUED);
          continue;
        }
        // Q, K_0 .. K_{nc-1}, then V^T_j for every chunk (the P slots in between are skipped)
        for (uint32_t j = 0; j < 1u + 2u * nc; ++j) {
          if (j > nc) a_cnt += (j == nc + 1u) ? 0u : 2u;  // step over the previous chunk's P slots
          const uint32_t slot = a_cnt % kASlots, use = a_cnt / kASlots;
          WAIT_OR_RETURN(mbar_wait(c, &c.ctrl->a_empty[slot], (use & 1u) ^ 1u, 0x202));
          const uint32_t full = smem_u32(&c.ctrl->a_full[slot]);
          const uint32_t dst = c.a_ring + slot * kSlotBytes;
          if (issuer) mbar_arrive_expect_tx(full, kSlotBytes);
          if (j == 0) {
            tma_issue(issuer, false, dst, tm, static_cast<int32_t>(op.q_col + t.h * 64u),
                        static_cast<int32_t>(t.b * op.seq + t.mt * 128u), full, 0ull);
          } else if (j <= nc) {
            tma_issue(issuer, false, dst, tmk, static_cast<int32_t>(op.k_col + t.h * 64u),
                        static_cast<int32_t>(t.b * op.seq + (j - 1u) * 128u), full, 0ull);
          } else {
            const int32_t x = static_cast<int32_t>((j - nc - 1u) * 128u);
            const int32_t y = static_cast<int32_t>((t.b * op.heads + t.h) * 64u);
            tma_issue(issuer, false, dst, tmv, x, y, full, 0ull);
            tma_issue(issuer, false, dst + 8192u, tmv, x + 64, y, full, 0ull);
          }
          ++a_cnt;
        }
        a_cnt += 2;  // the last chunk's P slots
      }
      if (issuer) trace(P, s, TR_ACT_ISSUED);
    }
  }
}

// ----------------------------------------------------------------------------
// Role: MMA issuer (warp 2). All 32 lanes run the loop converged and one elected lane issues the
// tcgen05 instructions: the operands of a converged warp can be kept in uniform registers, and
// a loop of four instructions, a commit and a wait per k block measured 88 cycles per
// instruction this way against 121 when a single lane ran it (probe: mononn_debug_mma_issue).
// ----------------------------------------------------------------------------
__device__ void role_mma(Ctx c, uint32_t tmem_base, uint32_t lane) {
  const KernelParams& P = *c.P;
  const bool issuer = elect_one_sync();
  uint32_t a_cnt = 0, b_cnt = 0, acc_cnt = 0;
  for (uint32_t s = P.stage_begin; s < P.stage_end; ++s) {
    c.stage = s;
    const StageDesc st = load_stage(P, s);
    for (uint32_t item = blockIdx.x; item < st.n_items; item += gridDim.x) {
      const Item it = fetch_item<true>(P, st, item, c.ctrl->desc[2], lane);
      const OpDesc& op = *it.op;
      if (op.kind == OP_GEMM) {
        const uint32_t nkb = op.kb_per_split, kbps = op.kb_per_bslot;
        const uint32_t buf = acc_cnt & 1u;
        WAIT_OR_RETURN(mbar_wait(c, &c.ctrl->acc_empty[buf], ((acc_cnt >> 1) & 1u) ^ 1u, 0x300));
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + buf * kAccCols;
        const uint32_t idesc = umma_idesc_m128(op.n_tile);
        uint32_t b_slot = 0;
        for (uint32_t kb = 0, next_sub = 0; kb < nkb; ++kb) {
          const uint32_t sub = next_sub;  // kb % kbps without the division (this loop is bound by its issue path)
          next_sub = (sub + 1u == kbps) ? 0u : sub + 1u;
          if (sub == 0) {
            b_slot = b_cnt % kBSlots;
            WAIT_OR_RETURN(mbar_wait(c, &c.ctrl->b_full[b_slot], (b_cnt / kBSlots) & 1u, 0x301));
          }
          const uint32_t a_slot = a_cnt % kASlots;
          WAIT_OR_RETURN(mbar_wait(c, &c.ctrl->a_full[a_slot], (a_cnt / kASlots) & 1u, 0x302));
          if (kb == 0) if (issuer) trace(P, s, TR_MMA_FIRST);
          tc_fence_after();
          const uint64_t ad = umma_desc_sw128(c.a_ring + a_slot * kSlotBytes);
          const uint64_t bd =
              umma_desc_sw128(c.b_ring + b_slot * kBSlotBytes + sub * op.n_tile * 128u);
#pragma unroll
          for (uint32_t k = 0; k < 4; ++k)
            if (issuer) tc_mma_f16(tmem_d, ad + 2u * k, bd + 2u * k, idesc, (kb | k) != 0u);
          if (issuer) tc_commit(smem_u32(&c.ctrl->a_empty[a_slot]));
          ++a_cnt;
          if (sub + 1 == kbps || kb + 1 == nkb) {
            if (issuer) tc_commit(smem_u32(&c.ctrl->b_empty[b_slot]));
            ++b_cnt;
          }
        }
        if (issuer) tc_commit(smem_u32(&c.ctrl->acc_full[buf]));
        ++acc_cnt;
        if (issuer) trace(P, s, TR_MMA_LAST);
      } else if (op.kind == OP_ATTENTION) {
        const uint32_t nc = attn_chunks(op);
        uint32_t base = a_cnt, ph = acc_cnt;
        a_cnt += attn_slots(op);
        auto slot_of = [](uint32_t cnt) { return cnt % kASlots; };
        auto par_of = [](uint32_t cnt) { return (cnt / kASlots) & 1u; };
        if (attn_fused(op)) {
          // [Q_h | K_h | V_h] = x_b W_h into 192 columns; the accumulator overlaps both GEMM buffers
          const uint32_t phQ = ph++, nkb = op.kb_per_split;
          WAIT_OR_RETURN(mbar_wait(c, &c.ctrl->acc_empty[phQ & 1u], ((phQ >> 1) & 1u) ^ 1u, 0x320));
          WAIT_OR_RETURN(mbar_wait(c, &c.ctrl->acc_empty[ph & 1u], ((ph >> 1) & 1u) ^ 1u, 0x321));
          tc_fence_after();
          const uint32_t idesc = umma_idesc_m128(192);
          for (uint32_t kb = 0; kb < nkb; ++kb) {
            const uint32_t b_slot = b_cnt % kBSlots, a_c = base + kb;
            WAIT_OR_RETURN(mbar_wait(c, &c.ctrl->b_full[b_slot], (b_cnt / kBSlots) & 1u, 0x322));
            WAIT_OR_RETURN(mbar_wait(c, &c.ctrl->a_full[slot_of(a_c)], par_of(a_c), 0x323));
            if (kb == 0) if (issuer) trace(P, s, TR_MMA_FIRST);
            tc_fence_after();
            const uint64_t ad = umma_desc_sw128(c.a_ring + slot_of(a_c) * kSlotBytes);
            const uint64_t bd = umma_desc_sw128(c.b_ring + b_slot * kBSlotBytes);
#pragma unroll
            for (uint32_t k = 0; k < 4; ++k)
              if (issuer) tc_mma_f16(tmem_base + kAttnQkvCol, ad + 2u * k, bd + 2u * k, idesc, (kb | k) != 0u);
            if (issuer) tc_commit(smem_u32(&c.ctrl->a_empty[slot_of(a_c)]));
            if (issuer) tc_commit(smem_u32(&c.ctrl->b_empty[b_slot]));
            ++b_cnt;
          }
          if (issuer) tc_commit(smem_u32(&c.ctrl->acc_full[phQ & 1u]));
          if (issuer) trace(P, s, TR_MMA_LAST);
          base += nkb;
        }
        // the scores may span both accumulator buffers: both must have been drained
        const uint32_t phS = ph, phO = ph + 1u;
        WAIT_OR_RETURN(mbar_wait(c, &c.ctrl->acc_empty[phS & 1u], ((phS >> 1) & 1u) ^ 1u, 0x310));
        WAIT_OR_RETURN(mbar_wait(c, &c.ctrl->acc_empty[phO & 1u], ((phO >> 1) & 1u) ^ 1u, 0x313));
        // S_j = Q K_j^T  (128 x 128, K = 64) into columns j*128
        WAIT_OR_RETURN(mbar_wait(c, &c.ctrl->a_full[slot_of(base)], par_of(base), 0x311));
        for (uint32_t j = 0; j < nc; ++j) {
          const uint32_t kc = base + 1u + j;
          WAIT_OR_RETURN(mbar_wait(c, &c.ctrl->a_full[slot_of(kc)], par_of(kc), 0x312));
          tc_fence_after();
          const uint64_t ad = umma_desc_sw128(c.a_ring + slot_of(base) * kSlotBytes);
          const uint64_t bd = umma_desc_sw128(c.a_ring + slot_of(kc) * kSlotBytes);
          const uint32_t idesc = umma_idesc_m128(128);
#pragma unroll
          for (uint32_t k = 0; k < 4; ++k)
            if (issuer) tc_mma_f16(tmem_base + j * 128u, ad + 2u * k, bd + 2u * k, idesc, k != 0u);
          if (issuer) tc_commit(smem_u32(&c.ctrl->a_empty[slot_of(kc)]));
        }
        if (issuer) tc_commit(smem_u32(&c.ctrl->a_empty[slot_of(base)]));
        if (issuer) tc_commit(smem_u32(&c.ctrl->acc_full[phS & 1u]));
        // O += P_j V_j  (128 x 64, K = 128 per chunk) into columns kAttnOutCol..
        for (uint32_t j = 0; j < nc; ++j) {
          const uint32_t vc = base + 1u + nc + 3u * j;
          WAIT_OR_RETURN(mbar_wait(c, &c.ctrl->a_full[slot_of(vc)], par_of(vc), 0x314));
          WAIT_OR_RETURN(mbar_wait(c, &c.ctrl->a_full[slot_of(vc + 1u)], par_of(vc + 1u), 0x315));
          WAIT_OR_RETURN(mbar_wait(c, &c.ctrl->a_full[slot_of(vc + 2u)], par_of(vc + 2u), 0x316));
          tc_fence_after();
          const uint32_t idesc = umma_idesc_m128(64);
#pragma unroll
          for (uint32_t kb = 0; kb < 2; ++kb) {
            const uint64_t ad = umma_desc_sw128(c.a_ring + slot_of(vc + 1u + kb) * kSlotBytes);
            const uint64_t bd = umma_desc_sw128(c.a_ring + slot_of(vc) * kSlotBytes + kb * 8192u);
#pragma unroll
            for (uint32_t k = 0; k < 4; ++k)
              if (issuer) tc_mma_f16(tmem_base + kAttnOutCol, ad + 2u * k, bd + 2u * k, idesc, (j | kb | k) != 0u);
          }
          for (uint32_t q = 0; q < 3; ++q) if (issuer) tc_commit(smem_u32(&c.ctrl->a_empty[slot_of(vc + q)]));
        }
        if (issuer) tc_commit(smem_u32(&c.ctrl->acc_full[phO & 1u]));
        acc_cnt = ph + 2u;
      }
    }
  }
}

// ----------------------------------------------------------------------------
// Epilogue / SIMT math. Everything here runs once per stage on four warps, so the code
// is kept compact (chunk loops are not unrolled, slow paths are out of line): the whole
// kernel has to stay resident in the instruction cache across a layer's stages.
// ----------------------------------------------------------------------------
__device__ __forceinline__ float gelu_erf_f(float x) {
  // erf by the rational form 1 - (a1 t + .. + a5 t^5) exp(-z^2), t = 1/(1 + p z), whose
  // absolute error (1.5e-7) is far below the f16 resolution of the stored result
  const float z = fabsf(x) * 0.70710678118654752f;
  const float t = __fdividef(1.0f, fmaf(0.3275911f, z, 1.0f));
  float p = fmaf(t, 1.061405429f, -1.453152027f);
  p = fmaf(t, p, 1.421413741f);
  p = fmaf(t, p, -0.284496736f);
  p = fmaf(t, p, 0.254829592f);
  const float e = 1.0f - p * t * __expf(-z * z);
  return 0.5f * x * (1.0f + copysignf(e, x));
}

__device__ __forceinline__ void apply_act16(float (&v)[16], uint32_t act) {
  if (act == ACT_GELU_ERF) {
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = gelu_erf_f(v[i]);
  } else if (act == ACT_RELU) {
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = fmaxf(v[i], 0.0f);
  } else if (act == ACT_QUICK_GELU) {
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __fdividef(v[i], 1.0f + __expf(-1.702f * v[i]));
  } else if (act == ACT_GELU_TANH) {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const float u = 0.7978845608028654f * fmaf(0.044715f * v[i] * v[i], v[i], v[i]);
      // 0.5 (1 + tanh u) = 1 / (1 + exp(-2u))
      v[i] = __fdividef(v[i], 1.0f + __expf(-2.0f * u));
    }
  }
}

// 32 consecutive floats of a shared-memory table (16-byte aligned) as eight vector loads issued
// back to back. Per-element scalar loads next to their uses left each multiply waiting for its
// own load: with one warp per scheduler that was ~20 cycles per element.
__device__ __forceinline__ void lds32(const float* p, float (&m)[32]) {
  const float4* q = reinterpret_cast<const float4*>(p);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float4 t = q[i];
    m[4 * i] = t.x; m[4 * i + 1] = t.y; m[4 * i + 2] = t.z; m[4 * i + 3] = t.w;
  }
}
// mk[i] += log2(e) * bias[i] for 32 consecutive f16 values (64-byte aligned: four vector loads)
__device__ __forceinline__ void add_bias32(const __half* p, float (&mk)[32]) {
  const uint4* q = reinterpret_cast<const uint4*>(p);
  uint4 r[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) r[i] = __ldg(q + i);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __half2* h = reinterpret_cast<const __half2*>(&r[i]);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __half22float2(h[j]);
      mk[8 * i + 2 * j] = fmaf(f.x, 1.4426950408889634f, mk[8 * i + 2 * j]);
      mk[8 * i + 2 * j + 1] = fmaf(f.y, 1.4426950408889634f, mk[8 * i + 2 * j + 1]);
    }
  }
}
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
  const __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&h);
}
__device__ __forceinline__ float4 h4_to_f4(uint2 u) {
  const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&u.x));
  const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&u.y));
  return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void add4(float4& a, const float4 b) {
  a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
}

// Accumulator row `quarter * 32 + lane` (TMEM lane = row) is shared by the two warps of the
// quarter: warp `half` takes every other column group of the tile (groups of 32 columns, of 16
// for tiles up to 32 wide so that both warps have work).
__device__ __noinline__ void gemm_epilogue(const OpDesc& op, const GemmTile t, uint32_t tmem_acc,
                                           uint32_t quarter, uint32_t half, uint32_t lane,
                                           const float* bias_s, uint8_t* stg) {
  const uint32_t grow = t.mt * 128u + quarter * 32u + lane;
  const bool row_ok = grow < op.M;
  const bool lead = (t.ks == 0);
  const uint32_t n0 = t.nt * op.n_tile;
  const uint32_t flags = op.flags, act = op.act, out_mode = op.out_mode, N = op.N;
  const uint32_t ldo = op.ldo, ldr = op.ldr, n_tile = op.n_tile;
  const float alpha = op.alpha;
  const uint64_t pout = op.p[0], presid = op.p[2];
  const bool bias_on = (flags & F_BIAS) && lead, resid_on = (flags & F_RESID) && lead;
  // row-major f16 output: a 32-column group is collected in the warp's staging block (32 rows x
  // 64 bytes, swizzled) and stored four lanes to a row instead of one row per lane
  const bool staged = (out_mode == OUT_F16);
  // transposed output: batch and row inside the batch of this thread's row, once per item
  const uint32_t t_batch = (out_mode == OUT_F16_T) ? grow / op.rows_per_batch : 0u;
  const uint32_t t_row = (out_mode == OUT_F16_T) ? grow - t_batch * op.rows_per_batch : 0u;
  const uint32_t sw = (lane >> 1) & 3u;
  const uint32_t gstep = (n_tile <= 32u) ? 16u : 32u;
#pragma unroll 1
  for (uint32_t g0 = half * gstep; g0 < n_tile; g0 += 2u * gstep) {
    const uint32_t gw = (n_tile - g0 < gstep) ? n_tile - g0 : gstep;  // 16 or 32 columns
#pragma unroll 1
    for (uint32_t c0 = g0; c0 < g0 + gw; c0 += 16) {
      float v[16];
      tc_ld16(tmem_acc + ((quarter * 32u) << 16) + c0, v);
      const uint32_t col = n0 + c0;
      if (row_ok && col < N) {
        if (alpha != 1.0f) {
#pragma unroll
          for (int i = 0; i < 16; ++i) v[i] *= alpha;
        }
        if (bias_on) {
          const float4* bq = reinterpret_cast<const float4*>(bias_s + c0);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float4 t = bq[i];
            v[4 * i] += t.x; v[4 * i + 1] += t.y; v[4 * i + 2] += t.z; v[4 * i + 3] += t.w;
          }
        }
        apply_act16(v, act);
        if (resid_on) {
          if (flags & F_RESID_F32) {
            const float4* r = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(presid) +
                                                              static_cast<size_t>(grow) * ldr + col);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const float4 x = __ldcg(r + i);
              v[4 * i] += x.x; v[4 * i + 1] += x.y; v[4 * i + 2] += x.z; v[4 * i + 3] += x.w;
            }
          } else {
            const uint2* r = reinterpret_cast<const uint2*>(reinterpret_cast<const __half*>(presid) +
                                                            static_cast<size_t>(grow) * ldr + col);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const float4 x = h4_to_f4(__ldcg(r + i));
              v[4 * i] += x.x; v[4 * i + 1] += x.y; v[4 * i + 2] += x.z; v[4 * i + 3] += x.w;
            }
          }
        }
        if (out_mode == OUT_F16) {
          const uint32_t ch = (c0 - g0) >> 3;  // 0 or 2
          *reinterpret_cast<uint4*>(stg + lane * 64u + ((ch ^ sw) << 4)) =
              make_uint4(pack_h2(v[0], v[1]), pack_h2(v[2], v[3]), pack_h2(v[4], v[5]), pack_h2(v[6], v[7]));
          *reinterpret_cast<uint4*>(stg + lane * 64u + (((ch + 1u) ^ sw) << 4)) =
              make_uint4(pack_h2(v[8], v[9]), pack_h2(v[10], v[11]), pack_h2(v[12], v[13]), pack_h2(v[14], v[15]));
        } else if (out_mode == OUT_F32_RED) {
          float* o = reinterpret_cast<float*>(pout) + static_cast<size_t>(grow) * ldo + col;
#pragma unroll
          for (int i = 0; i < 4; ++i)
            red_add_f32x4(o + 4 * i, v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
        } else if (out_mode == OUT_F16_T) {
          const uint32_t b = t_batch, rib = t_row;
          const uint32_t ldt = op.ldt;
          __half* o = reinterpret_cast<__half*>(pout) + (static_cast<size_t>(b) * N + col) * ldt + rib;
#pragma unroll
          for (int i = 0; i < 16; ++i) o[static_cast<size_t>(i) * ldt] = __float2half_rn(v[i]);
        } else {
          float4* o = reinterpret_cast<float4*>(reinterpret_cast<float*>(pout) +
                                                static_cast<size_t>(grow) * ldo + col);
#pragma unroll
          for (int i = 0; i < 4; ++i)
            o[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
        }
      }  // row_ok && col < N
    }
    if (staged) {
      __syncwarp();
      const uint32_t chunks = gw >> 3;  // 16-byte chunks per row in this group (2 or 4)
      const uint32_t chunk_shift = chunks >> 1;  // log2(chunks): no division in the store loop
      const uint32_t row0 = t.mt * 128u + quarter * 32u;
      for (uint32_t idx = lane; idx < 32u * chunks; idx += 32u) {
        const uint32_t r = idx >> chunk_shift, q = idx & (chunks - 1u);
        const uint32_t gcol = n0 + g0 + q * 8u;
        if (row0 + r < op.M && gcol < N)
          *reinterpret_cast<uint4*>(reinterpret_cast<__half*>(pout) + static_cast<size_t>(row0 + r) * ldo + gcol) =
              *reinterpret_cast<const uint4*>(stg + r * 64u + ((q ^ ((r >> 1) & 3u)) << 4));
      }
      __syncwarp();
    }
  }
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Sources of one row of a row-wise op (LayerNorm or embedding): up to three addends.
struct RowSrc {
  const float4* f32;   // f32 accumulator row (LayerNorm), cleared after reading when `zero`
  const uint2* h0;     // f16 row: LayerNorm source, or the gathered word row
  const uint2* h1;     // f16 row: residual, or the position row
  const uint2* h2;     // f16 row: token-type row
  bool zero;
};
// Loads only: the optional clearing of the f32 source is a separate step, because a store
// between the loads would keep the compiler from issuing them back to back.
__device__ __forceinline__ float4 row_chunk(const RowSrc& s, uint32_t vi) {
  float4 a;
  if (s.f32 != nullptr) {
    a = __ldcg(s.f32 + vi);
  } else {
    a = h4_to_f4(__ldcg(s.h0 + vi));
  }
  if (s.h1 != nullptr) add4(a, h4_to_f4(__ldcg(s.h1 + vi)));
  if (s.h2 != nullptr) add4(a, h4_to_f4(__ldcg(s.h2 + vi)));
  return a;
}
__device__ __forceinline__ void row_emit(float4 a, float mean, float rstd, uint32_t vi,
                                         uint2 gv, uint2 bv, uint2 b2v, uint2* out, float4* out2,
                                         bool add_bias2, bool no_norm, bool l2 = false) {
  float4 g = h4_to_f4(gv), b = h4_to_f4(bv);
  if (l2) {
    g = make_float4(1.f, 1.f, 1.f, 1.f);
    b = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  float4 y = a;
  if (!no_norm) {
    y.x = (a.x - mean) * rstd * g.x + b.x;
    y.y = (a.y - mean) * rstd * g.y + b.y;
    y.z = (a.z - mean) * rstd * g.z + b.z;
    y.w = (a.w - mean) * rstd * g.w + b.w;
  }
  if (out != nullptr) {
    uint2 o;
    o.x = pack_h2(y.x, y.y);
    o.y = pack_h2(y.z, y.w);
    out[vi] = o;
  }
  if (out2 != nullptr) {
    if (add_bias2) add4(y, h4_to_f4(b2v));
    out2[vi] = y;
  }
}

// LayerNorm / embedding item: eight rows, one warp each. Rows up to 1024 columns stay in
// registers between the statistics and the normalisation; wider rows are re-read.
__device__ __noinline__ void rowwise_item(const OpDesc& op, uint32_t local, uint32_t warp_in_group,
                                          uint32_t lane, const KernelParams& P, uint32_t stage) {
  const uint32_t row = local * kRowsPerItem + warp_in_group;
  if (row >= op.rows) return;
  const bool mark = (warp_in_group == 0 && lane == 0);
  if (mark) trace(P, stage, TR_MARK0);
  const uint32_t cols = op.cols, nvec = cols >> 2, flags = op.flags;
  const bool embed = (op.kind == OP_EMBED), assemble = (op.kind == OP_ASSEMBLE);
  const bool no_norm = (flags & F_NO_NORM) != 0u, l2 = (flags & F_L2NORM) != 0u, rms = (flags & F_RMSNORM) != 0u;
  RowSrc s{nullptr, nullptr, nullptr, nullptr, false};
  if (assemble) {
    // token row t of batch b: the first k_col rows come from a constant table (class token),
    // the others from the patch GEMM's output plus its bias; every row adds its position row
    const uint32_t t = row % op.seq, b = row / op.seq, prefix = op.k_col;
    if (t < prefix) {
      s.h0 = reinterpret_cast<const uint2*>(reinterpret_cast<const __half*>(op.p[3]) +
                                            static_cast<size_t>(t) * cols);
    } else {
      s.h0 = reinterpret_cast<const uint2*>(
          reinterpret_cast<const __half*>(op.p[1]) +
          (static_cast<size_t>(b) * (op.seq - prefix) + (t - prefix)) * op.lds);
      if (flags & F_BIAS) s.h2 = reinterpret_cast<const uint2*>(op.p[5]);
    }
    s.h1 = reinterpret_cast<const uint2*>(reinterpret_cast<const __half*>(op.p[4]) +
                                          static_cast<size_t>(t) * cols);
  } else if (embed) {
    const int32_t id = reinterpret_cast<const int32_t*>(op.p[1])[row];
    s.h0 = reinterpret_cast<const uint2*>(reinterpret_cast<const __half*>(op.p[3]) +
                                          static_cast<int64_t>(id) * cols);
    if (op.p[4] != 0)  // (a model without learned positions has no table: T5)
      s.h1 = reinterpret_cast<const uint2*>(reinterpret_cast<const __half*>(op.p[4]) +
                                            static_cast<size_t>(row % op.seq + op.q_col) * cols);
    if (flags & F_TYPE_IDS) {
      const int32_t ty = reinterpret_cast<const int32_t*>(op.p[2])[row];
      s.h2 = reinterpret_cast<const uint2*>(reinterpret_cast<const __half*>(op.p[5]) +
                                            static_cast<int64_t>(ty) * cols);
    }
    if ((flags & F_MASK_BIAS) && lane == 0) {
      const int32_t m = reinterpret_cast<const int32_t*>(op.q[0])[row];
      reinterpret_cast<float*>(op.q[1])[row] = (1.0f - static_cast<float>(m)) * op.alpha;
    }
  } else {
    if (flags & F_SRC_F32) {
      s.f32 = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(op.p[1]) +
                                              static_cast<size_t>(row) * op.lds);
      s.zero = (flags & F_ZERO_SRC) != 0u;
    } else {
      s.h0 = reinterpret_cast<const uint2*>(reinterpret_cast<const __half*>(op.p[1]) +
                                            static_cast<size_t>(row) * op.lds);
    }
    if (flags & F_RESID)
      s.h1 = reinterpret_cast<const uint2*>(reinterpret_cast<const __half*>(op.p[4]) +
                                            static_cast<size_t>(row) * op.ldr);
  }
  // (row ops without normalisation still get valid scale/shift pointers from the host, so
  // that the loads below stay unconditional)
  const uint2* gamma = reinterpret_cast<const uint2*>((embed || assemble) ? op.p[6] : op.p[2]);
  const uint2* beta = reinterpret_cast<const uint2*>((embed || assemble) ? op.p[7] : op.p[3]);
  uint2* out = op.p[0] ? reinterpret_cast<uint2*>(reinterpret_cast<__half*>(op.p[0]) +
                                                  static_cast<size_t>(row) * op.ldo)
                       : nullptr;
  float4* out2 = op.q[2] ? reinterpret_cast<float4*>(reinterpret_cast<float*>(op.q[2]) +
                                                     static_cast<size_t>(row) * cols)
                         : nullptr;
  const uint2* bias2 = reinterpret_cast<const uint2*>(op.q[3]);
  const float inv_n = 1.0f / static_cast<float>(cols), eps = op.eps;

  const bool add_bias2 = (out2 != nullptr) && (bias2 != nullptr);
  if (nvec <= 256u) {
    // Every global load of the row is issued before anything waits on one of them. The
    // loops are straight-line code (source kind decided outside, out-of-range chunks read
    // chunk 0 and are zeroed afterwards): a branch between two loads would make the
    // hardware wait for the first before issuing the second.
    float4 x[8];
    uint2 gv[8], bv[8], b2v[8];
    uint32_t vj[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) vj[i] = (i * 32u + lane < nvec) ? i * 32u + lane : 0u;
    if (s.f32 != nullptr) {
#pragma unroll
      for (int i = 0; i < 8; ++i) x[i] = __ldcg(s.f32 + vj[i]);
    } else {
      uint2 h[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) h[i] = __ldcg(s.h0 + vj[i]);
#pragma unroll
      for (int i = 0; i < 8; ++i) x[i] = h4_to_f4(h[i]);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      gv[i] = __ldg(gamma + vj[i]);
      bv[i] = __ldg(beta + vj[i]);
    }
    if (add_bias2) {
#pragma unroll
      for (int i = 0; i < 8; ++i) b2v[i] = __ldg(bias2 + vj[i]);
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) b2v[i] = make_uint2(0u, 0u);
    }
    if (s.h1 != nullptr) {
      uint2 h[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) h[i] = __ldcg(s.h1 + vj[i]);
#pragma unroll
      for (int i = 0; i < 8; ++i) add4(x[i], h4_to_f4(h[i]));
    }
    if (s.h2 != nullptr) {
      uint2 h[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) h[i] = __ldcg(s.h2 + vj[i]);
#pragma unroll
      for (int i = 0; i < 8; ++i) add4(x[i], h4_to_f4(h[i]));
    }
    if (s.zero) {
#pragma unroll
      for (int i = 0; i < 8; ++i)
        if (i * 32u + lane < nvec)
          const_cast<float4*>(s.f32)[i * 32u + lane] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (i * 32u + lane >= nvec) x[i] = make_float4(0.f, 0.f, 0.f, 0.f);
      sum += x[i].x + x[i].y + x[i].z + x[i].w;
    }
    if (mark) trace(P, stage, TR_MARK0 + 1);
    const float mean = (l2 || rms) ? 0.f : warp_sum(sum) * inv_n;
    float sq = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (i * 32u + lane < nvec) {
        const float a = x[i].x - mean, b = x[i].y - mean, c = x[i].z - mean, d = x[i].w - mean;
        sq += a * a + b * b + c * c + d * d;
      }
    const float rstd = l2 ? rsqrtf(warp_sum(sq)) : rsqrtf(warp_sum(sq) * inv_n + eps);
    if (rms) {  // no shift: the host binds the scale vector as the shift pointer too
#pragma unroll
      for (int i = 0; i < 8; ++i) bv[i] = make_uint2(0u, 0u);
    }
    if (!no_norm && !l2 && out != nullptr) {
      // the common LayerNorm: the per-item choices are made once here, not per 8-byte group (a
      // branch costs a warp that is alone on its scheduler some twenty cycles)
      const bool two = (out2 != nullptr);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const uint32_t vi = i * 32u + lane;
        if (vi < nvec) {
          const float4 g = h4_to_f4(gv[i]), b = h4_to_f4(bv[i]);
          float4 y;
          y.x = (x[i].x - mean) * rstd * g.x + b.x;
          y.y = (x[i].y - mean) * rstd * g.y + b.y;
          y.z = (x[i].z - mean) * rstd * g.z + b.z;
          y.w = (x[i].w - mean) * rstd * g.w + b.w;
          uint2 o;
          o.x = pack_h2(y.x, y.y);
          o.y = pack_h2(y.z, y.w);
          out[vi] = o;
          x[i] = y;
        }
      }
      if (two) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const uint32_t vi = i * 32u + lane;
          if (vi < nvec) {
            float4 y = x[i];
            add4(y, h4_to_f4(b2v[i]));  // zero when there is no bias to pre-load
            out2[vi] = y;
          }
        }
      }
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const uint32_t vi = i * 32u + lane;
        if (vi < nvec) row_emit(x[i], mean, rstd, vi, gv[i], bv[i], b2v[i], out, out2, add_bias2, no_norm, l2);
      }
    }
  } else {
    // wide rows: three passes over the (L2-resident) sources
    float sum = 0.f;
#pragma unroll 1
    for (uint32_t vi = lane; vi < nvec; vi += 32u) {
      const float4 a = row_chunk(s, vi);
      sum += a.x + a.y + a.z + a.w;
    }
    const float mean = (l2 || rms) ? 0.f : warp_sum(sum) * inv_n;
    float sq = 0.f;
#pragma unroll 1
    for (uint32_t vi = lane; vi < nvec; vi += 32u) {
      const float4 a = row_chunk(s, vi);
      const float e = a.x - mean, f = a.y - mean, g = a.z - mean, h = a.w - mean;
      sq += e * e + f * f + g * g + h * h;
    }
    const float rstd = l2 ? rsqrtf(warp_sum(sq)) : rsqrtf(warp_sum(sq) * inv_n + eps);
#pragma unroll 1
    for (uint32_t vi = lane; vi < nvec; vi += 32u) {
      const float4 a = row_chunk(s, vi);
      if (s.zero) const_cast<float4*>(s.f32)[vi] = make_float4(0.f, 0.f, 0.f, 0.f);
      row_emit(a, mean, rstd, vi, __ldg(gamma + vi), rms ? make_uint2(0u, 0u) : __ldg(beta + vi),
               add_bias2 ? __ldg(bias2 + vi) : make_uint2(0u, 0u), out, out2, add_bias2, no_norm, l2);
    }
  }
  if (mark) trace(P, stage, TR_MARK0 + 2);
}

// Scale, shift and pre-load bias of a row op are small constants that every layer reads once.
// The weight stream (larger than L2) evicts them between their uses, so a row op asks for them
// again while it waits for its inputs (grid barrier or arrival counter): the loads in
// rowwise_item then hit L2 instead of paying an HBM round trip on the critical path.
__device__ __forceinline__ void prefetch_row_consts(const OpDesc& op, uint32_t lane) {
  const bool alt = (op.kind == OP_EMBED || op.kind == OP_ASSEMBLE);
  const uint64_t g = alt ? op.p[6] : op.p[2], b = alt ? op.p[7] : op.p[3], b2 = op.q[3];
  const uint32_t off = lane * 128u;
  if (off < op.cols * 2u) {
    if (g != 0) asm volatile("prefetch.global.L2 [%0];" ::"l"(g + off));
    if (b != 0) asm volatile("prefetch.global.L2 [%0];" ::"l"(b + off));
    if (b2 != 0) asm volatile("prefetch.global.L2 [%0];" ::"l"(b2 + off));
  }
}

// LayerNorm / RMS norm of few rows: four warps share a row (two rows per work item), each
// taking a quarter of the columns; the partial sums meet in shared memory. With 128 rows this
// puts 512 warps on 64 SMs instead of 128 warps on 16, and cuts the per-warp chain of loads,
// reductions, conversions and stores (about 2 us for a 768-column row on one warp) to a quarter.
__device__ __noinline__ bool rowwise_split_item(Ctx& c, const OpDesc& op, uint32_t local, uint32_t widx,
                                                uint32_t lane) {
  const uint32_t r_in = widx >> 2, part = widx & 3u;
  const uint32_t row = local * kSplitRowsPerItem + r_in;
  const bool live = row < op.rows;
  const uint32_t safe_row = live ? row : 0u;
  const uint32_t cols = op.cols, per = cols >> 4;  // 16-byte f32 vectors per warp (<= 64)
  const uint32_t flags = op.flags;
  const bool rms = (flags & F_RMSNORM) != 0u, src32 = (flags & F_SRC_F32) != 0u;
  const uint32_t v0 = part * per;
  uint32_t vi[2];
  bool on[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    on[i] = lane + 32u * i < per;
    vi[i] = v0 + (on[i] ? lane + 32u * i : 0u);
  }
  const uint2* gamma = reinterpret_cast<const uint2*>(op.p[2]);
  const uint2* beta = reinterpret_cast<const uint2*>(op.p[3]);
  const bool two = op.q[2] != 0, add_b2 = two && op.q[3] != 0;
  const uint2* b2p = add_b2 ? reinterpret_cast<const uint2*>(op.q[3]) : gamma;
  uint2 gv[2], bv[2], b2v[2];
  float4 x[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    gv[i] = __ldg(gamma + vi[i]);
    bv[i] = __ldg(beta + vi[i]);
    b2v[i] = __ldg(b2p + vi[i]);
  }
  if (src32) {
    const float4* src = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(op.p[1]) +
                                                        static_cast<size_t>(safe_row) * op.lds);
#pragma unroll
    for (int i = 0; i < 2; ++i) x[i] = __ldcg(src + vi[i]);
    if ((flags & F_ZERO_SRC) && live) {
#pragma unroll
      for (int i = 0; i < 2; ++i)
        if (on[i]) const_cast<float4*>(src)[vi[i]] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
  } else {
    const uint2* src = reinterpret_cast<const uint2*>(reinterpret_cast<const __half*>(op.p[1]) +
                                                      static_cast<size_t>(safe_row) * op.lds);
#pragma unroll
    for (int i = 0; i < 2; ++i) x[i] = h4_to_f4(__ldcg(src + vi[i]));
  }
  if (flags & F_RESID) {
    const uint2* res = reinterpret_cast<const uint2*>(reinterpret_cast<const __half*>(op.p[4]) +
                                                      static_cast<size_t>(safe_row) * op.ldr);
#pragma unroll
    for (int i = 0; i < 2; ++i) add4(x[i], h4_to_f4(__ldcg(res + vi[i])));
  }
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    if (!on[i]) x[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    sum += x[i].x + x[i].y + x[i].z + x[i].w;
  }
  // Each warp reduces its quarter to (sum, sum of squared deviations from its own mean); the
  // four pairs are combined after ONE meeting in shared memory:
  //   M2 = sum_w [ M2_w + n_w (mean_w - mean)^2 ]       (pairwise variance combination)
  // which is as accurate as the two-pass form and saves its second group barrier.
  const float inv_n = 1.0f / static_cast<float>(cols);
  const float n_w = static_cast<float>(cols >> 2), inv_nw = 1.0f / n_w;
  sum = warp_sum(sum);
  const float mean_w = rms ? 0.f : sum * inv_nw;
  float sq = 0.f;
#pragma unroll
  for (int i = 0; i < 2; ++i)
    if (on[i]) {
      const float a = x[i].x - mean_w, b = x[i].y - mean_w, d = x[i].z - mean_w, e = x[i].w - mean_w;
      sq += a * a + b * b + d * d + e * e;
    }
  sq = warp_sum(sq);
  if (lane == 0) {
    c.ctrl->ln_part[0][r_in][part] = sum;
    c.ctrl->ln_part[1][r_in][part] = sq;
  }
  if (!group_sync(c, 0x431)) return false;
  const float* p0 = c.ctrl->ln_part[0][r_in];
  const float* p1 = c.ctrl->ln_part[1][r_in];
  const float mean = rms ? 0.f : (p0[0] + p0[1] + p0[2] + p0[3]) * inv_n;
  float m2 = p1[0] + p1[1] + p1[2] + p1[3];
  if (!rms) {
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float dm = p0[w] * inv_nw - mean;
      m2 = fmaf(n_w * dm, dm, m2);
    }
  }
  const float rstd = rsqrtf(m2 * inv_n + op.eps);
  if (live) {
    uint2* out = op.p[0] ? reinterpret_cast<uint2*>(reinterpret_cast<__half*>(op.p[0]) +
                                                    static_cast<size_t>(row) * op.ldo)
                         : nullptr;
    float4* out2 = two ? reinterpret_cast<float4*>(reinterpret_cast<float*>(op.q[2]) +
                                                   static_cast<size_t>(row) * cols)
                       : nullptr;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      if (!on[i]) continue;
      const float4 g = h4_to_f4(gv[i]);
      const float4 b = rms ? make_float4(0.f, 0.f, 0.f, 0.f) : h4_to_f4(bv[i]);
      float4 y;
      y.x = (x[i].x - mean) * rstd * g.x + b.x;
      y.y = (x[i].y - mean) * rstd * g.y + b.y;
      y.z = (x[i].z - mean) * rstd * g.z + b.z;
      y.w = (x[i].w - mean) * rstd * g.w + b.w;
      if (out != nullptr) {
        uint2 o;
        o.x = pack_h2(y.x, y.y);
        o.y = pack_h2(y.z, y.w);
        out[vi[i]] = o;
      }
      if (out2 != nullptr) {
        if (add_b2) add4(y, h4_to_f4(b2v[i]));
        out2[vi[i]] = y;
      }
    }
  }
  return true;
}

// Arg-max item: one f16 row per 256-thread group. Each thread scans every 256th 16-byte
// vector in ascending order (so "strictly greater" keeps its first maximum), then the
// partial results are merged by (larger value, then smaller index): the first index of the
// row maximum, which is what XLA's (value, index) reduce returns
// (reduction functors: mononn_engine/codegen/reduction_functor_generator.cc:296-441).
__device__ __noinline__ bool argmax_item(Ctx& c, const OpDesc& op, uint32_t row, uint32_t widx,
                                         uint32_t lane, uint32_t tid_in_group) {
  const uint32_t nvec = op.cols >> 3;
  const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const __half*>(op.p[1]) +
                                                    static_cast<size_t>(row) * op.lds);
  float best = -INFINITY;
  uint32_t best_i = 0;
#pragma unroll 1
  for (uint32_t v0 = tid_in_group; v0 < nvec; v0 += 4u * kSimtThreads) {
    uint4 h[4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
      h[i] = __ldcg(src + ((v0 + i * kSimtThreads < nvec) ? v0 + i * kSimtThreads : v0));
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t vi = v0 + i * kSimtThreads;
      if (vi < nvec) {
        const __half2* hp = reinterpret_cast<const __half2*>(&h[i]);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __half22float2(hp[j]);
          if (f.x > best) { best = f.x; best_i = vi * 8u + 2u * j; }
          if (f.y > best) { best = f.y; best_i = vi * 8u + 2u * j + 1u; }
        }
      }
    }
  }
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, off);
    const uint32_t oi = __shfl_xor_sync(0xffffffffu, best_i, off);
    if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
  }
  if (lane == 0) {
    c.ctrl->red_val[widx] = best;
    c.ctrl->red_idx[widx] = best_i;
  }
  if (!group_sync(c, 0x420)) return false;
  if (tid_in_group == 0) {
#pragma unroll
    for (int w = 1; w < static_cast<int>(kSimtWarps); ++w) {
      const float ov = c.ctrl->red_val[w];
      const uint32_t oi = c.ctrl->red_idx[w];
      if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
    }
    reinterpret_cast<int32_t*>(op.p[0])[row] = static_cast<int32_t>(best_i);
  }
  // the partial-result slots are reused by the group's next row
  return group_sync(c, 0x421);
}

// Pooling at the largest token id: out[b, :] = src[b * seq + argmax(ids[b, :]), :], the first
// maximum on ties (the end-of-text row of a CLIP text tower). One warp per output row.
__device__ __noinline__ void rowsel_item(const OpDesc& op, uint32_t local, uint32_t warp_in_group,
                                         uint32_t lane) {
  const uint32_t b = local * kRowsPerItem + warp_in_group;
  if (b >= op.rows) return;
  const int32_t* ids = reinterpret_cast<const int32_t*>(op.p[2]) + static_cast<size_t>(b) * op.seq;
  int32_t best = INT32_MIN;
  uint32_t best_i = 0;
  for (uint32_t i = lane; i < op.seq; i += 32u) {
    const int32_t v = __ldg(ids + i);
    if (v > best || (v == best && i < best_i)) { best = v; best_i = i; }
  }
  if (lane >= op.seq) best_i = 0xffffffffu;  // lanes without an element never win a tie
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) {
    const int32_t ov = __shfl_xor_sync(0xffffffffu, best, off);
    const uint32_t oi = __shfl_xor_sync(0xffffffffu, best_i, off);
    if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
  }
  const uint2* src = reinterpret_cast<const uint2*>(reinterpret_cast<const __half*>(op.p[1]) +
                                                    (static_cast<size_t>(b) * op.seq + best_i) * op.lds);
  uint2* out = reinterpret_cast<uint2*>(reinterpret_cast<__half*>(op.p[0]) + static_cast<size_t>(b) * op.ldo);
  for (uint32_t vi = lane; vi < (op.cols >> 2); vi += 32u) out[vi] = __ldcg(src + vi);
}

// out[i, j] = alpha * <a[i, :], b[j, :]> for two small f16 activations (the image-text logits
// of a dual encoder: a few dozen rows each). One warp per row i, lanes over j.
__device__ __noinline__ void pairdot_item(const OpDesc& op, uint32_t local, uint32_t warp_in_group,
                                          uint32_t lane) {
  const uint32_t i = local * kRowsPerItem + warp_in_group;
  if (i >= op.M) return;
  const uint4* a = reinterpret_cast<const uint4*>(reinterpret_cast<const __half*>(op.p[1]) +
                                                  static_cast<size_t>(i) * op.lds);
  __half* out = reinterpret_cast<__half*>(op.p[0]) + static_cast<size_t>(i) * op.ldo;
  const uint32_t kv = op.K >> 3;
  for (uint32_t j = lane; j < op.N; j += 32u) {
    const uint4* bj = reinterpret_cast<const uint4*>(reinterpret_cast<const __half*>(op.p[2]) +
                                                     static_cast<size_t>(j) * op.ldr);
    float acc = 0.f;
#pragma unroll 4
    for (uint32_t k = 0; k < kv; ++k) {
      const uint4 av = __ldcg(a + k), bv = __ldcg(bj + k);
      const __half2* ah = reinterpret_cast<const __half2*>(&av);
      const __half2* bh = reinterpret_cast<const __half2*>(&bv);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 x = __half22float2(ah[q]), y = __half22float2(bh[q]);
        acc = fmaf(x.x, y.x, acc);
        acc = fmaf(x.y, y.y, acc);
      }
    }
    out[j] = __float2half_rn(acc * op.alpha);
  }
}

// Window extraction for a forward convolution over the image (the ViT / CLIP patch embedding
// with stride = window, or an overlapping, zero-padded stem): row (b, py, px) of the f16 output
// holds the window's pixels in (ky, kx, c) order, read from the NCHW f32 image, zero where the
// window hangs over the edge and in the columns that pad the row to a multiple of 64. With
// that operand the convolution is a plain GEMM against the [out_channels, ky*kx*c] filter. The
// reference runs these through CUTLASS implicit-GEMM fprop
// (mononn_engine/core/op_impl/conv_impl.cc:36-106, 252-345).
__device__ __noinline__ void patchify_item(const OpDesc& op, uint32_t local, uint32_t warp_in_group,
                                           uint32_t lane) {
  const uint32_t row = local * kRowsPerItem + warp_in_group;
  if (row >= op.rows) return;
  const uint32_t C = op.heads, Himg = op.seq, Wimg = op.batches, kh = op.head_dim, kw = op.q_col;
  const uint32_t gw = op.k_col, per_img = op.vocab;  // windows per image row / per image
  const uint32_t b = row / per_img, pr = row % per_img, py = pr / gw, px = pr % gw;
  const uint32_t y0 = py * op.M - op.rows_per_batch, x0 = px * op.N - op.ldt;  // may wrap below 0
  const uint32_t valid = op.K;
  (void)kh;
  const float* src = reinterpret_cast<const float*>(op.p[1]);
  __half* dst = reinterpret_cast<__half*>(op.p[0]) + static_cast<size_t>(row) * op.ldo;
  // (ky, kx, c) of column j = lane, then of every 32nd column after it: the step of 32 columns is
  // split once into whole window rows, whole pixels and channels, and added with carries (three
  // divisions per element made this stage 16 % longer at batch 64; the scattered pixel reads are
  // the rest)
  const uint32_t per_row = C * kw;
  const uint32_t step_ky = 32u / per_row, step_kx = (32u % per_row) / C, step_c = 32u % C;
  uint32_t ky = lane / per_row, kx = (lane % per_row) / C, ch = lane % C;
#pragma unroll 4
  for (uint32_t j = lane; j < op.cols; j += 32u) {
    const uint32_t y = y0 + ky, x = x0 + kx;  // a wrapped (negative) coordinate fails the bound test
    float v = 0.f;
    if (j < valid && y < Himg && x < Wimg) v = src[((static_cast<size_t>(b) * C + ch) * Himg + y) * Wimg + x];
    dst[j] = __float2half_rn(v);
    ch += step_c;
    if (ch >= C) {
      ch -= C;
      ++kx;
    }
    kx += step_kx;
    if (kx >= kw) {
      kx -= kw;
      ++ky;
    }
    ky += step_ky;
  }
}

// Softmax + output of one attention tile. Query row `row` belongs to two threads (the warps
// `half` = 0, 1 of the row's TMEM quarter): each takes one 64-key half of every 128-key score
// chunk (which is also one of the chunk's two P tiles) and 32 of the 64 output columns; the row
// maximum and the row sum are combined through shared memory.
__device__ __noinline__ bool attention_simt(Ctx& c, const OpDesc& op, uint32_t local,
                                            uint32_t tmem_base, uint32_t& a_cnt, uint32_t& acc_cnt,
                                            uint32_t quarter, uint32_t half, uint32_t lane,
                                            uint32_t tid_in_group) {
  const AttnTile t = attn_tile(op, local);
  const uint32_t row = quarter * 32u + lane;
  const uint32_t qrow = t.mt * 128u + row;  // query index inside the sequence
  const uint32_t nc = attn_chunks(op);
  const bool fused = attn_fused(op);
  uint32_t base = a_cnt;
  a_cnt += attn_slots(op);
  const uint32_t phQ = acc_cnt;
  const uint32_t phS = acc_cnt + (fused ? 1u : 0u), phO = phS + 1u;
  acc_cnt = phO + 1u;
  const uint32_t seq = op.seq, n_cols = nc * 128u;
  const float alpha = op.alpha * 1.4426950408889634f;  // scores in log2 units: exp(x) = 2^(x log2 e)
  // Stage the additive key mask of this batch row while Q, K load and QK^T runs; keys past
  // the sequence end are masked out here so the loops below need no bound check.
  float* mb = c.ctrl->mask_row;
  {
    const bool has_mask = (op.flags & F_MASK_BIAS) != 0u;
    const float* gm = reinterpret_cast<const float*>(op.p[1]) + static_cast<size_t>(t.b) * seq;
    for (uint32_t i = tid_in_group; i < n_cols; i += kSimtThreads) {
      float m = -1.0e30f;
      if (i < seq) m = has_mask ? __ldcg(gm + i) : 0.f;
      mb[i] = m * 1.4426950408889634f;
    }
    if (fused && tid_in_group < 192u) {  // biases of this head's Q, K, V columns
      float* bs = c.ctrl->bias_tile[0];
      const uint32_t i = tid_in_group;
      const __half* bp = reinterpret_cast<const __half*>(op.p[2u + (i >> 6)]);
      bs[i] = bp ? __half2float(__ldg(bp + t.h * 64u + (i & 63u))) : 0.f;
    }
    if (!group_sync(c, 0x415)) return false;
  }
  if (fused) {
    // accumulator [tokens, Q | K | V] -> f16 operand tiles: Q and K row-major (token, d), V
    // transposed (d, token) in two 64-key halves, all in the 128-byte-swizzled K-major layout
    base += op.kb_per_split;
    const uint32_t cQ = base, cK = base + 1u, cV = base + 2u;
    // The accumulator is complete when every x tile has been consumed, and the commits that free
    // the tiles' slots precede the accumulator's: after this wait the three slots written below
    // (which x tiles occupied) are free. (Testing their empty barriers before it could be
    // fooled: two uses of a slot may be pending at once, and a parity wait cannot tell 0 from 2.)
    if (!mbar_wait_warp(c, &c.ctrl->acc_full[phQ & 1u], (phQ >> 1) & 1u, 0x419)) return false;
    if (!mbar_wait_warp(c, &c.ctrl->a_empty[cQ % kASlots], ((cQ / kASlots) & 1u) ^ 1u, 0x416)) return false;
    if (!mbar_wait_warp(c, &c.ctrl->a_empty[cK % kASlots], ((cK / kASlots) & 1u) ^ 1u, 0x417)) return false;
    if (!mbar_wait_warp(c, &c.ctrl->a_empty[cV % kASlots], ((cV / kASlots) & 1u) ^ 1u, 0x418)) return false;
    if (tid_in_group == 0) trace(*c.P, c.stage, TR_MARK0 + 4);
    tc_fence_after();
    const float* bs = c.ctrl->bias_tile[0];
    const uint32_t tQ = tmem_base + kAttnQkvCol + ((quarter * 32u) << 16);
    uint8_t* tileV = c.a_ring_ptr + (cV % kASlots) * kSlotBytes + (row >> 6) * 8192u;
    // one 32-column load is in flight while the previous one is converted and stored
    auto convert = [&](const uint32_t (&r)[32], uint32_t c0) {
      float v[32], bb[32];
      lds32(bs + c0, bb);
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]) + bb[i];
      if (c0 < 128u) {
        uint8_t* tile = c.a_ring_ptr + (((c0 < 64u) ? cQ : cK) % kASlots) * kSlotBytes;
        const uint32_t chunk = (c0 & 63u) >> 3;
#pragma unroll
        for (uint32_t q = 0; q < 4; ++q) {
          uint4* d = reinterpret_cast<uint4*>(tile + row * 128u + (((chunk + q) ^ (row & 7u)) << 4));
          *d = make_uint4(pack_h2(v[8 * q], v[8 * q + 1]), pack_h2(v[8 * q + 2], v[8 * q + 3]),
                          pack_h2(v[8 * q + 4], v[8 * q + 5]), pack_h2(v[8 * q + 6], v[8 * q + 7]));
        }
      } else {
        const uint32_t d0 = c0 - 128u, kc = (row & 63u) >> 3, kw = (row & 7u) << 1;
#pragma unroll
        for (uint32_t i = 0; i < 32; ++i) {
          const uint32_t d = d0 + i;
          *reinterpret_cast<__half*>(tileV + d * 128u + ((kc ^ (d & 7u)) << 4) + kw) = __float2half_rn(v[i]);
        }
      }
    };
    // warp `half` converts columns [32*half, +32) of each of Q, K and V
    uint32_t ra[32], rb[32];
    const uint32_t h32 = half * 32u;
    tc_ld32_issue(tQ + h32, ra);
    tc_wait_ld();
    tc_ld32_issue(tQ + 64u + h32, rb);
    convert(ra, h32);
    tc_wait_ld();
    tc_ld32_issue(tQ + 128u + h32, ra);
    convert(rb, 64u + h32);
    tc_wait_ld();
    convert(ra, 128u + h32);
    if (tid_in_group == 0) trace(*c.P, c.stage, TR_MARK0 + 5);
    // Every warp makes its part of the tiles visible to the tensor core (proxy fence) and counts
    // itself; the warp that counts last hands the three tiles to the MMA issuer. Nobody waits
    // for anybody here (a barrier over the eight warps plus an arrival by its first thread put
    // one more wake-up on the critical chain).
    fence_proxy_async_smem();
    if (last_warp_of(&c.ctrl->tiles_done[0], lane)) {
      mbar_arrive(smem_u32(&c.ctrl->a_full[cQ % kASlots]));
      mbar_arrive(smem_u32(&c.ctrl->a_full[cK % kASlots]));
      mbar_arrive(smem_u32(&c.ctrl->a_full[cV % kASlots]));
      trace(*c.P, c.stage, TR_MARK0 + 6);
    }
    tc_fence_before();
    warp_arrive(&c.ctrl->acc_empty[phQ & 1u]);
  }
  // causal: keys after the query are masked
  const uint32_t key_limit = (op.flags & F_CAUSAL) ? qrow : 0xffffffffu;
  if (!mbar_wait_warp(c, &c.ctrl->acc_full[phS & 1u], (phS >> 1) & 1u, 0x410)) return false;
  if (tid_in_group == 0) trace(*c.P, c.stage, TR_MARK0);
  tc_fence_after();
  const uint32_t tS = tmem_base + ((quarter * 32u) << 16);
  const uint32_t h64 = half * 64u;
  // additive bias per (head, query, key): this thread's row of the head's [seq, seq] table
  // (rows past the sequence end read the last row; their results are never stored)
  const __half* pb = nullptr;
  if (op.flags & F_POS_BIAS)
    pb = reinterpret_cast<const __half*>(op.q[0]) +
         (static_cast<size_t>(t.h) * seq + (qrow < seq ? qrow : seq - 1u)) * seq;
  float sum0 = 0.f, sum1 = 0.f;
  if (nc == 1u && key_limit == 0xffffffffu && pb == nullptr) {
    // One key chunk, no causal mask, no position bias (the encoder case): the 64 scaled and masked
    // scores of this thread stay in registers between the maximum and the exponentials, so the
    // accumulator and the mask row are read once.
    float z[64];
#pragma unroll
    for (uint32_t c0 = 0; c0 < 64u; c0 += 32u) {
      float v[32], mk[32];
      lds32(mb + h64 + c0, mk);
      tc_ld32(tS + h64 + c0, v);
#pragma unroll
      for (int i = 0; i < 32; ++i) z[c0 + i] = fmaf(v[i], alpha, mk[i]);
    }
    float m0 = z[0], m1 = z[1], m2 = z[2], m3 = z[3];
#pragma unroll
    for (int i = 4; i < 64; i += 4) {
      m0 = fmaxf(m0, z[i]);
      m1 = fmaxf(m1, z[i + 1]);
      m2 = fmaxf(m2, z[i + 2]);
      m3 = fmaxf(m3, z[i + 3]);
    }
    float mx = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
    c.ctrl->row_max[half][row] = mx;
    if (!group_sync(c, 0x41b)) return false;
    mx = fmaxf(mx, c.ctrl->row_max[half ^ 1u][row]);
    if (tid_in_group == 0) trace(*c.P, c.stage, TR_MARK0 + 1);
    const uint32_t cP = base + 2u + nc + half;
    const uint32_t slotP = cP % kASlots;
    if (!mbar_wait_warp(c, &c.ctrl->a_empty[slotP], ((cP / kASlots) & 1u) ^ 1u, 0x411)) return false;
    uint8_t* tile = c.a_ring_ptr + slotP * kSlotBytes;
#pragma unroll
    for (int i = 0; i < 64; i += 2) {
      z[i] = fast_exp2(z[i] - mx);
      z[i + 1] = fast_exp2(z[i + 1] - mx);
      sum0 += z[i];
      sum1 += z[i + 1];
    }
#pragma unroll
    for (uint32_t q = 0; q < 8; ++q) {
      uint4* d = reinterpret_cast<uint4*>(tile + row * 128u + ((q ^ (row & 7u)) << 4));
      *d = make_uint4(pack_h2(z[8 * q], z[8 * q + 1]), pack_h2(z[8 * q + 2], z[8 * q + 3]),
                      pack_h2(z[8 * q + 4], z[8 * q + 5]), pack_h2(z[8 * q + 6], z[8 * q + 7]));
    }
    c.ctrl->row_sum[half][row] = sum0 + sum1;
    fence_proxy_async_smem();
    if (last_warp_of(&c.ctrl->tiles_done[1], lane)) {
      const uint32_t cP0 = cP - half;
      mbar_arrive(smem_u32(&c.ctrl->a_full[cP0 % kASlots]));
      mbar_arrive(smem_u32(&c.ctrl->a_full[(cP0 + 1u) % kASlots]));
    }
  } else {
    // pass 1: row maximum of scale*s + mask over this warp's key halves (four independent chains)
    float m0 = -3.0e38f, m1 = -3.0e38f, m2 = -3.0e38f, m3 = -3.0e38f;
  #pragma unroll 1
    for (uint32_t c0 = h64; c0 < n_cols; c0 += ((c0 & 32u) ? 96u : 32u)) {  // 64 of every 128 columns
      float v[32], mk[32];
      lds32(mb + c0, mk);
      if (pb != nullptr) add_bias32(pb + c0, mk);
      tc_ld32(tS + c0, v);
      if (key_limit == 0xffffffffu) {  // not causal (warp-uniform): no per-element test
  #pragma unroll
        for (int i = 0; i < 32; i += 4) {
          m0 = fmaxf(m0, fmaf(v[i], alpha, mk[i]));
          m1 = fmaxf(m1, fmaf(v[i + 1], alpha, mk[i + 1]));
          m2 = fmaxf(m2, fmaf(v[i + 2], alpha, mk[i + 2]));
          m3 = fmaxf(m3, fmaf(v[i + 3], alpha, mk[i + 3]));
        }
      } else {
  #pragma unroll
        for (int i = 0; i < 32; i += 4) {
          m0 = fmaxf(m0, (c0 + i <= key_limit) ? fmaf(v[i], alpha, mk[i]) : -1.0e30f);
          m1 = fmaxf(m1, (c0 + i + 1 <= key_limit) ? fmaf(v[i + 1], alpha, mk[i + 1]) : -1.0e30f);
          m2 = fmaxf(m2, (c0 + i + 2 <= key_limit) ? fmaf(v[i + 2], alpha, mk[i + 2]) : -1.0e30f);
          m3 = fmaxf(m3, (c0 + i + 3 <= key_limit) ? fmaf(v[i + 3], alpha, mk[i + 3]) : -1.0e30f);
        }
      }
    }
    float mx = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
    c.ctrl->row_max[half][row] = mx;
    if (!group_sync(c, 0x41b)) return false;
    mx = fmaxf(mx, c.ctrl->row_max[half ^ 1u][row]);
    if (tid_in_group == 0) trace(*c.P, c.stage, TR_MARK0 + 1);
    // pass 2: p = exp(z - max), row sum, this warp's P tile of every chunk in the swizzled
    // K-major operand layout
  #pragma unroll 1
    for (uint32_t j = 0; j < nc; ++j) {
      const uint32_t cP = base + 2u + nc + 3u * j + half;  // the chunk's two P slots: one per warp half
      const uint32_t slotP = cP % kASlots;
      // the P slot must be free before it is overwritten
      if (!mbar_wait_warp(c, &c.ctrl->a_empty[slotP], ((cP / kASlots) & 1u) ^ 1u, 0x411)) return false;
      uint8_t* tile = c.a_ring_ptr + slotP * kSlotBytes;
  #pragma unroll 1
      for (uint32_t c0 = 0; c0 < 64u; c0 += 32) {
        const uint32_t cc = j * 128u + h64 + c0;
        float v[32], mk[32];
        lds32(mb + cc, mk);
        if (pb != nullptr) add_bias32(pb + cc, mk);
        tc_ld32(tS + cc, v);
        if (key_limit == 0xffffffffu) {
          // exp2(s*alpha + mask - max) with the subtraction folded into the multiply-add
  #pragma unroll
          for (int i = 0; i < 32; ++i) mk[i] -= mx;
  #pragma unroll
          for (int i = 0; i < 32; i += 2) {
            v[i] = fast_exp2(fmaf(v[i], alpha, mk[i]));
            v[i + 1] = fast_exp2(fmaf(v[i + 1], alpha, mk[i + 1]));
            sum0 += v[i];
            sum1 += v[i + 1];
          }
        } else {
  #pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const float z0 = (cc + i <= key_limit) ? fmaf(v[i], alpha, mk[i]) : -1.0e30f;
            const float z1 = (cc + i + 1 <= key_limit) ? fmaf(v[i + 1], alpha, mk[i + 1]) : -1.0e30f;
            v[i] = fast_exp2(z0 - mx);
            v[i + 1] = fast_exp2(z1 - mx);
            sum0 += v[i];
            sum1 += v[i + 1];
          }
        }
        const uint32_t chunk = c0 >> 3;  // 16-byte chunk index inside the 128-byte row
  #pragma unroll
        for (uint32_t q = 0; q < 4; ++q) {
          uint4* d = reinterpret_cast<uint4*>(tile + row * 128u + (((chunk + q) ^ (row & 7u)) << 4));
          *d = make_uint4(pack_h2(v[8 * q], v[8 * q + 1]), pack_h2(v[8 * q + 2], v[8 * q + 3]),
                          pack_h2(v[8 * q + 4], v[8 * q + 5]), pack_h2(v[8 * q + 6], v[8 * q + 7]));
        }
      }
      if (j + 1u == nc) c.ctrl->row_sum[half][row] = sum0 + sum1;
      // as above: the last warp to finish the chunk's two P tiles hands them over (one counter per
      // chunk: a warp may be a chunk ahead of another)
      fence_proxy_async_smem();
      if (last_warp_of(&c.ctrl->tiles_done[1u + j], lane)) {
        const uint32_t cP0 = cP - half;
        mbar_arrive(smem_u32(&c.ctrl->a_full[cP0 % kASlots]));
        mbar_arrive(smem_u32(&c.ctrl->a_full[(cP0 + 1u) % kASlots]));
      }
    }
  }
  if (tid_in_group == 0) trace(*c.P, c.stage, TR_MARK0 + 2);
  tc_fence_before();
  warp_arrive(&c.ctrl->acc_empty[phS & 1u]);

  // O = sum_j P_j V_j: this warp stores 32 of the head's 64 columns
  if (!mbar_wait_warp(c, &c.ctrl->acc_full[phO & 1u], (phO >> 1) & 1u, 0x413)) return false;
  if (tid_in_group == 0) trace(*c.P, c.stage, TR_MARK0 + 3);
  tc_fence_after();
  // the other half's row sum: its warp counted itself after writing it, the MMAs whose completion
  // was just observed were issued after the last count, so the value is visible here
  const float inv = 1.0f / (sum0 + sum1 + c.ctrl->row_sum[half ^ 1u][row]);
  const uint32_t tO = tmem_base + kAttnOutCol + half * 32u + ((quarter * 32u) << 16);
  // A thread owns a row, but a store instruction whose 32 lanes hit 32 different rows costs 32
  // memory transactions. The warp's 32 x 64-byte block goes through shared memory (swizzled, so
  // neither side has bank conflicts) and is stored four lanes to a row.
  uint8_t* stg = c.store_stage + (tid_in_group >> 5) * 2048u;
  {
    float v[32];
    tc_ld32(tO, v);
    const uint32_t sw = (lane >> 1) & 3u;
#pragma unroll
    for (uint32_t q = 0; q < 4; ++q)
      *reinterpret_cast<uint4*>(stg + lane * 64u + ((q ^ sw) << 4)) =
          make_uint4(pack_h2(v[8 * q] * inv, v[8 * q + 1] * inv), pack_h2(v[8 * q + 2] * inv, v[8 * q + 3] * inv),
                     pack_h2(v[8 * q + 4] * inv, v[8 * q + 5] * inv), pack_h2(v[8 * q + 6] * inv, v[8 * q + 7] * inv));
  }
  __syncwarp();
  {
    const uint32_t q = lane & 3u;
    __half* obase = reinterpret_cast<__half*>(op.p[0]) + t.h * 64u + half * 32u + q * 8u;
#pragma unroll
    for (uint32_t j = 0; j < 4; ++j) {
      const uint32_t r = 8u * j + (lane >> 2), qr = t.mt * 128u + quarter * 32u + r;
      const uint4 val = *reinterpret_cast<const uint4*>(stg + r * 64u + ((q ^ ((r >> 1) & 3u)) << 4));
      if (qr < seq)
        *reinterpret_cast<uint4*>(obase + (static_cast<size_t>(t.b) * seq + qr) * op.ldo) = val;
    }
  }
  // a GEMM of this stage may wait for this item's output: the warp that stores last counts the item
  if (op.flag != 0 && last_warp_of(&c.ctrl->tiles_done[4], lane))
    red_release_gpu_add(reinterpret_cast<uint32_t*>(op.flag), 1u);
  __syncwarp();  // the staging block is reused by the warp's next item
  tc_fence_before();
  warp_arrive(&c.ctrl->acc_empty[phO & 1u]);
  return true;
}

// ----------------------------------------------------------------------------
// Role: epilogue + SIMT stages + grid barrier (warps 4..11)
// ----------------------------------------------------------------------------
__device__ void role_simt(Ctx c, uint32_t tmem_base, uint32_t tid_in_group) {
  const KernelParams& P = *c.P;
  // warp w of the CTA reads TMEM lanes 32*(w%4)..: the SIMT warps 4..11 form two sets of quarters
  const uint32_t widx = tid_in_group >> 5, quarter = widx & 3u, half = widx >> 2, lane = tid_in_group & 31u;
  uint32_t a_cnt = 0, acc_cnt = 0;
  for (uint32_t s = P.stage_begin; s < P.stage_end; ++s) {
    c.stage = s;
    const StageDesc st = load_stage(P, s);
    uint4* slot = c.ctrl->desc[3 + widx];
    Item first{nullptr, 0};
    if (blockIdx.x < st.n_items) {
      first = fetch_item<true>(P, st, blockIdx.x, slot, lane);
      const uint32_t k0 = first.op->kind;
      if (k0 == OP_LAYERNORM || k0 == OP_EMBED || k0 == OP_ASSEMBLE) prefetch_row_consts(*first.op, lane);
    }
    // All CTAs must have finished the previous stage before this CTA reads its
    // results or arrives for this stage.
    WAIT_OR_RETURN(grid_wait_warp(c, s, 0x400));
    if (tid_in_group == 0) trace(P, s, TR_SIMT_READY);
    if (P.stamps != nullptr && blockIdx.x == 0 && tid_in_group == 0)
      P.stamps[s - P.stage_begin] = globaltimer_ns();
    for (uint32_t item = blockIdx.x; item < st.n_items; item += gridDim.x) {
      const Item it = (item == blockIdx.x) ? first : fetch_item<true>(P, st, item, slot, lane);
      const OpDesc& op = *it.op;
      switch (op.kind) {
        case OP_GEMM: {
          const uint32_t buf = acc_cnt & 1u;
          float* bias_s = c.ctrl->bias_tile[buf];
          if (op.flags & F_BIAS) {
            // stage the tile's bias while the MMAs run
            const uint32_t n0 = ((it.local / op.k_split) % op.n_tiles) * op.n_tile;
            if (tid_in_group < op.n_tile)
              bias_s[tid_in_group] =
                  (n0 + tid_in_group < op.N)
                      ? __half2float(__ldg(reinterpret_cast<const __half*>(op.p[1]) + n0 + tid_in_group))
                      : 0.f;
            WAIT_OR_RETURN(group_sync(c, 0x403));
          }
          const GemmTile tile = gemm_tile(op, it.local);  // (its divisions are done while the MMAs run)
          if (tid_in_group == 0) trace(P, s, TR_MARK0);
          WAIT_OR_RETURN(mbar_wait_warp(c, &c.ctrl->acc_full[buf], (acc_cnt >> 1) & 1u, 0x401));
          if (tid_in_group == 0) trace(P, s, TR_MARK0 + 1);
          tc_fence_after();
          gemm_epilogue(op, tile, tmem_base + buf * kAccCols, quarter, half, lane, bias_s,
                        c.store_stage + widx * 2048u);
          tc_fence_before();
          // A row op of this stage may wait for this item. The warps count themselves per
          // accumulator buffer in shared memory before they free the buffer (so the counts of two
          // items never mix: the buffer is not filled again until all eight have counted), and the
          // warp that counts last publishes the item: its release at GPU scope is cumulative over
          // the reductions of the other seven, observed through the counter. (Eight global arrivals
          // per item, one per warp, measured 6 us slower per inference.)
          bool last_of_item = false;
          if (op.flag != 0) {
            __syncwarp();
            if (lane == 0)
              last_of_item = (atom_add_acq_rel_cta_smem(&c.ctrl->items_done[buf], 1u) & (kSimtWarps - 1u)) ==
                             kSimtWarps - 1u;
          }
          warp_arrive(&c.ctrl->acc_empty[buf]);
          ++acc_cnt;
          a_cnt += op.kb_per_split;
          if (last_of_item) red_release_gpu_add(reinterpret_cast<uint32_t*>(op.flag), 1u);
          break;
        }
        case OP_ATTENTION:
          WAIT_OR_RETURN(attention_simt(c, op, it.local, tmem_base, a_cnt, acc_cnt, quarter, half, lane,
                                        tid_in_group));
          break;
        case OP_LAYERNORM:
        case OP_EMBED:
        case OP_ASSEMBLE:
          if (op.flag_target != 0) {
            prefetch_row_consts(op, lane);
            WAIT_OR_RETURN(flag_wait_warp(c, op.flag, op.flag_target, 0x430));
          }
          if (op.flags & F_ROW_SPLIT) {
            WAIT_OR_RETURN(rowwise_split_item(c, op, it.local, widx, lane));
          } else {
            rowwise_item(op, it.local, widx, lane, P, s);
          }
          break;
        case OP_PATCHIFY:
          patchify_item(op, it.local, widx, lane);
          break;
        case OP_ARGMAX:
          WAIT_OR_RETURN(argmax_item(c, op, it.local, widx, lane, tid_in_group));
          break;
        case OP_ROWSEL:
          rowsel_item(op, it.local, widx, lane);
          break;
        case OP_PAIRDOT:
          pairdot_item(op, it.local, widx, lane);
          break;
        default:
          break;
      }
    }
    // publish this CTA's stores of the stage, then arrive
    if (tid_in_group == 0) trace(P, s, TR_SIMT_DONE);
    // Results that later stages read through TMA need a generic->async proxy fence somewhere
    // between the store and the load. It sits on the reader side (the activation producer
    // issues fence.proxy.async after it has acquired the barrier): a second fence here, on
    // all the writers, cost about half a microsecond per stage.
    if (P.warp_arrive == 1u) {
      // every warp publishes its own stores (a warp stores whole rows or its own reductions) and
      // arrives for itself: no CTA-wide sync in front of the release
      __syncwarp();
      if (lane == 0) red_release_gpu_add(P.barrier, 1u);
      if (tid_in_group == 0) trace(P, s, TR_SIMT_ARRIVED);
      continue;
    }
    if (P.warp_arrive == 2u) {
      // every warp counts itself in shared memory (acquire + release at CTA scope) and moves on;
      // the warp that counts last arrives for the CTA. Its release at GPU scope is cumulative over
      // the other warps' stores, which it observed through the counter. One global arrival per
      // CTA and still no CTA-wide sync in front of it.
      __syncwarp();
      if (lane == 0) {
        const uint32_t seen = atom_add_acq_rel_cta_smem(&c.ctrl->warps_done, 1u);
        if ((seen & (kSimtWarps - 1u)) == kSimtWarps - 1u) red_release_gpu_add(P.barrier, 1u);
      }
      if (tid_in_group == 0) trace(P, s, TR_SIMT_ARRIVED);
      continue;
    }
    if (blockIdx.x < st.n_items) WAIT_OR_RETURN(group_sync(c, 0x402));
    if (tid_in_group == 0) {
      if (P.cluster > 1u) {
        // Cluster-scoped arrival: every CTA of the cluster arrives (release at cluster scope) on
        // an mbarrier in the first CTA's shared memory; that CTA acquires the phase and adds one
        // arrival for the whole cluster to the global counter (release at GPU scope, cumulative
        // over what it acquired).
        mbar_arrive_remote_release_cluster(mapa_smem(smem_u32(&c.ctrl->cl_bar), 0u));
        if (cluster_ctarank() == 0u) {
          const uint32_t bar = smem_u32(&c.ctrl->cl_bar), parity = (s - P.stage_begin) & 1u;
          bool ok = mbar_try_wait_acquire_cluster(bar, parity) != 0u;
          if (!ok) {
            const uint64_t t0 = globaltimer_ns();
            for (uint32_t it = 1; !ok; ++it) {
              ok = mbar_try_wait_acquire_cluster(bar, parity) != 0u;
              if (!ok && (it & 63u) == 0u) {
                if (*reinterpret_cast<volatile uint32_t*>(&c.ctrl->abort_flag)) break;
                if (globaltimer_ns() - t0 > c.timeout_ns) {
                  report_failure(c.P, c.ctrl, s, ST_GRID_BARRIER_TIMEOUT, 0x440);
                  break;
                }
              }
            }
          }
          if (ok) red_release_gpu_add(P.barrier, 1u);
        }
      } else {
        // release at gpu scope is cumulative over the group's stores ordered by group_sync
        red_release_gpu_add(P.barrier, 1u);
      }
      trace(P, s, TR_SIMT_ARRIVED);
    }
  }
  if (P.stamps != nullptr && blockIdx.x == 0 && tid_in_group == 0)
    P.stamps[P.stage_end - P.stage_begin] = globaltimer_ns();
}

// ----------------------------------------------------------------------------
// Kernel
// ----------------------------------------------------------------------------
extern "C" __global__ void __launch_bounds__(kThreads, 1)
mononn_megakernel(const __grid_constant__ KernelParams P) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t pad = (1024u - (raw & 1023u)) & 1023u;
  uint8_t* base = smem_raw + pad;
  Ctrl* ctrl = reinterpret_cast<Ctrl*>(base + kASlots * kSlotBytes + kBSlots * kBSlotBytes);

  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
  if (threadIdx.x == 0) {
    for (uint32_t i = 0; i < kASlots; ++i) {
      mbar_init(smem_u32(&ctrl->a_full[i]), 1);
      mbar_init(smem_u32(&ctrl->a_empty[i]), 1);
    }
    for (uint32_t i = 0; i < kBSlots; ++i) {
      mbar_init(smem_u32(&ctrl->b_full[i]), 1);
      mbar_init(smem_u32(&ctrl->b_empty[i]), 1);
    }
    for (uint32_t i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&ctrl->acc_full[i]), 1);
      mbar_init(smem_u32(&ctrl->acc_empty[i]), kSimtWarps);
    }
    mbar_init(smem_u32(&ctrl->group_bar), kSimtWarps);
    mbar_init(smem_u32(&ctrl->cl_bar), P.cluster);
    ctrl->abort_flag = 0;
    ctrl->barriers_seen = 0;
    ctrl->warps_done = 0;
    ctrl->items_done[0] = ctrl->items_done[1] = 0;
    for (uint32_t i = 0; i < 5; ++i) ctrl->tiles_done[i] = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 2) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(&ctrl->tmem_base)),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  // no CTA may arrive on a peer's mbarrier before that peer has initialised it
  if (P.cluster > 1u) cluster_sync_all();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&ctrl->tmem_base);

  // Biases and LayerNorm scale/shift of every layer sit in one small region; touching it now
  // puts it in L2 (and its page in the TLBs) long before the row-wise stages ask for it.
  for (uint64_t off = (static_cast<uint64_t>(blockIdx.x) * kThreads + threadIdx.x) * 128ull;
       off < P.hot_const_bytes; off += static_cast<uint64_t>(gridDim.x) * kThreads * 128ull)
    asm volatile("prefetch.global.L2 [%0];" ::"l"(P.hot_consts + off));
  // The same for the stage table, the operator descriptors and the tensor maps (one image): every
  // role of every CTA reads its descriptor at each stage, from L2 instead of HBM when the launch
  // starts with a cold cache.
  for (uint64_t off = (static_cast<uint64_t>(blockIdx.x) * kThreads + threadIdx.x) * 128ull;
       off < P.table_bytes; off += static_cast<uint64_t>(gridDim.x) * kThreads * 128ull)
    asm volatile("prefetch.global.L2 [%0];" ::"l"(reinterpret_cast<const uint8_t*>(P.stages) + off));

  Ctx c;
  c.P = &P;
  c.ctrl = ctrl;
  c.a_ring = smem_u32(base);
  c.b_ring = c.a_ring + kASlots * kSlotBytes;
  c.a_ring_ptr = base;
  c.store_stage = base + kASlots * kSlotBytes + kBSlots * kBSlotBytes + kCtrlBytes;
  c.stage = P.stage_begin;
  c.group_phase = 0;
  c.timeout_ns = static_cast<uint64_t>(P.timeout_us) * 1000ull;

  // 384 threads share the 64 K registers: 168 each, which every role fits without spilling.
  if (warp < 4) {
    if (warp == 0) role_weight_producer(c, lane);
    else if (warp == 1) role_act_producer(c, lane);
    else if (warp == 2) role_mma(c, tmem_base, lane);
  } else {
    role_simt(c, tmem_base, threadIdx.x - kRoleThreads);
  }
  __syncwarp();

  // Teardown. On the abort path give copies and MMAs still in flight time to land
  // before the shared memory and TMEM they target are released.
  if (*reinterpret_cast<volatile uint32_t*>(&ctrl->abort_flag)) __nanosleep(2000000);
  tc_fence_before();
  __syncthreads();
  if (*reinterpret_cast<volatile uint32_t*>(&ctrl->abort_flag)) __nanosleep(2000000);
  if (warp == 2) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(kTmemCols)
                 : "memory");
  }
  // a CTA's shared memory must outlive the last remote arrival aimed at it
  if (P.cluster > 1u) cluster_sync_all();
}

}  // namespace mononn
