// Issue-cost probe for tcgen05.mma (sm_100a): how long does the tensor pipe take per
// instruction when nothing else is in the way?
//
// One CTA per SM, operands resident in shared memory (zero-filled K-major 128-byte-swizzled
// tiles: A 128x64, B 256x64), no TMA and no mbarrier inside the timed loop. One thread issues
// `count` instructions of shape 128 x n x 16 (kind::f16, f32 accumulate) back to back, cycling
// through the four k-steps of the 64-wide tile and through `accumulators` TMEM buffers, then one
// tcgen05.commit; clock64 brackets first issue .. commit observed. The tile choice of the
// persistent kernel (how narrow a tile may be before the instruction count, not the operand
// bytes, bounds a main loop) rests on this table. Modes add the per-k-block bookkeeping of the
// kernel's MMA role one piece at a time, so that a stall can be told from pipe time.
//
// The reference has no counterpart: its GEMM tiles are a CUTLASS 2.x menu
// (mononn_engine/core/op_impl/gemm_impl.cc:505-566) timed whole by the tuner.
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>
#include <utility>
#include <vector>

#include "../../include/mononn.h"
#include "runtime.h"

namespace mononn {
namespace {

struct ProbeOut {
  unsigned long long cycles_issue;  // first issue .. last issue returned
  unsigned long long cycles_done;   // first issue .. commit observed
  unsigned long long ns_done;
  unsigned int ok;
  unsigned int pad;
};

__device__ __forceinline__ uint32_t s_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ uint64_t desc_sw128(uint32_t saddr) {
  return static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4) | (1ull << 16) | (64ull << 32) | (1ull << 46) |
         (2ull << 61);
}
__device__ __forceinline__ void mma(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}" ::"r"(d),
      "l"(a), "l"(b), "r"(idesc), "r"(acc), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
      : "memory");
}
// A operand read from tensor memory (128 lanes x 8 columns hold one 128 x 16 f16 slice)
__device__ __forceinline__ void mma_ts(uint32_t d, uint32_t a_tmem, uint64_t b, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %6, %7, %8}, p;\n\t}" ::"r"(d),
      "r"(a_tmem), "l"(b), "r"(idesc), "r"(acc), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
      : "memory");
}
// The same instruction without the optional disable-output-lane vector
__device__ __forceinline__ void mma_plain(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d),
      "l"(a), "l"(b), "r"(idesc), "r"(acc)
      : "memory");
}
__device__ __forceinline__ uint32_t elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred)::"memory");
  return pred;
}
__device__ __forceinline__ void commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}
__device__ __forceinline__ uint32_t try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}

// mode bit 0: a commit (to a barrier nobody waits on) after every four instructions
// mode bit 1: a try_wait on an already completed barrier + tcgen05.fence before every four
// mode bit 2: M = 64 instead of 128 (half of the A rows per instruction)
// mode bit 3: the A operand is read from tensor memory (columns 448..479) instead of shared memory
// mode bit 4: the instruction is written without the disable-output-lane vector
// mode bit 5: the whole first warp runs the loop converged and one elected lane issues (operands
//             can then live in uniform registers)
// mode bit 6: the operand descriptors are rebuilt for every group of four from a ring-slot index
//             (slot stride `slot_stride` bytes, 0 from the host: same data, but nothing the compiler
//             can hoist), as a main loop over a ring of tiles has to
// The mode is a template parameter: a run-time test inside the loop would be part of what is timed.
template <uint32_t mode>
__global__ void __launch_bounds__(128, 1)
mma_probe_kernel(ProbeOut* out, uint32_t n, uint32_t count, uint32_t accumulators, uint32_t slot_stride) {
  extern __shared__ uint8_t raw[];
  __shared__ uint64_t bar_done, bar_side, bar_ready;
  __shared__ uint32_t tmem_slot;
  const uint32_t pad = (1024u - (s_u32(raw) & 1023u)) & 1023u;
  uint8_t* base = raw + pad;
  for (uint32_t i = threadIdx.x; i < (16384u + 32768u) / 16u; i += blockDim.x)
    reinterpret_cast<uint4*>(base)[i] = make_uint4(0u, 0u, 0u, 0u);
  if (threadIdx.x == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(s_u32(&bar_done)) : "memory");
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(s_u32(&bar_side)) : "memory");
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(s_u32(&bar_ready)) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(s_u32(&bar_ready)) : "memory");
  }
  if (threadIdx.x < 32) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(s_u32(&tmem_slot))
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(&tmem_slot);
  if ((mode & 32u) ? (threadIdx.x < 32) : (threadIdx.x == 0)) {
    const bool issuer = (mode & 32u) ? (elect_one() != 0u) : true;
    const uint32_t m = (mode & 4u) ? 64u : 128u;
    const uint32_t idesc = (1u << 4) | ((n >> 3) << 17) | ((m >> 4) << 24);
    uint64_t ad = desc_sw128(s_u32(base)), bd = desc_sw128(s_u32(base) + 16384u);
    const uint32_t acc_stride = 512u / accumulators;
    const unsigned long long t0 = clock64();
    uint64_t g0;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(g0));
    for (uint32_t i = 0; i < count; i += 4) {
      if (mode & 2u) {
        while (!try_wait(s_u32(&bar_ready), 0)) {
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      }
      const uint32_t d = tmem + ((i >> 2) % accumulators) * acc_stride;
      if (mode & 64u) {
        ad = desc_sw128(s_u32(base) + ((i >> 2) % 6u) * slot_stride);
        bd = desc_sw128(s_u32(base) + 16384u + ((i >> 2) % 3u) * slot_stride);
      }
#pragma unroll
      for (uint32_t k = 0; k < 4; ++k) {
        if (issuer) {
          if (mode & 8u) {
            mma_ts(d, tmem + 448u + 8u * k, bd + 2u * k, idesc, (i | k) != 0u);
          } else if (mode & 16u) {
            mma_plain(d, ad + 2u * k, bd + 2u * k, idesc, (i | k) != 0u);
          } else {
            mma(d, ad + 2u * k, bd + 2u * k, idesc, (i | k) != 0u);
          }
        }
      }
      if ((mode & 1u) && issuer) commit(s_u32(&bar_side));
    }
    const unsigned long long t1 = clock64();
    if (issuer) commit(s_u32(&bar_done));
    uint32_t ok = 0;
    for (uint32_t it = 0; it < 20000000u && !ok; ++it) ok = try_wait(s_u32(&bar_done), 0);
    const unsigned long long t2 = clock64();
    uint64_t g1;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(g1));
    ProbeOut o;
    o.cycles_issue = t1 - t0;
    o.cycles_done = t2 - t0;
    o.ns_done = g1 - g0;
    o.ok = ok;
    o.pad = 0;
    if (threadIdx.x == 0) out[blockIdx.x] = o;
    if (!ok) __nanosleep(2000000);  // give the pipe time to drain before TMEM is released
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (threadIdx.x < 32) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem) : "memory");
  }
}

template <uint32_t... kModes>
auto probe_kernel_table(std::integer_sequence<uint32_t, kModes...>) {
  static void (*const table[])(ProbeOut*, uint32_t, uint32_t, uint32_t, uint32_t) = {mma_probe_kernel<kModes>...};
  return table;
}
void (*probe_kernel_for(uint32_t mode))(ProbeOut*, uint32_t, uint32_t, uint32_t, uint32_t) {
  return probe_kernel_table(std::make_integer_sequence<uint32_t, 128>{})[mode];
}

int probe_fail(int code, const std::string& msg) {
  set_last_error(msg);
  return code;
}

}  // namespace
}  // namespace mononn

using namespace mononn;

extern "C" int mononn_debug_mma_issue(int device, unsigned n, unsigned count, unsigned accumulators,
                                      unsigned mode, unsigned ctas, double* cycles_per_mma,
                                      double* issue_cycles_per_mma, double* ns_per_mma) {
  if (n < 16 || n > 256 || (n % 16u) != 0u) return probe_fail(MONONN_ERR_INVALID_ARGUMENT, "n must be a multiple of 16 in 16..256");
  if (count < 4 || count > (1u << 20) || (count % 4u) != 0u)
    return probe_fail(MONONN_ERR_INVALID_ARGUMENT, "count must be a multiple of 4 in 4..1048576");
  if (accumulators < 1 || accumulators > 4 || accumulators * n > 512u || (512u % accumulators) != 0u)
    return probe_fail(MONONN_ERR_INVALID_ARGUMENT, "accumulators x n must fit 512 TMEM columns");
  if (mode > 127u) return probe_fail(MONONN_ERR_INVALID_ARGUMENT, "mode has seven bits");
  if ((mode & 8u) && (mode & 16u)) return probe_fail(MONONN_ERR_INVALID_ARGUMENT, "mode bits 3 and 4 exclude each other");
  if ((mode & 8u) && (accumulators != 1u || n > 256u))
    return probe_fail(MONONN_ERR_INVALID_ARGUMENT, "with A in tensor memory one accumulator of at most 256 columns");
  if (ctas < 1 || ctas > 1024) return probe_fail(MONONN_ERR_INVALID_ARGUMENT, "ctas out of range");
  int prev = 0;
  if (cudaGetDevice(&prev) != cudaSuccess) return probe_fail(MONONN_ERR_NO_DEVICE, "no CUDA device");
  if (cudaSetDevice(device) != cudaSuccess) return probe_fail(MONONN_ERR_NO_DEVICE, "cannot select the device");
  cudaDeviceProp prop;
  int rc = MONONN_OK;
  ProbeOut* d = nullptr;
  std::vector<ProbeOut> h(ctas);
  const size_t smem = 16384 + 32768 + 1024;
  auto bail = [&](int code, const std::string& msg) {
    if (d) cudaFree(d);
    cudaSetDevice(prev);
    return probe_fail(code, msg);
  };
  if (cudaGetDeviceProperties(&prop, device) != cudaSuccess || prop.major != 10)
    return bail(MONONN_ERR_NO_DEVICE, "the probe is built for sm_100a only");
  if (ctas > static_cast<unsigned>(prop.multiProcessorCount))
    return bail(MONONN_ERR_INVALID_ARGUMENT, "more CTAs than SMs: TMEM allocation would serialise them");
  if (cudaMalloc(&d, ctas * sizeof(ProbeOut)) != cudaSuccess) return bail(MONONN_ERR_CUDA, "cudaMalloc failed");
  if (cudaMemset(d, 0, ctas * sizeof(ProbeOut)) != cudaSuccess) return bail(MONONN_ERR_CUDA, "cudaMemset failed");
  using Kernel = void (*)(ProbeOut*, uint32_t, uint32_t, uint32_t, uint32_t);
  Kernel kernel = probe_kernel_for(mode);
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) !=
      cudaSuccess)
    return bail(MONONN_ERR_CUDA, "cannot raise the shared-memory limit");
  for (int rep = 0; rep < 2; ++rep) {  // the second launch is the warm one
    kernel<<<ctas, 128, smem>>>(d, n, count, accumulators, 0u);
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return bail(MONONN_ERR_CUDA, std::string("probe launch: ") + cudaGetErrorString(e));
  }
  if (cudaMemcpy(h.data(), d, ctas * sizeof(ProbeOut), cudaMemcpyDeviceToHost) != cudaSuccess)
    return bail(MONONN_ERR_CUDA, "cudaMemcpy failed");
  double cyc = 0, iss = 0, ns = 0;
  for (unsigned i = 0; i < ctas; ++i) {
    if (!h[i].ok) rc = MONONN_ERR_BARRIER_TIMEOUT;
    cyc += static_cast<double>(h[i].cycles_done);
    iss += static_cast<double>(h[i].cycles_issue);
    ns += static_cast<double>(h[i].ns_done);
  }
  cudaFree(d);
  cudaSetDevice(prev);
  if (rc) return probe_fail(rc, "the commit of the probe's instructions was not observed");
  const double denom = static_cast<double>(ctas) * count;
  if (cycles_per_mma) *cycles_per_mma = cyc / denom;
  if (issue_cycles_per_mma) *issue_cycles_per_mma = iss / denom;
  if (ns_per_mma) *ns_per_mma = ns / denom;
  return MONONN_OK;
}
