// Allocation-free launch variant of the persistent kernel: one attention stage
// (QK^T -> masked softmax -> PV for every batch and head) on caller-owned buffers.
//
// Who needs it: hosts in which this library must not allocate device memory. Under
// TensorFlow/XLA the framework's own allocator has usually reserved the whole GPU, so a
// cudaMalloc made by a plug-in can fail or fragment the pool; latency-critical serving
// threads also avoid cudaMalloc because it synchronises the device. The regular path
// (mononn_compile_* / mononn_launch) keeps its stage table, tensor maps, barrier counter,
// status word and f32 work buffers in memory it allocates when a module is lowered. Here the
// same kernel reads all of that from one file-scope device array, so the call itself
// allocates nothing: no cudaMalloc / cudaFree, no allocating library call.
//
// Consequences of the shared array (documented in include/mononn.h as well):
//   * sizes are bounded: batches * seq <= MONONN_NOALLOC_MAX_TOKENS;
//   * every call on a device uses the same array and rewrites it, so two calls that overlap
//     on the GPU (different streams, or another host thread) race; serialise them;
//   * the first call on a device performs the one-time set-up (symbol address, kernel
//     attribute, SM count) and should therefore be made before any stream capture.
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>

#include "../../include/mononn.h"
#include "plan.h"
#include "runtime.h"
#include "stage_table.h"

namespace mononn {

extern "C" __global__ void mononn_megakernel(const __grid_constant__ KernelParams P);

namespace {

constexpr size_t kOffBarrier = 0, kOffStatus = 256, kOffStage = 512, kOffOp = 768, kOffTmaps = 1280,
                 kOffMask = 2048;
constexpr size_t kScratchBytes = kOffMask + static_cast<size_t>(MONONN_NOALLOC_MAX_TOKENS) * 4;
static_assert(sizeof(OpDesc) <= kOffTmaps - kOffOp, "operator descriptor does not fit its slot");

// The scratch of the allocation-free path. Every GPU that loads the library holds these
// ~66 KB until the process exits. In host code this name is only a handle for
// cudaGetSymbolAddress; the device address is obtained once per device below.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kScratchBytes];

__global__ void noalloc_mask_bias(const int32_t* __restrict__ mask, float* __restrict__ bias,
                                  uint32_t n, float scale) {
  const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) bias[i] = (1.0f - static_cast<float>(mask[i])) * scale;
}

struct DeviceState {
  bool ready = false;
  unsigned char* scratch = nullptr;
  int sm_count = 0;
};
constexpr int kMaxDevices = 64;
DeviceState g_state[kMaxDevices];
std::mutex g_mutex;
void* g_encode = nullptr;

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int fail(int code, const std::string& msg) {
  set_last_error(msg);
  return code;
}

#define NA_TRY(expr)                                                                      \
  do {                                                                                    \
    cudaError_t e__ = (expr);                                                             \
    if (e__ != cudaSuccess)                                                               \
      return fail(MONONN_ERR_CUDA, std::string(#expr) + ": " + cudaGetErrorString(e__));  \
  } while (0)

// One-time set-up for the current device.
int setup(int dev, DeviceState** out) {
  std::lock_guard<std::mutex> lock(g_mutex);
  DeviceState& st = g_state[dev];
  if (!st.ready) {
    cudaDeviceProp prop;
    NA_TRY(cudaGetDeviceProperties(&prop, dev));
    if (prop.major != 10) return fail(MONONN_ERR_NO_DEVICE, "the kernel is built for sm_100a only");
    void* p = nullptr;
    NA_TRY(cudaGetSymbolAddress(&p, g_noalloc_scratch));
    if (p == nullptr) return fail(MONONN_ERR_CUDA, "cudaGetSymbolAddress returned a null address");
    NA_TRY(cudaFuncSetAttribute(mononn_megakernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                static_cast<int>(kSmemBytes)));
    if (g_encode == nullptr) {
      cudaDriverEntryPointQueryResult q;
      NA_TRY(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &g_encode, cudaEnableDefault, &q));
      if (q != cudaDriverEntryPointSuccess || g_encode == nullptr)
        return fail(MONONN_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    }
    st.scratch = static_cast<unsigned char*>(p);
    st.sm_count = prop.multiProcessorCount;
    st.ready = true;
  }
  *out = &st;
  return MONONN_OK;
}

int encode_f16(CUtensorMap* tm, const void* base, uint64_t dim0, uint64_t dim1, uint64_t stride_bytes,
               uint32_t box0, uint32_t box1, const char* what) {
  if ((reinterpret_cast<uintptr_t>(base) & 15u) || (stride_bytes & 15u))
    return fail(MONONN_ERR_INVALID_ARGUMENT,
                std::string(what) + ": base address and row pitch must be multiples of 16 bytes");
  const cuuint64_t dims[2] = {dim0, dim1};
  const cuuint64_t strides[1] = {stride_bytes};
  const cuuint32_t box[2] = {box0, box1};
  const cuuint32_t es[2] = {1, 1};
  CUresult r = reinterpret_cast<EncodeTiledFn>(g_encode)(
      tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), dims, strides, box, es,
      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(MONONN_ERR_CUDA, std::string(what) + ": cuTensorMapEncodeTiled failed (CUresult " +
                                     std::to_string(static_cast<int>(r)) + ")");
  return MONONN_OK;
}

}  // namespace
}  // namespace mononn

using namespace mononn;

extern "C" int mononn_attention_noalloc(const void* q, const void* k, const void* v_t,
                                        const int32_t* mask, void* out, unsigned batches,
                                        unsigned heads, unsigned seq, unsigned ld_qk, unsigned ld_vt,
                                        unsigned ld_out, float scale, float mask_scale, int causal,
                                        void* cuda_stream) {
  if (!q || !k || !v_t || !out) return fail(MONONN_ERR_INVALID_ARGUMENT, "null buffer");
  if (batches == 0 || heads == 0 || seq == 0) return fail(MONONN_ERR_INVALID_ARGUMENT, "empty problem");
  if (seq > 128)
    return fail(MONONN_ERR_TOO_LARGE, "sequence length " + std::to_string(seq) + " exceeds 128");
  const uint64_t tokens = static_cast<uint64_t>(batches) * seq;
  if (tokens > MONONN_NOALLOC_MAX_TOKENS)
    return fail(MONONN_ERR_TOO_LARGE, "batches * seq = " + std::to_string(tokens) + " exceeds the " +
                                          std::to_string(MONONN_NOALLOC_MAX_TOKENS) +
                                          " tokens the static scratch is sized for");
  // geometry in 64 bits: heads * 64 and batches * heads must not wrap for absurd inputs
  const uint64_t width64 = static_cast<uint64_t>(heads) * 64u;
  const uint64_t items64 = static_cast<uint64_t>(batches) * heads * ((seq + 127u) / 128u);
  if (width64 > 65536u || items64 > (1u << 24))
    return fail(MONONN_ERR_TOO_LARGE, "heads * 64 exceeds 65536 columns or batches * heads exceeds 2^24 tiles");
  const unsigned width = static_cast<unsigned>(width64);
  if (ld_qk < width || ld_out < width || ld_vt < seq)
    return fail(MONONN_ERR_INVALID_ARGUMENT, "leading dimensions are smaller than the rows they hold");
  if ((ld_out % 8u) != 0u || (reinterpret_cast<uintptr_t>(out) & 15u) != 0u)
    return fail(MONONN_ERR_INVALID_ARGUMENT,
                "out: base address and row pitch must be multiples of 16 bytes (the kernel stores 16-byte vectors)");
  if (mask && (reinterpret_cast<uintptr_t>(mask) & 3u) != 0u)
    return fail(MONONN_ERR_INVALID_ARGUMENT, "mask: int32 elements must be 4-byte aligned");
  int dev = 0;
  NA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return fail(MONONN_ERR_INVALID_ARGUMENT, "device ordinal out of range");
  DeviceState* st = nullptr;
  int rc = setup(dev, &st);
  if (rc) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  {
    // Each call stages its table image from a stack buffer with cudaMemcpyAsync. A capturing
    // stream would record that copy as a node that reads the buffer at replay time, long after
    // this frame is gone, and would freeze this call's pointers into the tensor maps.
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    NA_TRY(cudaStreamIsCapturing(stream, &cap));
    if (cap != cudaStreamCaptureStatusNone)
      return fail(MONONN_ERR_INVALID_ARGUMENT, "the stream is being captured; this call stages host data per call");
  }
  unsigned char* s = st->scratch;

  // host image of the table part of the scratch: stage, operator, three tensor maps
  alignas(64) unsigned char img[kOffMask];
  std::memset(img, 0, sizeof(img));  // barrier counter and status word start at zero
  StageDesc sd{};
  sd.op_begin = 0;
  sd.op_count = 1;
  OpDesc od;
  std::memset(&od, 0, sizeof(od));
  od.kind = OP_ATTENTION;
  od.flags = (mask ? F_MASK_BIAS : 0u) | (causal ? F_CAUSAL : 0u);
  od.n_items = static_cast<uint32_t>(items64);
  od.alpha = scale;
  od.heads = heads;
  od.seq = seq;
  od.batches = batches;
  od.head_dim = 64;
  od.tmap_a = 0;
  od.tmap_b = 1;
  od.tmap_vt = 2;
  od.ldo = ld_out;
  od.p[0] = reinterpret_cast<uint64_t>(out);
  od.p[1] = mask ? reinterpret_cast<uint64_t>(s + kOffMask) : 0;
  sd.n_items = od.n_items;
  for (uint32_t i = 0; i < kMaxStageOps; ++i) sd.item_end[i] = 0xffffffffu;
  sd.item_end[0] = od.n_items;
  std::memcpy(img + kOffStage, &sd, sizeof(sd));
  std::memcpy(img + kOffOp, &od, sizeof(od));
  CUtensorMap tm;
  rc = encode_f16(&tm, q, width, tokens, static_cast<uint64_t>(ld_qk) * 2, 64, 128, "q");
  if (rc) return rc;
  std::memcpy(img + kOffTmaps, &tm, 128);
  rc = encode_f16(&tm, k, width, tokens, static_cast<uint64_t>(ld_qk) * 2, 64, 128, "k");
  if (rc) return rc;
  std::memcpy(img + kOffTmaps + 128, &tm, 128);
  rc = encode_f16(&tm, v_t, seq, static_cast<uint64_t>(batches) * width, static_cast<uint64_t>(ld_vt) * 2,
                  64, 64, "v_t");
  if (rc) return rc;
  std::memcpy(img + kOffTmaps + 256, &tm, 128);
  // the copy is from pageable host memory: the runtime stages it before returning, so `img`
  // may go out of scope; it also clears the counter and the status word of the last call
  NA_TRY(cudaMemcpyAsync(s, img, sizeof(img), cudaMemcpyHostToDevice, stream));
  if (mask) {
    const uint32_t n = static_cast<uint32_t>(tokens);
    noalloc_mask_bias<<<(n + 255u) / 256u, 256, 0, stream>>>(mask, reinterpret_cast<float*>(s + kOffMask), n,
                                                           mask_scale);
    NA_TRY(cudaGetLastError());
  }
  KernelParams kp;
  std::memset(&kp, 0, sizeof(kp));
  kp.stages = reinterpret_cast<const StageDesc*>(s + kOffStage);
  kp.ops = reinterpret_cast<const OpDesc*>(s + kOffOp);
  kp.tmaps = s + kOffTmaps;
  kp.barrier = reinterpret_cast<uint32_t*>(s + kOffBarrier);
  kp.status = reinterpret_cast<KernelStatus*>(s + kOffStatus);
  kp.n_stages = 1;
  kp.epoch_base = 0;
  kp.timeout_us = 2000000u;
  kp.stage_begin = 0;
  kp.stage_end = 1;
  kp.cluster = 1;
  kp.l2_hints = 0;
  kp.warp_arrive = 0;
  kp.flag_epoch = 0;
  const unsigned grid = od.n_items < static_cast<unsigned>(st->sm_count) ? od.n_items
                                                                        : static_cast<unsigned>(st->sm_count);
  void* kargs[1] = {&kp};
  NA_TRY(cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(mononn_megakernel), dim3(grid),
                                     dim3(kThreads), kargs, kSmemBytes, stream));
  return MONONN_OK;
}

// Status of the allocation-free path: the kernel's status word lives in the static array, where a
// bounded wait that expired leaves {code, stage, CTA, wait site}. Waits for `cuda_stream`, copies
// the word out (no allocation) and reports it. The next mononn_attention_noalloc call clears it.
extern "C" int mononn_attention_noalloc_status(void* cuda_stream) {
  int dev = 0;
  NA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return fail(MONONN_ERR_INVALID_ARGUMENT, "device ordinal out of range");
  DeviceState* st = nullptr;
  int rc = setup(dev, &st);
  if (rc) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  NA_TRY(cudaStreamSynchronize(stream));
  KernelStatus ks;
  NA_TRY(cudaMemcpy(&ks, st->scratch + kOffStatus, sizeof(ks), cudaMemcpyDeviceToHost));
  if (ks.code != ST_OK)
    return fail(MONONN_ERR_BARRIER_TIMEOUT, "a bounded wait expired in the attention kernel (code " +
                                                std::to_string(ks.code) + ", CTA " + std::to_string(ks.cta) +
                                                ", wait site 0x" + [&] {
                                                  char b[16];
                                                  std::snprintf(b, sizeof(b), "%x", ks.where);
                                                  return std::string(b);
                                                }() + "); `out` is incomplete");
  return MONONN_OK;
}
