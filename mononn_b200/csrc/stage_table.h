// Stage table shared by the host lowering and the persistent sm_100a kernel.
//
// The reference emits one CUDA source per graph: per-node device functions in
// wave-front order with a grid barrier at every depth boundary
// (mononn_engine/codegen/graph_codegen.cc:768-800).  Here the same structure
// is data: a list of stages (one per barrier depth), each holding a span of
// operator descriptors whose work items are dealt round-robin to the CTAs of
// one cooperative launch.
#pragma once
#include <stdint.h>

namespace mononn {

enum OpKind : uint32_t {
  OP_NONE = 0,
  OP_GEMM = 1,       // tcgen05 GEMM, 128-row tiles, fused epilogue
  OP_ATTENTION = 2,  // per (batch, head, 128 query rows): QK^T -> softmax -> PV
  OP_LAYERNORM = 3,  // row-wise LayerNorm over an f32 or f16 source
  OP_EMBED = 4,      // row gather + position + type + LayerNorm, mask bias
  OP_L2NORM_LOGITS = 5,
  OP_ASSEMBLE = 6,   // token rows = [constant prefix rows | GEMM rows + bias] + position rows -> f32
  OP_PATCHIFY = 7,   // NCHW f32 image -> f16 window rows (operand of the convolution's GEMM)
  OP_ARGMAX = 8,     // s32 index of the maximum of every f16 row (first index on ties)
  OP_ROWSEL = 9,     // out[b,:] = src[b*seq + argmax(ids[b,:]), :] (pooling at the largest token id)
  OP_PAIRDOT = 10,   // out[i,j] = alpha * <a[i,:], b[j,:]> for two small f16 activations (SIMT)
};

enum ActKind : uint32_t {
  ACT_NONE = 0,
  ACT_GELU_ERF = 1,
  ACT_RELU = 2,
  ACT_QUICK_GELU = 3,
  ACT_GELU_TANH = 4,
};

enum OutMode : uint32_t {
  OUT_F16 = 0,      // out[row*ldo + col] = half(v)
  OUT_F16_T = 1,    // out[batch][col][row_in_batch] = half(v)  (V^T for attention)
  OUT_F32_RED = 2,  // red.add into f32 out[row*ldo + col] (split-K partials)
  OUT_F32 = 3,      // out[row*ldo + col] = v
};

enum OpFlags : uint32_t {
  F_BIAS = 1u << 0,
  F_RESID = 1u << 1,       // residual add (f16 source)
  F_ZERO_SRC = 1u << 2,    // LayerNorm: clear the f32 source after reading it
  F_CAUSAL = 1u << 3,      // attention: key index > query index is masked
  F_MASK_BIAS = 1u << 4,   // attention: additive f32 bias per (batch, key)
  F_SRC_F32 = 1u << 5,     // LayerNorm source is f32 (else f16)
  F_TYPE_IDS = 1u << 6,    // embed: token-type table present
  F_OUT2_F16 = 1u << 7,    // LayerNorm: also write the un-normalised sum as f16
  F_RESID_F32 = 1u << 8,   // residual source is f32
  F_NO_NORM = 1u << 9,     // row op: no LayerNorm, the row sum is the result
  F_L2NORM = 1u << 10,     // row op: x / sqrt(sum x^2) instead of LayerNorm (scale and shift unused)
  F_FUSED_QKV = 1u << 11,  // attention: the item first computes its own Q, K, V = x W_h + b_h
  F_POS_BIAS = 1u << 12,   // attention: additive f16 bias per (head, query, key), q[0] = [heads, seq, seq]
  F_RMSNORM = 1u << 13,    // row op: x * rsqrt(mean(x^2) + eps) * scale (no mean subtraction, no shift)
  F_ROW_SPLIT = 1u << 14,  // LayerNorm: a row is shared by four warps (two rows per work item), for few rows
};

// Pointer slots p[0..7]; meaning per kind:
//  GEMM:      0 out, 1 bias(f16), 2 resid
//  ATTENTION: 0 out ctx(f16), 1 mask bias(f32 [B,S]); with F_FUSED_QKV also 2/3/4 = bias of Q/K/V
//             (f16 [heads*64]), tmap_a = x [tokens, K], tmap_b / tmap_vt / vocab = tensor maps of the
//             Q / K / V weights packed in 64-row tiles, K = hidden size, kb_per_split = K/64
//  LAYERNORM: 0 out(f16), 1 src, 2 gamma(f16), 3 beta(f16), 4 resid(f16, optional), 5 out2
//  EMBED:     0 out(f16), 1 ids(i32), 2 type ids(i32), 3 word table(f16), 4 pos table(f16),
//             5 type table(f16), 6 gamma, 7 beta ; mask(i32) -> q[0], mask bias out(f32) -> q[1]
//  ASSEMBLE:  0 out(f16, optional), 1 GEMM rows(f16), 3 prefix rows(f16), 4 position rows(f16),
//             5 bias(f16), 6/7 valid dummies; seq = tokens per batch, k_col = prefix rows
//  PATCHIFY:  0 out(f16 [rows, cols]), 1 image(f32 NCHW); heads = C, seq = H, batches = W,
//             head_dim = kh, q_col = kw, k_col = windows per image row, vocab = windows per image,
//             M / N = vertical / horizontal stride, rows_per_batch / ldt = rows / columns of zero
//             padding above / left of the image, K = kh*kw*C (columns K..cols-1 are written as 0)
//  EMBED: q_col = offset added to the position index; p[4] = 0: no position table
//  ATTENTION with F_POS_BIAS: q[0] = f16 [heads, seq, seq] added to the scaled scores (seq % 32 == 0)
//  LAYERNORM and EMBED may also write q[2] = f32 copy of the result plus the f16 bias q[3]
//  (residual + bias pre-loaded into the accumulator of the next split-K GEMM)
struct alignas(16) OpDesc {
  uint32_t kind;
  uint32_t flags;
  uint32_t n_items;  // work items of this op
  uint32_t act;
  // GEMM geometry
  uint32_t tmap_a, tmap_b;  // tensor-map indices
  uint32_t m_tiles, n_tiles, k_split, kb_per_split;  // kb = 64-element k block
  uint32_t n_tile;          // UMMA N (multiple of 16, <= 256)
  uint32_t kb_per_bslot;    // k blocks fetched per weight-ring slot
  uint32_t M, N, K;         // valid extents
  uint32_t out_mode;
  uint32_t ldo, ldr;        // leading dims (elements) of out / resid
  uint32_t rows_per_batch;  // OUT_F16_T: rows per batch (sequence length)
  uint32_t ldt;             // OUT_F16_T: leading dim of the transposed output
  float alpha;
  float eps;
  // attention geometry
  uint32_t heads, seq, batches, head_dim;
  uint32_t q_col, k_col;    // column offsets of Q and K inside the tmap_a tensor
  uint32_t tmap_vt;         // tensor map over V^T [batches*heads*head_dim, seq]
  uint32_t cols;            // row length for row-wise ops
  uint32_t rows;            // row count for row-wise ops
  uint32_t lds;             // leading dim of row-wise source
  uint32_t vocab;           // embed: word-table rows (ids are not clamped, as in the reference)
  uint32_t pad0;
  uint32_t flag_target;     // row op that follows its producer GEMM inside one stage: arrivals to wait for
  uint32_t wait_target;     // GEMM that follows the attention it reads inside one stage: arrivals to wait for
  uint64_t p[8];
  uint64_t q[4];  // LAYERNORM / EMBED: q[2] second output (f32, + q[3] bias f16), see plan
  // Arrival counter shared by a split-K GEMM and the row op that consumes its accumulator in the
  // same stage: every GEMM item adds 1 after its reductions, the row items wait for flag_target.
  uint64_t flag;
  // Arrival counter of the attention operator whose output this GEMM reads in the same stage: every
  // attention item adds 1 after its stores, the GEMM's activation producer waits for wait_target.
  uint64_t wait_flag;
};
static_assert(sizeof(OpDesc) == 256, "operator descriptor is copied as sixteen 16-byte words");

constexpr uint32_t kMaxStageOps = 8;

struct alignas(16) StageDesc {
  uint32_t op_begin;
  uint32_t op_count;  // at most kMaxStageOps
  uint32_t n_items;   // sum over the ops
  // Work items up to and including the last attention operator that computes its own projections
  // (0: the stage has none): the CTAs from this index on prefetch those projections' weights to L2.
  uint32_t attn_prefetch_from;
  // item_end[k] = work items of ops 0..k; entries past the last op are 0xffffffff, so the
  // owner of an item is found by comparisons alone
  uint32_t item_end[kMaxStageOps];
};

// Status word written by the kernel when a bounded wait expires.
struct KernelStatus {
  uint32_t code;   // 0 ok
  uint32_t stage;
  uint32_t cta;
  uint32_t where;  // which wait gave up
};

enum StatusCode : uint32_t {
  ST_OK = 0,
  ST_GRID_BARRIER_TIMEOUT = 1,
  ST_MBARRIER_TIMEOUT = 2,
};

// Shared-memory ring geometry (bytes).
constexpr uint32_t kSlotBytes = 16384;   // activation ring slot: one 128x64 f16 operand tile
constexpr uint32_t kBSlotBytes = 32768;  // weight ring slot: up to 256 rows of 64 f16 (one TMA box)
#ifndef MONONN_A_SLOTS
#define MONONN_A_SLOTS 6
#endif
#ifndef MONONN_B_SLOTS
#define MONONN_B_SLOTS 3
#endif
constexpr uint32_t kASlots = MONONN_A_SLOTS;
constexpr uint32_t kBSlots = MONONN_B_SLOTS;
constexpr uint32_t kStoreStageBytes = 16384;  // per epilogue warp 32 rows x 64 B, to store rows in 64-byte runs
constexpr uint32_t kCtrlBytes = 12288;        // shared-memory reserve of the control block
constexpr uint32_t kRoleThreads = 128;        // warps 0..3: producers and the MMA issuer (one lane each)
constexpr uint32_t kSimtThreads = 256;        // warps 4..11: epilogue / row-wise work
constexpr uint32_t kSimtWarps = kSimtThreads / 32;
constexpr uint32_t kThreads = kRoleThreads + kSimtThreads;
constexpr uint32_t kRowsPerItem = kSimtWarps;  // row-wise operators: one row per SIMT warp per work item
constexpr uint32_t kSplitRowsPerItem = 2;      // LayerNorm with F_ROW_SPLIT: four warps per row
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kTraceEvents = 16;  // per (CTA, stage) slots of the optional event trace
constexpr uint32_t kAccCols = 256;  // two accumulator buffers of 256 columns

struct KernelParams {
  const StageDesc* stages;
  const OpDesc* ops;
  const void* tmaps;     // CUtensorMap[]
  uint32_t* barrier;     // monotonically increasing arrival counter
  KernelStatus* status;
  uint64_t* stamps;      // optional per-stage %globaltimer stamps (CTA 0), or null
  uint64_t* trace;       // optional [cta][stage][kTraceEvents] event times, or null
  const uint8_t* hot_consts;  // small constants (biases, scale/shift), prefetched to L2 at start
  uint64_t hot_const_bytes;
  uint32_t n_stages;
  uint32_t epoch_base;   // counter value at kernel entry
  uint32_t timeout_us;   // bound on every wait
  uint32_t stage_begin;  // run stages [stage_begin, stage_end)
  uint32_t stage_end;
  uint32_t cluster;      // CTAs per cluster of this launch (1: no cluster-scoped arrival)
  uint32_t l2_hints;     // 1: weight tiles are loaded evict-first, GEMM activation tiles evict-last (default)
  uint32_t warp_arrive;  // 1: every epilogue warp arrives at the grid barrier for itself (8 arrivals per
                         // CTA and stage, no CTA-wide sync before the arrival); 2: the warps count themselves
                         // in shared memory and the last one arrives for the CTA; 0: one arrival per CTA
                         // after a CTA-wide sync
  uint32_t flag_epoch;   // launches that have added to the arrival counters since they were cleared,
                         // this one included (row ops wait for flag_epoch * their GEMM items)
  uint32_t table_bytes;  // size of the stage / operator / tensor-map image that starts at `stages`
                         // (prefetched to L2 at kernel start; 0: not prefetched)
  uint32_t* host_flag;   // optional word in pinned host memory, set to the status code when a bounded
                         // wait expires: the host learns of a failure without copying the status back
};

}  // namespace mononn
