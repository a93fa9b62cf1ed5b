// Host-side intermediate forms between the HLO graph and the device stage table.
//
//   HLO text --parser--> HloModule --recogniser--> FGraph --scheduler--> Plan --runtime--> device
//
// FGraph is the graph after this build's fusion passes: each node is one of the
// kernel's operator kinds with its fused prologue/epilogue.  It plays the part of
// the reference's clustered core::graph::Graph after run_group_pre_impl_assignment
// (mononn_engine/optimization/optimization_runner.cc:61-84).  Plan is the result
// of implementation/buffer assignment (optimization_runner.cc:86-163) and of
// GraphCodegen::generate (mononn_engine/codegen/graph_codegen.cc:637-842), as
// tables rather than source text.
#pragma once
#include <stdint.h>

#include <map>
#include <string>
#include <vector>

#include "stage_table.h"

namespace mononn {

// ---------------------------------------------------------------- tuning spec
struct GemmTileSpec {
  uint32_t n_tile = 0;   // 0 = choose by heuristic
  uint32_t k_split = 0;
};

struct TuningSpec {
  uint32_t grid = 0;       // CTAs; 0 = one per SM
  uint32_t block = kThreads;
  uint32_t smem_bytes = 0; // filled by the scheduler
  std::map<std::string, GemmTileSpec> gemm;  // per GEMM node
  std::vector<std::string> allow_list;       // run only these nodes (single-node profiling)
  std::vector<std::string> reject_list;
  // 0: fuse the Q/K/V projections into an attention stage that cannot fill the GPU anyway
  // (batches*heads <= CTAs, sequence <= 128); 1: never; 2: whenever the sequence allows it
  uint32_t qkv_fusion = 0;
  // 2: a LayerNorm that reads a split-K accumulator joins its GEMMs' stage and waits on an
  // arrival counter instead of a grid barrier; 1: it keeps a stage of its own; 0: the scheduler
  // decides (joined when the LayerNorm's rows are at most one wave of work items) and writes
  // its choice back
  uint32_t row_fusion = 0;
  // CTAs per thread-block cluster (1, 2 or 4; 0 = 1). With more than one, the CTAs of a cluster
  // arrive at the grid barrier through an mbarrier in the first CTA's shared memory and that
  // CTA alone adds to the global counter.
  uint32_t cluster = 0;
  // L2 eviction-priority hints on the TMA loads: 2 weights evict-first and GEMM activation
  // tiles evict-last, 1 none, 0 the scheduler decides (hints when no GEMM has more than four row
  // tiles, i.e. when a weight tile is read by few CTAs) and writes its choice back
  uint32_t l2_hints = 0;
  // grid-barrier arrival: 0 / 3 one per CTA by the epilogue warp that finishes the stage last (the
  // warps count themselves in shared memory), 2 one per epilogue warp (each releases its own
  // stores), 1 one per CTA after a CTA-wide sync (always the case inside a cluster launch)
  uint32_t barrier_arrive = 0;
  // 0 / 2: a LayerNorm with few rows shares each row among four warps; 1: always one warp per row
  uint32_t row_split = 0;
  // 2: the GEMM that reads an attention's output shares its stage and waits on its arrival counter;
  // 3: only behind an attention that computes its own projections; 1: it keeps a stage of its own;
  // 0: the scheduler decides (3 when the attention's work items occupy at most half of the CTAs
  // and the LayerNorms are joined too, else 1) and writes it back
  uint32_t out_fusion = 0;
  // 2: a GEMM that reads the output of another GEMM shares that GEMM's stage too and waits on its
  // arrival counter (FFN-up and FFN-down in one stage); 1: no; 0: the scheduler decides (no: it
  // measured no faster than the barrier) and writes it back
  uint32_t chain_fusion = 0;
};

// ------------------------------------------------------------------- FGraph
enum class TKind : uint32_t {
  ActF16,   // f16 activation [rows, ld] living in the caller's temp buffer
  ActF16T,  // per-batch transposed f16 activation [batches*cols, ldt] (V^T), temp buffer
  AccF32,   // f32 [rows, cols] accumulator in module scratch, zero whenever it is not live
  VecF32,   // f32 vector [rows] in module scratch (mask bias)
  Const,    // HLO constant (weights, biases, tables)
  Arg,      // kernel argument (parameter or live-out)
};

struct FTensor {
  std::string name;
  TKind kind = TKind::ActF16;
  uint32_t rows = 0, cols = 0, ld = 0;
  uint32_t batches = 1, seq = 0;  // ActF16T geometry
  uint32_t elem_bytes = 2;
  int arg_index = -1;             // Arg
  std::string const_name;         // Const: HLO constant name
  std::vector<uint32_t> const_dims;
  bool const_transposed = false;  // Const weight given as [N, K] instead of [K, N]
};

struct FOp {
  OpKind kind = OP_NONE;
  std::string name;
  uint32_t flags = 0;
  ActKind act = ACT_NONE;
  float alpha = 1.f, eps = 0.f;
  // GEMM: a (ActF16 [M,K]), w (Const [K,N]), bias (Const [N]), resid (ActF16), out
  int a = -1, w = -1, bias = -1, resid = -1, out = -1;
  uint32_t M = 0, N = 0, K = 0;
  // ATTENTION: q, k (ActF16 with column offsets), vt (ActF16T), mask (VecF32), out
  int q = -1, k = -1, vt = -1, mask = -1;
  // ATTENTION fused with its projections: a = x, w / wk / wv and bias / bias_k / bias_v, K = width of x
  int wk = -1, wv = -1, bias_k = -1, bias_v = -1;
  // ATTENTION: optional additive bias per (head, query, key), a constant [heads*seq, seq] (the
  // relative position bias of T5, folded to a tensor by the compiler that wrote the HLO)
  int pos_bias = -1;
  uint32_t q_col = 0, k_col = 0, heads = 0, seq = 0, batches = 0, head_dim = 64;
  // LAYERNORM: src (AccF32 | ActF16), resid, gamma, beta, out
  int src = -1, gamma = -1, beta = -1;
  // LAYERNORM / EMBED: optional f32 copy of the result (+ bias2) into an accumulator
  int out2 = -1, bias2 = -1;
  // EMBED: ids, type_ids, mask_in (Arg), word/pos/type tables (Const), mask_out (VecF32)
  int ids = -1, type_ids = -1, mask_in = -1, word = -1, pos = -1, type = -1, mask_out = -1;
  uint32_t rows = 0, cols = 0, vocab = 0;
  // PATCHIFY: M / N = strides, K = window elements, zero padding above / left of the image
  uint32_t pad_top = 0, pad_left = 0;
  int stage = -1;  // filled by the scheduler
};

struct ArgDesc {
  std::string name;
  size_t bytes = 0;
  int kind = 0;  // 0 parameter, 1 live-out, 2 temp
  int param_number = -1;
};

struct FGraph {
  std::string module_name;
  std::vector<FTensor> tensors;
  std::vector<FOp> ops;
  std::vector<ArgDesc> args;  // parameters.., live-outs.. ; the scheduler appends temp
  // constants whose values were printed in the HLO text, in their element type, by constant name:
  // given to the runtime when the module is compiled, so that nobody has to set them
  std::map<std::string, std::vector<uint8_t>> literals;
  int add_tensor(const FTensor& t) {
    tensors.push_back(t);
    return static_cast<int>(tensors.size()) - 1;
  }
};

// --------------------------------------------------------------------- Plan
enum BufSpace : int32_t { SPACE_NONE = -1, SPACE_ARG = 0, SPACE_CONST = 1, SPACE_SCRATCH = 2 };

struct BufRef {
  int32_t space = SPACE_NONE;
  int32_t index = 0;  // argument index for SPACE_ARG
  uint64_t offset = 0;
};

struct TmapSpec {
  BufRef base;
  uint64_t dim0 = 0, dim1 = 0;  // elements; dim0 is contiguous
  uint64_t stride1_bytes = 0;
  uint32_t box0 = 0, box1 = 0;
};

struct PlanOp {
  std::string name;
  OpDesc d{};
  BufRef p[8];
  BufRef q[4];
  // arrival counter shared by a split-K GEMM (signals) and the row op of the same stage that
  // reads its accumulator (waits); flag_index < 0: none
  BufRef flag;
  int flag_index = -1;
  bool waits = false;
  // arrival counter of an attention operator of the same stage that a GEMM reading its output
  // waits for before it loads its A operand; wflag_index < 0: none
  BufRef wflag;
  int wflag_index = -1;
};

// How one HLO constant lands in the constant arena.
struct ConstBinding {
  std::string const_name;
  enum Kind { RAW, PACK_B } kind = RAW;
  uint64_t offset = 0, bytes = 0;
  // PACK_B: source is row-major [K, N] (or [N, K] when transposed) f16;
  // destination is [n_tiles][K/64][n_tile][64] so every (n tile, k block) is one
  // contiguous 128-byte-row tile a single TMA box can fetch.
  uint32_t K = 0, N = 0, n_tile = 0;
  uint32_t K_src = 0;  // rows of the source when it has fewer than K (the rest packs as zeros)
  bool transposed = false;
  size_t src_bytes = 0;
};

// Where a graph tensor lives (for inspection and intermediate-tensor parity checks).
struct TensorPlacement {
  std::string name;
  TKind kind = TKind::ActF16;
  BufRef at;
  uint32_t rows = 0, cols = 0, ld = 0, batches = 1, seq = 0;
  int def_stage = -1, last_stage = -1;
};

struct Plan {
  std::string module_name;
  std::vector<TensorPlacement> tensors;
  std::vector<PlanOp> ops;
  std::vector<StageDesc> stages;
  std::vector<std::string> stage_names;
  std::vector<TmapSpec> tmaps;
  std::vector<ArgDesc> args;
  std::vector<ConstBinding> consts;
  uint64_t const_bytes = 0;
  uint64_t hot_const_bytes = 0;  // leading part of the constant arena holding the small constants
  uint64_t scratch_bytes = 0;  // module-owned, zero-initialised
  uint64_t flag_offset = 0, flag_bytes = 0;  // arrival counters of row ops fused into GEMM stages
  uint64_t temp_bytes = 0;
  uint32_t grid = 0, block = kThreads, smem_bytes = 0;
  uint32_t cluster = 1;  // CTAs per cluster of the launch
  TuningSpec spec;             // the spec this plan realises (with heuristics filled in)
  double algorithmic_bytes = 0, algorithmic_flops = 0;
};

// Scheduler: stage assignment by dependency depth, tile selection, buffer and
// tensor-map assignment. Returns 0 or a negative mononn error code; `err` gets a message.
int schedule(const FGraph& g, const TuningSpec& spec, uint32_t sm_count, Plan* plan,
             std::string* err);

// Host-side check of every invariant the kernel assumes (ring-slot sizes, TMA boxes, tile
// coverage, buffer presence). schedule() ends with it; the runtime repeats it before loading.
int validate_plan(const Plan& plan, std::string* err);

// Default tile choice for one GEMM given how many CTAs it may occupy.
GemmTileSpec default_gemm_tile(uint32_t M, uint32_t N, uint32_t K, bool can_split_k,
                               uint32_t cta_budget);
// Legal alternatives for the tuner.
std::vector<GemmTileSpec> gemm_tile_candidates(uint32_t M, uint32_t N, uint32_t K,
                                               bool can_split_k, uint32_t cta_budget);

// Fixed head of the module scratch: barrier counter, status word, per-stage time stamps.
constexpr uint64_t kScratchBarrierOff = 0, kScratchStatusOff = 256, kScratchStampsOff = 512;

constexpr uint32_t kSmemBytes =
    kASlots * kSlotBytes + kBSlots * kBSlotBytes + kCtrlBytes + kStoreStageBytes + 1024 /*align*/;

}  // namespace mononn
