// FGraph -> Plan: barrier-depth stage assignment, tile selection, buffer and tensor-map
// assignment, constant-arena layout.
//
// Counterparts in the reference:
//   stage assignment  GlobalSynchronizationEliminationPass (BFS depth over Global edges,
//                     mononn_engine/optimization/global_synchronization_elimination_pass.cc:98-147)
//   horizontal merge  MergeIndependentPass (.../merge_independent_pass.cc:103-194): here all
//                     operators of one depth share a stage and split the CTAs between them
//   tile selection    ImplementationAssignmentPass (.../implementation_assignment_pass.cc:49-193)
//   buffers           BufferAssignmentPass + XLA's BufferAssignment offsets
//                     (mononn_engine/codegen/graph_codegen.cc:113-257); XLA is absent, so a
//                     liveness-based first-fit allocator decides the temp-arena offsets
#include <functional>
#include <algorithm>
#include <cstring>
#include <set>

#include "../../include/mononn.h"
#include "plan.h"

namespace mononn {

static inline uint64_t align_up(uint64_t v, uint64_t a) { return (v + a - 1) / a * a; }

// ------------------------------------------------------------ tile selection
static bool tile_legal(uint32_t N, uint32_t K, const GemmTileSpec& t, bool can_split_k) {
  // UMMA N is a multiple of 16 up to 256, and one k-block of the tile (n_tile rows of 128
  // bytes) has to fit a weight-ring slot
  if (t.n_tile < 16 || t.n_tile > 256 || (t.n_tile % 16) != 0) return false;
  if (t.n_tile * 128u > kBSlotBytes) return false;
  if (t.k_split < 1) return false;
  const uint32_t kb = (K + 63) / 64;
  if (kb % t.k_split != 0) return false;
  if (t.k_split > 1 && !can_split_k) return false;
  (void)N;
  return true;
}

// Relative cost of one work item. On the device the main loop costs a fixed time per 64-wide
// k-block (one MMA instruction takes about as long for a 16-column tile as for a 128-column
// one) and the epilogue grows with the tile width; the byte count below is a proxy with the
// same ordering (k-blocks weigh most, width a little, split-K adds its reduction). The tuner
// measures the candidates on the device; at batch 1 it confirms these defaults.
static double tile_cost(uint32_t M, uint32_t N, uint32_t K, const GemmTileSpec& t,
                        uint32_t cta_budget) {
  const uint32_t m_tiles = (M + 127) / 128, n_tiles = (N + t.n_tile - 1) / t.n_tile;
  const uint32_t items = m_tiles * n_tiles * t.k_split;
  const uint32_t waves = (items + cta_budget - 1) / cta_budget;
  const double kchunk = static_cast<double>(K) / t.k_split;
  double per_item = (128.0 + t.n_tile) * kchunk * 2.0;
  if (t.k_split > 1) per_item += 128.0 * t.n_tile * 4.0 * 2.0;  // f32 atomics
  per_item += 2000.0;                                            // fixed pipeline fill
  return per_item * waves;
}

std::vector<GemmTileSpec> gemm_tile_candidates(uint32_t M, uint32_t N, uint32_t K,
                                               bool can_split_k, uint32_t cta_budget) {
  std::vector<GemmTileSpec> out;
  const uint32_t kb = (K + 63) / 64;
  const uint32_t m_tiles = (M + 127) / 128;
  for (uint32_t n_tile : {16u, 32u, 48u, 64u, 96u, 128u, 192u, 256u}) {
    if (n_tile > std::max(16u, (N + 15) / 16 * 16)) continue;
    for (uint32_t ks = 1; ks <= kb; ++ks) {
      GemmTileSpec t;
      t.n_tile = n_tile;
      t.k_split = ks;
      if (!tile_legal(N, K, t, can_split_k)) continue;
      const uint32_t items = m_tiles * ((N + n_tile - 1) / n_tile) * ks;
      // more than two waves of tiny tiles is never a good trade at these sizes
      if (items > 2 * cta_budget && n_tile < 128) continue;
      out.push_back(t);
    }
  }
  return out;
}

GemmTileSpec default_gemm_tile(uint32_t M, uint32_t N, uint32_t K, bool can_split_k,
                               uint32_t cta_budget) {
  GemmTileSpec best;
  best.n_tile = 16;
  best.k_split = 1;
  double best_cost = 1e300;
  for (const GemmTileSpec& t : gemm_tile_candidates(M, N, K, can_split_k, cta_budget)) {
    const double c = tile_cost(M, N, K, t, cta_budget);
    if (c < best_cost) {
      best_cost = c;
      best = t;
    }
  }
  return best;
}

// ---------------------------------------------------------- liveness arena
namespace {
struct Interval {
  int tensor;
  int def_stage, last_stage;
  uint64_t bytes;
  uint64_t offset;
};

// First-fit by address among intervals whose live ranges overlap. A buffer may be
// reused by a tensor defined in a later stage than the previous owner's last use:
// the grid barrier between the two stages orders the last read before the first write.
uint64_t assign_offsets(std::vector<Interval>& iv, uint64_t base, uint64_t align) {
  std::sort(iv.begin(), iv.end(), [](const Interval& a, const Interval& b) {
    return a.def_stage != b.def_stage ? a.def_stage < b.def_stage : a.bytes > b.bytes;
  });
  uint64_t top = base;
  std::vector<Interval*> placed;
  for (Interval& x : iv) {
    std::vector<std::pair<uint64_t, uint64_t>> busy;
    for (Interval* y : placed)
      if (!(y->last_stage < x.def_stage || x.last_stage < y->def_stage))
        busy.push_back({y->offset, y->offset + y->bytes});
    std::sort(busy.begin(), busy.end());
    uint64_t off = base;
    for (auto& b : busy) {
      if (off + x.bytes <= b.first) break;
      off = std::max(off, align_up(b.second, align));
    }
    x.offset = off;
    top = std::max(top, off + x.bytes);
    placed.push_back(&x);
  }
  return align_up(top, align);
}
}  // namespace

// Checks every invariant the kernel relies on without checking it itself. A plan that fails
// here would read or write outside its shared-memory rings, TMEM columns or buffers.
int validate_plan(const Plan& P, std::string* err) {
  auto bad = [&](const std::string& m) {
    if (err) *err = "plan validation: " + m;
    return MONONN_ERR_INVALID_ARGUMENT;
  };
  if (P.block != kThreads) return bad("block size");
  if ((P.cluster != 1 && P.cluster != 2 && P.cluster != 4) || P.grid % P.cluster != 0) return bad("cluster shape");
  if (P.smem_bytes != kSmemBytes) return bad("shared memory size");
  for (size_t s = 0; s < P.stages.size(); ++s) {
    const StageDesc& sd = P.stages[s];
    if (sd.op_begin + sd.op_count > P.ops.size() || sd.op_count == 0 || sd.op_count > kMaxStageOps)
      return bad("stage op range");
    {
      uint32_t run = 0;
      for (uint32_t k = 0; k < kMaxStageOps; ++k) {
        if (k < sd.op_count) run += P.ops[sd.op_begin + k].d.n_items;
        if (sd.item_end[k] != ((k < sd.op_count) ? run : 0xffffffffu)) return bad("stage item prefix sums");
      }
    }
    uint32_t items = 0;
    for (uint32_t i = 0; i < sd.op_count; ++i) items += P.ops[sd.op_begin + i].d.n_items;
    if (items != sd.n_items) return bad("stage item count");
  }
  for (const PlanOp& op : P.ops) {
    const OpDesc& d = op.d;
    const std::string n = op.name + ": ";
    switch (d.kind) {
      case OP_GEMM: {
        if (d.n_tile < 16 || d.n_tile > 256 || d.n_tile % 16) return bad(n + "n_tile");
        if (d.n_tile > kAccCols) return bad(n + "n_tile exceeds an accumulator buffer");
        if (d.kb_per_bslot == 0 || d.n_tile * d.kb_per_bslot * 128u > kBSlotBytes)
          return bad(n + "weight tile exceeds a ring slot");
        if (d.n_tile * d.kb_per_bslot > 256) return bad(n + "TMA box taller than 256 rows");
        if (d.k_split == 0 || d.kb_per_split == 0 || d.k_split * d.kb_per_split * 64u != d.K)
          return bad(n + "K split does not cover K");
        if (d.n_tiles * d.n_tile < d.N || d.m_tiles * 128u < d.M) return bad(n + "tiles do not cover the output");
        if (d.n_items != d.m_tiles * d.n_tiles * d.k_split) return bad(n + "item count");
        if (d.N % 16) return bad(n + "N must be a multiple of 16");
        if (d.tmap_a >= P.tmaps.size() || d.tmap_b >= P.tmaps.size()) return bad(n + "tensor map index");
        if (P.tmaps[d.tmap_b].box1 != d.n_tile * d.kb_per_bslot || P.tmaps[d.tmap_b].box0 != 64)
          return bad(n + "weight tensor-map box");
        if (P.tmaps[d.tmap_a].box0 != 64 || P.tmaps[d.tmap_a].box1 != 128) return bad(n + "activation box");
        if (d.k_split > 1 && (d.out_mode != OUT_F32_RED || d.act != ACT_NONE))
          return bad(n + "K split needs an accumulating output without activation");
        if (op.p[0].space == SPACE_NONE) return bad(n + "no output buffer");
        if ((d.flags & F_BIAS) && op.p[1].space == SPACE_NONE) return bad(n + "no bias buffer");
        if ((d.flags & F_RESID) && op.p[2].space == SPACE_NONE) return bad(n + "no residual buffer");
        if (d.out_mode == OUT_F16_T && (d.rows_per_batch == 0 || d.ldt == 0)) return bad(n + "transposed output geometry");
        break;
      }
      case OP_ATTENTION:
        if (d.head_dim != 64 || d.seq == 0 || d.seq > 384) return bad(n + "attention geometry");
        if (d.tmap_a >= P.tmaps.size() || d.tmap_b >= P.tmaps.size() || d.tmap_vt >= P.tmaps.size())
          return bad(n + "tensor map index");
        if (P.tmaps[d.tmap_vt].box0 != 64 || P.tmaps[d.tmap_vt].box1 != 64) return bad(n + "V^T box");
        if (d.flags & F_FUSED_QKV) {
          if (d.seq > 128 || d.K == 0 || d.K % 64 || d.kb_per_split != d.K / 64) return bad(n + "fused projection geometry");
          if (d.vocab >= P.tmaps.size()) return bad(n + "tensor map index");
          for (uint32_t tmi : {d.tmap_b, d.vocab})
            if (P.tmaps[tmi].box0 != 64 || P.tmaps[tmi].box1 != 64) return bad(n + "projection weight box");
          if (P.tmaps[d.tmap_a].box0 != 64 || P.tmaps[d.tmap_a].box1 != 128) return bad(n + "activation box");
        }
        if (d.n_items != d.batches * d.heads * ((d.seq + 127) / 128)) return bad(n + "item count");
        if ((d.flags & F_POS_BIAS) && (op.q[0].space == SPACE_NONE || d.seq % 32 != 0)) return bad(n + "position bias");
        if (op.p[0].space == SPACE_NONE) return bad(n + "no output buffer");
        break;
      case OP_LAYERNORM:
      case OP_EMBED:
      case OP_ASSEMBLE:
        if (d.cols == 0 || d.cols % 4 || d.cols > 2048) return bad(n + "row length");
        if (d.flags & F_ROW_SPLIT) {
          if (d.kind != OP_LAYERNORM || d.cols % 16 || d.cols > 1024 || (d.flags & (F_L2NORM | F_NO_NORM)))
            return bad(n + "row split geometry");
          if (d.n_items != (d.rows + kSplitRowsPerItem - 1) / kSplitRowsPerItem) return bad(n + "item count");
        } else if (d.n_items != (d.rows + kRowsPerItem - 1) / kRowsPerItem) return bad(n + "item count");
        if (op.p[0].space == SPACE_NONE && op.q[2].space == SPACE_NONE) return bad(n + "no output buffer");
        if (op.p[6].space == SPACE_NONE && d.kind != OP_LAYERNORM) return bad(n + "no scale pointer");
        if (d.kind == OP_ASSEMBLE && (d.seq == 0 || d.k_col >= d.seq)) return bad(n + "token geometry");
        break;
      case OP_ROWSEL:
        if (d.cols == 0 || d.cols % 4 || d.lds % 4 || d.ldo % 4 || d.seq == 0) return bad(n + "row geometry");
        if (d.n_items != (d.rows + kRowsPerItem - 1) / kRowsPerItem) return bad(n + "item count");
        if (op.p[0].space == SPACE_NONE || op.p[1].space == SPACE_NONE || op.p[2].space == SPACE_NONE)
          return bad(n + "buffers");
        break;
      case OP_PAIRDOT:
        if (d.K == 0 || d.K % 8 || d.lds % 8 || d.ldr % 8) return bad(n + "K and row pitches must be multiples of 8");
        if (d.n_items != (d.M + kRowsPerItem - 1) / kRowsPerItem) return bad(n + "item count");
        if (op.p[0].space == SPACE_NONE || op.p[1].space == SPACE_NONE || op.p[2].space == SPACE_NONE)
          return bad(n + "buffers");
        break;
      case OP_ARGMAX:
        if (d.cols == 0 || d.cols % 8 || d.lds % 8) return bad(n + "row length must be a multiple of 8");
        if (d.n_items != d.rows) return bad(n + "item count");
        if (op.p[0].space == SPACE_NONE || op.p[1].space == SPACE_NONE) return bad(n + "buffers");
        break;
      case OP_PATCHIFY:
        if (d.K != d.heads * d.head_dim * d.q_col || d.cols < d.K || d.vocab == 0 || d.k_col == 0 ||
            d.vocab % d.k_col || d.M == 0 || d.N == 0 || d.rows_per_batch >= d.head_dim || d.ldt >= d.q_col)
          return bad(n + "window geometry");
        // the last window may hang over the bottom / right edge (padding), never start beyond it
        if ((d.vocab / d.k_col - 1) * d.M >= d.seq + d.rows_per_batch || (d.k_col - 1) * d.N >= d.batches + d.ldt)
          return bad(n + "windows start outside the image");
        if (d.n_items != (d.rows + kRowsPerItem - 1) / kRowsPerItem) return bad(n + "item count");
        if (op.p[0].space == SPACE_NONE || op.p[1].space == SPACE_NONE) return bad(n + "buffers");
        break;
      default:
        return bad(n + "unknown operator kind");
    }
  }
  for (const StageDesc& sd : P.stages) {
    // An operator that waits on an arrival counter needs the operators that add to that counter
    // earlier in the same stage's item order (so that no CTA meets a waiting item before an item it
    // waits for), their item counts adding up to its target.
    auto signalled_before = [&](uint32_t a, int counter) {
      uint32_t target = 0;
      for (uint32_t b = sd.op_begin; b < a; ++b) {
        const PlanOp& s = P.ops[b];
        if (!s.waits && s.flag_index == counter) target += s.d.n_items;
      }
      return target;
    };
    for (uint32_t a = sd.op_begin; a < sd.op_begin + sd.op_count; ++a) {
      const PlanOp& op = P.ops[a];
      if (op.wflag_index >= 0) {
        // a GEMM behind the operator of the same stage that writes its A operand
        const uint32_t target = signalled_before(a, op.wflag_index);
        if (op.d.kind != OP_GEMM || op.wflag.space != SPACE_SCRATCH || target == 0 || target != op.d.wait_target)
          return bad(op.name + ": wait target does not match the operator it waits for");
      } else if (op.d.wait_target != 0) {
        return bad(op.name + ": wait target without a counter");
      }
      if (op.flag_index < 0) {
        if (op.d.flag_target != 0) return bad(op.name + ": wait target without a counter");
        continue;
      }
      if (op.flag.space != SPACE_SCRATCH) return bad(op.name + ": arrival counter outside the scratch");
      if (!op.waits) {
        if (op.d.kind != OP_GEMM && op.d.kind != OP_ATTENTION) return bad(op.name + ": operator cannot signal");
        continue;
      }
      const uint32_t target = signalled_before(a, op.flag_index);
      if (target == 0 || target != op.d.flag_target) return bad(op.name + ": wait target does not match its GEMMs");
    }
  }
  for (const TmapSpec& t : P.tmaps) {
    if (t.box0 * 2u > 128u || (t.box0 * 2u) % 16u) return bad("tensor-map inner box must be 16..128 bytes");
    if (t.box1 == 0 || t.box1 > 256) return bad("tensor-map box rows");
    if (t.stride1_bytes % 16) return bad("tensor-map stride");
  }
  return MONONN_OK;
}

static bool listed(const std::vector<std::string>& l, const std::string& n) {
  return std::find(l.begin(), l.end(), n) != l.end();
}

int schedule(const FGraph& g, const TuningSpec& spec_in, uint32_t sm_count, Plan* plan,
             std::string* err) {
  Plan& P = *plan;
  P = Plan();
  P.module_name = g.module_name;
  P.spec = spec_in;
  P.grid = spec_in.grid ? spec_in.grid : sm_count;
  P.block = kThreads;
  P.smem_bytes = kSmemBytes;
  P.cluster = spec_in.cluster ? spec_in.cluster : 1u;
  if ((P.cluster != 1 && P.cluster != 2 && P.cluster != 4) || P.grid % P.cluster != 0) {
    if (err) *err = "cluster of " + std::to_string(P.cluster) + " CTAs: must be 1, 2 or 4 and divide the grid";
    return MONONN_ERR_INVALID_ARGUMENT;
  }
  P.spec.cluster = P.cluster;
  P.spec.grid = P.grid;
  P.spec.block = P.block;
  P.spec.smem_bytes = P.smem_bytes;
  P.args = g.args;
  const int n_t = static_cast<int>(g.tensors.size());

  // ---- inputs / outputs of every op
  auto inputs_of = [](const FOp& o) {
    std::vector<int> v;
    for (int t : {o.a, o.w, o.bias, o.resid, o.q, o.k, o.vt, o.mask, o.src, o.gamma, o.beta, o.ids,
                  o.type_ids, o.mask_in, o.word, o.pos, o.type, o.bias2, o.wk, o.wv, o.bias_k, o.bias_v, o.pos_bias})
      if (t >= 0) v.push_back(t);
    return v;
  };
  auto outputs_of = [](const FOp& o) {
    std::vector<int> v;
    for (int t : {o.out, o.mask_out, o.out2})
      if (t >= 0) v.push_back(t);
    return v;
  };

  std::vector<FOp> ops;
  for (const FOp& o : g.ops) {
    if (!spec_in.allow_list.empty() && !listed(spec_in.allow_list, o.name)) continue;
    if (listed(spec_in.reject_list, o.name)) continue;
    ops.push_back(o);
  }
  if (ops.empty()) {
    if (err) *err = "no operators left after allow/reject lists";
    return MONONN_ERR_INVALID_ARGUMENT;
  }

  // ---- Q/K/V projections fused into the attention stage. With few (batch, head) pairs the
  // attention stage leaves most CTAs idle and the projection stage before it costs a full
  // barrier round trip; and an MMA instruction takes as long for a 16-column tile as for a
  // 192-column one. So each (batch, head) item computes its own [Q_h | K_h | V_h] =
  // x_b [W_q,h | W_k,h | W_v,h] + bias (one 192-column accumulator over K/64 k-blocks: as long
  // as the projection stage's main loop took with 148 CTAs), turns it into the f16 operand
  // tiles in shared memory and goes on with QK^T, softmax and PV. One stage and three
  // round trips through global memory disappear.
  {
    const uint32_t ctas = spec_in.grid ? spec_in.grid : sm_count;
    for (size_t ai = 0; ai < ops.size(); ++ai) {
      FOp& att = ops[ai];
      if (att.kind != OP_ATTENTION || att.a >= 0 || spec_in.qkv_fusion == 1) continue;
      if (att.seq > 128 || att.head_dim != 64) continue;
      if (spec_in.qkv_fusion == 0 && att.batches * att.heads > ctas) continue;
      int gi[3] = {-1, -1, -1};
      const int want[3] = {att.q, att.k, att.vt};
      bool ok = true;
      for (int j = 0; j < 3 && ok; ++j) {
        int readers = 0;
        for (size_t i = 0; i < ops.size(); ++i) {
          if (ops[i].out == want[j] && ops[i].kind == OP_GEMM) gi[j] = static_cast<int>(i);
          for (int in : inputs_of(ops[i]))
            if (in == want[j]) ++readers;
        }
        ok = gi[j] >= 0 && readers == 1 && g.tensors[want[j]].kind != TKind::Arg;
      }
      if (!ok) continue;
      const FOp &gq = ops[gi[0]], &gk = ops[gi[1]], &gv = ops[gi[2]];
      const uint32_t width = att.heads * 64u;
      for (const FOp* gp : {&gq, &gk, &gv})
        ok = ok && gp->a == gq.a && gp->K == gq.K && gp->N == width && gp->act == ACT_NONE && gp->resid < 0 &&
             gp->alpha == 1.f && gp->K % 64 == 0 && gp->M == att.batches * att.seq &&
             g.tensors[gp->w].const_name != "" ;
      if (!ok || att.q_col != 0 || att.k_col != 0) continue;
      // wide models: a head's three weight slabs (3 * K * 128 bytes) no longer stream through the
      // three-slot ring as fast as the MMAs consume them (measured: OPT-1.3B, K = 2048, is 2 %
      // slower fused), so the automatic choice stops at K = 1024
      if (spec_in.qkv_fusion == 0 && gq.K > 1024) continue;
      att.flags |= F_FUSED_QKV;
      att.a = gq.a;
      att.K = gq.K;
      att.w = gq.w;
      att.wk = gk.w;
      att.wv = gv.w;
      att.bias = gq.bias;
      att.bias_k = gk.bias;
      att.bias_v = gv.bias;
      att.q = att.k = att.vt = -1;
      std::vector<FOp> kept;
      for (size_t i = 0; i < ops.size(); ++i)
        if (static_cast<int>(i) != gi[0] && static_cast<int>(i) != gi[1] && static_cast<int>(i) != gi[2])
          kept.push_back(ops[i]);
      ops.swap(kept);
      ai = 0;  // indices moved: rescan (fused ops are skipped by the att.a >= 0 test)
    }
  }

  // ---- residual hoisting: a split-K GEMM that accumulates into an f32 buffer and adds a
  // residual produced by a LayerNorm / embedding row op gets that residual (and its bias)
  // pre-loaded into the accumulator by the producer, so its own epilogue is a bare
  // reduction with no global loads on the critical path.
  for (FOp& gop : ops) {
    if (gop.kind != OP_GEMM || gop.resid < 0 || gop.out < 0) continue;
    if (g.tensors[gop.out].kind != TKind::AccF32) continue;
    if (g.tensors[gop.resid].kind != TKind::ActF16 && g.tensors[gop.resid].kind != TKind::Arg) continue;
    for (FOp& pop : ops) {
      if ((pop.kind != OP_LAYERNORM && pop.kind != OP_EMBED) || pop.out != gop.resid) continue;
      if (pop.out2 >= 0 || pop.cols != gop.N) break;
      pop.out2 = gop.out;
      pop.bias2 = gop.bias;
      gop.resid = -1;
      gop.bias = -1;
      // the accumulator is now fully overwritten before use: its reader need not clear it
      for (FOp& rop : ops)
        if (rop.kind == OP_LAYERNORM && rop.src == gop.out) rop.flags &= ~F_ZERO_SRC;
      break;
    }
  }

  // ---- stage = dependency depth
  // A LayerNorm over an f32 accumulator whose last writers are split-K GEMMs normally sits one
  // barrier after them. When nothing else holds it back it joins their stage instead: every GEMM
  // item adds 1 to an arrival counter after its reductions and the row items, dealt to the CTAs
  // after the GEMM items, wait for the full count (a wait for CTAs that never wait themselves,
  // all co-resident: it cannot deadlock). One grid barrier per LayerNorm disappears. The
  // reference splits the same pair into a GEMM node and a reduce cluster with a barrier between
  // (mononn_engine/optimization/global_synchronization_elimination_pass.cc:98-147).
  std::vector<int> producer(n_t, -1), last_reader(n_t, -1);
  std::vector<std::vector<int>> writers(n_t);
  std::vector<int> flag_of(ops.size(), -1);   // arrival counter an op signals (GEMM) or waits on (row op)
  std::vector<char> waits(ops.size(), 0);
  // a GEMM that shares the stage of the attention whose output it reads waits on that attention's
  // counter (its own flag_of stays free for the row op that may follow it in the same stage)
  std::vector<int> wflag_of(ops.size(), -1);
  // ... or, with chain fusion, of the GEMM whose output it reads
  std::vector<int> wprod(ops.size(), -1);     // the operator a GEMM with wflag_of waits for
  std::vector<uint32_t> ops_at;               // operators per depth so far (a stage holds kMaxStageOps)
  // does the chain of waits that starts at operator `from` pass through operator `target`?
  std::function<bool(int, int)> chain_reaches = [&](int from, int target) -> bool {
    if (from < 0) return false;
    if (from == target) return true;
    if (wflag_of[from] >= 0) return chain_reaches(wprod[from], target);
    if (waits[from]) {
      for (size_t w = 0; w < ops.size(); ++w)
        if (!waits[w] && flag_of[w] == flag_of[from] && ops[w].stage == ops[from].stage &&
            chain_reaches(static_cast<int>(w), target))
          return true;
    }
    return false;
  };
  int n_flags = 0;
  int n_stages = 0;
  // Left to the scheduler (0), a LayerNorm joins its GEMMs' stage when its rows are one wave of
  // work items at most: with many rows the row items of the early row tiles would sit waiting
  // for the whole GEMM (BERT-large b16 and ViT b64 measured 2-4 % faster apart), and the
  // L2 hints are given only when a weight tile is read by few row tiles (evict-first on weights
  // that 48 row tiles re-read cost BERT-large b16 5 %).
  uint32_t max_ln_rows = 0, max_m_tiles = 1;
  for (const FOp& o : ops) {
    if (o.kind == OP_LAYERNORM) max_ln_rows = std::max(max_ln_rows, o.rows);
    if (o.kind == OP_GEMM) max_m_tiles = std::max(max_m_tiles, (o.M + 127u) / 128u);
  }
  if (P.spec.row_fusion == 0) P.spec.row_fusion = (max_ln_rows <= kRowsPerItem * P.grid) ? 2u : 1u;
  if (P.spec.l2_hints == 0) P.spec.l2_hints = (max_m_tiles <= 4u) ? 2u : 1u;
  // An attention stage that leaves most CTAs idle takes the GEMM that consumes its output (the
  // out-projection) into the same stage: the GEMM's items wait for the attention's arrival counter
  // instead of a grid barrier, and their weights are already on chip when the counter fills.
  uint32_t max_attn_items = 0;
  for (const FOp& o : ops)
    if (o.kind == OP_ATTENTION)
      max_attn_items = std::max(max_attn_items, o.batches * o.heads * ((o.seq + 127u) / 128u));
  // Left to the scheduler this is done only behind an attention that computes its own projections
  // (a long stage on few CTAs, the others idle: BERT-base b1 -5 us); behind a short attention
  // stage it measured slower (BERT-large b1 s384 +46 us, OPT-1.3B b1 +50 us, CLIP +94 us).
  if (P.spec.out_fusion == 0)
    P.spec.out_fusion = (P.spec.row_fusion == 2 && max_attn_items != 0 && max_attn_items * 2u <= P.grid) ? 3u : 1u;
  // Chain fusion goes on from there: a GEMM whose A operand is written by another GEMM joins that
  // GEMM's stage too and waits for its counter (FFN-up, FFN-down and the LayerNorm behind it in
  // one stage). With LayerNorms signalling as well a whole layer was one stage of operators chained
  // by counters; measured on BERT-base b1 that chain cost what the grid barriers it replaced cost
  // (512 us either way: release, observation and first tile make the hop, not the barrier), and
  // the signalling code cost the other configurations half a per cent, so it was taken out again;
  // left to the scheduler it stays off; the tuner tries it.
  if (P.spec.chain_fusion == 0) P.spec.chain_fusion = 1u;
  for (size_t i = 0; i < ops.size(); ++i) {
    int fuse_src = -1, fuse_stage = -1;
    bool gemm_after_producer = false;
    if (ops[i].kind == OP_GEMM && ops[i].a >= 0 && producer[ops[i].a] >= 0 && writers[ops[i].a].size() == 1) {
      const int pr = producer[ops[i].a];
      const OpKind pk = ops[pr].kind;
      const bool allowed = (pk == OP_ATTENTION && (P.spec.out_fusion == 2 ||
                                                   (P.spec.out_fusion == 3 && (ops[pr].flags & F_FUSED_QKV)))) ||
                           (pk == OP_GEMM && P.spec.chain_fusion == 2 &&
                            g.tensors[ops[i].a].kind == TKind::ActF16);
      if (allowed && ops_at.size() > static_cast<size_t>(ops[pr].stage) &&
          ops_at[ops[pr].stage] < kMaxStageOps) {
        fuse_src = ops[i].a;
        fuse_stage = ops[pr].stage;
        gemm_after_producer = true;
      }
    }
    if (ops[i].kind == OP_LAYERNORM && P.spec.row_fusion != 1 && ops[i].src >= 0 &&
        g.tensors[ops[i].src].kind == TKind::AccF32 && !writers[ops[i].src].empty()) {
      const int T = ops[i].src;
      int d = -1;
      for (int w : writers[T]) d = std::max(d, ops[w].stage);
      // the writers at that depth must be GEMMs free to signal, or operators those GEMMs already
      // wait for through their chain of counters (a LayerNorm that pre-loaded the accumulator)
      bool ok = true;
      for (int w : writers[T]) {
        if (ops[w].stage != d) continue;
        if (ops[w].kind == OP_GEMM && flag_of[w] < 0) continue;
        bool ordered = false;
        for (int v : writers[T])
          if (v != w && ops[v].stage == d && ops[v].kind == OP_GEMM && flag_of[v] < 0 && chain_reaches(v, w))
            ordered = true;
        if (!ordered) ok = false;
      }
      if (ok && d >= 0 && ops_at[d] < kMaxStageOps) {
        fuse_src = T;
        fuse_stage = d;
      }
    }
    int depth = 0;
    for (int t : inputs_of(ops[i]))
      if (producer[t] >= 0 && t != fuse_src) depth = std::max(depth, ops[producer[t]].stage + 1);
    // an op that adds into a live tensor (the f32 residual stream of pre-LN models) also
    // runs after every earlier reader of the old value
    for (int t : outputs_of(ops[i]))
      if (producer[t] >= 0) depth = std::max(depth, last_reader[t] + 1);
    // an op that accumulates into a tensor someone pre-loaded runs after that producer (which it
    // does inside one stage too when the chain of counters it waits on passes through that producer)
    for (int t : outputs_of(ops[i]))
      if (producer[t] >= 0 && !(gemm_after_producer && ops[producer[t]].stage == fuse_stage &&
                                chain_reaches(producer[fuse_src], producer[t])))
        depth = std::max(depth, ops[producer[t]].stage + 1);
    if (fuse_src >= 0) {
      if (depth <= fuse_stage && gemm_after_producer) {
        const int pr = producer[fuse_src];
        depth = fuse_stage;
        // several GEMMs may read one operator's output: they share its counter
        if (flag_of[pr] < 0) flag_of[pr] = n_flags++;
        wflag_of[i] = flag_of[pr];
        wprod[i] = pr;
      } else if (gemm_after_producer) {
        depth = std::max(depth, fuse_stage + 1);  // stays a stage behind its producer
      } else if (depth <= fuse_stage) {
        depth = fuse_stage;
        flag_of[i] = n_flags;
        waits[i] = 1;
        for (int w : writers[fuse_src])
          if (ops[w].stage == fuse_stage && ops[w].kind == OP_GEMM && flag_of[w] < 0) flag_of[w] = n_flags;
        ++n_flags;
      } else {
        depth = std::max(depth, fuse_stage + 1);
      }
    }
    ops[i].stage = depth;
    n_stages = std::max(n_stages, depth + 1);
    if (ops_at.size() <= static_cast<size_t>(depth)) ops_at.resize(depth + 1, 0);
    ++ops_at[depth];
    for (int t : inputs_of(ops[i])) last_reader[t] = std::max(last_reader[t], depth);
    for (int t : outputs_of(ops[i])) {
      producer[t] = static_cast<int>(i);
      writers[t].push_back(static_cast<int>(i));
    }
  }

  // ---- a stage holds at most kMaxStageOps operators (its descriptor has that many item
  // ranges). Many independent operators can share a depth (the cross-attention K / V projections
  // of every decoder layer depend on the encoder output alone); those whose results are not
  // needed in the next stage move one stage later, which no dependent operator can notice.
  {
    auto depends = [&](size_t j, size_t i) {  // does op j (later in program order) depend on op i?
      for (int t : inputs_of(ops[j]))
        for (int o : outputs_of(ops[i]))
          if (t == o) return true;
      for (int t : outputs_of(ops[j])) {
        for (int o : outputs_of(ops[i]))
          if (t == o) return true;
        for (int r : inputs_of(ops[i]))
          if (t == r && g.tensors[t].kind != TKind::Const) return true;
      }
      return false;
    };
    for (int st = 0; st < n_stages; ++st) {
      std::vector<size_t> here;
      for (size_t i = 0; i < ops.size(); ++i)
        if (ops[i].stage == st) here.push_back(i);
      for (size_t k = here.size(); here.size() > kMaxStageOps && k-- > 0;) {
        const size_t i = here[k];
        if (flag_of[i] >= 0 || wflag_of[i] >= 0) continue;  // tied to its partner's stage
        bool free_to_move = true;
        for (size_t j = i + 1; j < ops.size() && free_to_move; ++j)
          if (ops[j].stage <= st + 1 && depends(j, i)) free_to_move = false;
        if (!free_to_move) continue;
        ops[i].stage = st + 1;
        n_stages = std::max(n_stages, st + 2);
        here.erase(here.begin() + static_cast<long>(k));
      }
    }
  }

  // ---- liveness
  std::vector<int> def_stage(n_t, -1), last_stage(n_t, -1);
  std::vector<char> first_write_accumulates(n_t, 0);
  for (const FOp& o : ops) {
    for (int t : outputs_of(o)) {
      if (def_stage[t] < 0) {
        def_stage[t] = o.stage;
        first_write_accumulates[t] = (o.kind == OP_GEMM);
      }
      last_stage[t] = std::max(last_stage[t], o.stage);
    }
    for (int t : inputs_of(o)) {
      if (def_stage[t] < 0) def_stage[t] = 0;  // produced outside (or cut away by allow-list)
      last_stage[t] = std::max(last_stage[t], o.stage);
    }
  }

  // ---- scratch layout: barrier counter, status, stamps, then f32 tensors
  uint64_t scratch = kScratchStampsOff + align_up(8ull * (n_stages + 2), 256);
  // arrival counters of the row ops that share a stage with their GEMMs (one per pair, 8 bytes apart)
  const uint64_t flags_off = scratch;
  scratch += align_up(8ull * n_flags, 256);
  P.flag_offset = flags_off;
  P.flag_bytes = n_flags ? align_up(8ull * n_flags, 256) : 0;

  // f32 tensors come in two kinds that must not inherit each other's memory. A GEMM
  // accumulator whose first write is a reduction needs zeros when its life starts and is
  // cleared again by its reader (F_ZERO_SRC), so such tensors can follow one another. A tensor
  // whose first write is a plain store (a residual stream, a pre-loaded accumulator, the mask
  // bias) is left dirty when it dies; only other tensors of that kind may reuse its memory.
  std::vector<Interval> temp_iv, scratch_iv, dirty_iv;
  for (int t = 0; t < n_t; ++t) {
    if (def_stage[t] < 0) continue;
    const FTensor& T = g.tensors[t];
    Interval iv{t, def_stage[t], last_stage[t], 0, 0};
    switch (T.kind) {
      case TKind::ActF16:
        iv.bytes = align_up(static_cast<uint64_t>(T.rows) * T.ld * 2, 256);
        temp_iv.push_back(iv);
        break;
      case TKind::ActF16T:
        iv.bytes = align_up(static_cast<uint64_t>(T.batches) * T.cols * T.ld * 2, 256);
        temp_iv.push_back(iv);
        break;
      case TKind::AccF32:
        iv.bytes = align_up(static_cast<uint64_t>(T.rows) * T.cols * 4, 256);
        (first_write_accumulates[t] ? scratch_iv : dirty_iv).push_back(iv);
        break;
      case TKind::VecF32:
        iv.bytes = align_up(static_cast<uint64_t>(T.rows) * 4, 256);
        // the mask bias is produced once and read by every layer
        dirty_iv.push_back(iv);
        break;
      default:
        break;
    }
  }
  P.temp_bytes = assign_offsets(temp_iv, 0, 256);
  if (P.temp_bytes == 0) P.temp_bytes = 256;
  P.scratch_bytes = assign_offsets(scratch_iv, scratch, 256);
  P.scratch_bytes = assign_offsets(dirty_iv, P.scratch_bytes, 256);

  std::vector<BufRef> where(n_t);
  const int temp_arg = static_cast<int>(P.args.size());
  {
    ArgDesc a;
    a.name = "temp_buffer";
    a.bytes = P.temp_bytes;
    a.kind = 2;
    a.param_number = 0;
    P.args.push_back(a);
  }
  for (const Interval& iv : temp_iv) where[iv.tensor] = BufRef{SPACE_ARG, temp_arg, iv.offset};
  for (const Interval& iv : scratch_iv) where[iv.tensor] = BufRef{SPACE_SCRATCH, 0, iv.offset};
  for (const Interval& iv : dirty_iv) where[iv.tensor] = BufRef{SPACE_SCRATCH, 0, iv.offset};
  for (int t = 0; t < n_t; ++t)
    if (g.tensors[t].kind == TKind::Arg) where[t] = BufRef{SPACE_ARG, g.tensors[t].arg_index, 0};

  for (int t = 0; t < n_t; ++t) {
    const FTensor& T = g.tensors[t];
    if (def_stage[t] < 0 || T.kind == TKind::Const) continue;
    TensorPlacement tp;
    tp.name = T.name;
    tp.kind = T.kind;
    tp.at = where[t];
    tp.rows = T.rows;
    tp.cols = T.cols;
    tp.ld = T.ld;
    tp.batches = T.batches;
    tp.seq = T.seq;
    tp.def_stage = def_stage[t];
    tp.last_stage = last_stage[t];
    P.tensors.push_back(tp);
  }

  // ---- constants: RAW bindings are shared, PACK_B bindings are per (constant, n_tile)
  uint64_t const_top = 0;
  std::map<std::string, size_t> raw_binding;
  std::map<std::pair<std::string, uint32_t>, size_t> packed_binding;
  auto raw_const = [&](int t) -> BufRef {
    const FTensor& T = g.tensors[t];
    auto it = raw_binding.find(T.const_name);
    if (it == raw_binding.end()) {
      ConstBinding b;
      b.const_name = T.const_name;
      b.kind = ConstBinding::RAW;
      b.bytes = static_cast<uint64_t>(T.rows) * T.cols * T.elem_bytes;
      b.src_bytes = b.bytes;
      b.offset = const_top;
      const_top = align_up(const_top + b.bytes, 256);
      P.consts.push_back(b);
      it = raw_binding.emplace(T.const_name, P.consts.size() - 1).first;
    }
    return BufRef{SPACE_CONST, 0, P.consts[it->second].offset};
  };

  // Small constants first, contiguously: biases and LayerNorm scale/shift of all layers share
  // a few pages, which the kernel prefetches to L2 when it starts.
  for (const FOp& o : ops)
    for (int t : {o.bias, o.gamma, o.beta, o.bias2, o.bias_k, o.bias_v})
      if (t >= 0 && static_cast<uint64_t>(g.tensors[t].rows) * g.tensors[t].cols *
                            g.tensors[t].elem_bytes <= 65536)
        raw_const(t);
  P.hot_const_bytes = const_top;

  // ---- tensor maps
  std::map<int, uint32_t> act_tmap;  // tensor -> tmap index (box 64 x 128)
  auto tmap_for_act = [&](int t) -> uint32_t {
    auto it = act_tmap.find(t);
    if (it != act_tmap.end()) return it->second;
    const FTensor& T = g.tensors[t];
    TmapSpec s;
    s.base = where[t];
    s.dim0 = T.cols;
    s.dim1 = T.rows;
    s.stride1_bytes = static_cast<uint64_t>(T.ld) * 2;
    s.box0 = 64;
    s.box1 = 128;
    P.tmaps.push_back(s);
    return act_tmap[t] = static_cast<uint32_t>(P.tmaps.size() - 1);
  };

  // Packed copy of a weight ([n_tiles][K/64][n_tile][64], one binding per (constant, n_tile)) and
  // a tensor map whose box is `kbps` k-blocks of one tile; returns the tensor-map index.
  auto packed_weight = [&](int w, uint32_t K, uint32_t N, uint32_t n_tile, uint32_t kbps) -> uint32_t {
    const FTensor& W = g.tensors[w];
    const uint32_t n_tiles = (N + n_tile - 1) / n_tile, kb = K / 64;
    auto key = std::make_pair(W.const_name, n_tile);
    auto pit = packed_binding.find(key);
    if (pit == packed_binding.end()) {
      ConstBinding b;
      b.const_name = W.const_name;
      b.kind = ConstBinding::PACK_B;
      b.K = K;
      b.N = N;
      b.n_tile = n_tile;
      b.transposed = W.const_transposed;
      b.K_src = (W.rows && W.rows < K) ? W.rows : K;
      b.src_bytes = static_cast<uint64_t>(b.K_src) * N * 2;
      b.bytes = static_cast<uint64_t>(n_tiles) * n_tile * K * 2;
      b.offset = const_top;
      const_top = align_up(const_top + b.bytes, 1024);
      P.consts.push_back(b);
      pit = packed_binding.emplace(key, P.consts.size() - 1).first;
    }
    const ConstBinding& b = P.consts[pit->second];
    TmapSpec tm;
    tm.base = BufRef{SPACE_CONST, 0, b.offset};
    tm.dim0 = 64;
    tm.dim1 = static_cast<uint64_t>(n_tiles) * kb * n_tile;
    tm.stride1_bytes = 128;
    tm.box0 = 64;
    tm.box1 = n_tile * kbps;
    P.tmaps.push_back(tm);
    return static_cast<uint32_t>(P.tmaps.size() - 1);
  };

  // Operators that wait for others of their own stage come after them, so that a CTA meets the
  // items that never wait before any item that does, and every waiting item only items it does
  // not wait for: ordered by the length of the chain of counters behind them.
  std::vector<int> level(ops.size(), 0);
  for (size_t i = 0; i < ops.size(); ++i) {
    if (wflag_of[i] >= 0) level[i] = level[wprod[i]] + 1;
    if (waits[i])
      for (size_t w = 0; w < i; ++w)
        if (!waits[w] && flag_of[w] == flag_of[i] && ops[w].stage == ops[i].stage)
          level[i] = std::max(level[i], level[w] + 1);
  }
  // ---- emit ops stage by stage
  std::vector<std::vector<size_t>> by_stage(n_stages);
  for (int lv = 0; lv <= static_cast<int>(kMaxStageOps); ++lv)
    for (size_t i = 0; i < ops.size(); ++i)
      if (level[i] == lv) by_stage[ops[i].stage].push_back(i);

  // ---- the GEMMs that run side by side (same stage, same place in the chains of counters) share
  // the CTAs that the stage's attention items leave free
  std::vector<std::vector<uint32_t>> gemms_side_by_side(n_stages, std::vector<uint32_t>(kMaxStageOps + 1, 0));
  std::vector<uint32_t> attn_items_in_stage(n_stages, 0);
  for (size_t i = 0; i < ops.size(); ++i) {
    const FOp& o = ops[i];
    if (o.kind == OP_ATTENTION) attn_items_in_stage[o.stage] += o.batches * o.heads * ((o.seq + 127u) / 128u);
    if (o.kind == OP_GEMM) gemms_side_by_side[o.stage][std::min<int>(level[i], kMaxStageOps)]++;
  }

  for (int s = 0; s < n_stages; ++s) {
    StageDesc sd{};
    sd.op_begin = static_cast<uint32_t>(P.ops.size());
    std::string sname;
    for (size_t oi : by_stage[s]) {
      const FOp& o = ops[oi];
      PlanOp po;
      po.name = o.name;
      OpDesc& d = po.d;
      std::memset(&d, 0, sizeof(d));
      d.kind = o.kind;
      d.flags = o.flags;
      d.act = o.act;
      d.alpha = o.alpha;
      d.eps = o.eps;
      switch (o.kind) {
        case OP_GEMM: {
          const FTensor& A = g.tensors[o.a];
          const FTensor& W = g.tensors[o.w];
          const FTensor& O = g.tensors[o.out];
          if (o.K % 64 != 0 || o.N % 16 != 0) {
            if (err) *err = "GEMM " + o.name + ": K must be a multiple of 64 and N of 16";
            return MONONN_ERR_UNSUPPORTED;
          }
          const bool can_split = (O.kind == TKind::AccF32) && o.act == ACT_NONE;
          // CTAs busy with a few attention items of the same stage are not available to its GEMMs
          // (attention items that fill the grid take whole waves and then leave all of it)
          const uint32_t reserved = attn_items_in_stage[s] * 2u <= P.grid ? attn_items_in_stage[s] : 0u;
          const uint32_t free_ctas = P.grid - reserved;
          const uint32_t budget =
              std::max(1u, free_ctas / std::max(1u, gemms_side_by_side[s][std::min<int>(level[oi], kMaxStageOps)]));
          GemmTileSpec ts;
          auto it = spec_in.gemm.find(o.name);
          if (it != spec_in.gemm.end()) ts = it->second;
          if (ts.n_tile == 0 || ts.k_split == 0 || !tile_legal(o.N, o.K, ts, can_split))
            ts = default_gemm_tile(o.M, o.N, o.K, can_split, budget);
          P.spec.gemm[o.name] = ts;
          d.M = o.M;
          d.N = o.N;
          d.K = o.K;
          d.n_tile = ts.n_tile;
          d.k_split = ts.k_split;
          d.m_tiles = (o.M + 127) / 128;
          d.n_tiles = (o.N + ts.n_tile - 1) / ts.n_tile;
          const uint32_t kb = o.K / 64;
          d.kb_per_split = kb / ts.k_split;
          d.kb_per_bslot = std::max(1u, std::min(d.kb_per_split, kBSlotBytes / (ts.n_tile * 128u)));
          d.n_items = d.m_tiles * d.n_tiles * d.k_split;
          d.tmap_a = tmap_for_act(o.a);
          (void)A;
          d.tmap_b = packed_weight(o.w, o.K, o.N, ts.n_tile, d.kb_per_bslot);
          po.p[0] = where[o.out];
          if (o.bias >= 0) {
            po.p[1] = raw_const(o.bias);
            d.flags |= F_BIAS;
          }
          if (o.resid >= 0) {
            po.p[2] = where[o.resid];
            d.flags |= F_RESID;
            d.ldr = g.tensors[o.resid].ld;
            if (g.tensors[o.resid].kind == TKind::AccF32) {
              d.flags |= F_RESID_F32;
              d.ldr = g.tensors[o.resid].cols;
            }
          }
          switch (O.kind) {
            case TKind::ActF16:
              d.out_mode = OUT_F16;
              d.ldo = O.ld;
              break;
            case TKind::ActF16T:
              d.out_mode = OUT_F16_T;
              d.rows_per_batch = O.seq;
              d.ldt = O.ld;
              break;
            case TKind::AccF32:
              d.out_mode = OUT_F32_RED;
              d.ldo = O.cols;
              break;
            case TKind::Arg:
              d.out_mode = O.elem_bytes == 4 ? OUT_F32 : OUT_F16;
              d.ldo = O.ld;
              break;
            default:
              if (err) *err = "GEMM " + o.name + ": unsupported output tensor kind";
              return MONONN_ERR_UNSUPPORTED;
          }
          P.algorithmic_flops += 2.0 * o.M * o.N * o.K;
          break;
        }
        case OP_ATTENTION: {
          if (o.head_dim != 64 || o.seq > 384) {
            if (err) *err = "attention " + o.name + ": head_dim must be 64 and seq <= 384";
            return MONONN_ERR_UNSUPPORTED;
          }
          d.heads = o.heads;
          d.seq = o.seq;
          d.batches = o.batches;
          d.head_dim = o.head_dim;
          d.q_col = o.q_col;
          d.k_col = o.k_col;
          if (o.flags & F_FUSED_QKV) {
            const uint32_t width = o.heads * 64u;
            d.K = o.K;
            d.kb_per_split = o.K / 64;
            d.tmap_a = tmap_for_act(o.a);
            d.tmap_b = packed_weight(o.w, o.K, width, 64, 1);
            d.tmap_vt = packed_weight(o.wk, o.K, width, 64, 1);
            d.vocab = packed_weight(o.wv, o.K, width, 64, 1);
            // bases of the three packed weights: CTAs without an item pre-fetch them into L2
            po.p[5] = P.tmaps[d.tmap_b].base;
            po.p[6] = P.tmaps[d.tmap_vt].base;
            po.p[7] = P.tmaps[d.vocab].base;
            if (o.bias >= 0) po.p[2] = raw_const(o.bias);
            if (o.bias_k >= 0) po.p[3] = raw_const(o.bias_k);
            if (o.bias_v >= 0) po.p[4] = raw_const(o.bias_v);
            P.algorithmic_flops += 2.0 * o.batches * o.seq * 3.0 * width * o.K;
          } else {
            d.tmap_a = tmap_for_act(o.q);
            d.tmap_b = tmap_for_act(o.k);
            const FTensor& VT = g.tensors[o.vt];
            TmapSpec tm;
            tm.base = where[o.vt];
            tm.dim0 = VT.seq;
            tm.dim1 = static_cast<uint64_t>(VT.batches) * VT.cols;
            tm.stride1_bytes = static_cast<uint64_t>(VT.ld) * 2;
            tm.box0 = 64;
            tm.box1 = 64;
            P.tmaps.push_back(tm);
            d.tmap_vt = static_cast<uint32_t>(P.tmaps.size() - 1);
          }
          d.n_items = o.batches * o.heads * ((o.seq + 127) / 128);
          d.ldo = g.tensors[o.out].ld;
          po.p[0] = where[o.out];
          if (o.mask >= 0) {
            po.p[1] = where[o.mask];
            d.flags |= F_MASK_BIAS;
          }
          if (o.pos_bias >= 0) {
            if (o.seq % 32 != 0) {
              if (err) *err = "attention " + o.name + ": a position bias needs a sequence length that is a multiple of 32";
              return MONONN_ERR_UNSUPPORTED;
            }
            po.q[0] = raw_const(o.pos_bias);
            d.flags |= F_POS_BIAS;
          }
          P.algorithmic_flops += 2.0 * 2.0 * o.seq * o.seq * o.head_dim * o.heads * o.batches;
          break;
        }
        case OP_LAYERNORM: {
          const FTensor& S = g.tensors[o.src];
          d.rows = o.rows;
          d.cols = o.cols;
          if (o.cols % 4 != 0 || o.cols > 2048) {
            if (err) *err = "layernorm " + o.name + ": row length must be <= 2048 and a multiple of 4";
            return MONONN_ERR_UNSUPPORTED;
          }
          d.n_items = (o.rows + kRowsPerItem - 1) / kRowsPerItem;
          // Few rows (batch 1): one warp per row leaves most CTAs idle while each row's load ->
          // reduce -> normalise -> store chain runs on a single warp. Four warps per row, two rows
          // per item, when all items still fit one wave of the CTAs.
          if (spec_in.row_split != 1 && !(o.flags & (F_L2NORM | F_NO_NORM)) && o.cols % 16 == 0 && o.cols <= 1024 &&
              (o.rows + kSplitRowsPerItem - 1) / kSplitRowsPerItem <= P.grid) {
            d.flags |= F_ROW_SPLIT;
            d.n_items = (o.rows + kSplitRowsPerItem - 1) / kSplitRowsPerItem;
          }
          po.p[0] = where[o.out];
          d.ldo = g.tensors[o.out].ld;
          po.p[1] = where[o.src];
          // rows taken every `k_col`-th source row starting at row `q_col` (class-token pooling)
          const uint32_t stride = o.k_col ? o.k_col : 1u;
          if (S.kind == TKind::AccF32) {
            d.flags |= F_SRC_F32;
            d.lds = S.cols * stride;
            po.p[1].offset += static_cast<uint64_t>(o.q_col) * S.cols * 4;
          } else {
            d.lds = S.ld * stride;
            po.p[1].offset += static_cast<uint64_t>(o.q_col) * S.ld * 2;
          }
          if (o.flags & F_L2NORM) {  // scale and shift are unused; any readable row will do
            po.p[2] = po.p[1];
            po.p[3] = po.p[1];
          } else {
            po.p[2] = raw_const(o.gamma);
            po.p[3] = raw_const(o.beta >= 0 ? o.beta : o.gamma);  // RMS norm: no shift, any valid row
          }
          if (o.resid >= 0) {
            po.p[4] = where[o.resid];
            d.flags |= F_RESID;
            d.ldr = g.tensors[o.resid].ld;
          }
          if (o.out2 >= 0) {
            po.q[2] = where[o.out2];
            if (o.bias2 >= 0) po.q[3] = raw_const(o.bias2);
          }
          break;
        }
        case OP_PATCHIFY: {
          d.rows = o.rows;
          d.cols = o.cols;
          d.heads = o.heads;
          d.seq = o.seq;
          d.batches = o.batches;
          d.head_dim = o.head_dim;
          d.q_col = o.q_col;
          d.k_col = o.k_col;
          d.vocab = o.vocab;
          d.M = o.M;
          d.N = o.N;
          d.K = o.K;
          d.rows_per_batch = o.pad_top;
          d.ldt = o.pad_left;
          d.n_items = (o.rows + kRowsPerItem - 1) / kRowsPerItem;
          po.p[0] = where[o.out];
          d.ldo = g.tensors[o.out].ld;
          po.p[1] = where[o.src];
          break;
        }
        case OP_ROWSEL: {
          d.rows = o.rows;
          d.cols = o.cols;
          d.seq = o.seq;
          d.lds = g.tensors[o.src].ld;
          d.ldo = g.tensors[o.out].ld;
          d.n_items = (o.rows + kRowsPerItem - 1) / kRowsPerItem;
          po.p[0] = where[o.out];
          po.p[1] = where[o.src];
          po.p[2] = where[o.ids];
          break;
        }
        case OP_PAIRDOT: {
          d.M = o.M;
          d.N = o.N;
          d.K = o.K;
          d.lds = g.tensors[o.a].ld;
          d.ldr = g.tensors[o.src].ld;
          d.ldo = g.tensors[o.out].ld;
          d.n_items = (o.M + kRowsPerItem - 1) / kRowsPerItem;
          po.p[0] = where[o.out];
          po.p[1] = where[o.a];
          po.p[2] = where[o.src];
          P.algorithmic_flops += 2.0 * o.M * o.N * o.K;
          break;
        }
        case OP_ARGMAX: {
          d.rows = o.rows;
          d.cols = o.cols;
          d.lds = g.tensors[o.src].ld;
          d.n_items = o.rows;  // one row per 128-thread group
          po.p[0] = where[o.out];
          po.p[1] = where[o.src];
          break;
        }
        case OP_ASSEMBLE: {
          d.rows = o.rows;
          d.cols = o.cols;
          d.seq = o.seq;
          d.k_col = o.k_col;
          if (o.cols % 4 != 0 || o.cols > 2048) {
            if (err) *err = "assemble " + o.name + ": row length must be <= 2048 and a multiple of 4";
            return MONONN_ERR_UNSUPPORTED;
          }
          d.n_items = (o.rows + kRowsPerItem - 1) / kRowsPerItem;
          d.flags |= F_NO_NORM;
          if (o.out >= 0) {
            po.p[0] = where[o.out];
            d.ldo = g.tensors[o.out].ld;
          }
          po.p[1] = where[o.a];
          d.lds = g.tensors[o.a].ld;
          po.p[3] = raw_const(o.word);
          po.p[4] = raw_const(o.pos);
          if (o.bias >= 0) {
            po.p[5] = raw_const(o.bias);
            d.flags |= F_BIAS;
          }
          po.p[6] = po.p[4];
          po.p[7] = po.p[4];
          if (o.out2 >= 0) po.q[2] = where[o.out2];
          break;
        }
        case OP_EMBED: {
          d.rows = o.rows;
          d.cols = o.cols;
          d.seq = o.seq;
          d.vocab = o.vocab;
          if (o.cols % 4 != 0 || o.cols > 2048) {
            if (err) *err = "embed " + o.name + ": row length must be <= 2048 and a multiple of 4";
            return MONONN_ERR_UNSUPPORTED;
          }
          d.n_items = (o.rows + kRowsPerItem - 1) / kRowsPerItem;
          d.q_col = o.q_col;  // offset of the position index
          if (o.out >= 0) {
            po.p[0] = where[o.out];
            d.ldo = g.tensors[o.out].ld;
          }
          po.p[1] = where[o.ids];
          po.p[3] = raw_const(o.word);
          if (o.pos >= 0) po.p[4] = raw_const(o.pos);
          if (o.type_ids >= 0 && o.type >= 0) {
            po.p[2] = where[o.type_ids];
            po.p[5] = raw_const(o.type);
            d.flags |= F_TYPE_IDS;
          }
          if (o.gamma >= 0 && o.beta >= 0) {
            po.p[6] = raw_const(o.gamma);
            po.p[7] = raw_const(o.beta);
          } else {  // no embedding LayerNorm: the row sum is the result
            d.flags |= F_NO_NORM;
            po.p[6] = po.p[3];
            po.p[7] = po.p[3];
          }
          if (o.mask_in >= 0 && o.mask_out >= 0) {
            po.q[0] = where[o.mask_in];
            po.q[1] = where[o.mask_out];
            d.flags |= F_MASK_BIAS;
          }
          if (o.out2 >= 0) {
            po.q[2] = where[o.out2];
            if (o.bias2 >= 0) po.q[3] = raw_const(o.bias2);
          }
          break;
        }
        default:
          if (err) *err = "operator " + o.name + ": unknown kind";
          return MONONN_ERR_UNSUPPORTED;
      }
      if (flag_of[oi] >= 0) {
        po.flag = BufRef{SPACE_SCRATCH, 0, flags_off + 8ull * flag_of[oi]};
        po.flag_index = flag_of[oi];
        po.waits = waits[oi] != 0;
      }
      if (wflag_of[oi] >= 0) {
        po.wflag = BufRef{SPACE_SCRATCH, 0, flags_off + 8ull * wflag_of[oi]};
        po.wflag_index = wflag_of[oi];
      }
      sd.n_items += d.n_items;
      if (!sname.empty()) sname += "+";
      sname += o.name;
      P.ops.push_back(po);
    }
    sd.op_count = static_cast<uint32_t>(P.ops.size()) - sd.op_begin;
    for (size_t a = sd.op_begin; a < P.ops.size(); ++a) {
      if (!P.ops[a].waits) continue;
      uint32_t target = 0;
      for (size_t b = sd.op_begin; b < P.ops.size(); ++b)
        if (!P.ops[b].waits && P.ops[b].flag_index == P.ops[a].flag_index) target += P.ops[b].d.n_items;
      P.ops[a].d.flag_target = target;
    }
    for (size_t a = sd.op_begin; a < P.ops.size(); ++a) {
      if (P.ops[a].wflag_index < 0) continue;
      uint32_t target = 0;
      for (size_t b = sd.op_begin; b < a; ++b)
        if (!P.ops[b].waits && P.ops[b].flag_index == P.ops[a].wflag_index) target += P.ops[b].d.n_items;
      P.ops[a].d.wait_target = target;
    }
    if (sd.op_count > kMaxStageOps) {
      if (err) *err = "more than " + std::to_string(kMaxStageOps) + " independent operators at one depth";
      return MONONN_ERR_UNSUPPORTED;
    }
    {
      uint32_t run = 0;
      for (uint32_t k = 0; k < kMaxStageOps; ++k) {
        if (k < sd.op_count) run += P.ops[sd.op_begin + k].d.n_items;
        sd.item_end[k] = (k < sd.op_count) ? run : 0xffffffffu;
        if (k < sd.op_count && P.ops[sd.op_begin + k].d.kind == OP_ATTENTION &&
            (P.ops[sd.op_begin + k].d.flags & F_FUSED_QKV))
          sd.attn_prefetch_from = run;
      }
    }
    P.stages.push_back(sd);
    P.stage_names.push_back(sname);
  }
  P.const_bytes = std::max<uint64_t>(const_top, 256);

  // ---- algorithmic bytes: every constant once, except gathered tables (rows touched only)
  std::set<std::string> gathered;
  for (const FOp& o : ops)
    if (o.kind == OP_EMBED) {
      for (int t : {o.word, o.pos, o.type})
        if (t >= 0) gathered.insert(g.tensors[t].const_name);
      P.algorithmic_bytes += 2.0 * o.rows * o.cols;                 // word rows
      P.algorithmic_bytes += 2.0 * std::min(o.rows, o.seq) * o.cols;  // position rows
      if (o.type >= 0) P.algorithmic_bytes += 2.0 * o.cols;           // one type row
    }
  std::set<std::string> counted;
  for (const ConstBinding& b : P.consts) {
    if ((b.kind == ConstBinding::RAW && gathered.count(b.const_name)) || counted.count(b.const_name)) continue;
    counted.insert(b.const_name);
    P.algorithmic_bytes += static_cast<double>(b.src_bytes);
  }
  for (const ArgDesc& a : P.args)
    if (a.kind != 2) P.algorithmic_bytes += static_cast<double>(a.bytes);
  return validate_plan(P, err);
}

}  // namespace mononn
