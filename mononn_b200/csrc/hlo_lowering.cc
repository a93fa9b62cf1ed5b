// HLO module -> fused operator graph.
//
// Replaces, for the hot path, the reference's parser + clustering passes:
//   IRParserFused::from_hlo_module_impl     mononn_engine/parser/ir_parser_fused.cc:319-385
//   initialize_custom_call (__cublas$gemm)  ir_parser_fused.cc:740-826, op_impl/gemm_impl.cc:182-253
//   kLoop / kInput fusion -> cluster        ir_parser_fused.cc:489-539
//   MergeDependent / ElementWiseConcatenation (vertical fusion)
//                                           optimization/merge_dependent_pass.cc:37-190
// The reference never fuses across a GEMM custom-call (its epilogue is alpha*AB + beta*C,
// gemm_impl.cc:72-90); here the elementwise / reduce fusion that follows a GEMM becomes that
// GEMM's epilogue (bias, activation, residual) or a LayerNorm stage fed by its accumulator,
// and scores-GEMM -> softmax fusion -> PV-GEMM collapses into one attention operator.
//
// A fused computation is classified by hypothesis + numeric check (hlo_interp.h), so the
// same arithmetic printed in a different instruction order is still recognised, and anything
// that matches no hypothesis is rejected (the reference LOG(FATAL)s on unsupported input,
// e.g. ir_parser_fused.cc:95,311; here the caller gets MONONN_ERR_UNSUPPORTED).
#include "hlo_lowering.h"

#include <cstring>
#include <algorithm>
#include <cmath>
#include <functional>

#include "../../include/mononn.h"
#include "hlo_interp.h"
#include "hlo_parser.h"
#include "json.h"

namespace mononn {

namespace {

// IEEE binary16 bits of a float, round to nearest even (the device type of every weight).
uint16_t half_bits(float f) {
  uint32_t x;
  std::memcpy(&x, &f, 4);
  const uint32_t sign = (x >> 16) & 0x8000u;
  const uint32_t mant = x & 0x007fffffu;
  const int32_t exp = static_cast<int32_t>((x >> 23) & 0xffu);
  if (exp == 0xff) return static_cast<uint16_t>(sign | 0x7c00u | (mant ? 0x200u : 0u));  // inf / nan
  const int32_t e = exp - 127 + 15;
  if (e >= 31) return static_cast<uint16_t>(sign | 0x7c00u);  // overflow
  if (e <= 0) {                                                // subnormal or zero
    if (e < -10) return static_cast<uint16_t>(sign);
    const uint32_t m = mant | 0x00800000u;
    const uint32_t shift = static_cast<uint32_t>(14 - e);
    uint32_t h = m >> shift;
    const uint32_t rem = m & ((1u << shift) - 1u), halfway = 1u << (shift - 1);
    if (rem > halfway || (rem == halfway && (h & 1u))) ++h;
    return static_cast<uint16_t>(sign | h);
  }
  uint32_t h = (static_cast<uint32_t>(e) << 10) | (mant >> 13);
  const uint32_t rem = mant & 0x1fffu;
  if (rem > 0x1000u || (rem == 0x1000u && (h & 1u))) ++h;      // may carry into the exponent: still right
  return static_cast<uint16_t>(sign | h);
}

// The printed values of a constant in its element type; false for a type no operand can have.
bool encode_literal(const std::string& dtype, const std::vector<double>& v, std::vector<uint8_t>* raw) {
  if (dtype == "f16") {
    raw->resize(v.size() * 2);
    for (size_t i = 0; i < v.size(); ++i) {
      const uint16_t h = half_bits(static_cast<float>(v[i]));
      std::memcpy(raw->data() + 2 * i, &h, 2);
    }
  } else if (dtype == "f32") {
    raw->resize(v.size() * 4);
    for (size_t i = 0; i < v.size(); ++i) {
      const float f = static_cast<float>(v[i]);
      std::memcpy(raw->data() + 4 * i, &f, 4);
    }
  } else if (dtype == "s32" || dtype == "u32") {
    raw->resize(v.size() * 4);
    for (size_t i = 0; i < v.size(); ++i) {
      const int32_t k = static_cast<int32_t>(v[i]);
      std::memcpy(raw->data() + 4 * i, &k, 4);
    }
  } else {
    return false;
  }
  return true;
}

struct Rng {
  uint64_t s = 0x9E3779B97F4A7C15ull;
  float uni(float lo, float hi) {
    s = s * 6364136223846793005ull + 1442695040888963407ull;
    const float u = static_cast<float>((s >> 40) & 0xFFFFFF) / 16777216.0f;
    return lo + (hi - lo) * u;
  }
};

HTensor rand_tensor(const std::vector<int64_t>& dims, Rng& rng, float lo, float hi) {
  HTensor t = HTensor::zeros(dims);
  for (float& x : t.v) x = rng.uni(lo, hi);
  return t;
}

bool all_close(const std::vector<float>& a, const std::vector<float>& b, float atol, float rtol) {
  if (a.size() != b.size()) return false;
  for (size_t i = 0; i < a.size(); ++i) {
    const float d = std::fabs(a[i] - b[i]);
    if (!(d <= atol + rtol * std::fabs(b[i]))) return false;
  }
  return true;
}

float act_ref(float x, ActKind k) {
  switch (k) {
    case ACT_GELU_ERF: return 0.5f * x * (1.0f + std::erf(x * 0.70710678118654752f));
    case ACT_RELU: return std::max(x, 0.0f);
    case ACT_QUICK_GELU: return x / (1.0f + std::exp(-1.702f * x));
    case ACT_GELU_TANH:
      return 0.5f * x * (1.0f + std::tanh(0.7978845608028654f * (x + 0.044715f * x * x * x)));
    default: return x;
  }
}

struct Val {
  // STREAM: the f32 residual stream of a pre-LN model (an accumulator that GEMMs add into);
  // IMAGE: NCHW f32 image argument seen through its NHWC/f16 layout fusion; CONVOUT: result
  // tuple of a patch convolution (its element 0 is a pending GEMM)
  enum Kind { NONE, ARG, CONST, ACT, GEMM, HEADS, SCORES, PROBS, ATTN, MASK, EMBED_SUM, STREAM, IMAGE, CONVOUT } kind = NONE;
  int tensor = -1;  // FGraph tensor (ARG, CONST-as-instr, ACT, HEADS, MASK)
  int op = -1;      // producing FGraph op (ACT, GEMM, HEADS, ATTN)
  int instr = -1;   // HLO instruction that defines the (unaliased) value
  uint32_t rows = 0, cols = 0;        // logical 2-D shape of ACT / GEMM
  uint32_t B = 0, heads = 0, S = 0, D = 0;  // head-shaped values
  int q_tensor = -1, k_tensor = -1;   // SCORES / PROBS
  float alpha = 1.f;
  int mask_tensor = -1;               // PROBS
  int pbias_tensor = -1;              // PROBS: constant bias per (head, query, key)
  float mask_scale = 0.f;             // MASK
  int mask_arg = -1;                  // MASK: the s32 argument it derives from
  int ids = -1, types = -1, word = -1, pos = -1, type = -1;  // EMBED_SUM (FGraph tensors)
  uint32_t vocab = 0;
  uint32_t pos_off = 0;               // EMBED_SUM: first row of the position table that is used
  bool causal = false;                // PROBS
};

class Lowering {
 public:
  Lowering(const HloModule& m, FGraph* g, std::string* err) : m_(m), e_(m.comps[m.entry]), g_(*g), err_(err) {}

  int run() {
    g_ = FGraph();
    g_.module_name = m_.name;
    vals_.assign(e_.instrs.size(), Val());
    uses_.assign(e_.instrs.size(), 0);
    for (const HloInstr& i : e_.instrs)
      for (int o : i.operands) uses_[o]++;
    // parameters first: argument order is by parameter_number (mononn_module.cc:91-143)
    for (size_t k = 0; k < e_.params.size(); ++k) {
      if (e_.params[k] < 0) return fail(MONONN_ERR_PARSE, "parameter " + std::to_string(k) + " is missing");
      const HloInstr& p = e_.instrs[e_.params[k]];
      if (p.shape.is_tuple()) return unsupported(p, "tuple parameters");
      ArgDesc a;
      a.name = p.name;
      a.kind = 0;
      a.param_number = static_cast<int>(k);
      a.bytes = static_cast<size_t>(p.shape.elements()) * p.shape.elem_bytes();
      g_.args.push_back(a);
      FTensor t;
      t.name = p.name;
      t.kind = TKind::Arg;
      t.cols = p.shape.dims.empty() ? 1 : static_cast<uint32_t>(p.shape.dims.back());
      t.rows = static_cast<uint32_t>(p.shape.elements() / std::max<uint32_t>(1, t.cols));
      t.ld = t.cols;
      t.elem_bytes = static_cast<uint32_t>(p.shape.elem_bytes());
      t.arg_index = static_cast<int>(k);
      Val v;
      v.kind = Val::ARG;
      v.tensor = g_.add_tensor(t);
      v.instr = e_.params[k];
      vals_[e_.params[k]] = v;
    }
    for (size_t idx = 0; idx < e_.instrs.size(); ++idx) {
      const HloInstr& ins = e_.instrs[idx];
      int rc = MONONN_OK;
      if (ins.opcode == "parameter" || ins.opcode == "split-fusion") continue;
      if (ins.opcode == "constant") {
        Val v;
        v.kind = Val::CONST;
        v.instr = static_cast<int>(idx);
        vals_[idx] = v;
      } else if (ins.opcode == "custom-call") {
        rc = lower_custom_call(static_cast<int>(idx));
      } else if (ins.opcode == "fusion") {
        rc = lower_fusion(static_cast<int>(idx));
      } else if (ins.opcode == "bitcast" || ins.opcode == "reshape" || ins.opcode == "copy") {
        if (ins.operands.size() != 1) return unsupported(ins, "expects one operand");
        const Val& s = vals_[ins.operands[0]];
        if (s.kind != Val::ACT && s.kind != Val::ARG && s.kind != Val::CONST &&
            !(s.kind == Val::GEMM && uses_[ins.operands[0]] == 1))
          return unsupported(ins, "reshape of this kind of value at the top level");
        if (ins.shape.elements() != e_.instrs[ins.operands[0]].shape.elements())
          return unsupported(ins, "element count changes");
        vals_[idx] = s;  // same buffer, row-major in both shapes
        if (s.kind == Val::GEMM) vals_[idx].instr = static_cast<int>(idx);  // consumers are counted on the alias
      } else if (ins.opcode == "get-tuple-element") {
        if (ins.operands.size() != 1) return unsupported(ins, "expects one operand");
        const Val& s = vals_[ins.operands[0]];
        const auto gi = ins.int_list("index");
        if (s.kind != Val::CONVOUT || gi.size() != 1 || gi[0] != 0)
          return unsupported(ins, "get-tuple-element of anything but element 0 of a convolution result");
        Val v = s;  // element 0 of the cuDNN result tuple is the output (ir_parser_fused.cc:803-823)
        v.kind = Val::GEMM;
        v.instr = static_cast<int>(idx);
        vals_[idx] = v;
      } else if (ins.opcode == "tuple") {
        if (static_cast<int>(idx) != e_.root) return unsupported(ins, "tuple that is not the entry root");
      } else {
        // the reference wraps bare top-level ops into one-node clusters
        // (optimization/clustering_single_node_pass.cc:41-219); none occurs on this path
        return unsupported(ins, "top-level instruction outside {parameter, constant, fusion, custom-call, bitcast, tuple}");
      }
      if (rc) return rc;
    }
    int rc = finish_outputs();
    if (rc) return rc;
    return attach_mask();
  }

 private:
  // ------------------------------------------------------------------ errors
  int fail(int code, const std::string& msg) {
    if (err_) *err_ = msg;
    return code;
  }
  int unsupported(const HloInstr& ins, const std::string& why) {
    return fail(MONONN_ERR_UNSUPPORTED, "%" + ins.name + " (" + ins.opcode + ", HLO line " +
                                            std::to_string(ins.line) + "): " + why);
  }

  // ----------------------------------------------------------------- tensors
  int const_tensor(int instr, uint32_t rows, uint32_t cols, bool transposed = false) {
    const HloInstr& c = e_.instrs[instr];
    const std::pair<int, bool> key(instr, transposed);
    auto it = const_tensors_.find(key);
    if (it != const_tensors_.end()) return it->second;
    FTensor t;
    t.name = c.name;
    t.kind = TKind::Const;
    t.rows = rows;
    t.cols = cols;
    t.ld = cols;
    t.elem_bytes = static_cast<uint32_t>(c.shape.elem_bytes());
    t.const_name = c.name;
    t.const_transposed = transposed;
    for (int64_t d : c.shape.dims) t.const_dims.push_back(static_cast<uint32_t>(d));
    if (!c.payload.empty() && static_cast<int64_t>(c.payload.size()) == c.shape.elements() &&
        !g_.literals.count(c.name)) {
      std::vector<uint8_t> raw;
      if (encode_literal(c.shape.dtype, c.payload, &raw)) g_.literals[c.name] = std::move(raw);
    }
    return const_tensors_[key] = g_.add_tensor(t);
  }
  int act_tensor(const std::string& name, uint32_t rows, uint32_t cols) {
    FTensor t;
    t.name = name;
    t.kind = TKind::ActF16;
    t.rows = rows;
    t.cols = cols;
    t.ld = cols;
    return g_.add_tensor(t);
  }
  bool is_f16(const HloInstr& i) const { return i.shape.dtype == "f16"; }

  // Runs a fused computation on probe inputs.
  int probe(const HloComputation& c, const std::vector<HTensor>& params, HTensor* out) {
    std::string e;
    int rc = eval_computation(m_, c, params, out, &e);
    if (rc) return fail(rc, "fused computation " + c.name + ": " + e);
    return MONONN_OK;
  }
  // Probe tensors shaped like the fusion's parameters; `fill` decides the contents.
  std::vector<HTensor> probe_inputs(const HloComputation& c,
                                    const std::function<void(size_t, HTensor&)>& fill) {
    std::vector<HTensor> ps(c.params.size());
    for (size_t k = 0; k < c.params.size(); ++k) {
      ps[k] = HTensor::zeros(c.instrs[c.params[k]].shape.dims);
      fill(k, ps[k]);
    }
    return ps;
  }

  // Every layer of a model repeats the same fused computations; a computation that has been
  // classified once (same instructions, shapes and attributes, same operand roles) is not
  // evaluated again. Instruction names are not part of the key.
  std::string memo_key(const char* what, const HloComputation& c, std::initializer_list<int> roles) const {
    std::string k = what;
    for (int r : roles) k += "," + std::to_string(r);
    k += "|";
    for (const HloInstr& i : c.instrs) {
      k += i.opcode + ":" + i.shape.str() + "(";
      for (int o : i.operands) k += std::to_string(o) + " ";
      k += ")";
      if (i.opcode == "parameter") k += std::to_string(i.param_number);
      if (i.opcode == "constant") k += std::to_string(i.literal);
      for (const auto& a : i.attrs) k += a.first + "=" + a.second + ";";
      k += "\n";
    }
    return k;
  }

  // ------------------------------------------------------------- custom-call
  int lower_custom_call(int idx) {
    const HloInstr& ins = e_.instrs[idx];
    const std::string target = ins.attr("custom_call_target");
    if (target == "__cudnn$convForward") return lower_conv(idx);  // custom_call.cc:96-103
    if (target != "__cublas$gemm")
      return unsupported(ins, "custom-call target " + target);
    if (ins.operands.size() != 2) return unsupported(ins, "GEMM with a C operand (beta != 0)");
    Json cfg;
    std::string je;
    if (!Json::parse(ins.attr("backend_config"), &cfg, &je))
      return fail(MONONN_ERR_PARSE, "%" + ins.name + ": backend_config is not JSON: " + je);
    const Json* dn = cfg.find("dot_dimension_numbers");
    if (!dn) return fail(MONONN_ERR_PARSE, "%" + ins.name + ": backend_config lacks dot_dimension_numbers");
    auto list = [&](const char* key) {
      std::vector<int> v;
      if (const Json* a = dn->find(key))
        if (a->is_array())
          for (const Json& x : a->arr) v.push_back(static_cast<int>(x.as_number()));
      return v;
    };
    const auto lc = list("lhs_contracting_dimensions"), rc_ = list("rhs_contracting_dimensions");
    const auto lb = list("lhs_batch_dimensions"), rb = list("rhs_batch_dimensions");
    if (lc.size() != 1 || rc_.size() != 1) return unsupported(ins, "exactly one contracting dimension per side");
    if (cfg.get_number("beta", 0) != 0 || cfg.get_number("alpha_imag", 0) != 0)
      return unsupported(ins, "beta or imaginary alpha");
    const float alpha = static_cast<float>(cfg.get_number("alpha_real", 1));
    const HloInstr& lhs = e_.instrs[ins.operands[0]];
    const HloInstr& rhs = e_.instrs[ins.operands[1]];
    if (!is_f16(lhs) || !is_f16(rhs) || !is_f16(ins))
      return unsupported(ins, "GEMM operand types other than f16 (accumulation is fp32)");
    const Val& a = vals_[ins.operands[0]];
    const Val& b = vals_[ins.operands[1]];

    if (lb.empty() && rb.empty()) {
      // ---- dense layer: activation [M,K] x constant weight
      if (a.kind != Val::ACT) return unsupported(ins, "left operand is not a materialised activation");
      if (b.kind == Val::ACT) return lower_pairdot(idx, alpha, lc[0], rc_[0]);
      if (b.kind != Val::CONST) return unsupported(ins, "right operand is not a constant weight");
      if (lhs.shape.dims.size() != 2 || rhs.shape.dims.size() != 2 || lc[0] != 1)
        return unsupported(ins, "left operand must be [M,K] contracting its last dimension");
      const uint32_t M = static_cast<uint32_t>(lhs.shape.dims[0]), K = static_cast<uint32_t>(lhs.shape.dims[1]);
      const bool transposed = (rc_[0] == 1);
      const uint32_t Kw = static_cast<uint32_t>(rhs.shape.dims[transposed ? 1 : 0]);
      const uint32_t N = static_cast<uint32_t>(rhs.shape.dims[transposed ? 0 : 1]);
      if (Kw != K || a.rows != M || a.cols != K) return unsupported(ins, "operand shapes are inconsistent");
      FOp o;
      o.kind = OP_GEMM;
      o.name = canonical_node_name(ins.name);
      o.a = a.tensor;
      o.w = const_tensor(b.instr, K, N, transposed);
      o.M = M;
      o.N = N;
      o.K = K;
      o.alpha = alpha;
      g_.ops.push_back(o);
      Val v;
      v.kind = Val::GEMM;
      v.op = static_cast<int>(g_.ops.size()) - 1;
      v.instr = idx;
      v.rows = M;
      v.cols = N;
      vals_[idx] = v;
      return MONONN_OK;
    }
    // ---- batched over (batch, head): the two GEMMs of attention
    if (lb != std::vector<int>{0, 1} || rb != std::vector<int>{0, 1} || lhs.shape.dims.size() != 4)
      return unsupported(ins, "batched GEMM other than [B,heads,.,.] x [B,heads,.,.]");
    if (a.kind == Val::HEADS && b.kind == Val::HEADS && lc[0] == 3 && rc_[0] == 3) {
      Val v;
      v.kind = Val::SCORES;
      v.instr = idx;
      v.q_tensor = a.tensor;
      v.k_tensor = b.tensor;
      v.alpha = alpha;
      v.B = a.B; v.heads = a.heads; v.S = a.S; v.D = a.D;
      if (b.B != a.B || b.heads != a.heads || b.S != a.S || b.D != a.D)
        return unsupported(ins, "query and key shapes differ");
      vals_[idx] = v;
      return MONONN_OK;
    }
    if (a.kind == Val::PROBS && b.kind == Val::HEADS && lc[0] == 3 && rc_[0] == 2) {
      if (alpha != 1.f) return unsupported(ins, "alpha on the probability x value GEMM");
      if (uses_[b.instr] != 1) return unsupported(ins, "value tensor has other consumers");
      FTensor& vt = g_.tensors[b.tensor];
      vt.kind = TKind::ActF16T;  // the V projection writes its output transposed per batch
      vt.batches = b.B;
      vt.seq = b.S;
      vt.ld = (b.S + 7) / 8 * 8;
      FOp o;
      o.kind = OP_ATTENTION;
      o.name = canonical_node_name(ins.name);
      o.q = a.q_tensor;
      o.k = a.k_tensor;
      o.vt = b.tensor;
      o.mask = a.mask_tensor;
      o.pos_bias = a.pbias_tensor;
      o.heads = a.heads;
      o.seq = a.S;
      o.batches = a.B;
      o.head_dim = a.D;
      o.alpha = a.alpha;
      if (a.causal) o.flags |= F_CAUSAL;
      g_.ops.push_back(o);
      Val v;
      v.kind = Val::ATTN;
      v.op = static_cast<int>(g_.ops.size()) - 1;
      v.instr = idx;
      v.B = a.B; v.heads = a.heads; v.S = a.S; v.D = a.D;
      vals_[idx] = v;
      return MONONN_OK;
    }
    return unsupported(ins, "batched GEMM that is neither Q.K^T nor P.V of an attention block");
  }

  // ------------------------------------------------------------------ fusion
  int lower_fusion(int idx) {
    const HloInstr& ins = e_.instrs[idx];
    const HloComputation* c = m_.find(ins.attr("calls"));
    if (!c) return fail(MONONN_ERR_PARSE, "%" + ins.name + ": fused computation " + ins.attr("calls") + " not found");
    if (c->params.size() != ins.operands.size())
      return fail(MONONN_ERR_PARSE, "%" + ins.name + ": operand count does not match " + c->name);
    if (ins.shape.is_tuple()) return unsupported(ins, "multi-output fusion that is not read through get-tuple-element");
    bool has_reduce = false, has_gather = false;
    for (const HloInstr& i : c->instrs) {
      has_reduce = has_reduce || i.opcode == "reduce";
      has_gather = has_gather || i.opcode == "gather";
    }
    bool has_concat = false;
    for (const HloInstr& i : c->instrs) has_concat = has_concat || i.opcode == "concatenate";
    if (has_gather && has_reduce) return lower_rowsel(idx, *c);
    if (has_gather) return lower_embed_sum(idx, *c);
    if (has_reduce && ins.shape.dtype == "s32" && ins.operands.size() == 1) return lower_argmax(idx, *c);
    if (has_concat) {  // token assembly: the result has more rows than the patch GEMM
      for (size_t k = 0; k < ins.operands.size(); ++k)
        if (vals_[ins.operands[k]].kind == Val::GEMM) return lower_tokens(idx, *c, static_cast<int>(k));
      return unsupported(ins, "concatenating fusion that does not follow a patch convolution");
    }
    // the "main" operand: same element count as the result and not a constant
    int main_k = -1;
    for (size_t k = 0; k < ins.operands.size(); ++k) {
      const Val& v = vals_[ins.operands[k]];
      if (v.kind == Val::CONST || v.kind == Val::NONE || v.kind == Val::MASK) continue;
      if (e_.instrs[ins.operands[k]].shape.elements() != ins.shape.elements()) continue;
      if (main_k < 0 || v.kind == Val::GEMM) main_k = static_cast<int>(k);
    }
    if (main_k < 0 && ins.operands.size() == 1 && vals_[ins.operands[0]].kind == Val::ARG &&
        e_.instrs[ins.operands[0]].shape.dims.size() == 4)
      return lower_image_layout(idx, *c);
    if (main_k < 0 && has_reduce) {
      // a row-wise reduction over selected rows of a larger tensor (class-token LayerNorm)
      for (size_t k = 0; k < ins.operands.size(); ++k) {
        const Val& v = vals_[ins.operands[k]];
        const int64_t ne = e_.instrs[ins.operands[k]].shape.elements();
        if ((v.kind == Val::ACT || v.kind == Val::STREAM) && ne > ins.shape.elements() && ne % ins.shape.elements() == 0)
          return lower_layernorm(idx, *c, static_cast<int>(k));
      }
    }
    if (main_k < 0) return unsupported(ins, "fusion without a tensor operand of the result's size");
    const Val& mv = vals_[ins.operands[main_k]];
    if (has_reduce && ins.operands.size() == 1 && (mv.kind == Val::GEMM || mv.kind == Val::ACT))
      return lower_l2norm(idx, *c);
    switch (mv.kind) {
      case Val::GEMM:
        return has_reduce ? lower_layernorm(idx, *c, main_k) : lower_epilogue(idx, *c, main_k);
      case Val::ACT:
      case Val::STREAM:
      case Val::EMBED_SUM:
        if (has_reduce) return lower_layernorm(idx, *c, main_k);
        return unsupported(ins, "elementwise fusion that does not follow a GEMM");
      case Val::SCORES:
        return lower_softmax(idx, *c, main_k);
      case Val::ATTN:
        return lower_merge(idx, *c, main_k);
      case Val::ARG:
        if (e_.instrs[ins.operands[main_k]].shape.dims.size() == 4) return lower_image_layout(idx, *c);
        return lower_mask(idx, *c, main_k);
      default:
        return unsupported(ins, "fusion over this kind of value");
    }
  }

  // bias / activation / residual (/ head split) after a GEMM -> that GEMM's epilogue
  int lower_epilogue(int idx, const HloComputation& c, int main_k) {
    const HloInstr& ins = e_.instrs[idx];
    Val gv = vals_[ins.operands[main_k]];
    if (uses_[gv.instr] != 1) return unsupported(ins, "GEMM result with more than one consumer");
    FOp& gop = g_.ops[gv.op];
    const uint32_t M = gop.M, N = gop.N;
    int bias_k = -1, resid_k = -1;
    for (size_t k = 0; k < ins.operands.size(); ++k) {
      if (static_cast<int>(k) == main_k) continue;
      const Val& v = vals_[ins.operands[k]];
      const HloInstr& oi = e_.instrs[ins.operands[k]];
      if (v.kind == Val::CONST && oi.shape.elements() == N && bias_k < 0) bias_k = static_cast<int>(k);
      else if ((v.kind == Val::ACT || v.kind == Val::STREAM) && v.rows == M && v.cols == N && resid_k < 0)
        resid_k = static_cast<int>(k);
      else return unsupported(ins, "operand %" + oi.name + " has no role in a GEMM epilogue");
    }
    // result layout: [M,N] row-major, or [B,heads,S,D] with B*S = M and heads*D = N
    bool split = false;
    uint32_t B = 0, H = 0, S = 0, D = 0;
    const auto& od = ins.shape.dims;
    if (od.size() == 4 && od[0] * od[2] == M && od[1] * od[3] == N) {
      split = true;
      B = static_cast<uint32_t>(od[0]); H = static_cast<uint32_t>(od[1]);
      S = static_cast<uint32_t>(od[2]); D = static_cast<uint32_t>(od[3]);
    } else if (ins.shape.elements() != static_cast<int64_t>(M) * N) {
      return unsupported(ins, "result shape");
    }
    ActKind found = ACT_NONE;
    bool ok = false;
    const std::string mkey = memo_key("epilogue", c, {main_k, bias_k, resid_k, split ? 1 : 0});
    const auto hit = memo_.find(mkey);
    if (hit != memo_.end()) {
      found = static_cast<ActKind>(static_cast<int>(hit->second[0]));
      ok = true;
    } else {
    Rng rng;
    std::vector<HTensor> ps = probe_inputs(c, [&](size_t k, HTensor& t) {
      for (float& x : t.v) x = rng.uni(-2.f, 2.f);
      (void)k;
    });
    HTensor got;
    int rc = probe(c, ps, &got);
    if (rc) return rc;
    const HTensor& x = ps[main_k];
    for (ActKind act : {ACT_NONE, ACT_GELU_ERF, ACT_RELU, ACT_QUICK_GELU, ACT_GELU_TANH}) {
      std::vector<float> want(static_cast<size_t>(M) * N);
      for (uint32_t r = 0; r < M; ++r)
        for (uint32_t col = 0; col < N; ++col) {
          float y = x.v[static_cast<size_t>(r) * N + col];
          if (bias_k >= 0) y += ps[bias_k].v[col];
          y = act_ref(y, act);
          if (resid_k >= 0) y += ps[resid_k].v[static_cast<size_t>(r) * N + col];
          size_t dst = static_cast<size_t>(r) * N + col;
          if (split) {
            const uint32_t b = r / S, s = r % S, h = col / D, d = col % D;
            dst = ((static_cast<size_t>(b) * H + h) * S + s) * D + d;
          }
          want[dst] = y;
        }
      if (all_close(got.v, want, 1e-4f, 1e-4f)) {
        found = act;
        ok = true;
        break;
      }
    }
    if (ok) memo_[mkey] = {static_cast<double>(found)};
    }
    if (!ok) return unsupported(ins, "fused computation " + c.name + " matches no epilogue form act(x + bias) + residual");
    if (bias_k >= 0) gop.bias = const_tensor(vals_[ins.operands[bias_k]].instr, 1, N);
    if (resid_k >= 0 && vals_[ins.operands[resid_k]].kind == Val::ACT && found == ACT_NONE && !split) {
      // x + (A W + b) where x is a LayerNorm output that starts a pre-LN residual stream (the
      // LayerNorm before the blocks of a CLIP vision tower): that LayerNorm also writes an f32
      // copy, and from here on the stream is the accumulator the GEMMs add into.
      Val& rv = vals_[ins.operands[resid_k]];
      if (rv.op >= 0 && g_.ops[rv.op].kind == OP_LAYERNORM && g_.ops[rv.op].out == rv.tensor &&
          g_.ops[rv.op].out2 < 0 && g_.ops[rv.op].rows == M && g_.ops[rv.op].cols == N) {
        FTensor st;
        st.name = g_.ops[rv.op].name + "_stream";
        st.kind = TKind::AccF32;
        st.rows = M;
        st.cols = N;
        st.ld = N;
        st.elem_bytes = 4;
        g_.ops[rv.op].out2 = g_.add_tensor(st);
        Val sv;
        sv.kind = Val::STREAM;
        sv.instr = rv.instr;
        sv.tensor = g_.ops[rv.op].out2;
        sv.op = rv.op;
        sv.rows = M;
        sv.cols = N;
        stream_of_[rv.tensor] = sv;
      }
    }
    if (resid_k >= 0 && vals_[ins.operands[resid_k]].kind == Val::ACT &&
        stream_of_.count(vals_[ins.operands[resid_k]].tensor) && found == ACT_NONE && !split) {
      Val sv = stream_of_[vals_[ins.operands[resid_k]].tensor];
      gop.act = ACT_NONE;
      gop.out = sv.tensor;
      sv.instr = idx;
      sv.op = gv.op;
      vals_[idx] = sv;
      return MONONN_OK;
    }
    if (resid_k >= 0 && vals_[ins.operands[resid_k]].kind == Val::STREAM) {
      // pre-LN residual: x <- x + (A W + b). The stream is an f32 accumulator the GEMM adds
      // its (split-K) partial sums into; nothing is copied.
      if (found != ACT_NONE || split) return unsupported(ins, "activation or head split on a residual update");
      gop.act = ACT_NONE;
      gop.out = vals_[ins.operands[resid_k]].tensor;
      Val sv = vals_[ins.operands[resid_k]];
      sv.instr = idx;
      sv.op = gv.op;
      vals_[idx] = sv;
      return MONONN_OK;
    }
    if (resid_k >= 0) gop.resid = vals_[ins.operands[resid_k]].tensor;
    gop.act = found;
    gop.out = act_tensor(canonical_node_name(ins.name), M, N);
    Val v;
    v.instr = idx;
    v.tensor = gop.out;
    v.op = gv.op;
    v.rows = M;
    v.cols = N;
    if (split) {
      if (D != 64) return unsupported(ins, "head dimension other than 64");
      v.kind = Val::HEADS;
      v.B = B; v.heads = H; v.S = S; v.D = D;
    } else {
      v.kind = Val::ACT;
    }
    vals_[idx] = v;
    return MONONN_OK;
  }

  // LayerNorm of (x [+ bias] [+ residual]) where x is a GEMM result, an activation or the
  // embedding sum.
  int lower_layernorm(int idx, const HloComputation& c, int main_k) {
    const HloInstr& ins = e_.instrs[idx];
    const Val mv = vals_[ins.operands[main_k]];
    if (ins.shape.dims.empty()) return unsupported(ins, "scalar LayerNorm result");
    const uint32_t cols = static_cast<uint32_t>(ins.shape.dims.back());
    const uint32_t rows = static_cast<uint32_t>(ins.shape.elements() / cols);
    std::vector<int> vec_k;
    int resid_k = -1;
    for (size_t k = 0; k < ins.operands.size(); ++k) {
      if (static_cast<int>(k) == main_k) continue;
      const Val& v = vals_[ins.operands[k]];
      const HloInstr& oi = e_.instrs[ins.operands[k]];
      if (v.kind == Val::CONST && oi.shape.elements() == cols) vec_k.push_back(static_cast<int>(k));
      else if (v.kind == Val::ACT && v.rows == rows && v.cols == cols && resid_k < 0) resid_k = static_cast<int>(k);
      else return unsupported(ins, "operand %" + oi.name + " has no role in a LayerNorm fusion");
    }
    // Row selection: the result has one row per `stride` source rows, taken at offset `off`
    // (a slice inside the fusion: the class-token row of every image).
    uint32_t stride = 1;
    std::vector<uint32_t> off_cands{0};
    if ((mv.kind == Val::STREAM || mv.kind == Val::ACT) && (mv.rows != rows || mv.cols != cols)) {
      if (mv.cols != cols || rows == 0 || mv.rows % rows != 0 || resid_k >= 0)
        return unsupported(ins, "LayerNorm shape differs from its source");
      stride = mv.rows / rows;
      for (const HloInstr& i : c.instrs)
        if (i.opcode == "slice") {
          const std::string sl = i.attr("slice");
          for (size_t p = sl.find('['); p != std::string::npos; p = sl.find('[', p + 1)) {
            const uint32_t st = static_cast<uint32_t>(std::strtoul(sl.c_str() + p + 1, nullptr, 10));
            if (st < stride && std::find(off_cands.begin(), off_cands.end(), st) == off_cands.end())
              off_cands.push_back(st);
          }
        }
    }
    uint32_t off_found = 0;
    if (vec_k.size() == 1) return lower_rmsnorm(idx, c, main_k, vec_k[0], resid_k, stride);
    if (vec_k.size() < 2 || vec_k.size() > 3) return unsupported(ins, "expected scale, shift and at most one bias vector");
    std::vector<float> eps_cands;
    for (const HloInstr& i : c.instrs)
      if (i.opcode == "constant" && i.literal_is_scalar && i.literal > 0 && i.literal < 0.1)
        eps_cands.push_back(static_cast<float>(i.literal));
    if (eps_cands.empty()) eps_cands.push_back(0.f);
    int bias_k = -1, gamma_k = -1, beta_k = -1;
    float eps_found = 0.f;
    bool ok = false;
    const std::string mkey = memo_key("layernorm", c, {main_k, resid_k, static_cast<int>(stride),
                                                       static_cast<int>(mv.kind == Val::GEMM)});
    const auto hit = memo_.find(mkey);
    if (hit != memo_.end()) {
      bias_k = static_cast<int>(hit->second[0]);
      gamma_k = static_cast<int>(hit->second[1]);
      beta_k = static_cast<int>(hit->second[2]);
      eps_found = static_cast<float>(hit->second[3]);
      off_found = static_cast<uint32_t>(hit->second[4]);
      ok = true;
    } else {
    // Probe with small-magnitude rows (variance ~1e-4) so that the epsilon under the square
    // root changes the result visibly; scale/shift stay O(1).
    Rng rng;
    std::vector<HTensor> ps = probe_inputs(c, [&](size_t k, HTensor& t) {
      const bool is_vec = std::find(vec_k.begin(), vec_k.end(), static_cast<int>(k)) != vec_k.end();
      for (float& x : t.v) x = is_vec ? rng.uni(0.5f, 1.5f) : rng.uni(-0.02f, 0.02f);
    });
    HTensor got;
    int rc = probe(c, ps, &got);
    if (rc) return rc;
    // closed form for a given assignment of the vectors to (bias?, gamma, beta) and epsilon
    std::vector<float> want(static_cast<size_t>(rows) * cols), sum(cols);
    uint32_t off = 0;
    auto max_error = [&](int bk, int gk, int ek, float eps, uint32_t n_rows) {
      float worst = 0.f;
      for (uint32_t r = 0; r < n_rows; ++r) {
        double mean = 0;
        for (uint32_t j = 0; j < cols; ++j) {
          float y = ps[main_k].v[(static_cast<size_t>(r) * stride + off) * cols + j];
          if (bk >= 0) y += ps[bk].v[j];
          if (resid_k >= 0) y += ps[resid_k].v[static_cast<size_t>(r) * cols + j];
          sum[j] = y;
          mean += y;
        }
        mean /= cols;
        double var = 0;
        for (uint32_t j = 0; j < cols; ++j) var += (sum[j] - mean) * (sum[j] - mean);
        var /= cols;
        const double rstd = 1.0 / std::sqrt(var + eps);
        for (uint32_t j = 0; j < cols; ++j) {
          const float w = static_cast<float>((sum[j] - mean) * rstd) * ps[gk].v[j] + ps[ek].v[j];
          worst = std::max(worst, std::fabs(w - got.v[static_cast<size_t>(r) * cols + j]));
        }
      }
      return worst;
    };
    std::vector<int> perm = vec_k;
    std::sort(perm.begin(), perm.end());
    float best = 1e30f;
    do {
      const int bk = perm.size() == 3 ? perm[0] : -1;
      const int gk = perm[perm.size() - 2], ek = perm[perm.size() - 1];
      for (float eps : eps_cands)
        for (uint32_t oc : off_cands) {
          off = oc;
          const float e = max_error(bk, gk, ek, eps, std::min<uint32_t>(rows, 4));
          if (e < best) {
            best = e;
            bias_k = bk; gamma_k = gk; beta_k = ek;
            eps_found = eps;
            off_found = oc;
          }
        }
    } while (std::next_permutation(perm.begin(), perm.end()));
    off = off_found;
    ok = best < 1e-3f && max_error(bias_k, gamma_k, beta_k, eps_found, rows) < 1e-3f;
    if (ok) memo_[mkey] = {static_cast<double>(bias_k), static_cast<double>(gamma_k), static_cast<double>(beta_k),
                           static_cast<double>(eps_found), static_cast<double>(off_found)};
    }
    if (!ok) return unsupported(ins, "fused computation " + c.name + " matches no LayerNorm(x + bias + residual) form");

    FOp n;
    n.kind = OP_LAYERNORM;
    n.name = canonical_node_name(ins.name);
    n.rows = rows;
    n.cols = cols;
    n.eps = eps_found;
    n.gamma = const_tensor(vals_[ins.operands[gamma_k]].instr, 1, cols);
    n.beta = const_tensor(vals_[ins.operands[beta_k]].instr, 1, cols);
    if (mv.kind == Val::GEMM) {
      if (uses_[mv.instr] != 1) return unsupported(ins, "GEMM result with more than one consumer");
      FOp& gop = g_.ops[mv.op];
      if (gop.M != rows || gop.N != cols) return unsupported(ins, "GEMM and LayerNorm shapes differ");
      if (bias_k >= 0) gop.bias = const_tensor(vals_[ins.operands[bias_k]].instr, 1, cols);
      if (resid_k >= 0) gop.resid = vals_[ins.operands[resid_k]].tensor;
      FTensor acc;
      acc.name = gop.name + "_sum";
      acc.kind = TKind::AccF32;
      acc.rows = rows;
      acc.cols = cols;
      acc.ld = cols;
      acc.elem_bytes = 4;
      gop.out = g_.add_tensor(acc);
      n.src = gop.out;
      n.flags = F_ZERO_SRC;
    } else if (mv.kind == Val::EMBED_SUM) {
      if (bias_k >= 0 || resid_k >= 0) return unsupported(ins, "bias or residual on the embedding LayerNorm");
      n.kind = OP_EMBED;
      n.ids = mv.ids;
      n.type_ids = mv.types;
      n.word = mv.word;
      n.pos = mv.pos;
      n.type = mv.type;
      n.seq = mv.S;
      n.vocab = mv.vocab;
      n.q_col = mv.pos_off;
      n.alpha = -10000.f;
    } else {
      if (bias_k >= 0) return unsupported(ins, "bias vector on a LayerNorm that does not follow a GEMM");
      n.src = mv.tensor;  // f16 activation, or the f32 residual stream (read, not cleared)
      if (resid_k >= 0) n.resid = vals_[ins.operands[resid_k]].tensor;
      if (stride > 1) {
        n.k_col = stride;
        n.q_col = off_found;
      }
    }
    n.out = act_tensor(n.name, rows, cols);
    g_.ops.push_back(n);
    Val v;
    v.kind = Val::ACT;
    v.instr = idx;
    v.tensor = n.out;
    v.op = static_cast<int>(g_.ops.size()) - 1;
    v.rows = rows;
    v.cols = cols;
    vals_[idx] = v;
    return MONONN_OK;
  }

  // x * rsqrt(mean(x^2) + eps) * scale over the last dimension: the LayerNorm of T5 (no mean
  // subtraction, no shift), reading an activation or the f32 residual stream.
  int lower_rmsnorm(int idx, const HloComputation& c, int main_k, int gamma_k, int resid_k, uint32_t stride) {
    const HloInstr& ins = e_.instrs[idx];
    const Val mv = vals_[ins.operands[main_k]];
    const uint32_t cols = static_cast<uint32_t>(ins.shape.dims.back());
    const uint32_t rows = static_cast<uint32_t>(ins.shape.elements() / cols);
    if (resid_k >= 0 || stride != 1 || (mv.kind != Val::ACT && mv.kind != Val::STREAM))
      return unsupported(ins, "RMS normalisation of anything but a plain activation");
    std::vector<float> eps_cands;
    for (const HloInstr& i : c.instrs)
      if (i.opcode == "constant" && i.literal_is_scalar && i.literal > 0 && i.literal < 0.1)
        eps_cands.push_back(static_cast<float>(i.literal));
    if (eps_cands.empty()) eps_cands.push_back(0.f);
    float eps_found = 0.f;
    bool ok = false;
    const std::string mkey = memo_key("rmsnorm", c, {main_k, gamma_k});
    const auto hit = memo_.find(mkey);
    if (hit != memo_.end()) {
      eps_found = static_cast<float>(hit->second[0]);
      ok = true;
    } else {
      Rng rng;  // small rows, so that the epsilon under the root is visible in the result
      std::vector<HTensor> ps = probe_inputs(c, [&](size_t k, HTensor& t) {
        for (float& x : t.v) x = static_cast<int>(k) == gamma_k ? rng.uni(0.5f, 1.5f) : rng.uni(-0.02f, 0.02f);
      });
      HTensor got;
      int rc = probe(c, ps, &got);
      if (rc) return rc;
      float best = 1e30f;
      for (float eps : eps_cands) {
        float worst = 0.f;
        for (uint32_t r = 0; r < rows; ++r) {
          double sq = 0;
          for (uint32_t j = 0; j < cols; ++j) {
            const double y = ps[main_k].v[static_cast<size_t>(r) * cols + j];
            sq += y * y;
          }
          const double rstd = 1.0 / std::sqrt(sq / cols + eps);
          for (uint32_t j = 0; j < cols; ++j) {
            const float w = static_cast<float>(ps[main_k].v[static_cast<size_t>(r) * cols + j] * rstd) * ps[gamma_k].v[j];
            worst = std::max(worst, std::fabs(w - got.v[static_cast<size_t>(r) * cols + j]));
          }
        }
        if (worst < best) {
          best = worst;
          eps_found = eps;
        }
      }
      ok = best < 1e-3f;
      if (ok) memo_[mkey] = {static_cast<double>(eps_found)};
    }
    if (!ok) return unsupported(ins, "fused computation " + c.name + " is neither LayerNorm nor x * rsqrt(mean(x^2) + eps) * scale");
    FOp n;
    n.kind = OP_LAYERNORM;
    n.name = canonical_node_name(ins.name);
    n.flags = F_RMSNORM;
    n.rows = rows;
    n.cols = cols;
    n.eps = eps_found;
    n.gamma = const_tensor(vals_[ins.operands[gamma_k]].instr, 1, cols);
    n.src = mv.tensor;
    n.out = act_tensor(n.name, rows, cols);
    g_.ops.push_back(n);
    Val v;
    v.kind = Val::ACT;
    v.instr = idx;
    v.tensor = n.out;
    v.op = static_cast<int>(g_.ops.size()) - 1;
    v.rows = rows;
    v.cols = cols;
    vals_[idx] = v;
    return MONONN_OK;
  }

  // softmax(scores + mask) over the keys
  int lower_softmax(int idx, const HloComputation& c, int main_k) {
    const HloInstr& ins = e_.instrs[idx];
    const Val sv = vals_[ins.operands[main_k]];
    if (uses_[sv.instr] != 1) return unsupported(ins, "attention scores with more than one consumer");
    int mask_k = -1, pbias_k = -1;
    for (size_t k = 0; k < ins.operands.size(); ++k) {
      if (static_cast<int>(k) == main_k) continue;
      const Val& ov = vals_[ins.operands[k]];
      if (ov.kind == Val::MASK && mask_k < 0) mask_k = static_cast<int>(k);
      else if (ov.kind == Val::CONST && pbias_k < 0 &&
               e_.instrs[ins.operands[k]].shape.elements() == static_cast<int64_t>(sv.heads) * sv.S * sv.S)
        pbias_k = static_cast<int>(k);  // additive bias per (head, query, key)
      else return unsupported(ins, "operand %" + e_.instrs[ins.operands[k]].name + " has no role in a softmax fusion");
    }
    const uint32_t B = sv.B, H = sv.heads, S = sv.S;
    if (ins.shape.dims != std::vector<int64_t>{B, H, S, S}) return unsupported(ins, "result shape");
    bool causal = false, ok = false;
    const std::string mkey = memo_key("softmax", c, {main_k, mask_k, pbias_k});
    const auto hit = memo_.find(mkey);
    if (hit != memo_.end()) {
      causal = hit->second[0] != 0.0;
      ok = true;
    } else {
    Rng rng;
    std::vector<HTensor> ps = probe_inputs(c, [&](size_t k, HTensor& t) {
      for (float& x : t.v) x = (static_cast<int>(k) == mask_k) ? (rng.uni(0.f, 1.f) < 0.25f ? -50.f : 0.f)
                                                               : rng.uni(-4.f, 4.f);
    });
    HTensor got;
    int rc = probe(c, ps, &got);
    if (rc) return rc;
    std::vector<float> want(got.v.size());
    for (int trial = 0; trial < 2 && !ok; ++trial) {
      causal = (trial == 1);  // keys after the query position are excluded
      for (uint32_t b = 0; b < B; ++b)
        for (uint32_t h = 0; h < H; ++h)
          for (uint32_t q = 0; q < S; ++q) {
            const size_t base = ((static_cast<size_t>(b) * H + h) * S + q) * S;
            const uint32_t n_keys = causal ? q + 1 : S;
            float mx = -INFINITY;
            for (uint32_t k = 0; k < n_keys; ++k) {
              const float z = ps[main_k].v[base + k] + (mask_k >= 0 ? ps[mask_k].v[static_cast<size_t>(b) * S + k] : 0.f) +
                              (pbias_k >= 0 ? ps[pbias_k].v[(static_cast<size_t>(h) * S + q) * S + k] : 0.f);
              want[base + k] = z;
              mx = std::max(mx, z);
            }
            double sum = 0;
            for (uint32_t k = 0; k < n_keys; ++k) {
              want[base + k] = std::exp(want[base + k] - mx);
              sum += want[base + k];
            }
            for (uint32_t k = 0; k < n_keys; ++k) want[base + k] = static_cast<float>(want[base + k] / sum);
            for (uint32_t k = n_keys; k < S; ++k) want[base + k] = 0.f;
          }
      ok = all_close(got.v, want, 1e-5f, 1e-4f);
    }
    if (ok) memo_[mkey] = {causal ? 1.0 : 0.0};
    }
    if (!ok)
      return unsupported(ins, "fused computation " + c.name +
                                  " is not softmax(scores + mask) over the last dimension, plain or causal");
    Val v = sv;
    v.kind = Val::PROBS;
    v.instr = idx;
    v.mask_tensor = mask_k >= 0 ? vals_[ins.operands[mask_k]].tensor : -1;
    v.pbias_tensor = pbias_k >= 0 ? const_tensor(vals_[ins.operands[pbias_k]].instr, H * S, S) : -1;
    v.causal = causal;
    vals_[idx] = v;
    return MONONN_OK;
  }

  // [B,heads,S,D] -> [B*S, heads*D]
  int lower_merge(int idx, const HloComputation& c, int main_k) {
    const HloInstr& ins = e_.instrs[idx];
    const Val av = vals_[ins.operands[main_k]];
    if (ins.operands.size() != 1) return unsupported(ins, "extra operands on a head-merge fusion");
    if (uses_[av.instr] != 1) return unsupported(ins, "attention output with more than one consumer");
    const uint32_t B = av.B, H = av.heads, S = av.S, D = av.D;
    if (ins.shape.elements() != static_cast<int64_t>(B) * H * S * D) return unsupported(ins, "result shape");
    const std::string mkey = memo_key("merge", c, {main_k});
    if (!memo_.count(mkey)) {
      Rng rng;
      std::vector<HTensor> ps = probe_inputs(c, [&](size_t, HTensor& t) {
        for (float& x : t.v) x = rng.uni(-1.f, 1.f);
      });
      HTensor got;
      int rc = probe(c, ps, &got);
      if (rc) return rc;
      std::vector<float> want(got.v.size());
      for (uint32_t b = 0; b < B; ++b)
        for (uint32_t h = 0; h < H; ++h)
          for (uint32_t s = 0; s < S; ++s)
            for (uint32_t d = 0; d < D; ++d)
              want[(static_cast<size_t>(b) * S + s) * H * D + h * D + d] =
                  ps[0].v[((static_cast<size_t>(b) * H + h) * S + s) * D + d];
      if (!all_close(got.v, want, 0.f, 0.f))
        return unsupported(ins, "fused computation " + c.name + " is not the head merge [B,h,S,d] -> [B*S, h*d]");
      memo_[mkey] = {1.0};
    }
    FOp& aop = g_.ops[av.op];
    aop.out = act_tensor(canonical_node_name(ins.name), B * S, H * D);
    Val v;
    v.kind = Val::ACT;
    v.instr = idx;
    v.tensor = aop.out;
    v.op = av.op;
    v.rows = B * S;
    v.cols = H * D;
    vals_[idx] = v;
    return MONONN_OK;
  }

  // NCHW f32 image argument -> NHWC f16 (the layout XLA gives cuDNN)
  int lower_image_layout(int idx, const HloComputation& c) {
    const HloInstr& ins = e_.instrs[idx];
    const HloInstr& src = e_.instrs[ins.operands[0]];
    const auto& sd = src.shape.dims;
    if (src.shape.dtype != "f32" || sd.size() != 4 || ins.shape.dims.size() != 4)
      return unsupported(ins, "image layout fusion must map f32 [B,C,H,W] to [B,H,W,C]");
    const int64_t B = sd[0], C = sd[1], H = sd[2], W = sd[3];
    if (ins.shape.dims != std::vector<int64_t>{B, H, W, C}) return unsupported(ins, "result is not [B,H,W,C]");
    Rng rng;
    std::vector<HTensor> ps = probe_inputs(c, [&](size_t, HTensor& t) {
      for (float& x : t.v) x = rng.uni(-1.f, 1.f);
    });
    HTensor got;
    int rc = probe(c, ps, &got);
    if (rc) return rc;
    std::vector<float> want(got.v.size());
    for (int64_t b = 0; b < B; ++b)
      for (int64_t ch = 0; ch < C; ++ch)
        for (int64_t y = 0; y < H; ++y)
          for (int64_t x = 0; x < W; ++x)
            want[((b * H + y) * W + x) * C + ch] = ps[0].v[((b * C + ch) * H + y) * W + x];
    if (!all_close(got.v, want, 0.f, 0.f))
      return unsupported(ins, "fused computation " + c.name + " is not the NCHW -> NHWC layout change");
    Val v;
    v.kind = Val::IMAGE;
    v.instr = idx;
    v.tensor = vals_[ins.operands[0]].tensor;
    v.B = static_cast<uint32_t>(B);
    v.heads = static_cast<uint32_t>(C);
    v.S = static_cast<uint32_t>(H);
    v.D = static_cast<uint32_t>(W);
    vals_[idx] = v;
    return MONONN_OK;
  }

  // __cudnn$convForward over the image: a window-extraction stage (stride, zero padding) writes
  // one row per output position and the convolution is a GEMM over those rows. With stride =
  // window and no padding every position sees its own patch (the ViT / CLIP embedding)
  // (NHWC input, KRSC filter, cross-correlation: ir_parser_fused.cc:749-800, conv_impl.cc:252-345).
  int lower_conv(int idx) {
    const HloInstr& ins = e_.instrs[idx];
    if (ins.operands.size() != 2) return unsupported(ins, "convolution with a side input");
    const Val& img = vals_[ins.operands[0]];
    const Val& wv = vals_[ins.operands[1]];
    if (img.kind != Val::IMAGE || wv.kind != Val::CONST)
      return unsupported(ins, "convolution operands must be the image and a constant filter");
    if (ins.attr("dim_labels") != "b01f_o01i->b01f") return unsupported(ins, "dim_labels other than b01f_o01i->b01f");
    const std::string win = ins.attr("window");
    auto pair_after = [&](const std::string& key, int64_t* a, int64_t* b) {
      const size_t p = win.find(key + "=");
      if (p == std::string::npos) return false;
      char* e = nullptr;
      *a = std::strtoll(win.c_str() + p + key.size() + 1, &e, 10);
      if (!e || *e != 'x') return false;
      *b = std::strtoll(e + 1, nullptr, 10);
      return true;
    };
    int64_t kh = 0, kw = 0, sh = 1, sw = 1;
    if (!pair_after("size", &kh, &kw)) return unsupported(ins, "window without a size");
    pair_after("stride", &sh, &sw);
    if (win.find("dilat") != std::string::npos || win.find("rhs_reversal") != std::string::npos)
      return unsupported(ins, "dilated or reversed convolution");
    // pad=<top>_<bottom>x<left>_<right>
    int64_t pad[4] = {0, 0, 0, 0};
    const size_t pp = win.find("pad=");
    if (pp != std::string::npos) {
      const char* s = win.c_str() + pp + 4;
      for (int i = 0; i < 4; ++i) {
        char* e = nullptr;
        pad[i] = std::strtoll(s, &e, 10);
        const char want = i == 1 ? 'x' : '_';
        if (e == s || (i < 3 && *e != want)) return unsupported(ins, "window padding is not lo_hixlo_hi");
        s = e + 1;
      }
    }
    if (kh <= 0 || kw <= 0 || sh <= 0 || sw <= 0 || pad[0] < 0 || pad[1] < 0 || pad[2] < 0 || pad[3] < 0 ||
        pad[0] >= kh || pad[1] >= kh || pad[2] >= kw || pad[3] >= kw)
      return unsupported(ins, "window geometry (padding must be smaller than the window)");
    const HloInstr& wi = e_.instrs[ins.operands[1]];
    if (!ins.shape.is_tuple() || ins.shape.elems.empty() || ins.shape.elems[0].dims.size() != 4 ||
        wi.shape.dims.size() != 4)
      return unsupported(ins, "convolution result must be a tuple whose element 0 is [B,P,Q,K]");
    const auto& od = ins.shape.elems[0].dims;
    const uint32_t O = static_cast<uint32_t>(wi.shape.dims[0]);
    const int64_t span_h = img.S + pad[0] + pad[1] - kh, span_w = img.D + pad[2] + pad[3] - kw;
    if (wi.shape.dims[1] != kh || wi.shape.dims[2] != kw || wi.shape.dims[3] != img.heads || span_h < 0 ||
        span_w < 0 || od[0] != img.B || od[1] != span_h / sh + 1 || od[2] != span_w / sw + 1 || od[3] != O)
      return unsupported(ins, "convolution shapes are inconsistent");
    const uint32_t gh = static_cast<uint32_t>(od[1]), gw = static_cast<uint32_t>(od[2]);
    const uint32_t Kw = static_cast<uint32_t>(kh * kw) * img.heads;  // elements of one window
    const uint32_t M = img.B * gh * gw, K = (Kw + 63u) / 64u * 64u;   // GEMM rows are whole 64-element k blocks
    FOp pt;
    pt.kind = OP_PATCHIFY;
    pt.name = canonical_node_name(ins.name) + "_patches";
    pt.src = img.tensor;
    pt.out = act_tensor(pt.name, M, K);
    pt.rows = M;
    pt.cols = K;
    pt.heads = img.heads;
    pt.seq = img.S;
    pt.batches = img.D;
    pt.head_dim = static_cast<uint32_t>(kh);
    pt.q_col = static_cast<uint32_t>(kw);
    pt.k_col = gw;
    pt.vocab = gh * gw;
    pt.M = static_cast<uint32_t>(sh);
    pt.N = static_cast<uint32_t>(sw);
    pt.K = Kw;
    pt.pad_top = static_cast<uint32_t>(pad[0]);
    pt.pad_left = static_cast<uint32_t>(pad[2]);
    g_.ops.push_back(pt);
    FOp o;
    o.kind = OP_GEMM;
    o.name = canonical_node_name(ins.name);
    o.a = pt.out;
    o.w = const_tensor(wv.instr, Kw, O, /*transposed=*/true);  // filter [O, kh*kw*C] is [N, K], zero-extended to K
    o.M = M;
    o.N = O;
    o.K = K;
    g_.ops.push_back(o);
    Val v;
    v.kind = Val::CONVOUT;
    v.op = static_cast<int>(g_.ops.size()) - 1;
    v.instr = idx;
    v.rows = M;
    v.cols = O;
    v.B = img.B;
    vals_[idx] = v;
    return MONONN_OK;
  }

  // tokens = concat(class rows, patches + bias) + positions  -> the f32 residual stream
  int lower_tokens(int idx, const HloComputation& c, int main_k) {
    const HloInstr& ins = e_.instrs[idx];
    const Val gv = vals_[ins.operands[main_k]];
    if (uses_[gv.instr] != 1) return unsupported(ins, "patch embedding with more than one consumer");
    FOp& gop = g_.ops[gv.op];
    const uint32_t M = gop.M, O = gop.N, B = gv.B;
    if (ins.shape.dims.size() != 2 || ins.shape.dims[1] != O || B == 0 || ins.shape.dims[0] % B)
      return unsupported(ins, "token tensor must be [B*tokens, width]");
    const uint32_t T = static_cast<uint32_t>(ins.shape.dims[0]), S = T / B, P = M / B;
    if (S <= P) return unsupported(ins, "no prefix rows in a concatenating fusion");
    const uint32_t prefix = S - P;
    std::vector<int> small;  // operands of O or prefix*O elements: bias and prefix rows
    int pos_k = -1;
    for (size_t k = 0; k < ins.operands.size(); ++k) {
      if (static_cast<int>(k) == main_k) continue;
      const HloInstr& oi = e_.instrs[ins.operands[k]];
      if (vals_[ins.operands[k]].kind != Val::CONST) return unsupported(ins, "operand %" + oi.name + " must be a constant");
      if (oi.shape.elements() == static_cast<int64_t>(S) * O && pos_k < 0) pos_k = static_cast<int>(k);
      else small.push_back(static_cast<int>(k));
    }
    if (pos_k < 0 || small.empty() || small.size() > 2)
      return unsupported(ins, "expected prefix rows, position rows and at most one bias vector");
    const bool with_bias = small.size() == 2;
    if (!with_bias) small.push_back(-1);
    Rng rng;
    std::vector<HTensor> ps = probe_inputs(c, [&](size_t, HTensor& t) {
      for (float& x : t.v) x = rng.uni(-1.f, 1.f);
    });
    HTensor got;
    int rc = probe(c, ps, &got);
    if (rc) return rc;
    int bias_k = -1, cls_k = -1;
    for (int trial = 0; trial < 2; ++trial) {
      const int bk = small[trial], ck = small[1 - trial];
      if (ck < 0 || (with_bias && bk < 0)) continue;
      if ((bk >= 0 && e_.instrs[ins.operands[bk]].shape.elements() != O) ||
          e_.instrs[ins.operands[ck]].shape.elements() != static_cast<int64_t>(prefix) * O)
        continue;
      std::vector<float> want(static_cast<size_t>(T) * O);
      for (uint32_t b = 0; b < B; ++b)
        for (uint32_t t = 0; t < S; ++t)
          for (uint32_t j = 0; j < O; ++j) {
            float y = ps[pos_k].v[static_cast<size_t>(t) * O + j];
            if (t < prefix) y += ps[ck].v[static_cast<size_t>(t) * O + j];
            else y += ps[main_k].v[(static_cast<size_t>(b) * P + (t - prefix)) * O + j] + (bk >= 0 ? ps[bk].v[j] : 0.f);
            want[(static_cast<size_t>(b) * S + t) * O + j] = y;
          }
      if (all_close(got.v, want, 1e-5f, 1e-5f)) {
        bias_k = bk;
        cls_k = ck;
        break;
      }
    }
    if (cls_k < 0)
      return unsupported(ins, "fused computation " + c.name + " is not concat(prefix, patches + bias) + positions");
    gop.out = act_tensor(gop.name + "_out", M, O);
    FTensor st;
    st.name = canonical_node_name(ins.name);
    st.kind = TKind::AccF32;
    st.rows = T;
    st.cols = O;
    st.ld = O;
    st.elem_bytes = 4;
    FOp a;
    a.kind = OP_ASSEMBLE;
    a.name = canonical_node_name(ins.name);
    a.a = gop.out;
    if (bias_k >= 0) a.bias = const_tensor(vals_[ins.operands[bias_k]].instr, 1, O);
    a.word = const_tensor(vals_[ins.operands[cls_k]].instr, prefix, O);
    a.pos = const_tensor(vals_[ins.operands[pos_k]].instr, S, O);
    a.out2 = g_.add_tensor(st);
    a.rows = T;
    a.cols = O;
    a.seq = S;
    a.k_col = prefix;
    g_.ops.push_back(a);
    Val v;
    v.kind = Val::STREAM;
    v.instr = idx;
    v.tensor = a.out2;
    v.op = static_cast<int>(g_.ops.size()) - 1;
    v.rows = T;
    v.cols = O;
    vals_[idx] = v;
    return MONONN_OK;
  }

  // additive attention mask (1 - m) * c from the integer mask argument
  int lower_mask(int idx, const HloComputation& c, int main_k) {
    const HloInstr& ins = e_.instrs[idx];
    if (ins.operands.size() != 1) return unsupported(ins, "extra operands on a mask fusion");
    const Val mv = vals_[ins.operands[main_k]];
    const HloInstr& mi = e_.instrs[ins.operands[main_k]];
    if (mi.shape.dtype != "s32" || ins.shape.dims.size() != 2) return unsupported(ins, "mask must be s32 [B,S]");
    Rng rng;
    std::vector<HTensor> zero = probe_inputs(c, [&](size_t, HTensor&) {});
    HTensor z;
    int rc = probe(c, zero, &z);
    if (rc) return rc;
    const float scale = z.v.empty() ? 0.f : z.v[0];
    std::vector<HTensor> ps = probe_inputs(c, [&](size_t, HTensor& t) {
      for (float& x : t.v) x = rng.uni(0.f, 1.f) < 0.5f ? 0.f : 1.f;
    });
    HTensor got;
    rc = probe(c, ps, &got);
    if (rc) return rc;
    std::vector<float> want(got.v.size());
    for (size_t i = 0; i < want.size(); ++i) want[i] = (1.0f - ps[0].v[i]) * scale;
    if (!all_close(got.v, want, 1e-3f, 1e-5f))
      return unsupported(ins, "fused computation " + c.name + " is not the additive mask (1 - m) * c");
    FTensor t;
    t.name = canonical_node_name(ins.name);
    t.kind = TKind::VecF32;
    t.rows = static_cast<uint32_t>(ins.shape.elements());
    t.cols = 1;
    t.elem_bytes = 4;
    Val v;
    v.kind = Val::MASK;
    v.instr = idx;
    v.tensor = g_.add_tensor(t);
    v.mask_scale = scale;
    v.mask_arg = mv.tensor;
    vals_[idx] = v;
    masks_.push_back(v);
    return MONONN_OK;
  }

  // word[ids] + position[0:S] + type[type_ids]
  int lower_embed_sum(int idx, const HloComputation& c) {
    const HloInstr& ins = e_.instrs[idx];
    // roles from the structure: gather(table param, index param), slice(position table param)
    auto param_of = [&](int i) {
      while (c.instrs[i].opcode != "parameter") {
        const std::string& o = c.instrs[i].opcode;
        if ((o == "convert" || o == "reshape" || o == "bitcast" || o == "copy") && c.instrs[i].operands.size() == 1)
          i = c.instrs[i].operands[0];
        else
          return -1;
      }
      return static_cast<int>(c.instrs[i].param_number);
    };
    std::vector<std::pair<int, int>> gathers;  // (table param, index param)
    int pos_param = -1;
    uint32_t pos_off = 0;
    for (const HloInstr& i : c.instrs) {
      if (i.opcode == "gather" && i.operands.size() == 2)
        gathers.push_back({param_of(i.operands[0]), param_of(i.operands[1])});
      if (i.opcode == "slice" && i.operands.size() == 1) {
        pos_param = param_of(i.operands[0]);
        // first row taken from the position table: slice={[a:b], [0:H]}
        const std::string sl = i.attr("slice");
        const size_t lb = sl.find('[');
        pos_off = lb == std::string::npos ? 0 : static_cast<uint32_t>(std::strtoul(sl.c_str() + lb + 1, nullptr, 10));
      }
    }
    // (no position slice: a model with relative positions, e.g. T5, gathers token rows only)
    if (gathers.empty() || gathers.size() > 2 || (pos_param < 0 && gathers.size() != 1))
      return unsupported(ins, "embedding fusion must be word gather (+ position slice) (+ type gather)");
    for (auto& gp : gathers)
      if (gp.first < 0 || gp.second < 0) return unsupported(ins, "gather operands must come from fusion parameters");
    if (ins.shape.dims.size() != 2) return unsupported(ins, "embedding sum must be [tokens, hidden]");
    const uint32_t T = static_cast<uint32_t>(ins.shape.dims[0]), H = static_cast<uint32_t>(ins.shape.dims[1]);
    const HloInstr& ids_i = e_.instrs[ins.operands[gathers[0].second]];
    if (ids_i.shape.dims.size() != 2 || ids_i.shape.elements() != T) return unsupported(ins, "ids must be [B,S]");
    const uint32_t B = static_cast<uint32_t>(ids_i.shape.dims[0]), S = static_cast<uint32_t>(ids_i.shape.dims[1]);
    // numeric check
    Rng rng;
    std::vector<HTensor> ps = probe_inputs(c, [&](size_t k, HTensor& t) {
      const HloInstr& pi = c.instrs[c.params[k]];
      if (pi.shape.dtype == "s32") {
        int64_t rows = 1;
        for (auto& gp : gathers)
          if (gp.second == static_cast<int>(k)) rows = c.instrs[c.params[gp.first]].shape.dims[0];
        for (float& x : t.v) x = std::floor(rng.uni(0.f, static_cast<float>(rows) - 0.001f));
      } else {
        for (float& x : t.v) x = rng.uni(-1.f, 1.f);
      }
    });
    HTensor got;
    int rc = probe(c, ps, &got);
    if (rc) return rc;
    std::vector<float> want(static_cast<size_t>(T) * H);
    for (uint32_t t = 0; t < T; ++t)
      for (uint32_t j = 0; j < H; ++j) {
        float y = pos_param >= 0 ? ps[pos_param].v[static_cast<size_t>(t % S + pos_off) * H + j] : 0.f;
        for (auto& gp : gathers)
          y += ps[gp.first].v[static_cast<size_t>(ps[gp.second].v[t]) * H + j];
        want[static_cast<size_t>(t) * H + j] = y;
      }
    if (!all_close(got.v, want, 1e-5f, 1e-5f))
      return unsupported(ins, "fused computation " + c.name + " is not word[ids] + position[a:a+S] + type[type_ids]");
    if (pos_param >= 0 && static_cast<int64_t>(pos_off) + S > c.instrs[c.params[pos_param]].shape.dims[0])
      return unsupported(ins, "position slice runs past the table");
    auto table = [&](int param) {
      const int instr = vals_[ins.operands[param]].instr;
      const HloInstr& ti = e_.instrs[instr];
      return const_tensor(instr, static_cast<uint32_t>(ti.shape.dims[0]), static_cast<uint32_t>(ti.shape.dims[1]));
    };
    for (int p : {gathers[0].first, pos_param})
      if (p >= 0 && vals_[ins.operands[p]].kind != Val::CONST) return unsupported(ins, "embedding tables must be constants");
    Val v;
    v.kind = Val::EMBED_SUM;
    v.instr = idx;
    v.rows = T;
    v.cols = H;
    v.B = B;
    v.S = S;
    v.ids = vals_[ins.operands[gathers[0].second]].tensor;
    v.word = table(gathers[0].first);
    v.vocab = g_.tensors[v.word].rows;
    v.pos = pos_param >= 0 ? table(pos_param) : -1;
    if (gathers.size() == 2) {
      if (vals_[ins.operands[gathers[1].first]].kind != Val::CONST) return unsupported(ins, "type table must be a constant");
      v.types = vals_[ins.operands[gathers[1].second]].tensor;
      v.type = table(gathers[1].first);
    }
    v.pos_off = pos_off;
    if (uses_[idx] != 1) {
      // No LayerNorm follows directly (pre-LN decoder): the sum itself is the residual
      // stream, materialised in f32 by an embedding stage without normalisation.
      FTensor st;
      st.name = canonical_node_name(ins.name);
      st.kind = TKind::AccF32;
      st.rows = T;
      st.cols = H;
      st.ld = H;
      st.elem_bytes = 4;
      FOp e;
      e.kind = OP_EMBED;
      e.name = canonical_node_name(ins.name);
      e.ids = v.ids;
      e.type_ids = v.types;
      e.word = v.word;
      e.pos = v.pos;
      e.type = v.type;
      e.seq = S;
      e.vocab = v.vocab;
      e.q_col = pos_off;
      e.rows = T;
      e.cols = H;
      e.out2 = g_.add_tensor(st);
      g_.ops.push_back(e);
      Val sv;
      sv.kind = Val::STREAM;
      sv.instr = idx;
      sv.tensor = e.out2;
      sv.op = static_cast<int>(g_.ops.size()) - 1;
      sv.rows = T;
      sv.cols = H;
      vals_[idx] = sv;
      return MONONN_OK;
    }
    vals_[idx] = v;
    return MONONN_OK;
  }

  // A GEMM whose result is used as it is (no epilogue fusion follows): give it an f16 output.
  int materialise_gemm(int instr) {
    Val& v = vals_[instr];
    if (v.kind != Val::GEMM) return MONONN_OK;
    FOp& gop = g_.ops[v.op];
    if (gop.out < 0) gop.out = act_tensor(gop.name, gop.M, gop.N);
    v.kind = Val::ACT;
    v.tensor = gop.out;
    v.rows = gop.M;
    v.cols = gop.N;
    return MONONN_OK;
  }

  // index of the row maximum (first index on ties): XLA's variadic (value, index) reduce
  int lower_argmax(int idx, const HloComputation& c) {
    const HloInstr& ins = e_.instrs[idx];
    int rc = materialise_gemm(ins.operands[0]);
    if (rc) return rc;
    const Val sv = vals_[ins.operands[0]];
    if (sv.kind != Val::ACT) return unsupported(ins, "arg-max over something that is not an activation");
    const uint32_t rows = sv.rows, cols = sv.cols;
    if (ins.shape.elements() != rows) return unsupported(ins, "arg-max must reduce the last dimension");
    // few distinct values, so that every row has ties and the tie-break rule is checked
    Rng rng;
    std::vector<HTensor> ps = probe_inputs(c, [&](size_t, HTensor& t) {
      for (float& x : t.v) x = std::floor(rng.uni(0.f, 7.999f)) - 4.f;
    });
    HTensor got;
    rc = probe(c, ps, &got);
    if (rc) return rc;
    for (uint32_t r = 0; r < rows; ++r) {
      uint32_t best = 0;
      for (uint32_t j = 1; j < cols; ++j)
        if (ps[0].v[static_cast<size_t>(r) * cols + j] > ps[0].v[static_cast<size_t>(r) * cols + best]) best = j;
      if (got.v[r] != static_cast<float>(best))
        return unsupported(ins, "fused computation " + c.name + " is not arg-max over the last dimension (first index on ties)");
    }
    FTensor t;
    t.name = canonical_node_name(ins.name);
    t.kind = TKind::ActF16;
    t.rows = rows;
    t.cols = 1;
    t.ld = 2;  // one s32 per row, counted in 16-bit units
    t.elem_bytes = 4;
    FOp o;
    o.kind = OP_ARGMAX;
    o.name = canonical_node_name(ins.name);
    o.src = sv.tensor;
    o.rows = rows;
    o.cols = cols;
    o.out = g_.add_tensor(t);
    g_.ops.push_back(o);
    Val v;
    v.kind = Val::ACT;
    v.instr = idx;
    v.tensor = o.out;
    v.op = static_cast<int>(g_.ops.size()) - 1;
    v.rows = rows;
    v.cols = 1;
    vals_[idx] = v;
    return MONONN_OK;
  }

  // x / sqrt(sum x^2) over the last dimension (embedding normalisation of a dual encoder)
  int lower_l2norm(int idx, const HloComputation& c) {
    const HloInstr& ins = e_.instrs[idx];
    const Val mv = vals_[ins.operands[0]];
    if (ins.shape.dims.empty()) return unsupported(ins, "scalar result");
    const uint32_t cols = static_cast<uint32_t>(ins.shape.dims.back());
    const uint32_t rows = static_cast<uint32_t>(ins.shape.elements() / cols);
    if (mv.rows != rows || mv.cols != cols) return unsupported(ins, "shape differs from the operand");
    Rng rng;
    std::vector<HTensor> ps = probe_inputs(c, [&](size_t, HTensor& t) {
      for (float& x : t.v) x = rng.uni(-1.f, 1.f);
    });
    HTensor got;
    int rc = probe(c, ps, &got);
    if (rc) return rc;
    std::vector<float> want(got.v.size());
    for (uint32_t r = 0; r < rows; ++r) {
      double sq = 0;
      for (uint32_t j = 0; j < cols; ++j) sq += static_cast<double>(ps[0].v[static_cast<size_t>(r) * cols + j]) * ps[0].v[static_cast<size_t>(r) * cols + j];
      const double inv = 1.0 / std::sqrt(sq);
      for (uint32_t j = 0; j < cols; ++j)
        want[static_cast<size_t>(r) * cols + j] = static_cast<float>(ps[0].v[static_cast<size_t>(r) * cols + j] * inv);
    }
    if (!all_close(got.v, want, 1e-5f, 1e-4f))
      return unsupported(ins, "fused computation " + c.name + " is not x / sqrt(sum x^2) over the last dimension");
    FOp n;
    n.kind = OP_LAYERNORM;
    n.name = canonical_node_name(ins.name);
    n.rows = rows;
    n.cols = cols;
    n.flags = F_L2NORM;
    if (mv.kind == Val::GEMM) {
      if (uses_[mv.instr] != 1) return unsupported(ins, "GEMM result with more than one consumer");
      FOp& gop = g_.ops[mv.op];
      FTensor acc;
      acc.name = gop.name + "_sum";
      acc.kind = TKind::AccF32;
      acc.rows = rows;
      acc.cols = cols;
      acc.ld = cols;
      acc.elem_bytes = 4;
      gop.out = g_.add_tensor(acc);
      n.src = gop.out;
      n.flags |= F_ZERO_SRC;
    } else {
      n.src = mv.tensor;
    }
    n.out = act_tensor(n.name, rows, cols);
    g_.ops.push_back(n);
    Val v;
    v.kind = Val::ACT;
    v.instr = idx;
    v.tensor = n.out;
    v.op = static_cast<int>(g_.ops.size()) - 1;
    v.rows = rows;
    v.cols = cols;
    vals_[idx] = v;
    return MONONN_OK;
  }

  // out[b, :] = x[b * S + argmax(ids[b, :]), :]: pooling at the largest token id
  int lower_rowsel(int idx, const HloComputation& c) {
    const HloInstr& ins = e_.instrs[idx];
    int x_k = -1, ids_k = -1;
    for (size_t k = 0; k < ins.operands.size(); ++k) {
      const Val& v = vals_[ins.operands[k]];
      const HloInstr& oi = e_.instrs[ins.operands[k]];
      if (v.kind == Val::ACT && x_k < 0) x_k = static_cast<int>(k);
      else if (v.kind == Val::ARG && oi.shape.dtype == "s32" && oi.shape.dims.size() == 2 && ids_k < 0)
        ids_k = static_cast<int>(k);
      else return unsupported(ins, "operand %" + oi.name + " has no role in a pooling fusion");
    }
    if (x_k < 0 || ids_k < 0 || ins.shape.dims.size() != 2) return unsupported(ins, "expected an activation and s32 [B,S] ids");
    const Val xv = vals_[ins.operands[x_k]];
    const HloInstr& ids_i = e_.instrs[ins.operands[ids_k]];
    const uint32_t B = static_cast<uint32_t>(ids_i.shape.dims[0]), S = static_cast<uint32_t>(ids_i.shape.dims[1]);
    const uint32_t H = xv.cols;
    if (xv.rows != B * S || ins.shape.dims[0] != B || ins.shape.dims[1] != H) return unsupported(ins, "shapes");
    Rng rng;
    std::vector<HTensor> ps = probe_inputs(c, [&](size_t k, HTensor& t) {
      // few distinct ids, so that ties occur and the first-maximum rule is checked
      for (float& x : t.v) x = (static_cast<int>(k) == ids_k) ? std::floor(rng.uni(0.f, 4.999f)) : rng.uni(-1.f, 1.f);
    });
    HTensor got;
    int rc = probe(c, ps, &got);
    if (rc) return rc;
    std::vector<float> want(static_cast<size_t>(B) * H);
    for (uint32_t b = 0; b < B; ++b) {
      uint32_t best = 0;
      for (uint32_t t = 1; t < S; ++t)
        if (ps[ids_k].v[static_cast<size_t>(b) * S + t] > ps[ids_k].v[static_cast<size_t>(b) * S + best]) best = t;
      for (uint32_t j = 0; j < H; ++j)
        want[static_cast<size_t>(b) * H + j] = ps[x_k].v[(static_cast<size_t>(b) * S + best) * H + j];
    }
    if (!all_close(got.v, want, 0.f, 0.f))
      return unsupported(ins, "fused computation " + c.name + " is not the row at the largest id of every sequence");
    FOp o;
    o.kind = OP_ROWSEL;
    o.name = canonical_node_name(ins.name);
    o.src = xv.tensor;
    o.ids = vals_[ins.operands[ids_k]].tensor;
    o.rows = B;
    o.cols = H;
    o.seq = S;
    o.out = act_tensor(o.name, B, H);
    g_.ops.push_back(o);
    Val v;
    v.kind = Val::ACT;
    v.instr = idx;
    v.tensor = o.out;
    v.op = static_cast<int>(g_.ops.size()) - 1;
    v.rows = B;
    v.cols = H;
    vals_[idx] = v;
    return MONONN_OK;
  }

  // activation x activation^T (both operands contract their last dimension): small SIMT product
  int lower_pairdot(int idx, float alpha, int lhs_c, int rhs_c) {
    const HloInstr& ins = e_.instrs[idx];
    const Val a = vals_[ins.operands[0]], b = vals_[ins.operands[1]];
    if (lhs_c != 1 || rhs_c != 1 || a.cols != b.cols)
      return unsupported(ins, "activation x activation GEMM must contract the last dimension of both");
    if (a.rows > 1024 || b.rows > 1024)
      return unsupported(ins, "activation x activation GEMM larger than 1024 rows a side");
    FOp o;
    o.kind = OP_PAIRDOT;
    o.name = canonical_node_name(ins.name);
    o.a = a.tensor;
    o.src = b.tensor;
    o.M = a.rows;
    o.N = b.rows;
    o.K = a.cols;
    o.alpha = alpha;
    o.out = act_tensor(o.name, a.rows, b.rows);
    g_.ops.push_back(o);
    Val v;
    v.kind = Val::ACT;
    v.instr = idx;
    v.tensor = o.out;
    v.op = static_cast<int>(g_.ops.size()) - 1;
    v.rows = a.rows;
    v.cols = b.rows;
    vals_[idx] = v;
    return MONONN_OK;
  }

  // ------------------------------------------------------------------ outputs
  int finish_outputs() {
    const HloInstr& root = e_.instrs[e_.root];
    std::vector<int> outs;
    if (root.opcode == "tuple") outs = root.operands;
    else outs.push_back(e_.root);
    const int n_params = static_cast<int>(e_.params.size());
    int ordinal = 0;
    for (int o : outs) {
      materialise_gemm(o);
      const Val& v = vals_[o];
      const HloInstr& oi = e_.instrs[o];
      if (v.kind != Val::ACT || v.op < 0)
        return unsupported(oi, "module output must be the result of a fused operator");
      ArgDesc a;
      a.name = oi.name;
      a.kind = 1;
      a.param_number = ordinal;
      a.bytes = static_cast<size_t>(oi.shape.elements()) * oi.shape.elem_bytes();
      g_.args.push_back(a);
      // the producing operator writes straight into the live-out buffer
      FTensor& t = g_.tensors[v.tensor];
      t.kind = TKind::Arg;
      t.arg_index = n_params + ordinal;
      t.name = oi.name;
      ++ordinal;
    }
    return MONONN_OK;
  }

  // The additive mask is computed by the embedding stage (same launch, stage 0).
  int attach_mask() {
    if (masks_.empty()) return MONONN_OK;
    bool used = false;
    for (const FOp& o : g_.ops)
      if (o.kind == OP_ATTENTION && o.mask >= 0) used = true;
    if (!used) return MONONN_OK;
    if (masks_.size() > 1) return fail(MONONN_ERR_UNSUPPORTED, "more than one attention-mask fusion");
    for (FOp& o : g_.ops)
      if (o.kind == OP_EMBED) {
        o.mask_in = masks_[0].mask_arg;
        o.mask_out = masks_[0].tensor;
        o.alpha = masks_[0].mask_scale;
        return MONONN_OK;
      }
    return fail(MONONN_ERR_UNSUPPORTED, "attention mask without an embedding stage to compute it in");
  }

  const HloModule& m_;
  const HloComputation& e_;
  FGraph& g_;
  std::string* err_;
  std::vector<Val> vals_;
  std::vector<int> uses_;
  std::map<std::pair<int, bool>, int> const_tensors_;
  std::vector<Val> masks_;
  std::map<int, Val> stream_of_;
  std::map<std::string, std::vector<double>> memo_;  // classification results by memo_key  // f16 LayerNorm output -> the f32 stream it was promoted to
};

}  // namespace

// A multi-output fusion returns a tuple that the entry computation takes apart with
// get-tuple-element (the reference names those pointers get_tuple_element_<cluster>_<i>,
// mononn_engine/parser/ir_parser_fused.cc:447-455, codegen/graph_codegen.cc:491-543). Each
// element is a function of some of the fusion's operands: the fusion is split into one
// single-output fusion per element (the instructions its root reaches, parameters renumbered),
// every get-tuple-element becomes that fusion, and the tuple-valued instruction is left without
// operands or users. What shares work between the elements in the original is recomputed, which
// is free here: the pieces end up as epilogues of different GEMMs or as separate row ops anyway.
static int split_multi_output_fusions(HloModule* m, std::string* err) {
  HloComputation& entry = m->comps[m->entry];
  const size_t n_entry = entry.instrs.size();
  for (size_t fi = 0; fi < n_entry; ++fi) {
    if (entry.instrs[fi].opcode != "fusion" || !entry.instrs[fi].shape.is_tuple()) continue;
    const HloComputation* cp = m->find(entry.instrs[fi].attr("calls"));
    if (!cp || cp->root < 0 || cp->instrs[cp->root].opcode != "tuple") {
      if (err) *err = "%" + entry.instrs[fi].name + ": a tuple-shaped fusion must end in a tuple instruction";
      return MONONN_ERR_UNSUPPORTED;
    }
    const HloComputation base = *cp;  // (m->comps grows below)
    const std::vector<int> elems = base.instrs[base.root].operands;
    bool used_whole = false;
    for (size_t gi = 0; gi < n_entry; ++gi) {
      HloInstr& g = entry.instrs[gi];
      bool reads = false;
      for (int o : g.operands) reads = reads || o == static_cast<int>(fi);
      if (!reads) continue;
      const auto idx = g.int_list("index");
      if (g.opcode != "get-tuple-element" || g.operands.size() != 1 || idx.size() != 1 || idx[0] < 0 ||
          idx[0] >= static_cast<int64_t>(elems.size())) {
        used_whole = true;
        continue;
      }
      const int root = elems[idx[0]];
      std::vector<char> keep(base.instrs.size(), 0);
      std::vector<int> stack{root};
      while (!stack.empty()) {
        const int i = stack.back();
        stack.pop_back();
        if (keep[i]) continue;
        keep[i] = 1;
        for (int o : base.instrs[i].operands) stack.push_back(o);
      }
      HloComputation sub;
      sub.name = base.name + "_out" + std::to_string(idx[0]);
      std::vector<int> remap(base.instrs.size(), -1);
      std::vector<int> new_operands;
      for (size_t pn = 0; pn < base.params.size(); ++pn) {  // parameters in ascending number, renumbered
        const int pi = base.params[pn];
        if (pi < 0 || !keep[pi]) continue;
        new_operands.push_back(entry.instrs[fi].operands[pn]);
      }
      int next_param = 0;
      std::map<int64_t, int64_t> renum;
      for (size_t pn = 0; pn < base.params.size(); ++pn)
        if (base.params[pn] >= 0 && keep[base.params[pn]]) renum[static_cast<int64_t>(pn)] = next_param++;
      for (size_t i = 0; i < base.instrs.size(); ++i) {
        if (!keep[i]) continue;
        HloInstr c = base.instrs[i];
        for (int& o : c.operands) o = remap[o];
        c.is_root = static_cast<int>(i) == root;
        if (c.opcode == "parameter") c.param_number = renum[c.param_number];
        remap[i] = static_cast<int>(sub.instrs.size());
        sub.index[c.name] = remap[i];
        sub.instrs.push_back(c);
      }
      sub.root = remap[root];
      sub.params.assign(static_cast<size_t>(next_param), -1);
      for (size_t i = 0; i < sub.instrs.size(); ++i)
        if (sub.instrs[i].opcode == "parameter") sub.params[static_cast<size_t>(sub.instrs[i].param_number)] = static_cast<int>(i);
      m->comp_index[sub.name] = static_cast<int>(m->comps.size());
      m->comps.push_back(sub);
      HloComputation& e2 = m->comps[m->entry];  // (the vector may have moved)
      HloInstr& g2 = e2.instrs[gi];
      g2.opcode = "fusion";
      g2.operands = new_operands;
      g2.attrs.erase("index");
      g2.attrs["calls"] = "%" + sub.name;
      g2.attrs["kind"] = e2.instrs[fi].attr("kind");
    }
    HloComputation& e2 = m->comps[m->entry];
    if (used_whole) {
      if (err) *err = "%" + e2.instrs[fi].name + ": a multi-output fusion may only be read through get-tuple-element";
      return MONONN_ERR_UNSUPPORTED;
    }
    e2.instrs[fi].opcode = "split-fusion";  // no operands, no users: skipped by the lowering
    e2.instrs[fi].operands.clear();
    return split_multi_output_fusions(m, err);  // references were invalidated: start over for the next one
  }
  return MONONN_OK;
}

int hlo_text_to_fgraph(const std::string& text, FGraph* graph, std::string* err) {
  HloModule m;
  int rc = parse_hlo_text(text, &m, err);
  if (rc) return rc;
  rc = split_multi_output_fusions(&m, err);
  if (rc) return rc;
  Lowering l(m, graph, err);
  return l.run();
}

}  // namespace mononn
