// Compile-time fp32 evaluator for fused HLO computations (see hlo_interp.h).
#include "hlo_interp.h"

#include <algorithm>
#include <cmath>
#include <functional>
#include <map>

#include "../../include/mononn.h"

namespace mononn {

namespace {

std::vector<int64_t> strides_of(const std::vector<int64_t>& dims) {
  std::vector<int64_t> s(dims.size(), 1);
  for (int i = static_cast<int>(dims.size()) - 2; i >= 0; --i) s[i] = s[i + 1] * dims[i + 1];
  return s;
}

bool default_layout(const HloShape& s) {
  const int r = static_cast<int>(s.dims.size());
  if (static_cast<int>(s.minor_to_major.size()) != r) return true;
  for (int i = 0; i < r; ++i)
    if (s.minor_to_major[i] != r - 1 - i) return false;
  return true;
}

int unsupported(std::string* err, const HloInstr& ins, const std::string& why) {
  if (err) *err = "%" + ins.name + " (" + ins.opcode + ", HLO line " + std::to_string(ins.line) + "): " + why;
  return MONONN_ERR_UNSUPPORTED;
}

float round_to_dtype(float x, const std::string& dtype) {
  if (dtype == "s32" || dtype == "s64" || dtype == "s8" || dtype == "s16" || dtype == "u8" ||
      dtype == "u32" || dtype == "u64" || dtype == "u16")
    return std::trunc(x);
  if (dtype == "pred") return x != 0.f ? 1.f : 0.f;
  return x;  // f16 / f32: the evaluator works in fp32 throughout
}

// A reduction's to_apply computation compiled to a straight-line program over scalars, for
// combiners that are more than one operator (the (value, index) comparator of an arg-max:
// codegen/reduction_functor_generator.cc:296-441 supports add/max/min/and/select/compare/
// tuple/get-tuple-element there).
struct ScalarProgram {
  enum Code { PARAM, CONST, ADD, SUB, MUL, MAX, MIN, AND, OR, NOT, SELECT, EQ, NE, LT, LE, GT, GE, COPY };
  struct Step { Code code; int a, b, c; float k; };
  std::vector<Step> steps;
  std::vector<int> results;  // step index of each result element
  mutable std::vector<float> reg;

  static bool compile(const HloComputation& f, ScalarProgram* p, std::string* why) {
    p->steps.clear();
    p->results.clear();
    for (const HloInstr& i : f.instrs) {
      Step st{COPY, i.operands.size() > 0 ? i.operands[0] : -1, i.operands.size() > 1 ? i.operands[1] : -1,
              i.operands.size() > 2 ? i.operands[2] : -1, 0.f};
      const std::string& o = i.opcode;
      if (o == "parameter") { st.code = PARAM; st.a = static_cast<int>(i.param_number); }
      else if (o == "constant" && i.literal_is_scalar) { st.code = CONST; st.k = static_cast<float>(i.literal); }
      else if (o == "add") st.code = ADD;
      else if (o == "subtract") st.code = SUB;
      else if (o == "multiply") st.code = MUL;
      else if (o == "maximum") st.code = MAX;
      else if (o == "minimum") st.code = MIN;
      else if (o == "and") st.code = AND;
      else if (o == "or") st.code = OR;
      else if (o == "not") st.code = NOT;
      else if (o == "select") st.code = SELECT;
      else if (o == "convert" || o == "copy" || o == "bitcast") st.code = COPY;
      else if (o == "compare") {
        const std::string d = i.attr("direction");
        if (d == "EQ") st.code = EQ; else if (d == "NE") st.code = NE; else if (d == "LT") st.code = LT;
        else if (d == "LE") st.code = LE; else if (d == "GT") st.code = GT; else if (d == "GE") st.code = GE;
        else { *why = "comparison direction " + d; return false; }
      } else if (o == "tuple") {
        st.code = COPY;  // value unused; elements recorded below
        st.a = i.operands.empty() ? -1 : i.operands[0];
      } else { *why = "operator " + o + " in a reduction combiner"; return false; }
      p->steps.push_back(st);
    }
    if (f.root < 0) { *why = "combiner without a root"; return false; }
    const HloInstr& root = f.instrs[f.root];
    if (root.opcode == "tuple") p->results = root.operands;
    else p->results.push_back(f.root);
    p->reg.assign(p->steps.size(), 0.f);
    return true;
  }
  // args: accumulators then new elements (XLA's reducer signature); out: one per result
  void run(const float* args, float* out) const {
    float* r = reg.data();
    for (size_t i = 0; i < steps.size(); ++i) {
      const Step& s = steps[i];
      switch (s.code) {
        case PARAM: r[i] = args[s.a]; break;
        case CONST: r[i] = s.k; break;
        case ADD: r[i] = r[s.a] + r[s.b]; break;
        case SUB: r[i] = r[s.a] - r[s.b]; break;
        case MUL: r[i] = r[s.a] * r[s.b]; break;
        case MAX: r[i] = std::max(r[s.a], r[s.b]); break;
        case MIN: r[i] = std::min(r[s.a], r[s.b]); break;
        case AND: r[i] = (r[s.a] != 0.f && r[s.b] != 0.f) ? 1.f : 0.f; break;
        case OR: r[i] = (r[s.a] != 0.f || r[s.b] != 0.f) ? 1.f : 0.f; break;
        case NOT: r[i] = r[s.a] != 0.f ? 0.f : 1.f; break;
        case SELECT: r[i] = r[s.a] != 0.f ? r[s.b] : r[s.c]; break;
        case EQ: r[i] = r[s.a] == r[s.b] ? 1.f : 0.f; break;
        case NE: r[i] = r[s.a] != r[s.b] ? 1.f : 0.f; break;
        case LT: r[i] = r[s.a] < r[s.b] ? 1.f : 0.f; break;
        case LE: r[i] = r[s.a] <= r[s.b] ? 1.f : 0.f; break;
        case GT: r[i] = r[s.a] > r[s.b] ? 1.f : 0.f; break;
        case GE: r[i] = r[s.a] >= r[s.b] ? 1.f : 0.f; break;
        case COPY: r[i] = s.a >= 0 ? r[s.a] : 0.f; break;
      }
    }
    for (size_t k = 0; k < results.size(); ++k) out[k] = r[results[k]];
  }
};

}  // namespace

int eval_computation(const HloModule& m, const HloComputation& comp,
                     const std::vector<HTensor>& params, HTensor* out, std::string* err) {
  std::vector<HTensor> val(comp.instrs.size());
  std::map<int, std::vector<HTensor>> tuples;  // results of variadic reduces
  // last use, to free intermediates of large fusions early
  std::vector<int> last_use(comp.instrs.size(), -1);
  for (size_t i = 0; i < comp.instrs.size(); ++i)
    for (int o : comp.instrs[i].operands) last_use[o] = static_cast<int>(i);

  for (size_t idx = 0; idx < comp.instrs.size(); ++idx) {
    const HloInstr& ins = comp.instrs[idx];
    const std::string& op = ins.opcode;
    if (ins.shape.is_tuple()) {
      // Variadic reduce over one dimension: N inputs, N init values, N results.
      if (op != "reduce" || ins.operands.size() < 4 || ins.operands.size() % 2 != 0)
        return unsupported(err, ins, "tuple-shaped value inside a fusion");
      const size_t N = ins.operands.size() / 2;
      const std::vector<int64_t> rd = ins.int_list("dimensions");
      const HloComputation* f = m.find(ins.attr("to_apply"));
      if (rd.size() != 1 || !f || ins.shape.elems.size() != N)
        return unsupported(err, ins, "variadic reduce must reduce one dimension with a known combiner");
      ScalarProgram prog;
      std::string why;
      if (!ScalarProgram::compile(*f, &prog, &why)) return unsupported(err, ins, why);
      if (f->params.size() != 2 * N || prog.results.size() != N)
        return unsupported(err, ins, "combiner signature does not match the reduce");
      const HTensor& a0 = val[ins.operands[0]];
      const int64_t d = rd[0];
      if (d < 0 || d >= static_cast<int64_t>(a0.dims.size())) return unsupported(err, ins, "bad dimension");
      const auto as = strides_of(a0.dims);
      const int64_t len = a0.dims[d], inner = as[d], outer = a0.size() / (len * inner);
      std::vector<HTensor> res(N);
      for (size_t k = 0; k < N; ++k) {
        if (val[ins.operands[k]].size() != a0.size() || val[ins.operands[N + k]].size() != 1)
          return unsupported(err, ins, "variadic reduce operand shapes differ");
        res[k].dims = ins.shape.elems[k].dims;
        if (res[k].size() != outer * inner) return unsupported(err, ins, "result shape mismatch");
        res[k].v.resize(static_cast<size_t>(outer * inner));
      }
      std::vector<float> args(2 * N), acc(N);
      for (int64_t o = 0; o < outer; ++o)
        for (int64_t in = 0; in < inner; ++in) {
          for (size_t k = 0; k < N; ++k) acc[k] = val[ins.operands[N + k]].v[0];
          for (int64_t e = 0; e < len; ++e) {
            for (size_t k = 0; k < N; ++k) {
              args[k] = acc[k];
              args[N + k] = val[ins.operands[k]].v[(o * len + e) * inner + in];
            }
            prog.run(args.data(), acc.data());
          }
          for (size_t k = 0; k < N; ++k) res[k].v[o * inner + in] = acc[k];
        }
      tuples[static_cast<int>(idx)] = std::move(res);
      continue;
    }
    if (op == "get-tuple-element") {
      const auto gi = ins.int_list("index");
      auto it = ins.operands.size() == 1 ? tuples.find(ins.operands[0]) : tuples.end();
      if (it == tuples.end() || gi.size() != 1 || gi[0] < 0 || gi[0] >= static_cast<int64_t>(it->second.size()))
        return unsupported(err, ins, "get-tuple-element of something that is not a variadic reduce");
      val[idx] = it->second[gi[0]];
      continue;
    }
    if (!default_layout(ins.shape))
      return unsupported(err, ins, "non-default (not row-major) layout");
    HTensor r;
    r.dims = ins.shape.dims;
    const int64_t n = r.size();
    auto A = [&](int k) -> const HTensor& { return val[ins.operands[k]]; };
    auto need = [&](size_t k) { return ins.operands.size() == k; };

    if (op == "parameter") {
      if (ins.param_number < 0 || ins.param_number >= static_cast<int64_t>(params.size()))
        return unsupported(err, ins, "parameter number out of range");
      r = params[ins.param_number];
      if (r.size() != n) return unsupported(err, ins, "probe tensor does not match the parameter shape");
      r.dims = ins.shape.dims;
    } else if (op == "constant") {
      if (!ins.literal_is_scalar || n != 1)
        return unsupported(err, ins, "non-scalar constant inside a fusion");
      r.v.assign(1, static_cast<float>(ins.literal));
    } else if (op == "convert" || op == "copy" || op == "bitcast" || op == "reshape" ||
               op == "bitcast-convert") {
      if (!need(1)) return unsupported(err, ins, "expects one operand");
      if (A(0).size() != n) return unsupported(err, ins, "element count changes");
      r.v = A(0).v;
      if (op == "convert")
        for (float& x : r.v) x = round_to_dtype(x, ins.shape.dtype);
    } else if (op == "broadcast") {
      if (!need(1)) return unsupported(err, ins, "expects one operand");
      const std::vector<int64_t> bd = ins.int_list("dimensions");
      const HTensor& a = A(0);
      if (bd.size() != a.dims.size()) return unsupported(err, ins, "dimensions do not match operand rank");
      const auto os = strides_of(r.dims), as = strides_of(a.dims);
      r.v.resize(static_cast<size_t>(n));
      for (int64_t i = 0; i < n; ++i) {
        int64_t src = 0;
        for (size_t k = 0; k < bd.size(); ++k) src += ((i / os[bd[k]]) % r.dims[bd[k]]) * as[k];
        r.v[i] = a.v[src];
      }
    } else if (op == "transpose") {
      if (!need(1)) return unsupported(err, ins, "expects one operand");
      const std::vector<int64_t> perm = ins.int_list("dimensions");
      const HTensor& a = A(0);
      if (perm.size() != a.dims.size()) return unsupported(err, ins, "bad permutation");
      const auto os = strides_of(r.dims), as = strides_of(a.dims);
      r.v.resize(static_cast<size_t>(n));
      for (int64_t i = 0; i < n; ++i) {
        int64_t src = 0;
        for (size_t k = 0; k < perm.size(); ++k) src += ((i / os[k]) % r.dims[k]) * as[perm[k]];
        r.v[i] = a.v[src];
      }
    } else if (op == "slice") {
      if (!need(1)) return unsupported(err, ins, "expects one operand");
      // slice={[a:b], [c:d]} or with strides [a:b:s]
      const std::string s = ins.attr("slice");
      std::vector<int64_t> start, stride;
      size_t p = 0;
      while ((p = s.find('[', p)) != std::string::npos) {
        const size_t e = s.find(']', p);
        if (e == std::string::npos) break;
        const std::string part = s.substr(p + 1, e - p - 1);
        const size_t c1 = part.find(':');
        const size_t c2 = c1 == std::string::npos ? std::string::npos : part.find(':', c1 + 1);
        start.push_back(std::strtoll(part.c_str(), nullptr, 10));
        stride.push_back(c2 == std::string::npos ? 1 : std::strtoll(part.c_str() + c2 + 1, nullptr, 10));
        p = e + 1;
      }
      const HTensor& a = A(0);
      if (start.size() != a.dims.size()) return unsupported(err, ins, "slice rank mismatch");
      for (int64_t st : stride)
        if (st != 1) return unsupported(err, ins, "slice stride must be 1");  // ir_parser_fused.cc:1321-1327
      const auto os = strides_of(r.dims), as = strides_of(a.dims);
      r.v.resize(static_cast<size_t>(n));
      for (int64_t i = 0; i < n; ++i) {
        int64_t src = 0;
        for (size_t k = 0; k < start.size(); ++k) src += ((i / os[k]) % r.dims[k] + start[k]) * as[k];
        r.v[i] = a.v[src];
      }
    } else if (op == "pad") {
      // padding=lo_hi[_interior] per dimension joined by 'x'; no interior padding and no negative
      // edges (mononn_engine/parser/ir_parser_fused.cc:1143-1151); out-of-range reads give the
      // pad value (index_tracer.cc:368-401)
      if (!need(2) || A(1).size() != 1) return unsupported(err, ins, "expects an operand and a scalar pad value");
      const std::string ps = ins.attr("padding");
      std::vector<int64_t> lo;
      size_t p = 0;
      while (p < ps.size()) {
        const size_t e = ps.find('x', p);
        const std::string part = ps.substr(p, e == std::string::npos ? std::string::npos : e - p);
        char* q = nullptr;
        const long long l = std::strtoll(part.c_str(), &q, 10);
        const long long h = (q && *q == '_') ? std::strtoll(q + 1, &q, 10) : 0;
        const long long in = (q && *q == '_') ? std::strtoll(q + 1, &q, 10) : 0;
        if (l < 0 || h < 0 || in != 0) return unsupported(err, ins, "interior or negative padding");
        lo.push_back(l);
        if (e == std::string::npos) break;
        p = e + 1;
      }
      const HTensor& a = A(0);
      if (lo.size() != a.dims.size() || r.dims.size() != a.dims.size()) return unsupported(err, ins, "pad rank mismatch");
      const auto os = strides_of(r.dims), as = strides_of(a.dims);
      r.v.assign(static_cast<size_t>(n), A(1).v[0]);
      for (int64_t i = 0; i < a.size(); ++i) {
        int64_t dst = 0;
        for (size_t k = 0; k < a.dims.size(); ++k) dst += ((i / as[k]) % a.dims[k] + lo[k]) * os[k];
        if (dst >= n) return unsupported(err, ins, "padded extent smaller than the operand");
        r.v[dst] = a.v[i];
      }
    } else if (op == "dynamic-slice") {
      // operand, then one scalar start index per dimension, clamped to [0, dim - size]
      // (mononn_engine/core/context/index_tracer.cc:142-148)
      if (ins.operands.empty()) return unsupported(err, ins, "expects operands");
      const HTensor& a = A(0);
      const auto sizes = ins.int_list("dynamic_slice_sizes");
      if (ins.operands.size() != 1 + a.dims.size() || sizes.size() != a.dims.size() || r.dims.size() != a.dims.size())
        return unsupported(err, ins, "one start index per dimension is expected");
      std::vector<int64_t> start(a.dims.size());
      for (size_t k = 0; k < a.dims.size(); ++k) {
        if (A(static_cast<int>(k) + 1).size() != 1 || sizes[k] != r.dims[k] || sizes[k] > a.dims[k])
          return unsupported(err, ins, "start indices must be scalars and sizes must match the result");
        const int64_t st = static_cast<int64_t>(A(static_cast<int>(k) + 1).v[0]);
        start[k] = std::min(std::max<int64_t>(st, 0), a.dims[k] - sizes[k]);
      }
      const auto os = strides_of(r.dims), as = strides_of(a.dims);
      r.v.resize(static_cast<size_t>(n));
      for (int64_t i = 0; i < n; ++i) {
        int64_t src = 0;
        for (size_t k = 0; k < start.size(); ++k) src += ((i / os[k]) % r.dims[k] + start[k]) * as[k];
        r.v[i] = a.v[src];
      }
    } else if (op == "gather") {
      // Row lookup only (embedding): operand [V, H], indices [...] ->  [..., H]; the gathered
      // index is not clamped (mononn_engine/core/context/index_tracer.cc:235-280).
      if (!need(2)) return unsupported(err, ins, "expects two operands");
      const HTensor& table = A(0);
      const HTensor& ids = A(1);
      const auto off = ins.int_list("offset_dims"), col = ins.int_list("collapsed_slice_dims"),
                 sim = ins.int_list("start_index_map"), ss = ins.int_list("slice_sizes");
      const auto ivd = ins.int_list("index_vector_dim");
      if (table.dims.size() != 2 || off.size() != 1 || off[0] != static_cast<int64_t>(r.dims.size()) - 1 ||
          col.size() != 1 || col[0] != 0 || sim.size() != 1 || sim[0] != 0 || ss.size() != 2 ||
          ss[0] != 1 || ss[1] != table.dims[1] || ivd.size() != 1 ||
          ivd[0] != static_cast<int64_t>(ids.dims.size()) || ids.size() * table.dims[1] != n)
        return unsupported(err, ins, "only the row-lookup (embedding) form of gather is supported");
      const int64_t h = table.dims[1];
      r.v.resize(static_cast<size_t>(n));
      for (int64_t t = 0; t < ids.size(); ++t) {
        const int64_t row = static_cast<int64_t>(ids.v[t]);
        if (row < 0 || row >= table.dims[0]) return unsupported(err, ins, "probe index out of range");
        std::copy(table.v.begin() + row * h, table.v.begin() + (row + 1) * h, r.v.begin() + t * h);
      }
    } else if (op == "concatenate") {
      const auto cd = ins.int_list("dimensions");
      if (cd.size() != 1 || cd[0] < 0 || cd[0] >= static_cast<int64_t>(r.dims.size()))
        return unsupported(err, ins, "bad concatenate dimension");
      const int64_t d = cd[0];
      const auto os = strides_of(r.dims);
      r.v.resize(static_cast<size_t>(n));
      int64_t offset = 0;
      for (size_t k = 0; k < ins.operands.size(); ++k) {
        const HTensor& a = A(static_cast<int>(k));
        if (a.dims.size() != r.dims.size()) return unsupported(err, ins, "operand rank differs");
        const auto as = strides_of(a.dims);
        for (int64_t i = 0; i < a.size(); ++i) {
          int64_t dst = 0;
          for (size_t q = 0; q < a.dims.size(); ++q) {
            const int64_t c = (i / as[q]) % a.dims[q];
            dst += (static_cast<int64_t>(q) == d ? c + offset : c) * os[q];
          }
          r.v[dst] = a.v[i];
        }
        offset += a.dims[d];
      }
      if (offset != r.dims[d]) return unsupported(err, ins, "concatenated extent mismatch");
    } else if (op == "iota") {
      const auto d = ins.int_list("iota_dimension");
      if (d.size() != 1 || d[0] < 0 || d[0] >= static_cast<int64_t>(r.dims.size()))
        return unsupported(err, ins, "bad iota_dimension");
      const auto os = strides_of(r.dims);
      r.v.resize(static_cast<size_t>(n));
      for (int64_t i = 0; i < n; ++i) r.v[i] = static_cast<float>((i / os[d[0]]) % r.dims[d[0]]);
    } else if (op == "reduce") {
      if (!need(2)) return unsupported(err, ins, "variadic reduce is not supported here");
      const HTensor& a = A(0);
      const HTensor& init = A(1);
      const std::vector<int64_t> rd = ins.int_list("dimensions");
      if (rd.size() != 1) return unsupported(err, ins, "exactly one reduced dimension is supported");  // ir_parser_fused.cc:1169-1213
      const HloComputation* f = m.find(ins.attr("to_apply"));
      if (!f || f->root < 0) return unsupported(err, ins, "to_apply computation not found");
      const std::string fop = f->instrs[f->root].opcode;
      std::function<float(float, float)> comb;
      if (fop == "add") comb = [](float x, float y) { return x + y; };
      else if (fop == "maximum") comb = [](float x, float y) { return std::max(x, y); };
      else if (fop == "minimum") comb = [](float x, float y) { return std::min(x, y); };
      else if (fop == "multiply") comb = [](float x, float y) { return x * y; };
      else if (fop == "and") comb = [](float x, float y) { return (x != 0.f && y != 0.f) ? 1.f : 0.f; };
      else if (fop == "or") comb = [](float x, float y) { return (x != 0.f || y != 0.f) ? 1.f : 0.f; };
      else return unsupported(err, ins, "reduction combiner " + fop + " is not supported");
      const int64_t d = rd[0];
      if (d < 0 || d >= static_cast<int64_t>(a.dims.size())) return unsupported(err, ins, "bad dimension");
      const auto as = strides_of(a.dims);
      const int64_t len = a.dims[d], inner = as[d], outer = a.size() / (len * inner);
      if (outer * inner != n) return unsupported(err, ins, "result shape mismatch");
      // ±inf init values become the dtype limits in the reference (ir_parser_fused.cc:154-211);
      // with fp32 evaluation the infinities behave identically for max/min
      r.v.resize(static_cast<size_t>(n));
      for (int64_t o = 0; o < outer; ++o)
        for (int64_t in = 0; in < inner; ++in) {
          float acc = init.v[0];
          const float* p = a.v.data() + o * len * inner + in;
          for (int64_t k = 0; k < len; ++k) acc = comb(acc, p[k * inner]);
          r.v[o * inner + in] = acc;
        }
    } else if (op == "select") {
      if (!need(3)) return unsupported(err, ins, "expects three operands");
      r.v.resize(static_cast<size_t>(n));
      const bool scalar_pred = A(0).size() == 1;
      for (int64_t i = 0; i < n; ++i) r.v[i] = (A(0).v[scalar_pred ? 0 : i] != 0.f) ? A(1).v[i] : A(2).v[i];
    } else if (op == "clamp") {
      if (!need(3)) return unsupported(err, ins, "expects three operands");
      r.v.resize(static_cast<size_t>(n));
      const bool s0 = A(0).size() == 1, s2 = A(2).size() == 1;
      for (int64_t i = 0; i < n; ++i)
        r.v[i] = std::min(std::max(A(1).v[i], A(0).v[s0 ? 0 : i]), A(2).v[s2 ? 0 : i]);
    } else if (op == "compare") {
      if (!need(2)) return unsupported(err, ins, "expects two operands");
      const std::string dir = ins.attr("direction");
      r.v.resize(static_cast<size_t>(n));
      for (int64_t i = 0; i < n; ++i) {
        const float x = A(0).v[i], y = A(1).v[i];
        bool b;
        if (dir == "EQ") b = x == y;
        else if (dir == "NE") b = x != y;
        else if (dir == "LT") b = x < y;
        else if (dir == "LE") b = x <= y;
        else if (dir == "GT") b = x > y;
        else if (dir == "GE") b = x >= y;
        else return unsupported(err, ins, "unknown comparison direction " + dir);
        r.v[i] = b ? 1.f : 0.f;
      }
    } else if (ins.operands.size() == 2 &&
               (op == "add" || op == "subtract" || op == "multiply" || op == "divide" || op == "maximum" ||
                op == "minimum" || op == "power" || op == "and" || op == "or")) {
      if (A(0).size() != n || A(1).size() != n) return unsupported(err, ins, "operand shapes differ");
      r.v.resize(static_cast<size_t>(n));
      const float* x = A(0).v.data();
      const float* y = A(1).v.data();
      for (int64_t i = 0; i < n; ++i) {
        float z;
        if (op == "add") z = x[i] + y[i];
        else if (op == "subtract") z = x[i] - y[i];
        else if (op == "multiply") z = x[i] * y[i];
        else if (op == "divide") z = x[i] / y[i];
        else if (op == "maximum") z = std::max(x[i], y[i]);
        else if (op == "minimum") z = std::min(x[i], y[i]);
        else if (op == "power") z = std::pow(x[i], y[i]);
        else if (op == "and") z = (x[i] != 0.f && y[i] != 0.f) ? 1.f : 0.f;
        else z = (x[i] != 0.f || y[i] != 0.f) ? 1.f : 0.f;
        r.v[i] = z;
      }
    } else if (ins.operands.size() == 1 &&
               (op == "exponential" || op == "log" || op == "tanh" || op == "rsqrt" || op == "sqrt" ||
                op == "negate" || op == "abs" || op == "sign" || op == "erf" || op == "logistic" ||
                op == "not" || op == "floor" || op == "ceil")) {
      if (A(0).size() != n) return unsupported(err, ins, "operand shape differs");
      r.v.resize(static_cast<size_t>(n));
      const float* x = A(0).v.data();
      for (int64_t i = 0; i < n; ++i) {
        float z;
        if (op == "exponential") z = std::exp(x[i]);
        else if (op == "log") z = std::log(x[i]);
        else if (op == "tanh") z = std::tanh(x[i]);
        else if (op == "rsqrt") z = 1.0f / std::sqrt(x[i]);
        else if (op == "sqrt") z = std::sqrt(x[i]);
        else if (op == "negate") z = -x[i];
        else if (op == "abs") z = std::fabs(x[i]);
        else if (op == "sign") z = static_cast<float>((x[i] > 0.f) - (x[i] < 0.f));
        else if (op == "erf") z = std::erf(x[i]);
        else if (op == "logistic") z = 1.0f / (1.0f + std::exp(-x[i]));
        else if (op == "not") z = x[i] != 0.f ? 0.f : 1.f;
        else if (op == "floor") z = std::floor(x[i]);
        else z = std::ceil(x[i]);
        r.v[i] = z;
      }
    } else {
      return unsupported(err, ins, "operator is outside the supported set");
    }
    val[idx] = std::move(r);
    for (int o : ins.operands)
      if (last_use[o] == static_cast<int>(idx) && o != comp.root) {
        val[o].v.clear();
        val[o].v.shrink_to_fit();
      }
  }
  *out = std::move(val[comp.root]);
  return MONONN_OK;
}

}  // namespace mononn
