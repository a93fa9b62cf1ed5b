// XLA HLO text parser (see hlo_parser.h).
#include "hlo_parser.h"

#include <cctype>
#include <cmath>
#include <cstdlib>
#include <sstream>

#include "../../include/mononn.h"

namespace mononn {

int HloShape::elem_bytes() const {
  if (dtype == "pred" || dtype == "s8" || dtype == "u8") return 1;
  if (dtype == "s16" || dtype == "u16" || dtype == "f16" || dtype == "bf16") return 2;
  if (dtype == "s32" || dtype == "u32" || dtype == "f32") return 4;
  if (dtype == "s64" || dtype == "u64" || dtype == "f64") return 8;
  return 0;
}

std::string HloShape::str() const {
  std::ostringstream o;
  if (is_tuple()) {
    o << "(";
    for (size_t i = 0; i < elems.size(); ++i) o << (i ? ", " : "") << elems[i].str();
    o << ")";
    return o.str();
  }
  o << dtype << "[";
  for (size_t i = 0; i < dims.size(); ++i) o << (i ? "," : "") << dims[i];
  o << "]";
  return o.str();
}

std::vector<int64_t> HloInstr::int_list(const std::string& key) const {
  std::vector<int64_t> out;
  auto it = attrs.find(key);
  if (it == attrs.end()) return out;
  const std::string& s = it->second;
  size_t i = 0;
  while (i < s.size()) {
    if (std::isdigit(static_cast<unsigned char>(s[i])) || (s[i] == '-' && i + 1 < s.size() &&
                                                            std::isdigit(static_cast<unsigned char>(s[i + 1])))) {
      char* e = nullptr;
      out.push_back(std::strtoll(s.c_str() + i, &e, 10));
      i = static_cast<size_t>(e - s.c_str());
    } else {
      ++i;
    }
  }
  return out;
}

std::string canonical_node_name(const std::string& name) {
  std::string v = name;
  for (char& c : v)
    if (c == '.' || c == '-') c = '_';
  return v;
}

namespace {

struct Cursor {
  const std::string& s;
  size_t i;
  int line;
  std::string* err;
  bool fail(const std::string& m) {
    if (err) *err = "HLO line " + std::to_string(line) + ": " + m;
    return false;
  }
  void ws() {
    while (i < s.size() && (s[i] == ' ' || s[i] == '\t')) ++i;
  }
  bool eat(char c) {
    ws();
    if (i < s.size() && s[i] == c) {
      ++i;
      return true;
    }
    return false;
  }
};

std::string trim(const std::string& s) {
  size_t a = 0, b = s.size();
  while (a < b && std::isspace(static_cast<unsigned char>(s[a]))) ++a;
  while (b > a && std::isspace(static_cast<unsigned char>(s[b - 1]))) --b;
  return s.substr(a, b - a);
}

bool parse_shape(Cursor& c, HloShape* out) {
  c.ws();
  *out = HloShape();
  if (c.i < c.s.size() && c.s[c.i] == '(') {
    ++c.i;
    c.ws();
    if (c.eat(')')) return true;
    for (;;) {
      HloShape e;
      if (!parse_shape(c, &e)) return false;
      out->elems.push_back(e);
      if (c.eat(',')) continue;
      if (c.eat(')')) return true;
      return c.fail("expected ',' or ')' in tuple shape");
    }
  }
  size_t a = c.i;
  while (c.i < c.s.size() && std::isalnum(static_cast<unsigned char>(c.s[c.i]))) ++c.i;
  out->dtype = c.s.substr(a, c.i - a);
  if (out->dtype.empty() || c.i >= c.s.size() || c.s[c.i] != '[')
    return c.fail("expected a shape like f16[128,768]");
  ++c.i;
  while (c.i < c.s.size() && c.s[c.i] != ']') {
    if (std::isdigit(static_cast<unsigned char>(c.s[c.i]))) {
      char* e = nullptr;
      out->dims.push_back(std::strtoll(c.s.c_str() + c.i, &e, 10));
      c.i = static_cast<size_t>(e - c.s.c_str());
    } else if (c.s[c.i] == ',' || c.s[c.i] == ' ') {
      ++c.i;
    } else {
      return c.fail("dynamic or malformed dimension in shape (only static shapes are supported)");
    }
  }
  if (c.i >= c.s.size()) return c.fail("unterminated shape");
  ++c.i;  // ]
  if (c.i < c.s.size() && c.s[c.i] == '{') {
    size_t close = c.s.find('}', c.i);
    if (close == std::string::npos) return c.fail("unterminated layout");
    std::string lay = c.s.substr(c.i + 1, close - c.i - 1);
    const size_t colon = lay.find(':');  // tiling / memory space annotations are ignored
    if (colon != std::string::npos) lay = lay.substr(0, colon);
    size_t k = 0;
    while (k < lay.size()) {
      if (std::isdigit(static_cast<unsigned char>(lay[k]))) {
        char* e = nullptr;
        out->minor_to_major.push_back(static_cast<int>(std::strtol(lay.c_str() + k, &e, 10)));
        k = static_cast<size_t>(e - lay.c_str());
      } else {
        ++k;
      }
    }
    c.i = close + 1;
  }
  if (out->minor_to_major.empty())
    for (int d = static_cast<int>(out->dims.size()) - 1; d >= 0; --d) out->minor_to_major.push_back(d);
  return true;
}

// Splits s at top-level commas (outside (), {}, [], "").
std::vector<std::string> split_top(const std::string& s) {
  std::vector<std::string> out;
  int depth = 0;
  bool quote = false;
  std::string cur;
  for (size_t i = 0; i < s.size(); ++i) {
    const char ch = s[i];
    if (quote) {
      cur.push_back(ch);
      if (ch == '\\' && i + 1 < s.size()) cur.push_back(s[++i]);
      else if (ch == '"') quote = false;
      continue;
    }
    if (ch == '"') quote = true;
    if (ch == '(' || ch == '{' || ch == '[') ++depth;
    if (ch == ')' || ch == '}' || ch == ']') --depth;
    if (ch == ',' && depth == 0) {
      out.push_back(trim(cur));
      cur.clear();
    } else {
      cur.push_back(ch);
    }
  }
  if (!trim(cur).empty()) out.push_back(trim(cur));
  return out;
}

// Position of the ')' matching the '(' at `open`.
size_t match_paren(const std::string& s, size_t open) {
  int depth = 0;
  bool quote = false;
  for (size_t i = open; i < s.size(); ++i) {
    const char ch = s[i];
    if (quote) {
      if (ch == '\\') ++i;
      else if (ch == '"') quote = false;
      continue;
    }
    if (ch == '"') quote = true;
    else if (ch == '(' || ch == '{' || ch == '[') ++depth;
    else if (ch == ')' || ch == '}' || ch == ']') {
      --depth;
      if (depth == 0) return i;
    }
  }
  return std::string::npos;
}

std::string unquote(const std::string& v) {
  if (v.size() < 2 || v.front() != '"' || v.back() != '"') return v;
  std::string out;
  for (size_t i = 1; i + 1 < v.size(); ++i) {
    if (v[i] == '\\' && i + 2 < v.size()) {
      ++i;
      out.push_back(v[i] == 'n' ? '\n' : v[i]);
    } else {
      out.push_back(v[i]);
    }
  }
  return out;
}

bool parse_scalar_literal(const std::string& text, double* v) {
  const std::string t = trim(text);
  if (t.empty() || t[0] == '{') return false;
  if (t == "inf" || t == "+inf") { *v = INFINITY; return true; }
  if (t == "-inf") { *v = -INFINITY; return true; }
  if (t == "nan" || t == "-nan") { *v = NAN; return true; }
  if (t == "true") { *v = 1; return true; }
  if (t == "false") { *v = 0; return true; }
  char* e = nullptr;
  const double d = std::strtod(t.c_str(), &e);
  if (e == t.c_str() || *e != '\0') return false;
  *v = d;
  return true;
}

// "{ {1, 2}, /*i0=1*/ {3, inf} }" -> 1 2 3 inf. false for "{...}" (values elided) or anything
// that is not a brace list of numbers.
bool parse_array_literal(const std::string& text, std::vector<double>* out) {
  const std::string t = trim(text);
  if (t.size() < 2 || t[0] != '{' || t.find("...") != std::string::npos) return false;
  out->clear();
  size_t i = 0;
  while (i < t.size()) {
    const char ch = t[i];
    if (ch == '/' && i + 1 < t.size() && t[i + 1] == '*') {  // index comments of long literals
      const size_t e = t.find("*/", i + 2);
      if (e == std::string::npos) return false;
      i = e + 2;
      continue;
    }
    if (ch == '{' || ch == '}' || ch == ',' || ch == ' ' || ch == '\t') {
      ++i;
      continue;
    }
    size_t j = i;
    while (j < t.size() && t[j] != ',' && t[j] != '}' && t[j] != ' ' && t[j] != '{') ++j;
    double v = 0;
    if (!parse_scalar_literal(t.substr(i, j - i), &v)) return false;
    out->push_back(v);
    i = j;
  }
  return !out->empty();
}

}  // namespace

int parse_hlo_text(const std::string& text, HloModule* module, std::string* err) {
  *module = HloModule();
  std::istringstream in(text);
  std::string raw;
  int line_no = 0;
  HloComputation* cur = nullptr;
  bool in_block_comment = false;
  // operand names are resolved after the whole computation is read (forward references
  // do not occur in printed HLO, but resolving late keeps the error messages uniform)
  std::vector<std::vector<std::string>> pending_operands;

  auto finish = [&](int ln) -> int {
    HloComputation& c = *cur;
    for (size_t k = 0; k < c.instrs.size(); ++k) {
      for (const std::string& on : pending_operands[k]) {
        auto it = c.index.find(on);
        if (it == c.index.end()) {
          if (err) *err = "HLO line " + std::to_string(c.instrs[k].line) + ": operand %" + on +
                          " of %" + c.instrs[k].name + " is not defined in computation " + c.name;
          return MONONN_ERR_PARSE;
        }
        c.instrs[k].operands.push_back(it->second);
      }
    }
    if (c.root < 0) {
      if (c.instrs.empty()) {
        if (err) *err = "HLO line " + std::to_string(ln) + ": computation " + c.name + " is empty";
        return MONONN_ERR_PARSE;
      }
      c.root = static_cast<int>(c.instrs.size()) - 1;
    }
    int64_t np = 0;
    for (const HloInstr& ins : c.instrs)
      if (ins.opcode == "parameter") np = std::max<int64_t>(np, ins.param_number + 1);
    c.params.assign(static_cast<size_t>(np), -1);
    for (size_t k = 0; k < c.instrs.size(); ++k)
      if (c.instrs[k].opcode == "parameter") c.params[c.instrs[k].param_number] = static_cast<int>(k);
    pending_operands.clear();
    cur = nullptr;
    return MONONN_OK;
  };

  while (std::getline(in, raw)) {
    ++line_no;
    std::string line = raw;
    if (in_block_comment) {
      const size_t e = line.find("*/");
      if (e == std::string::npos) continue;
      line = line.substr(e + 2);
      in_block_comment = false;
    }
    for (;;) {
      const size_t b = line.find("/*");
      if (b == std::string::npos) break;
      const size_t e = line.find("*/", b + 2);
      if (e == std::string::npos) {
        line = line.substr(0, b);
        in_block_comment = true;
        break;
      }
      line = line.substr(0, b) + line.substr(e + 2);
    }
    line = trim(line);
    if (line.empty() || line.compare(0, 2, "//") == 0) continue;

    if (line.compare(0, 9, "HloModule") == 0) {
      std::string rest = trim(line.substr(9));
      size_t e = 0;
      while (e < rest.size() && rest[e] != ',' && !std::isspace(static_cast<unsigned char>(rest[e]))) ++e;
      module->name = rest.substr(0, e);
      continue;
    }
    if (line == "}") {
      if (!cur) {
        if (err) *err = "HLO line " + std::to_string(line_no) + ": unmatched '}'";
        return MONONN_ERR_PARSE;
      }
      int rc = finish(line_no);
      if (rc) return rc;
      continue;
    }
    if (!cur) {
      // computation header: [ENTRY] %name (params) -> shape {
      if (line.back() != '{') {
        if (err) *err = "HLO line " + std::to_string(line_no) + ": expected a computation header";
        return MONONN_ERR_PARSE;
      }
      bool entry = false;
      std::string h = line;
      if (h.compare(0, 6, "ENTRY ") == 0) {
        entry = true;
        h = trim(h.substr(6));
      }
      size_t e = 0;
      while (e < h.size() && h[e] != ' ' && h[e] != '(') ++e;
      std::string name = h.substr(0, e);
      if (!name.empty() && name[0] == '%') name = name.substr(1);
      if (name.empty()) {
        if (err) *err = "HLO line " + std::to_string(line_no) + ": computation without a name";
        return MONONN_ERR_PARSE;
      }
      module->comps.emplace_back();
      cur = &module->comps.back();
      cur->name = name;
      module->comp_index[name] = static_cast<int>(module->comps.size()) - 1;
      if (entry) module->entry = static_cast<int>(module->comps.size()) - 1;
      continue;
    }

    // instruction
    HloInstr ins;
    ins.line = line_no;
    std::string body = line;
    if (body.compare(0, 5, "ROOT ") == 0) {
      ins.is_root = true;
      body = trim(body.substr(5));
    }
    const size_t eq = body.find(" = ");
    if (eq == std::string::npos) {
      if (err) *err = "HLO line " + std::to_string(line_no) + ": expected '%name = shape opcode(...)'";
      return MONONN_ERR_PARSE;
    }
    ins.name = trim(body.substr(0, eq));
    if (!ins.name.empty() && ins.name[0] == '%') ins.name = ins.name.substr(1);
    Cursor c{body, eq + 3, line_no, err};
    if (!parse_shape(c, &ins.shape)) return MONONN_ERR_PARSE;
    c.ws();
    const size_t op_a = c.i;
    while (c.i < body.size() && (std::isalnum(static_cast<unsigned char>(body[c.i])) || body[c.i] == '-' ||
                                 body[c.i] == '_'))
      ++c.i;
    ins.opcode = body.substr(op_a, c.i - op_a);
    if (ins.opcode.empty() || c.i >= body.size() || body[c.i] != '(') {
      if (err) *err = "HLO line " + std::to_string(line_no) + ": expected an opcode followed by '('";
      return MONONN_ERR_PARSE;
    }
    const size_t close = match_paren(body, c.i);
    if (close == std::string::npos) {
      if (err) *err = "HLO line " + std::to_string(line_no) + ": unbalanced parentheses";
      return MONONN_ERR_PARSE;
    }
    const std::string args = body.substr(c.i + 1, close - c.i - 1);
    std::vector<std::string> operand_names;
    if (ins.opcode == "parameter") {
      ins.param_number = std::strtoll(args.c_str(), nullptr, 10);
    } else if (ins.opcode == "constant") {
      ins.literal_is_scalar = parse_scalar_literal(args, &ins.literal);
      if (!ins.literal_is_scalar) parse_array_literal(args, &ins.payload);
    } else {
      for (const std::string& a : split_top(args)) {
        // "f16[128,768]{1,0} %x" or "%x" or "x"
        size_t sp = a.find_last_of(" \t");
        std::string n = sp == std::string::npos ? a : a.substr(sp + 1);
        if (!n.empty() && n[0] == '%') n = n.substr(1);
        if (n.empty()) {
          if (err) *err = "HLO line " + std::to_string(line_no) + ": empty operand";
          return MONONN_ERR_PARSE;
        }
        operand_names.push_back(n);
      }
    }
    // attributes
    std::string rest = trim(body.substr(close + 1));
    if (!rest.empty() && rest[0] == ',') rest = rest.substr(1);
    for (const std::string& kv : split_top(rest)) {
      const size_t e2 = kv.find('=');
      if (e2 == std::string::npos) continue;
      ins.attrs[trim(kv.substr(0, e2))] = unquote(trim(kv.substr(e2 + 1)));
    }
    if (cur->index.count(ins.name)) {
      if (err) *err = "HLO line " + std::to_string(line_no) + ": duplicate instruction name %" + ins.name;
      return MONONN_ERR_PARSE;
    }
    cur->index[ins.name] = static_cast<int>(cur->instrs.size());
    if (ins.is_root) cur->root = static_cast<int>(cur->instrs.size());
    cur->instrs.push_back(ins);
    pending_operands.push_back(operand_names);
  }
  if (cur) {
    if (err) *err = "HLO text ends inside computation " + cur->name;
    return MONONN_ERR_PARSE;
  }
  if (module->comps.empty()) {
    if (err) *err = "no computation found in the HLO text";
    return MONONN_ERR_PARSE;
  }
  if (module->entry < 0) module->entry = static_cast<int>(module->comps.size()) - 1;
  if (module->name.empty()) module->name = module->comps[module->entry].name;
  return MONONN_OK;
}

}  // namespace mononn
