// Parser for XLA HLO text (the post-optimisation form a TF cluster reaches the hook in).
//
// The reference walks an in-memory xla::HloModule (IRParserFused::from_hlo_module_impl,
// mononn_engine/parser/ir_parser_fused.cc:319-385; the HLO-text entry points are
// from_text / from_file, ir_parser_fused.h:40-47).  XLA itself is not available to this
// build, so the textual form is parsed directly into a small module representation.
#pragma once
#include <stdint.h>

#include <map>
#include <string>
#include <vector>

namespace mononn {

struct HloShape {
  std::string dtype;  // "f16", "f32", "s32", "pred", ...; empty for a tuple
  std::vector<int64_t> dims;
  std::vector<int> minor_to_major;
  std::vector<HloShape> elems;  // tuple
  bool is_tuple() const { return dtype.empty(); }
  int64_t elements() const {
    int64_t n = 1;
    for (int64_t d : dims) n *= d;
    return n;
  }
  int elem_bytes() const;
  std::string str() const;
};

struct HloInstr {
  std::string name;    // without the leading '%'
  std::string opcode;
  HloShape shape;
  std::vector<int> operands;  // indices into the owning computation
  std::map<std::string, std::string> attrs;  // raw attribute text by key
  bool is_root = false;
  int64_t param_number = -1;
  bool literal_is_scalar = false;  // constant with a parsed scalar literal
  double literal = 0;
  // constant printed with its values ("constant({{1, 2}, {3, 4}})" instead of "constant({...})"):
  // the values in the printed (row-major, logical dimension) order
  std::vector<double> payload;
  int line = 0;

  std::vector<int64_t> int_list(const std::string& key) const;  // "{1,0}" -> {1,0}
  bool has(const std::string& key) const { return attrs.count(key) != 0; }
  std::string attr(const std::string& key) const {
    auto it = attrs.find(key);
    return it == attrs.end() ? std::string() : it->second;
  }
};

struct HloComputation {
  std::string name;
  std::vector<HloInstr> instrs;
  int root = -1;
  std::map<std::string, int> index;
  std::vector<int> params;  // instruction index by parameter number
};

struct HloModule {
  std::string name;
  std::vector<HloComputation> comps;
  int entry = -1;
  std::map<std::string, int> comp_index;
  const HloComputation* find(const std::string& comp_name) const {
    std::string n = comp_name;
    if (!n.empty() && n[0] == '%') n = n.substr(1);
    auto it = comp_index.find(n);
    return it == comp_index.end() ? nullptr : &comps[it->second];
  }
};

// Names as the reference canonicalises them: '.' and '-' become '_'
// (mononn_engine/helpers/string_helpers.cc:22-32).
std::string canonical_node_name(const std::string& name);

// Returns 0 or MONONN_ERR_PARSE / MONONN_ERR_UNSUPPORTED with a message that names the line.
int parse_hlo_text(const std::string& text, HloModule* module, std::string* err);

}  // namespace mononn
