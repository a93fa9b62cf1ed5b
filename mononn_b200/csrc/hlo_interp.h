// A small fp32 evaluator for fused HLO computations, used at COMPILE time only.
//
// The fusion recogniser does not pattern-match the instruction tree of a fused computation
// (XLA prints the same arithmetic in many shapes: operand order, extra converts, expanded
// polynomials).  It forms a hypothesis from the operand shapes ("bias + GELU epilogue",
// "LayerNorm of x + bias + residual", "softmax with additive mask", ...) and checks it by
// running the computation on random inputs with this evaluator and comparing with the
// closed form.  Nothing here runs at inference time and it is not a CPU fallback: a
// computation that matches no hypothesis is rejected with MONONN_ERR_UNSUPPORTED.
//
// Operator semantics follow the reference's index tracer and op implementations
// (mononn_engine/core/context/index_tracer.cc:67-434; op list core/op/op_type.h:20-65).
#pragma once
#include <stdint.h>

#include <string>
#include <vector>

#include "hlo_parser.h"

namespace mononn {

struct HTensor {
  std::vector<int64_t> dims;
  std::vector<float> v;  // integers are held exactly as floats (|x| < 2^24)
  int64_t size() const {
    int64_t n = 1;
    for (int64_t d : dims) n *= d;
    return n;
  }
  static HTensor zeros(const std::vector<int64_t>& d) {
    HTensor t;
    t.dims = d;
    t.v.assign(static_cast<size_t>(t.size()), 0.f);
    return t;
  }
};

// Evaluates `comp` on `params` (one tensor per parameter number). Returns 0 or a negative
// mononn error code (unsupported opcode / attribute form) with a message.
int eval_computation(const HloModule& m, const HloComputation& comp,
                     const std::vector<HTensor>& params, HTensor* out, std::string* err);

}  // namespace mononn
