// HLO text -> fused operator graph (parser + fusion recogniser).
#pragma once
#include <string>

#include "plan.h"

namespace mononn {
// Returns 0 or a negative mononn error code with a message in *err.
int hlo_text_to_fgraph(const std::string& text, FGraph* graph, std::string* err);
}  // namespace mononn
