#include "hlo_lowering.h"
#include "../../include/mononn.h"
namespace mononn {
int hlo_text_to_fgraph(const std::string&, FGraph*, std::string* err) {
  if (err) *err = "HLO front end not built yet";
  return MONONN_ERR_UNSUPPORTED;
}
}
