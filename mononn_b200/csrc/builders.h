// Programmatic FGraph builders (see builders.cc).
#pragma once
#include <string>

#include "plan.h"

namespace mononn {

struct EncoderConfig {
  std::string model = "bert";
  std::string name = "cluster_0";
  uint32_t layers = 12, hidden = 768, heads = 12, ffn = 3072;
  uint32_t vocab = 30522, max_pos = 512, types = 2;
  uint32_t batch = 1, seq = 128;
  float eps = 1e-12f;
  ActKind act = ACT_GELU_ERF;
};

int encoder_config_from_json(const std::string& text, EncoderConfig* c, std::string* err);
int build_bert_encoder(const EncoderConfig& c, FGraph* out, std::string* err);

}  // namespace mononn
