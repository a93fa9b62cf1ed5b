// Programmatic FGraph builders for the encoder families of the reference's examples
// (examples/utils/save_model.py:44-110 exports BERT / ViT / OPT / CLIP graphs). They
// produce the same fused graph the HLO recogniser produces from the XLA module of such a
// model, and serve the standalone (no HLO dump at hand) path.
#include "builders.h"

#include <cmath>

#include "../../include/mononn.h"
#include "json.h"

namespace mononn {

namespace {

int act_tensor(FGraph& g, const std::string& name, uint32_t rows, uint32_t cols) {
  FTensor t;
  t.name = name;
  t.kind = TKind::ActF16;
  t.rows = rows;
  t.cols = cols;
  t.ld = cols;
  return g.add_tensor(t);
}
int acc_tensor(FGraph& g, const std::string& name, uint32_t rows, uint32_t cols) {
  FTensor t;
  t.name = name;
  t.kind = TKind::AccF32;
  t.rows = rows;
  t.cols = cols;
  t.ld = cols;
  t.elem_bytes = 4;
  return g.add_tensor(t);
}
int const_tensor(FGraph& g, const std::string& name, uint32_t rows, uint32_t cols) {
  FTensor t;
  t.name = name;
  t.kind = TKind::Const;
  t.rows = rows;
  t.cols = cols;
  t.ld = cols;
  t.const_name = name;
  return g.add_tensor(t);
}
int arg_tensor(FGraph& g, const std::string& name, int kind, int number, uint32_t rows,
               uint32_t cols, uint32_t elem_bytes) {
  ArgDesc a;
  a.name = name;
  a.kind = kind;
  a.param_number = number;
  a.bytes = static_cast<size_t>(rows) * cols * elem_bytes;
  g.args.push_back(a);
  FTensor t;
  t.name = name;
  t.kind = TKind::Arg;
  t.rows = rows;
  t.cols = cols;
  t.ld = cols;
  t.elem_bytes = elem_bytes;
  t.arg_index = static_cast<int>(g.args.size()) - 1;
  return g.add_tensor(t);
}

FOp gemm(const std::string& name, int a, int w, int bias, int resid, int out, uint32_t M,
         uint32_t N, uint32_t K, ActKind act) {
  FOp o;
  o.kind = OP_GEMM;
  o.name = name;
  o.a = a;
  o.w = w;
  o.bias = bias;
  o.resid = resid;
  o.out = out;
  o.M = M;
  o.N = N;
  o.K = K;
  o.act = act;
  return o;
}

}  // namespace

int build_bert_encoder(const EncoderConfig& c, FGraph* out, std::string* err) {
  if (c.hidden != c.heads * 64) {
    if (err) *err = "head dimension must be 64";
    return MONONN_ERR_UNSUPPORTED;
  }
  FGraph& g = *out;
  g = FGraph();
  g.module_name = c.name.empty() ? "cluster_0" : c.name;
  const uint32_t T = c.batch * c.seq, H = c.hidden, F = c.ffn;
  const int ids = arg_tensor(g, "input_ids", 0, 0, c.batch, c.seq, 4);
  const int mask = arg_tensor(g, "attention_mask", 0, 1, c.batch, c.seq, 4);
  const int types = arg_tensor(g, "token_type_ids", 0, 2, c.batch, c.seq, 4);
  const int result = arg_tensor(g, "last_hidden_state", 1, 0, T, H, 2);

  FTensor mb;
  mb.name = "mask_bias";
  mb.kind = TKind::VecF32;
  mb.rows = T;
  mb.cols = 1;
  mb.elem_bytes = 4;
  const int mask_bias = g.add_tensor(mb);

  int x = act_tensor(g, "embeddings.out", T, H);
  {
    FOp e;
    e.kind = OP_EMBED;
    e.name = "embeddings";
    e.ids = ids;
    e.type_ids = types;
    e.mask_in = mask;
    e.mask_out = mask_bias;
    e.word = const_tensor(g, "embeddings.word", c.vocab, H);
    e.pos = const_tensor(g, "embeddings.position", c.max_pos, H);
    e.type = const_tensor(g, "embeddings.token_type", c.types, H);
    e.gamma = const_tensor(g, "embeddings.ln.gamma", 1, H);
    e.beta = const_tensor(g, "embeddings.ln.beta", 1, H);
    e.out = x;
    e.rows = T;
    e.cols = H;
    e.seq = c.seq;
    e.vocab = c.vocab;
    e.eps = c.eps;
    e.alpha = -10000.0f;  // additive mask (1 - m) * -10000, the HF convention
    g.ops.push_back(e);
  }
  for (uint32_t l = 0; l < c.layers; ++l) {
    const std::string p = "layer" + std::to_string(l) + ".";
    const int q = act_tensor(g, p + "q", T, H);
    const int k = act_tensor(g, p + "k", T, H);
    FTensor vt;
    vt.name = p + "v_t";
    vt.kind = TKind::ActF16T;
    vt.rows = T;
    vt.cols = H;
    vt.batches = c.batch;
    vt.seq = c.seq;
    vt.ld = (c.seq + 7) / 8 * 8;
    const int v_t = g.add_tensor(vt);
    g.ops.push_back(gemm(p + "attn.q", x, const_tensor(g, p + "attn.q.w", H, H),
                         const_tensor(g, p + "attn.q.b", 1, H), -1, q, T, H, H, ACT_NONE));
    g.ops.push_back(gemm(p + "attn.k", x, const_tensor(g, p + "attn.k.w", H, H),
                         const_tensor(g, p + "attn.k.b", 1, H), -1, k, T, H, H, ACT_NONE));
    g.ops.push_back(gemm(p + "attn.v", x, const_tensor(g, p + "attn.v.w", H, H),
                         const_tensor(g, p + "attn.v.b", 1, H), -1, v_t, T, H, H, ACT_NONE));
    const int ctx = act_tensor(g, p + "ctx", T, H);
    {
      FOp a;
      a.kind = OP_ATTENTION;
      a.name = p + "attn.core";
      a.q = q;
      a.k = k;
      a.vt = v_t;
      a.mask = mask_bias;
      a.out = ctx;
      a.heads = c.heads;
      a.seq = c.seq;
      a.batches = c.batch;
      a.alpha = 1.0f / std::sqrt(64.0f);
      g.ops.push_back(a);
    }
    const int acc1 = acc_tensor(g, p + "attn.sum", T, H);
    g.ops.push_back(gemm(p + "attn.o", ctx, const_tensor(g, p + "attn.o.w", H, H),
                         const_tensor(g, p + "attn.o.b", 1, H), x, acc1, T, H, H, ACT_NONE));
    const int x1 = act_tensor(g, p + "attn.ln.out", T, H);
    {
      FOp n;
      n.kind = OP_LAYERNORM;
      n.name = p + "attn.ln";
      n.src = acc1;
      n.gamma = const_tensor(g, p + "attn.ln.gamma", 1, H);
      n.beta = const_tensor(g, p + "attn.ln.beta", 1, H);
      n.out = x1;
      n.rows = T;
      n.cols = H;
      n.eps = c.eps;
      n.flags = F_ZERO_SRC;
      g.ops.push_back(n);
    }
    const int h = act_tensor(g, p + "ffn.h", T, F);
    g.ops.push_back(gemm(p + "ffn.up", x1, const_tensor(g, p + "ffn.up.w", H, F),
                         const_tensor(g, p + "ffn.up.b", 1, F), -1, h, T, F, H, c.act));
    const int acc2 = acc_tensor(g, p + "ffn.sum", T, H);
    g.ops.push_back(gemm(p + "ffn.down", h, const_tensor(g, p + "ffn.down.w", F, H),
                         const_tensor(g, p + "ffn.down.b", 1, H), x1, acc2, T, H, F, ACT_NONE));
    const int x2 = (l + 1 == c.layers) ? result : act_tensor(g, p + "ffn.ln.out", T, H);
    {
      FOp n;
      n.kind = OP_LAYERNORM;
      n.name = p + "ffn.ln";
      n.src = acc2;
      n.gamma = const_tensor(g, p + "ffn.ln.gamma", 1, H);
      n.beta = const_tensor(g, p + "ffn.ln.beta", 1, H);
      n.out = x2;
      n.rows = T;
      n.cols = H;
      n.eps = c.eps;
      n.flags = F_ZERO_SRC;
      g.ops.push_back(n);
    }
    x = x2;
  }
  return MONONN_OK;
}

int encoder_config_from_json(const std::string& text, EncoderConfig* c, std::string* err) {
  Json j;
  if (!Json::parse(text, &j, err)) return MONONN_ERR_PARSE;
  if (!j.is_object()) {
    if (err) *err = "config must be a JSON object";
    return MONONN_ERR_PARSE;
  }
  c->model = j.get_string("model", "bert");
  c->name = j.get_string("name", "cluster_0");
  c->layers = static_cast<uint32_t>(j.get_number("layers", 12));
  c->hidden = static_cast<uint32_t>(j.get_number("hidden", 768));
  c->heads = static_cast<uint32_t>(j.get_number("heads", 12));
  c->ffn = static_cast<uint32_t>(j.get_number("ffn", 3072));
  c->vocab = static_cast<uint32_t>(j.get_number("vocab", 30522));
  c->max_pos = static_cast<uint32_t>(j.get_number("max_pos", 512));
  c->types = static_cast<uint32_t>(j.get_number("types", 2));
  c->batch = static_cast<uint32_t>(j.get_number("batch", 1));
  c->seq = static_cast<uint32_t>(j.get_number("seq", 128));
  c->eps = static_cast<float>(j.get_number("eps", 1e-12));
  const std::string act = j.get_string("act", "gelu_erf");
  if (act == "gelu_erf") c->act = ACT_GELU_ERF;
  else if (act == "relu") c->act = ACT_RELU;
  else if (act == "quick_gelu") c->act = ACT_QUICK_GELU;
  else if (act == "gelu_tanh") c->act = ACT_GELU_TANH;
  else {
    if (err) *err = "unknown activation " + act;
    return MONONN_ERR_UNSUPPORTED;
  }
  if (c->model != "bert") {
    if (err) *err = "unknown model family " + c->model;
    return MONONN_ERR_UNSUPPORTED;
  }
  if (c->seq > c->max_pos || c->batch == 0 || c->seq == 0 || c->layers == 0) {
    if (err) *err = "inconsistent encoder configuration";
    return MONONN_ERR_INVALID_ARGUMENT;
  }
  return MONONN_OK;
}

}  // namespace mononn
