"""CPU fp32 restatement of the encoder graphs on the hot path.  TEST INFRASTRUCTURE ONLY:
imported by tests/, by ``__graft_entry__.smoke()`` and by ``bench.py``'s CPU-baseline leg,
never by the product path.

Parity status: UNPINNED by the reference.  The reference holds no golden outputs, no
known-answer tests and no weights for this path (its only fixture is the input file
examples/data/bert_bs1.npy), and its TF-XLA CPU execution cannot run here (TensorFlow 2.9
and both submodules are absent).  The restatement is instead pinned against the
`transformers` PyTorch BertModel on identical weights (tests/golden/make_golden.py).

What it follows:
  * graph and I/O signature: examples/utils/save_model.py:44-54 (BERT: int32 input_ids,
    attention_mask, token_type_ids of shape [B, S]); the output is the last hidden state.
  * GEMM semantics alpha*op(A)*op(B): mononn_engine/core/op_impl/gemm_impl.cc:233-469.
  * reduce semantics (one reduced dimension, row-wise): core/op/cluster_reduce.cc:72-84.
  * gather without clamping: mononn_engine/core/context/index_tracer.cc:235-280.
  * architecture math (public BERT definition): embeddings = word + position + type -> LN;
    post-LN blocks; attention scale 1/sqrt(64) with additive mask (1 - m) * -10000;
    exact-erf GELU; LayerNorm eps 1e-12 with biased variance.
"""
from __future__ import annotations

import math

import numpy as np


def _erf(x: np.ndarray) -> np.ndarray:
    try:
        from scipy.special import erf
        return erf(x).astype(x.dtype)
    except Exception:  # pragma: no cover - scipy is present in the image
        return np.vectorize(math.erf)(x).astype(x.dtype)


def layer_norm(x: np.ndarray, gamma: np.ndarray, beta: np.ndarray, eps: float) -> np.ndarray:
    mean = x.mean(-1, keepdims=True, dtype=np.float64)
    var = ((x - mean) ** 2).mean(-1, keepdims=True, dtype=np.float64)
    return (((x - mean) / np.sqrt(var + eps)) * gamma + beta).astype(np.float32)


def gelu_erf(x: np.ndarray) -> np.ndarray:
    return (0.5 * x * (1.0 + _erf(x * np.float32(0.7071067811865476)))).astype(np.float32)


def activation(x: np.ndarray, kind: str) -> np.ndarray:
    if kind == "gelu_erf":
        return gelu_erf(x)
    if kind == "relu":
        return np.maximum(x, 0)
    if kind == "quick_gelu":
        return (x / (1.0 + np.exp(-1.702 * x))).astype(np.float32)
    if kind == "gelu_tanh":
        return (0.5 * x * (1 + np.tanh(0.7978845608028654 * (x + 0.044715 * x ** 3)))).astype(np.float32)
    if kind == "none":
        return x
    raise ValueError(kind)


def softmax_rows(z: np.ndarray) -> np.ndarray:
    z = z - z.max(-1, keepdims=True)
    e = np.exp(z)
    return (e / e.sum(-1, keepdims=True)).astype(np.float32)


def attention(q, k, v, mask_bias, heads, causal=False):
    """q, k, v: [B, S, H]; mask_bias: [B, S] additive or None.  Returns [B, S, H]."""
    b, s, h = q.shape
    d = h // heads
    split = lambda t: t.reshape(b, s, heads, d).transpose(0, 2, 1, 3)
    qh, kh, vh = split(q), split(k), split(v)
    scores = np.matmul(qh, kh.transpose(0, 1, 3, 2)) * np.float32(1.0 / math.sqrt(d))
    if mask_bias is not None:
        scores = scores + mask_bias[:, None, None, :]
    if causal:
        scores = scores + np.triu(np.full((s, s), -1e30, np.float32), 1)
    p = softmax_rows(scores)
    ctx = np.matmul(p, vh)
    return ctx.transpose(0, 2, 1, 3).reshape(b, s, h)


def bert_embeddings(cfg, w, ids, types):
    pos = np.arange(cfg.seq)
    x = w["embeddings.word"][ids] + w["embeddings.position"][pos][None] + w["embeddings.token_type"][types]
    return layer_norm(x.astype(np.float32), w["embeddings.ln.gamma"], w["embeddings.ln.beta"], cfg.eps)


def bert_layer(cfg, w, x, mask_bias, l):
    p = f"layer{l}."
    lin = lambda t, n: t @ w[p + n + ".w"] + w[p + n + ".b"]
    q, k, v = lin(x, "attn.q"), lin(x, "attn.k"), lin(x, "attn.v")
    ctx = attention(q, k, v, mask_bias, cfg.heads)
    x1 = layer_norm(lin(ctx, "attn.o") + x, w[p + "attn.ln.gamma"], w[p + "attn.ln.beta"], cfg.eps)
    hmid = activation(lin(x1, "ffn.up"), cfg.act)
    return layer_norm(lin(hmid, "ffn.down") + x1, w[p + "ffn.ln.gamma"], w[p + "ffn.ln.beta"], cfg.eps)


def bert_encoder(cfg, w, inputs, return_all=False):
    """fp32 forward.  Returns the last hidden state [B*S, H] (the live-out of the module)."""
    ids, mask, types = inputs["input_ids"], inputs["attention_mask"], inputs["token_type_ids"]
    mask_bias = (1.0 - mask.astype(np.float32)) * np.float32(-10000.0)
    x = bert_embeddings(cfg, w, ids, types)
    hidden = [x]
    for l in range(cfg.layers):
        x = bert_layer(cfg, w, x, mask_bias, l)
        hidden.append(x)
    out = x.reshape(cfg.batch * cfg.seq, cfg.hidden)
    return (out, hidden) if return_all else out


def bert_encoder_torch(cfg, w, inputs, threads=0):
    """Same math through torch CPU ops (multi-threaded); the timed CPU baseline."""
    import torch
    import torch.nn.functional as F
    if threads:
        torch.set_num_threads(threads)
    tw = {k: torch.from_numpy(v) for k, v in w.items()}
    ids = torch.from_numpy(inputs["input_ids"]).long()
    types = torch.from_numpy(inputs["token_type_ids"]).long()
    mask = torch.from_numpy(inputs["attention_mask"]).float()
    mask_bias = (1.0 - mask) * -10000.0
    b, s, h, nh = cfg.batch, cfg.seq, cfg.hidden, cfg.heads
    with torch.no_grad():
        x = tw["embeddings.word"][ids] + tw["embeddings.position"][:s][None] + tw["embeddings.token_type"][types]
        x = F.layer_norm(x, (h,), tw["embeddings.ln.gamma"], tw["embeddings.ln.beta"], cfg.eps)
        for l in range(cfg.layers):
            p = f"layer{l}."
            lin = lambda t, n: t @ tw[p + n + ".w"] + tw[p + n + ".b"]
            split = lambda t: t.view(b, s, nh, h // nh).transpose(1, 2)
            q, k, v = split(lin(x, "attn.q")), split(lin(x, "attn.k")), split(lin(x, "attn.v"))
            sc = q @ k.transpose(-1, -2) / math.sqrt(h // nh) + mask_bias[:, None, None, :]
            ctx = (torch.softmax(sc, -1) @ v).transpose(1, 2).reshape(b, s, h)
            x = F.layer_norm(lin(ctx, "attn.o") + x, (h,), tw[p + "attn.ln.gamma"], tw[p + "attn.ln.beta"], cfg.eps)
            y = lin(x, "ffn.up")
            y = F.gelu(y) if cfg.act == "gelu_erf" else torch.relu(y)
            x = F.layer_norm(lin(y, "ffn.down") + x, (h,), tw[p + "ffn.ln.gamma"], tw[p + "ffn.ln.beta"], cfg.eps)
    return x.reshape(b * s, h).numpy()


def _torch_weights(w):
    import torch
    return {k: torch.from_numpy(np.ascontiguousarray(v)) for k, v in w.items()}


def _act_torch(x, kind):
    import torch
    import torch.nn.functional as F
    if kind == "gelu_erf":
        return F.gelu(x)
    if kind == "relu":
        return torch.relu(x)
    if kind == "quick_gelu":
        return x * torch.sigmoid(1.702 * x)
    if kind == "gelu_tanh":
        return F.gelu(x, approximate="tanh")
    raise ValueError(kind)


def preln_blocks_torch(cfg, tw, x, prefix="", causal=False):
    """_preln_blocks through torch CPU ops (multi-threaded): the full-size parity cases need the
    fp32 side in seconds. x: [B, S, H] torch tensor; tw: torch weights."""
    import torch
    import torch.nn.functional as F
    b, s, h = x.shape
    nh = cfg.heads
    d = h // nh
    tri = torch.triu(torch.full((s, s), -1e30), 1) if causal else None
    for l in range(cfg.layers):
        p = f"{prefix}layer{l}."
        lin = lambda t, n: t @ tw[p + n + ".w"] + tw[p + n + ".b"]
        split = lambda t: t.view(b, s, nh, d).transpose(1, 2)
        y = F.layer_norm(x, (h,), tw[p + "ln1.gamma"], tw[p + "ln1.beta"], cfg.eps)
        sc = split(lin(y, "attn.q")) @ split(lin(y, "attn.k")).transpose(-1, -2) / math.sqrt(d)
        if tri is not None:
            sc = sc + tri
        ctx = (torch.softmax(sc, -1) @ split(lin(y, "attn.v"))).transpose(1, 2).reshape(b, s, h)
        x = x + lin(ctx, "attn.o")
        y = F.layer_norm(x, (h,), tw[p + "ln2.gamma"], tw[p + "ln2.beta"], cfg.eps)
        x = x + lin(_act_torch(lin(y, "ffn.up"), cfg.act), "ffn.down")
    return x


def vit_encoder_torch(cfg, w, inputs, threads=0):
    """vit_encoder through torch CPU ops. Returns [B*tokens, H] as numpy f32."""
    import torch
    import torch.nn.functional as F
    if threads:
        torch.set_num_threads(threads)
    tw = _torch_weights(w)
    b, h = cfg.batch, cfg.hidden
    with torch.no_grad():
        pat = torch.from_numpy(vit_patches(cfg, inputs["pixel_values"].astype(np.float32)))
        pat = pat @ tw["embeddings.patch.w"].reshape(h, -1).T + tw["embeddings.patch.b"]
        cls = tw["embeddings.cls"].reshape(1, 1, h).expand(b, 1, h)
        x = torch.cat([cls, pat.reshape(b, cfg.seq - 1, h)], 1) + tw["embeddings.position"][None]
        x = preln_blocks_torch(cfg, tw, x)
        out = F.layer_norm(x, (h,), tw["ln.gamma"], tw["ln.beta"], cfg.eps)
    return out.reshape(b * cfg.seq, h).numpy()


def opt_decoder_torch(cfg, w, inputs, threads=0):
    """opt_decoder through torch CPU ops. Returns (logits [B*S, vocab], argmax [B*S])."""
    import torch
    import torch.nn.functional as F
    if threads:
        torch.set_num_threads(threads)
    tw = _torch_weights(w)
    b, s_, h = cfg.batch, cfg.seq, cfg.hidden
    with torch.no_grad():
        ids = torch.from_numpy(inputs["input_ids"]).long()
        x = tw["embeddings.word"][ids] + tw["embeddings.position"][2:2 + s_][None]
        x = preln_blocks_torch(cfg, tw, x, causal=True)
        y = F.layer_norm(x, (h,), tw["ln.gamma"], tw["ln.beta"], cfg.eps).reshape(b * s_, h)
        logits = y @ tw["embeddings.word"].T
    return logits.numpy(), logits.argmax(-1).to(torch.int32).numpy()


def vit_patches(cfg, pixels):
    """[B, C, H, W] -> [B * patches, ky * kx * C]: the operand of the patch-embedding
    convolution (any stride, symmetric zero padding, cross-correlation, NHWC/KRSC as the reference's conv,
    mononn_engine/core/op_impl/conv_impl.cc:252-345) written as a matrix product."""
    b, c, hh, ww = pixels.shape
    p = cfg.patch
    st, pad = getattr(cfg, "patch_stride", 0) or p, getattr(cfg, "patch_pad", 0)
    if st == p and pad == 0:
        g = hh // p
        x = pixels.reshape(b, c, g, p, g, p).transpose(0, 2, 4, 3, 5, 1)  # b, gy, gx, ky, kx, c
        return x.reshape(b * g * g, p * p * c)
    # overlapping / zero-padded windows: one output position at a time
    xp = np.zeros((b, c, hh + 2 * pad, ww + 2 * pad), pixels.dtype)
    xp[:, :, pad:pad + hh, pad:pad + ww] = pixels
    gy, gx = (hh + 2 * pad - p) // st + 1, (ww + 2 * pad - p) // st + 1
    out = np.empty((b, gy, gx, p, p, c), pixels.dtype)
    for y in range(gy):
        for x in range(gx):
            out[:, y, x] = xp[:, :, y * st:y * st + p, x * st:x * st + p].transpose(0, 2, 3, 1)
    return out.reshape(b * gy * gx, p * p * c)


def vit_encoder(cfg, w, inputs, return_all=False):
    """fp32 forward of the pre-LN vision encoder (patch embedding, class token, learned
    positions, pre-LN blocks with exact GELU, final LayerNorm). Returns [B*tokens, H]."""
    px = inputs["pixel_values"].astype(np.float32)
    b, h = cfg.batch, cfg.hidden
    pat = vit_patches(cfg, px) @ w["embeddings.patch.w"].reshape(h, -1).T + w["embeddings.patch.b"]
    pat = pat.reshape(b, cfg.seq - 1, h)
    cls = np.broadcast_to(w["embeddings.cls"].reshape(1, 1, h), (b, 1, h))
    x = np.concatenate([cls, pat], 1) + w["embeddings.position"][None]
    x = x.astype(np.float32)
    hidden = [x]
    for l in range(cfg.layers):
        p = f"layer{l}."
        lin = lambda t, n: t @ w[p + n + ".w"] + w[p + n + ".b"]
        y = layer_norm(x, w[p + "ln1.gamma"], w[p + "ln1.beta"], cfg.eps)
        ctx = attention(lin(y, "attn.q"), lin(y, "attn.k"), lin(y, "attn.v"), None, cfg.heads)
        x = x + lin(ctx, "attn.o")
        y = layer_norm(x, w[p + "ln2.gamma"], w[p + "ln2.beta"], cfg.eps)
        x = x + lin(activation(lin(y, "ffn.up"), cfg.act), "ffn.down")
        hidden.append(x)
    out = layer_norm(x, w["ln.gamma"], w["ln.beta"], cfg.eps).reshape(b * cfg.seq, h)
    return (out, hidden) if return_all else out


def opt_decoder(cfg, w, inputs):
    """fp32 prefill of the pre-LN causal decoder (OPT): token + learned position embeddings
    (position index + 2, attention mask all ones), causal attention, ReLU FFN, final
    LayerNorm, LM head tied to the token table. Returns (logits [B*S, vocab], argmax [B*S])."""
    ids = inputs["input_ids"]
    b, s_, h = cfg.batch, cfg.seq, cfg.hidden
    x = (w["embeddings.word"][ids] + w["embeddings.position"][2:2 + s_][None]).astype(np.float32)
    for l in range(cfg.layers):
        p = f"layer{l}."
        lin = lambda t, n: t @ w[p + n + ".w"] + w[p + n + ".b"]
        y = layer_norm(x, w[p + "ln1.gamma"], w[p + "ln1.beta"], cfg.eps)
        ctx = attention(lin(y, "attn.q"), lin(y, "attn.k"), lin(y, "attn.v"), None, cfg.heads, causal=True)
        x = x + lin(ctx, "attn.o")
        y = layer_norm(x, w[p + "ln2.gamma"], w[p + "ln2.beta"], cfg.eps)
        x = x + lin(activation(lin(y, "ffn.up"), cfg.act), "ffn.down")
    y = layer_norm(x, w["ln.gamma"], w["ln.beta"], cfg.eps).reshape(b * s_, h)
    logits = (y @ w["embeddings.word"].T).astype(np.float32)
    return logits, logits.argmax(-1).astype(np.int32)


def _preln_blocks(cfg, w, x, prefix="", causal=False):
    """The pre-LN transformer blocks of `cfg` applied to the residual stream x [B, S, H]."""
    for l in range(cfg.layers):
        p = f"{prefix}layer{l}."
        lin = lambda t, n: t @ w[p + n + ".w"] + w[p + n + ".b"]
        y = layer_norm(x, w[p + "ln1.gamma"], w[p + "ln1.beta"], cfg.eps)
        ctx = attention(lin(y, "attn.q"), lin(y, "attn.k"), lin(y, "attn.v"), None, cfg.heads, causal=causal)
        x = x + lin(ctx, "attn.o")
        y = layer_norm(x, w[p + "ln2.gamma"], w[p + "ln2.beta"], cfg.eps)
        x = x + lin(activation(lin(y, "ffn.up"), cfg.act), "ffn.down")
    return x


def clip_dual(cfg, w, inputs):
    """fp32 forward of the dual encoder (CLIP). Vision: bias-free patch convolution, class
    token + positions, LayerNorm, pre-LN blocks (quick-GELU), LayerNorm of the class row,
    projection. Text: token + position rows, causal pre-LN blocks, final LayerNorm, the row of
    the largest token id (first on ties), projection. Returns (logits_per_image [images,
    texts], image_embeds, text_embeds), the embeddings L2-normalised."""
    v, t = cfg.vision, cfg.text
    px = inputs["pixel_values"].astype(np.float32)
    pat = vit_patches(v, px) @ w["vision.embeddings.patch.w"].reshape(v.hidden, -1).T
    pat = pat.reshape(v.batch, v.seq - 1, v.hidden)
    cls = np.broadcast_to(w["vision.embeddings.cls"].reshape(1, 1, v.hidden), (v.batch, 1, v.hidden))
    x = (np.concatenate([cls, pat], 1) + w["vision.embeddings.position"][None]).astype(np.float32)
    x = layer_norm(x, w["vision.pre_ln.gamma"], w["vision.pre_ln.beta"], v.eps)
    x = _preln_blocks(v, w, x, "vision.")
    pooled = layer_norm(x[:, 0, :], w["vision.ln.gamma"], w["vision.ln.beta"], v.eps)
    img = pooled @ w["vision.proj.w"]

    ids = inputs["input_ids"]
    y = (w["text.embeddings.word"][ids] + w["text.embeddings.position"][: t.seq][None]).astype(np.float32)
    y = _preln_blocks(t, w, y, "text.", causal=True)
    y = layer_norm(y, w["text.ln.gamma"], w["text.ln.beta"], t.eps)
    eos = ids.argmax(-1)  # first occurrence of the largest id
    txt = y[np.arange(t.batch), eos] @ w["text.proj.w"]

    img = img / np.linalg.norm(img, axis=-1, keepdims=True)
    txt = txt / np.linalg.norm(txt, axis=-1, keepdims=True)
    logits = (cfg.logit_scale * img @ txt.T).astype(np.float32)
    return logits, img.astype(np.float32), txt.astype(np.float32)


# ------------------------------------------------------------------------------------ T5
def rms_norm(x: np.ndarray, gamma: np.ndarray, eps: float) -> np.ndarray:
    """T5's LayerNorm: x / sqrt(mean(x^2) + eps) * scale, no mean subtraction and no shift."""
    return (x / np.sqrt((x * x).mean(-1, keepdims=True) + eps) * gamma).astype(np.float32)


def _t5_attention(q, k, v, heads, bias, causal):
    """Un-scaled scores + per-(head, query, key) bias; q [B, Sq, H], k / v [B, Sk, H]."""
    b, sq, h = q.shape
    sk, d = k.shape[1], h // heads
    qh = q.reshape(b, sq, heads, d).transpose(0, 2, 1, 3)
    kh = k.reshape(b, sk, heads, d).transpose(0, 2, 1, 3)
    vh = v.reshape(b, sk, heads, d).transpose(0, 2, 1, 3)
    scores = np.matmul(qh, kh.transpose(0, 1, 3, 2))
    if bias is not None:
        scores = scores + bias[None]
    if causal:
        scores = scores + np.triu(np.full((sq, sk), -1e30, np.float32), 1)
    return np.matmul(softmax_rows(scores), vh).transpose(0, 2, 1, 3).reshape(b, sq, h)


def t5_model(cfg, w, inputs):
    """fp32 forward of the T5 encoder-decoder (the model of examples/utils/save_model.py:84-92,
    which returns the decoder's last hidden state): shared token table, pre-norm blocks with RMS
    LayerNorm, bias-free projections, un-scaled attention scores plus the relative position bias
    of the stack (bidirectional buckets in the encoder, causal ones in the decoder, none in
    cross-attention), ReLU FFN. Returns [B * S, H]."""
    from mononn_b200.models import t5_position_bias
    b, s_, h = cfg.batch, cfg.seq, cfg.hidden
    lin = lambda t, name: t @ w[name + ".w"]
    enc_bias = t5_position_bias(w["encoder.rel_bias"], s_, s_, True)
    dec_bias = t5_position_bias(w["decoder.rel_bias"], s_, s_, False)
    x = w["shared"][inputs["input_ids"]].astype(np.float32)
    for l in range(cfg.layers):
        p = f"encoder.layer{l}."
        y = rms_norm(x, w[p + "ln1.gamma"], cfg.eps)
        ctx = _t5_attention(lin(y, p + "attn.q"), lin(y, p + "attn.k"), lin(y, p + "attn.v"), cfg.heads, enc_bias, False)
        x = x + lin(ctx, p + "attn.o")
        y = rms_norm(x, w[p + "ln2.gamma"], cfg.eps)
        x = x + lin(activation(lin(y, p + "ffn.up"), cfg.act), p + "ffn.down")
    enc = rms_norm(x, w["encoder.ln.gamma"], cfg.eps)
    x = w["shared"][inputs["decoder_input_ids"]].astype(np.float32)
    for l in range(cfg.layers):
        p = f"decoder.layer{l}."
        y = rms_norm(x, w[p + "ln1.gamma"], cfg.eps)
        ctx = _t5_attention(lin(y, p + "attn.q"), lin(y, p + "attn.k"), lin(y, p + "attn.v"), cfg.heads, dec_bias, True)
        x = x + lin(ctx, p + "attn.o")
        y = rms_norm(x, w[p + "lnx.gamma"], cfg.eps)
        ctx = _t5_attention(lin(y, p + "xattn.q"), lin(enc, p + "xattn.k"), lin(enc, p + "xattn.v"), cfg.heads, None, False)
        x = x + lin(ctx, p + "xattn.o")
        y = rms_norm(x, w[p + "ln2.gamma"], cfg.eps)
        x = x + lin(activation(lin(y, p + "ffn.up"), cfg.act), p + "ffn.down")
    return rms_norm(x, w["decoder.ln.gamma"], cfg.eps).reshape(b * s_, h)
