"""Model configurations and seeded synthetic weights / inputs.

The reference exports its example graphs from HuggingFace checkpoints
(examples/utils/save_model.py:44-110).  No checkpoint or dataset is reachable here, so
every tensor is synthetic: weights ~ N(0, 0.02) as HF initialises them, inputs drawn
from ``numpy.random.default_rng(seed)``.  The *stress* variant also randomises biases and
LayerNorm scale/shift so every fused epilogue term is observable in a parity test.
"""
from __future__ import annotations

import dataclasses
import json

import numpy as np


@dataclasses.dataclass
class EncoderConfig:
    model: str = "bert"
    name: str = "cluster_0"
    layers: int = 12
    hidden: int = 768
    heads: int = 12
    ffn: int = 3072
    vocab: int = 30522
    max_pos: int = 512
    types: int = 2
    batch: int = 1
    seq: int = 128
    eps: float = 1e-12
    act: str = "gelu_erf"
    # vision models: square image / patch size and channels (seq = patches + 1 class token)
    image: int = 0
    patch: int = 0
    channels: int = 3
    # patch convolution with overlapping windows: stride (0 = the patch size) and zero padding on every side
    patch_stride: int = 0
    patch_pad: int = 0

    def to_json(self) -> str:
        return json.dumps(dataclasses.asdict(self))

    @property
    def tokens(self) -> int:
        return self.batch * self.seq

    @property
    def patch_grid(self) -> int:
        """Output positions of the patch convolution along one image side."""
        return (self.image + 2 * self.patch_pad - self.patch) // (self.patch_stride or self.patch) + 1


def bert_base(batch: int = 1, seq: int = 128) -> EncoderConfig:
    """BERT-base encoder: the headline configuration (b1, s128)."""
    return EncoderConfig(batch=batch, seq=seq)


def bert_tiny(batch: int = 1, seq: int = 16, layers: int = 1, hidden: int = 64, ffn: int = 256,
              vocab: int = 100, max_pos: int = 64) -> EncoderConfig:
    """Small shape for element-wise parity checks (one layer, hidden 64)."""
    return EncoderConfig(layers=layers, hidden=hidden, heads=hidden // 64, ffn=ffn, vocab=vocab,
                         max_pos=max(max_pos, seq), batch=batch, seq=seq)


def bert_weight_shapes(cfg: EncoderConfig) -> dict[str, tuple[int, ...]]:
    h, f = cfg.hidden, cfg.ffn
    shapes: dict[str, tuple[int, ...]] = {
        "embeddings.word": (cfg.vocab, h),
        "embeddings.position": (cfg.max_pos, h),
        "embeddings.token_type": (cfg.types, h),
        "embeddings.ln.gamma": (h,),
        "embeddings.ln.beta": (h,),
    }
    for l in range(cfg.layers):
        p = f"layer{l}."
        for n in ("q", "k", "v", "o"):
            shapes[p + f"attn.{n}.w"] = (h, h)
            shapes[p + f"attn.{n}.b"] = (h,)
        shapes[p + "attn.ln.gamma"] = (h,)
        shapes[p + "attn.ln.beta"] = (h,)
        shapes[p + "ffn.up.w"] = (h, f)
        shapes[p + "ffn.up.b"] = (f,)
        shapes[p + "ffn.down.w"] = (f, h)
        shapes[p + "ffn.down.b"] = (h,)
        shapes[p + "ffn.ln.gamma"] = (h,)
        shapes[p + "ffn.ln.beta"] = (h,)
    return shapes


def make_weights(cfg, seed: int = 1234, stress: bool = False) -> dict[str, np.ndarray]:
    """fp32 weights, already rounded to fp16-representable values so that the fp16 device
    copy and the fp32 CPU copy hold the same numbers.  Linear weights are [in, out]."""
    rng = np.random.default_rng(seed)
    out: dict[str, np.ndarray] = {}
    if isinstance(cfg, ClipConfig):
        shapes = clip_weight_shapes(cfg)
    else:
        shapes = {"vit": vit_weight_shapes, "opt": opt_weight_shapes, "t5": t5_weight_shapes}.get(
            cfg.model, bert_weight_shapes)(cfg)
    for name, shape in shapes.items():
        if name.endswith(".gamma"):
            w = np.ones(shape, np.float32)
            if stress:
                w += rng.normal(0.0, 0.02, shape).astype(np.float32)
        elif name.endswith(".beta") or name.endswith(".b"):
            w = rng.normal(0.0, 0.02, shape).astype(np.float32) if stress else np.zeros(shape, np.float32)
        else:
            w = rng.normal(0.0, 0.02, shape).astype(np.float32)
        out[name] = w.astype(np.float16).astype(np.float32)
    return out


def make_inputs(cfg: EncoderConfig, seed: int = 1234, pad_fraction: float = 0.0) -> dict[str, np.ndarray]:
    """Token ids uniform over the vocabulary, type ids 0, mask all ones (or the trailing
    `pad_fraction` of every sequence zeroed)."""
    rng = np.random.default_rng(seed + 7919)
    ids = rng.integers(0, cfg.vocab, (cfg.batch, cfg.seq), dtype=np.int32)
    mask = np.ones((cfg.batch, cfg.seq), np.int32)
    if pad_fraction > 0:
        mask[:, cfg.seq - int(cfg.seq * pad_fraction):] = 0
    types = np.zeros((cfg.batch, cfg.seq), np.int32)
    return {"input_ids": ids, "attention_mask": mask, "token_type_ids": types}


def vit_base(batch: int = 1) -> EncoderConfig:
    """ViT-B/16: 224x224x3 image, 16x16 patches (196 + class token = 197 tokens), pre-LN."""
    return EncoderConfig(model="vit", layers=12, hidden=768, heads=12, ffn=3072, batch=batch, seq=197,
                         image=224, patch=16, channels=3, max_pos=197, vocab=0, types=0)


def vit_tiny(batch: int = 1, image: int = 32, patch: int = 16, layers: int = 1, hidden: int = 64,
             ffn: int = 256, patch_stride: int = 0, patch_pad: int = 0) -> EncoderConfig:
    """Small vision encoder. `patch_stride` / `patch_pad` turn the patch embedding into an
    overlapping, zero-padded convolution (a strided NHWC fprop as the reference's
    mononn_engine/core/op_impl/conv_impl.cc:252-345 accepts)."""
    n = ((image + 2 * patch_pad - patch) // (patch_stride or patch) + 1) ** 2 + 1
    return EncoderConfig(model="vit", layers=layers, hidden=hidden, heads=hidden // 64, ffn=ffn, batch=batch,
                         seq=n, image=image, patch=patch, channels=3, max_pos=n, vocab=0, types=0,
                         patch_stride=patch_stride, patch_pad=patch_pad)


def vit_weight_shapes(cfg: EncoderConfig) -> dict[str, tuple[int, ...]]:
    h, f = cfg.hidden, cfg.ffn
    shapes: dict[str, tuple[int, ...]] = {
        "embeddings.patch.w": (h, cfg.patch, cfg.patch, cfg.channels),  # [out, ky, kx, in]
        "embeddings.patch.b": (h,),
        "embeddings.cls": (1, h),
        "embeddings.position": (cfg.seq, h),
    }
    for l in range(cfg.layers):
        p = f"layer{l}."
        shapes[p + "ln1.gamma"] = (h,)
        shapes[p + "ln1.beta"] = (h,)
        for n in ("q", "k", "v", "o"):
            shapes[p + f"attn.{n}.w"] = (h, h)
            shapes[p + f"attn.{n}.b"] = (h,)
        shapes[p + "ln2.gamma"] = (h,)
        shapes[p + "ln2.beta"] = (h,)
        shapes[p + "ffn.up.w"] = (h, f)
        shapes[p + "ffn.up.b"] = (f,)
        shapes[p + "ffn.down.w"] = (f, h)
        shapes[p + "ffn.down.b"] = (h,)
    shapes["ln.gamma"] = (h,)
    shapes["ln.beta"] = (h,)
    return shapes


def make_vit_inputs(cfg: EncoderConfig, seed: int = 1234) -> dict[str, np.ndarray]:
    """Pixels uniform in [-1, 1], NCHW f32 as the reference's exported graph takes them
    (examples/utils/save_model.py:76-82)."""
    rng = np.random.default_rng(seed + 7919)
    px = rng.uniform(-1.0, 1.0, (cfg.batch, cfg.channels, cfg.image, cfg.image)).astype(np.float32)
    return {"pixel_values": px}


def opt_1p3b(batch: int = 1, seq: int = 128) -> EncoderConfig:
    """OPT-1.3B-shaped decoder prefill: 24 pre-LN layers, hidden 2048, 32 heads, FFN 8192 with
    ReLU, causal attention, learned positions (offset 2), vocab 50272 with a tied LM head."""
    return EncoderConfig(model="opt", layers=24, hidden=2048, heads=32, ffn=8192, vocab=50272,
                         max_pos=2048, types=0, batch=batch, seq=seq, eps=1e-5, act="relu")


def opt_tiny(batch: int = 1, seq: int = 16, layers: int = 1, hidden: int = 64, ffn: int = 256,
             vocab: int = 128) -> EncoderConfig:
    return EncoderConfig(model="opt", layers=layers, hidden=hidden, heads=hidden // 64, ffn=ffn, vocab=vocab,
                         max_pos=max(64, seq), types=0, batch=batch, seq=seq, eps=1e-5, act="relu")


def opt_weight_shapes(cfg: EncoderConfig) -> dict[str, tuple[int, ...]]:
    h, f = cfg.hidden, cfg.ffn
    shapes: dict[str, tuple[int, ...]] = {
        "embeddings.word": (cfg.vocab, h),           # also the LM head (tied)
        "embeddings.position": (cfg.max_pos + 2, h),  # learned positions, index = position + 2
    }
    for l in range(cfg.layers):
        p = f"layer{l}."
        shapes[p + "ln1.gamma"] = (h,)
        shapes[p + "ln1.beta"] = (h,)
        for n in ("q", "k", "v", "o"):
            shapes[p + f"attn.{n}.w"] = (h, h)
            shapes[p + f"attn.{n}.b"] = (h,)
        shapes[p + "ln2.gamma"] = (h,)
        shapes[p + "ln2.beta"] = (h,)
        shapes[p + "ffn.up.w"] = (h, f)
        shapes[p + "ffn.up.b"] = (f,)
        shapes[p + "ffn.down.w"] = (f, h)
        shapes[p + "ffn.down.b"] = (h,)
    shapes["ln.gamma"] = (h,)
    shapes["ln.beta"] = (h,)
    return shapes


# ---------------------------------------------------------------------------- T5
T5_BUCKETS, T5_MAX_DISTANCE = 32, 128


def t5_small(batch: int = 1, seq: int = 128) -> EncoderConfig:
    """T5-small-shaped encoder-decoder (examples/utils/save_model.py:84-92, 107-110): 6 + 6
    layers, width 512, 8 heads of 64, ReLU FFN 2048, no biases, RMS LayerNorm, relative position
    bias shared by the layers of a stack; `seq` is both the encoder and the decoder length."""
    return EncoderConfig(model="t5", layers=6, hidden=512, heads=8, ffn=2048, vocab=32128, max_pos=0, types=0,
                         batch=batch, seq=seq, eps=1e-6, act="relu")


def t5_tiny(batch: int = 1, seq: int = 32, layers: int = 1, hidden: int = 64, ffn: int = 128,
            vocab: int = 96) -> EncoderConfig:
    return EncoderConfig(model="t5", layers=layers, hidden=hidden, heads=hidden // 64, ffn=ffn, vocab=vocab,
                         max_pos=0, types=0, batch=batch, seq=seq, eps=1e-6, act="relu")


def t5_weight_shapes(cfg: EncoderConfig) -> dict[str, tuple[int, ...]]:
    h, f = cfg.hidden, cfg.ffn
    shapes: dict[str, tuple[int, ...]] = {"shared": (cfg.vocab, h)}
    for stack in ("encoder", "decoder"):
        shapes[f"{stack}.rel_bias"] = (T5_BUCKETS, cfg.heads)   # the learned table; not a device constant
        for l in range(cfg.layers):
            p = f"{stack}.layer{l}."
            shapes[p + "ln1.gamma"] = (h,)
            for n in ("q", "k", "v", "o"):
                shapes[p + f"attn.{n}.w"] = (h, h)
            if stack == "decoder":
                shapes[p + "lnx.gamma"] = (h,)
                for n in ("q", "k", "v", "o"):
                    shapes[p + f"xattn.{n}.w"] = (h, h)
            shapes[p + "ln2.gamma"] = (h,)
            shapes[p + "ffn.up.w"] = (h, f)
            shapes[p + "ffn.down.w"] = (f, h)
        shapes[f"{stack}.ln.gamma"] = (h,)
    return shapes


def t5_relative_buckets(seq_q: int, seq_k: int, bidirectional: bool) -> np.ndarray:
    """Bucket index [seq_q, seq_k] of the relative position key - query, as T5 defines it: half
    of the buckets (of each sign when bidirectional) hold exact distances, the other half
    logarithmically growing ranges up to T5_MAX_DISTANCE, beyond which everything shares the
    last bucket; a causal stack only distinguishes keys at or before the query."""
    rel = np.arange(seq_k)[None, :] - np.arange(seq_q)[:, None]
    n = T5_BUCKETS
    out = np.zeros_like(rel)
    if bidirectional:
        n //= 2
        out += (rel > 0).astype(rel.dtype) * n
        dist = np.abs(rel)
    else:
        dist = -np.minimum(rel, 0)
    exact = n // 2
    big = exact + (np.log(np.maximum(dist, 1).astype(np.float32) / exact) / np.log(T5_MAX_DISTANCE / exact)
                   * (n - exact)).astype(rel.dtype)
    big = np.minimum(big, n - 1)
    return out + np.where(dist < exact, dist, big)


def t5_position_bias(table: np.ndarray, seq_q: int, seq_k: int, bidirectional: bool) -> np.ndarray:
    """[heads, seq_q, seq_k] additive attention bias gathered from the [buckets, heads] table."""
    return np.ascontiguousarray(table[t5_relative_buckets(seq_q, seq_k, bidirectional)].transpose(2, 0, 1))


def t5_device_weights(cfg: EncoderConfig, w: dict[str, np.ndarray]) -> dict[str, np.ndarray]:
    """The constants of the T5 HLO module: every weight, with each stack's relative-position
    table replaced by the [heads * seq, seq] bias tensor a compiler folds it into (the table,
    the bucket arithmetic and the gather involve no run-time input)."""
    out = {k: v for k, v in w.items() if not k.endswith(".rel_bias")}
    s = cfg.seq
    out["encoder.pos_bias"] = t5_position_bias(w["encoder.rel_bias"], s, s, True).reshape(cfg.heads * s, s)
    out["decoder.pos_bias"] = t5_position_bias(w["decoder.rel_bias"], s, s, False).reshape(cfg.heads * s, s)
    return out


def make_t5_inputs(cfg: EncoderConfig, seed: int = 1234) -> dict[str, np.ndarray]:
    rng = np.random.default_rng(seed + 7919)
    return {"input_ids": rng.integers(0, cfg.vocab, (cfg.batch, cfg.seq), dtype=np.int32),
            "decoder_input_ids": rng.integers(0, cfg.vocab, (cfg.batch, cfg.seq), dtype=np.int32)}


@dataclasses.dataclass
class ClipConfig:
    """Dual encoder: a pre-LN vision tower (class token, LayerNorm before the blocks, LayerNorm
    of the class row after them) and a pre-LN causal text tower (row of the largest token id
    pooled after the final LayerNorm); both projected to `proj` columns, L2-normalised and
    compared: logits[i, j] = logit_scale * <image_i, text_j>."""
    vision: EncoderConfig
    text: EncoderConfig
    proj: int = 512
    logit_scale: float = 1.0 / 0.07   # exp(2.6592), the initial value of the learned temperature
    name: str = "cluster_0"
    model: str = "clip"


def _clip_towers(batch_img, batch_txt, image, patch, vh, vl, vf, th, tl, tf, seq, vocab):
    n = (image // patch) ** 2 + 1
    vision = EncoderConfig(model="vit", layers=vl, hidden=vh, heads=vh // 64, ffn=vf, batch=batch_img, seq=n,
                           image=image, patch=patch, channels=3, max_pos=n, vocab=0, types=0, eps=1e-5,
                           act="quick_gelu")
    text = EncoderConfig(model="opt", layers=tl, hidden=th, heads=th // 64, ffn=tf, vocab=vocab, max_pos=seq,
                         types=0, batch=batch_txt, seq=seq, eps=1e-5, act="quick_gelu")
    return vision, text


def clip_b32(images: int = 32, texts: int = 32) -> ClipConfig:
    """CLIP ViT-B/32 shape: 224x224 image in 32x32 patches (50 tokens, width 768, 12 layers),
    text width 512 / 8 heads / 12 layers / 77 tokens over 49408 ids, projection 512."""
    v, t = _clip_towers(images, texts, 224, 32, 768, 12, 3072, 512, 12, 2048, 77, 49408)
    return ClipConfig(vision=v, text=t, proj=512)


def clip_tiny(images: int = 3, texts: int = 5, image: int = 64, patch: int = 32, layers: int = 1,
              vh: int = 128, th: int = 64, seq: int = 12, vocab: int = 200, proj: int = 64) -> ClipConfig:
    v, t = _clip_towers(images, texts, image, patch, vh, layers, 2 * vh, th, layers, 2 * th, seq, vocab)
    return ClipConfig(vision=v, text=t, proj=proj)


def clip_weight_shapes(cfg: ClipConfig) -> dict[str, tuple[int, ...]]:
    v, t = cfg.vision, cfg.text
    shapes: dict[str, tuple[int, ...]] = {}
    for k, shp in vit_weight_shapes(v).items():
        if k == "embeddings.patch.b":
            continue  # the patch convolution has no bias
        shapes["vision." + k] = shp
    shapes["vision.pre_ln.gamma"] = (v.hidden,)
    shapes["vision.pre_ln.beta"] = (v.hidden,)
    shapes["vision.proj.w"] = (v.hidden, cfg.proj)
    for k, shp in opt_weight_shapes(t).items():
        shapes["text." + k] = (t.max_pos, t.hidden) if k == "embeddings.position" else shp
    shapes["text.proj.w"] = (t.hidden, cfg.proj)
    return shapes


def make_clip_inputs(cfg: ClipConfig, seed: int = 1234) -> dict[str, np.ndarray]:
    """Pixels uniform in [-1, 1], token ids uniform over the vocabulary."""
    out = make_vit_inputs(cfg.vision, seed)
    out["input_ids"] = make_inputs(cfg.text, seed)["input_ids"]
    return out
