"""Parity of the CUDA path with the CPU oracle, through the C ABI (-m gpu)."""
import numpy as np
import pytest

from mononn_b200 import (bert_base, bert_tiny, clip_b32, clip_tiny, compile_encoder, compile_hlo, make_clip_inputs,
                         make_inputs, make_vit_inputs, make_weights, opt_tiny, vit_base, vit_tiny)
from mononn_b200 import make_t5_inputs, t5_device_weights, t5_small, t5_tiny
from mononn_b200.hlo_builder import bert_hlo, clip_hlo, opt_hlo, t5_hlo, vit_hlo
from mononn_b200.models import EncoderConfig
from oracle import ref_encoder as R
from tests.helpers import assert_parity, golden_cases, load_golden, reference_fixture_inputs

pytestmark = pytest.mark.gpu


def run_module(mod, cfg, inp):
    out = mod.run([inp["input_ids"], inp["attention_mask"], inp["token_type_ids"]])[0]
    return out[: cfg.tokens * cfg.hidden].reshape(cfg.tokens, cfg.hidden).astype(np.float32)


def build(cfg, w, frontend):
    if frontend == "hlo":
        text, names = bert_hlo(cfg)
        mod = compile_hlo(text, barrier_timeout_us=500000)
        mod.set_weights({names[k]: v for k, v in w.items()})
    else:
        mod = compile_encoder(cfg, barrier_timeout_us=500000)
        mod.set_weights(w)
    return mod


@pytest.mark.parametrize("name", sorted(golden_cases()))
@pytest.mark.parametrize("frontend", ["hlo", "builder"])
def test_golden_vectors(name, frontend):
    cfg, seed, stress, pad = golden_cases()[name]
    w = make_weights(cfg, seed, stress=stress)
    if cfg.model != "bert" and frontend == "builder":
        pytest.skip("the config builder covers the BERT family only")
    if cfg.model == "vit":
        got = run_vit(cfg, w, make_vit_inputs(cfg, seed))
    elif cfg.model == "clip":
        got = run_clip(cfg, w, make_clip_inputs(cfg, seed))[0]
    elif cfg.model == "t5":
        got = run_t5(cfg, w, make_t5_inputs(cfg, seed))
    elif cfg.model == "opt":
        got, ids = run_opt(cfg, w, make_inputs(cfg, seed))
        check_argmax(got, ids, load_golden(name)["last_hidden_state"])
    else:
        inp = make_inputs(cfg, seed, pad_fraction=pad)
        mod = build(cfg, w, frontend)
        got = run_module(mod, cfg, inp)
        mod.close()
    assert_parity(got, load_golden(name)["last_hidden_state"], name)


def run_t5(cfg, w, inp):
    """Decoder last hidden state [tokens, hidden] of the encoder-decoder, one launch."""
    text, names = t5_hlo(cfg)
    mod = compile_hlo(text, barrier_timeout_us=1000000)
    dw = t5_device_weights(cfg, w)
    mod.set_weights({names[k]: v for k, v in dw.items()})
    out = mod.run([inp["input_ids"], inp["decoder_input_ids"]])[0]
    mod.close()
    return out[: cfg.tokens * cfg.hidden].reshape(cfg.tokens, cfg.hidden).astype(np.float32)


@pytest.mark.parametrize("cfg", [
    t5_tiny(),                                                 # one layer per stack, one head, 32 tokens
    t5_tiny(batch=3, seq=64, layers=2, hidden=128, ffn=256),   # ragged rows (192), two heads
    t5_tiny(batch=1, seq=128, layers=1, hidden=192, ffn=384),  # a full 128-row tile, three heads
], ids=lambda c: f"b{c.batch}s{c.seq}h{c.hidden}l{c.layers}")
def test_t5_shapes_against_oracle(cfg):
    """Encoder-decoder: RMS LayerNorm, un-scaled scores with a per-(head, query, key) position
    bias (bidirectional in the encoder, causal in the decoder), cross-attention over the encoder
    output, bias-free projections; both stacks share stages until the decoder needs the encoder."""
    w = make_weights(cfg, 61, stress=True)
    inp = make_t5_inputs(cfg, 61)
    assert_parity(run_t5(cfg, w, inp), R.t5_model(cfg, w, inp), "T5 shape case")


def test_t5_small_full_size():
    """T5-small shape (6 + 6 layers, width 512, 8 heads, FFN 2048, vocab 32128), batch 1, 128 tokens."""
    cfg = t5_small()
    w = make_weights(cfg, 1239, stress=True)
    inp = make_t5_inputs(cfg, 1239)
    assert_parity(run_t5(cfg, w, inp), R.t5_model(cfg, w, inp), "T5-small b1 s128")


def run_vit(cfg, w, inp):
    text, names = vit_hlo(cfg)
    mod = compile_hlo(text, barrier_timeout_us=500000)
    mod.set_weights({names[k]: v for k, v in w.items()})
    out = mod.run([inp["pixel_values"]])[0]
    mod.close()
    return out[: cfg.tokens * cfg.hidden].reshape(cfg.tokens, cfg.hidden).astype(np.float32)


@pytest.mark.parametrize("cfg", [
    vit_tiny(),                                           # 4 patches + class token, one layer
    vit_tiny(batch=3, image=64, layers=2, hidden=128),    # 17 tokens, ragged rows
    vit_tiny(batch=2, image=224, layers=1, hidden=128),   # 197 tokens: two key chunks
], ids=lambda c: f"b{c.batch}img{c.image}h{c.hidden}l{c.layers}")
def test_vit_shapes_against_oracle(cfg):
    """Pre-LN vision encoder: patch convolution as patchify + GEMM, class token and positions
    assembled into the f32 residual stream, GEMMs accumulating into the stream."""
    w = make_weights(cfg, 41, stress=True)
    inp = make_vit_inputs(cfg, 41)
    assert_parity(run_vit(cfg, w, inp), R.vit_encoder(cfg, w, inp), "ViT shape case")


@pytest.mark.parametrize("cfg", [
    vit_tiny(batch=2, image=32, patch=7, patch_stride=4, patch_pad=3, hidden=128),  # 147-element windows -> 192
    vit_tiny(batch=1, image=48, patch=16, patch_stride=8),                          # overlap, no padding
    vit_tiny(batch=3, image=30, patch=8, patch_stride=8, patch_pad=1),              # padding only, 4x4 windows
], ids=lambda c: f"b{c.batch}img{c.image}k{c.patch}s{c.patch_stride}p{c.patch_pad}")
def test_strided_padded_patch_convolution_against_oracle(cfg):
    """The convolution in general form (stride != window, zero padding, a window that is not a
    whole number of 64-element blocks): window rows gathered with zeros at the edges, GEMM
    against the zero-extended filter."""
    w = make_weights(cfg, 43, stress=True)
    inp = make_vit_inputs(cfg, 43)
    assert_parity(run_vit(cfg, w, inp), R.vit_encoder(cfg, w, inp), "overlapping patch convolution")


def test_vit_base_full_size():
    cfg = vit_base()
    w = make_weights(cfg, 1236, stress=True)
    inp = make_vit_inputs(cfg, 1236)
    assert_parity(run_vit(cfg, w, inp), R.vit_encoder(cfg, w, inp), "ViT-B/16 b1")


@pytest.mark.parametrize("cfg", [
    bert_tiny(),                                                   # one 16-row tile, hidden 64
    bert_tiny(batch=3, seq=20, layers=2, hidden=128, ffn=512),     # ragged: 60 rows, 2 heads
    bert_tiny(batch=1, seq=128, layers=1, hidden=192, ffn=768),    # full 128-row tile, 3 heads
    bert_tiny(batch=2, seq=128, layers=1, hidden=128, ffn=512),    # two 128-row tiles
    bert_tiny(batch=5, seq=33, layers=1, hidden=64, ffn=256),      # rows straddle tile boundaries
    bert_tiny(batch=2, seq=200, layers=1, hidden=128, ffn=256),    # two key chunks, ragged second
    bert_tiny(batch=1, seq=384, layers=2, hidden=128, ffn=256),    # three key chunks, three row tiles
    bert_tiny(batch=3, seq=257, layers=1, hidden=64, ffn=256),     # third chunk holds a single key
], ids=lambda c: f"b{c.batch}s{c.seq}h{c.hidden}l{c.layers}")
def test_shapes_against_oracle(cfg):
    w = make_weights(cfg, 21, stress=True)
    inp = make_inputs(cfg, 21, pad_fraction=0.25)
    mod = build(cfg, w, "hlo")
    got = run_module(mod, cfg, inp)
    mod.close()
    assert_parity(got, R.bert_encoder(cfg, w, inp), "shape case")


@pytest.mark.parametrize("act", ["gelu_erf", "relu", "quick_gelu", "gelu_tanh"])
def test_activations(act):
    cfg = bert_tiny(seq=32, hidden=128, ffn=512)
    cfg.act = act
    w = make_weights(cfg, 5, stress=True)
    inp = make_inputs(cfg, 5)
    mod = build(cfg, w, "hlo")
    got = run_module(mod, cfg, inp)
    mod.close()
    assert_parity(got, R.bert_encoder(cfg, w, inp), act)


@pytest.fixture(scope="module")
def base():
    cfg = bert_base()
    w = make_weights(cfg, 1234, stress=True)
    text, names = bert_hlo(cfg)
    mod = compile_hlo(text, barrier_timeout_us=500000)
    mod.set_weights({names[k]: v for k, v in w.items()})
    yield cfg, w, mod
    mod.close()


def test_bert_base_full_size(base):
    cfg, w, mod = base
    inp = make_inputs(cfg, 1234)
    assert_parity(run_module(mod, cfg, inp), R.bert_encoder(cfg, w, inp), "BERT-base b1 s128")


def test_bert_base_reference_fixture_inputs(base):
    cfg, w, mod = base
    inp = reference_fixture_inputs()
    assert_parity(run_module(mod, cfg, inp), R.bert_encoder(cfg, w, inp), "bert_bs1 fixture inputs")


def test_bert_base_padding_mask(base):
    cfg, w, mod = base
    inp = make_inputs(cfg, 77, pad_fraction=0.25)
    got = run_module(mod, cfg, inp)
    assert_parity(got, R.bert_encoder(cfg, w, inp), "padding mask")
    # size-independent property: ids under the mask do not influence unmasked positions
    inp2 = {k: v.copy() for k, v in inp.items()}
    inp2["input_ids"][0, -5:] = 0
    got2 = run_module(mod, cfg, inp2)
    keep = inp["attention_mask"].reshape(-1) == 1
    assert np.abs(got[keep] - got2[keep]).max() <= 2e-2


def test_bert_base_relaunch_is_stable(base):
    """The f32 accumulators and the barrier epoch carry over between launches: the same
    inputs must give the same answer again (split-K sums are atomic, so allow rounding)."""
    cfg, w, mod = base
    inp = make_inputs(cfg, 3)
    a = run_module(mod, cfg, inp)
    for _ in range(3):
        mod.launch()
    b = run_module(mod, cfg, inp)
    assert np.abs(a - b).max() <= 4e-3


def test_bert_large_shape_two_layers_batch16():
    """BERT-large geometry (hidden 1024, 16 heads, FFN 4096, seq 384) at batch 16 = 6144 rows
    (48 row tiles), last quarter of every sequence padded; two layers keep the oracle quick."""
    cfg = EncoderConfig(layers=2, hidden=1024, heads=16, ffn=4096, batch=16, seq=384)
    w = make_weights(cfg, 1235, stress=True)
    inp = make_inputs(cfg, 1235, pad_fraction=0.25)
    mod = build(cfg, w, "hlo")
    got = run_module(mod, cfg, inp)
    mod.close()
    assert_parity(got, R.bert_encoder_torch(cfg, w, inp), "BERT-large geometry b16 s384")


def test_bert_large_full_depth_batch1():
    cfg = EncoderConfig(layers=24, hidden=1024, heads=16, ffn=4096, batch=1, seq=384)
    w = make_weights(cfg, 1235)
    inp = make_inputs(cfg, 1235, pad_fraction=0.25)
    mod = build(cfg, w, "builder")
    got = run_module(mod, cfg, inp)
    mod.close()
    assert_parity(got, R.bert_encoder_torch(cfg, w, inp), "BERT-large b1 s384")


def test_layernorm_output_statistics(base):
    # with gamma = 1 + small, beta small: every output row is close to zero mean, unit variance
    cfg, w, mod = base
    got = run_module(mod, cfg, make_inputs(cfg, 9))
    g, b = w[f"layer{cfg.layers - 1}.ffn.ln.gamma"], w[f"layer{cfg.layers - 1}.ffn.ln.beta"]
    z = (got - b) / g
    assert np.abs(z.mean(1)).max() < 2e-2 and np.abs(z.var(1) - 1).max() < 5e-2


def run_opt(cfg, w, inp):
    """(logits f32 [tokens, vocab], arg-max ids s32 [tokens]) of the decoder prefill."""
    text, names = opt_hlo(cfg)
    mod = compile_hlo(text, barrier_timeout_us=2000000)
    mod.set_weights({names[k]: v for k, v in w.items()})
    outs = mod.run([inp["input_ids"]])
    mod.close()
    logits = outs[0][: cfg.tokens * cfg.vocab].reshape(cfg.tokens, cfg.vocab)
    ids = outs[1].view(np.int32)[: cfg.tokens]
    return logits.astype(np.float32), ids


def check_argmax(logits, ids, ref_logits):
    """Token ids are bit-exact: equal to the first maximum of the device's own f16 logits on
    every row, and equal to the fp32 oracle's arg-max wherever the oracle's top-2 margin is
    larger than the f16 tolerance of the logits (a closer race is decided by rounding)."""
    assert np.array_equal(ids, logits.argmax(-1).astype(np.int32))
    top2 = np.sort(ref_logits, axis=-1)[:, -2:]
    clear = (top2[:, 1] - top2[:, 0]) > 2 * 2e-2
    assert clear.any()
    assert np.array_equal(ids[clear], ref_logits.argmax(-1)[clear].astype(np.int32))


@pytest.mark.parametrize("cfg", [
    opt_tiny(),                                                     # one layer, one head
    opt_tiny(batch=3, seq=40, layers=2, hidden=128, vocab=1008),    # ragged rows, vocab not a tile multiple
    opt_tiny(batch=2, seq=128, layers=1, hidden=256, ffn=1024, vocab=4096),
    opt_tiny(batch=1, seq=200, layers=1, hidden=128, vocab=512),    # causal mask across two key chunks
], ids=lambda c: f"b{c.batch}s{c.seq}h{c.hidden}v{c.vocab}")
def test_opt_shapes_against_oracle(cfg):
    """Pre-LN causal decoder: embedding rows (position offset 2) into the f32 stream, causal
    attention, LM head against the transposed token table, arg-max per position."""
    w = make_weights(cfg, 77, stress=True)
    inp = make_inputs(cfg, 77)
    logits, ids = run_opt(cfg, w, inp)
    ref, _ = R.opt_decoder(cfg, w, inp)
    assert_parity(logits, ref, "OPT shape case")
    check_argmax(logits, ids, ref)


def test_opt_wide_reduced_depth():
    """OPT-1.3B's widths (hidden 2048, 32 heads, FFN 8192, vocab 50272) on two layers: the
    three-pass LayerNorm for 2048 columns, the 50272-column LM head and its arg-max."""
    cfg = EncoderConfig(model="opt", layers=2, hidden=2048, heads=32, ffn=8192, vocab=50272, max_pos=2048,
                        types=0, batch=1, seq=128, eps=1e-5, act="relu")
    w = make_weights(cfg, 78)
    inp = make_inputs(cfg, 78)
    logits, ids = run_opt(cfg, w, inp)
    ref, _ = R.opt_decoder(cfg, w, inp)
    assert_parity(logits, ref, "OPT-1.3B widths, 2 layers")
    check_argmax(logits, ids, ref)


def run_clip(cfg, w, inp):
    """(logits_per_image [images, texts], image_embeds, text_embeds) as f32."""
    text, names = clip_hlo(cfg)
    mod = compile_hlo(text, barrier_timeout_us=2000000)
    mod.set_weights({names[k]: v for k, v in w.items()})
    outs = mod.run([inp["pixel_values"], inp["input_ids"]])
    mod.close()
    ni, nt, p = cfg.vision.batch, cfg.text.batch, cfg.proj
    return (outs[0][: ni * nt].reshape(ni, nt).astype(np.float32), outs[1][: ni * p].reshape(ni, p).astype(np.float32),
            outs[2][: nt * p].reshape(nt, p).astype(np.float32))


def check_clip(cfg, seed):
    w = make_weights(cfg, seed, stress=True)
    inp = make_clip_inputs(cfg, seed)
    # repeat the largest id inside some sequences: the pooled row is the first occurrence
    ids = inp["input_ids"]
    for b in range(0, cfg.text.batch, 2):
        ids[b, cfg.text.seq - 1] = ids[b].max()
    logits, img, txt = run_clip(cfg, w, inp)
    ref_logits, ref_img, ref_txt = R.clip_dual(cfg, w, inp)
    assert_parity(img, ref_img, "image embeddings")
    assert_parity(txt, ref_txt, "text embeddings")
    assert_parity(logits, ref_logits, "image-text logits")


@pytest.mark.parametrize("cfg", [
    clip_tiny(),                                                    # 5 image tokens, 12 text tokens
    clip_tiny(images=4, texts=7, image=96, layers=2, vh=128, th=128, seq=40, vocab=1000, proj=128),
    clip_tiny(images=2, texts=3, image=224, layers=1, vh=192, th=64, seq=77, vocab=49408, proj=64),
], ids=lambda c: f"i{c.vision.batch}t{c.text.batch}img{c.vision.image}s{c.text.seq}")
def test_clip_shapes_against_oracle(cfg):
    """Dual encoder: both towers scheduled into the same stages of one launch; LayerNorm that
    starts a residual stream, class-row LayerNorm, pooling at the largest token id, L2
    normalisation and the activation x activation logits product."""
    check_clip(cfg, 91)


def test_clip_b32_full_size():
    """CLIP ViT-B/32 shape, 32 images x 32 texts."""
    check_clip(clip_b32(), 1238)


@pytest.mark.parametrize("mode", ["off", "on"])
@pytest.mark.parametrize("cfg", [
    bert_tiny(batch=3, seq=40, layers=2, hidden=128, ffn=512),     # ragged rows, two heads, padded keys
    bert_tiny(batch=2, seq=128, layers=1, hidden=192, ffn=256),    # full 128-row tiles, three heads
    bert_tiny(batch=75, seq=16, layers=2, hidden=128, ffn=256),    # 150 items on 148 CTAs: two CTAs take a second item
], ids=lambda c: f"b{c.batch}s{c.seq}h{c.hidden}")
def test_projection_fusion_modes_agree_with_the_oracle(cfg, mode, tmp_path):
    """The Q/K/V projections as a stage of their own ("off") and computed inside the attention
    items ("on": x W_h accumulated in TMEM, converted on chip into the Q, K and V^T operand
    tiles) both meet the oracle."""
    import json
    from mononn_b200.module import describe
    w = make_weights(cfg, 55, stress=True)
    inp = make_inputs(cfg, 55, pad_fraction=0.25)
    text, names = bert_hlo(cfg)
    spec = describe("hlo", text)["spec"]
    spec["qkv_fusion"] = mode
    (tmp_path / "cluster_0").mkdir()
    (tmp_path / "cluster_0" / "best_tuning_spec.json").write_text(json.dumps(spec))
    mod = compile_hlo(text, spec_dir=str(tmp_path), barrier_timeout_us=500000)
    mod.set_weights({names[k]: v for k, v in w.items()})
    kinds = [[o["kind"] for o in st["ops"]] for st in mod.plan()["stages"]]
    assert (["gemm", "gemm", "gemm"] in kinds) == (mode == "off")
    got = run_module(mod, cfg, inp)
    mod.close()
    assert_parity(got, R.bert_encoder(cfg, w, inp), f"projection fusion {mode}")
