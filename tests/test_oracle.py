"""The CPU restatement (oracle/) against the golden vectors and against itself."""
import numpy as np
import pytest

from mononn_b200.models import (EncoderConfig, bert_tiny, make_clip_inputs, make_inputs, make_vit_inputs,
                                make_weights)
from oracle import ref_encoder as R
from tests.helpers import golden_cases, load_golden


@pytest.mark.parametrize("name", sorted(golden_cases()))
def test_oracle_matches_golden_vectors(name):
    cfg, seed, stress, pad = golden_cases()[name]
    g = load_golden(name)
    w = make_weights(cfg, seed, stress=stress)
    if cfg.model == "vit":
        out = R.vit_encoder(cfg, w, make_vit_inputs(cfg, seed))
    elif cfg.model == "clip":
        out, img, txt = R.clip_dual(cfg, w, make_clip_inputs(cfg, seed))
        assert np.allclose(np.linalg.norm(img, axis=-1), 1.0, atol=1e-5)
    elif cfg.model == "t5":
        from mononn_b200.models import make_t5_inputs
        out = R.t5_model(cfg, w, make_t5_inputs(cfg, seed))
    elif cfg.model == "opt":
        out, ids = R.opt_decoder(cfg, w, make_inputs(cfg, seed))
        assert np.array_equal(ids, g["last_hidden_state"].argmax(-1))  # the stored array holds the logits
    else:
        out = R.bert_encoder(cfg, w, make_inputs(cfg, seed, pad_fraction=pad))
    ref = g["last_hidden_state"]
    assert out.shape == ref.shape
    # two fp32 implementations of the same definition: agreement to rounding
    assert np.abs(out - ref).max() < 2e-4


def test_numpy_and_torch_restatements_agree():
    cfg = bert_tiny(batch=2, seq=24, layers=2, hidden=128, ffn=512)
    w = make_weights(cfg, 5, stress=True)
    inp = make_inputs(cfg, 5, pad_fraction=0.25)
    a = R.bert_encoder(cfg, w, inp)
    b = R.bert_encoder_torch(cfg, w, inp, threads=1)
    assert np.abs(a - b).max() < 2e-4


def test_torch_variants_of_vit_and_opt_agree_with_the_numpy_ones():
    """The full-size GPU parity cases use the torch-CPU variants (seconds instead of minutes);
    here they are pinned to the numpy restatement, which the golden vectors pin in turn."""
    from mononn_b200.models import opt_tiny, vit_tiny
    cfg = vit_tiny(batch=2, image=48, layers=2, hidden=128, ffn=256)
    w = make_weights(cfg, 6, stress=True)
    inp = make_vit_inputs(cfg, 6)
    assert np.abs(R.vit_encoder(cfg, w, inp) - R.vit_encoder_torch(cfg, w, inp, threads=1)).max() < 2e-4
    cfg = opt_tiny(batch=2, seq=24, layers=2, hidden=128, vocab=1008)
    w = make_weights(cfg, 7, stress=True)
    inp = make_inputs(cfg, 7)
    a, ia = R.opt_decoder(cfg, w, inp)
    b, ib = R.opt_decoder_torch(cfg, w, inp, threads=1)
    assert np.abs(a - b).max() < 2e-4
    margin = np.sort(a, -1)[:, -1] - np.sort(a, -1)[:, -2]
    assert np.array_equal(ia[margin > 1e-3], ib[margin > 1e-3])


def test_mask_changes_only_through_masked_keys():
    cfg = bert_tiny(seq=16)
    w = make_weights(cfg, 3, stress=True)
    inp = make_inputs(cfg, 3, pad_fraction=0.25)
    base = R.bert_encoder(cfg, w, inp)
    # changing a masked-out token id must not change any unmasked position
    inp2 = {k: v.copy() for k, v in inp.items()}
    inp2["input_ids"][0, -1] = (inp2["input_ids"][0, -1] + 1) % cfg.vocab
    other = R.bert_encoder(cfg, w, inp2)
    keep = inp["attention_mask"].reshape(-1) == 1
    assert np.abs(base[keep] - other[keep]).max() < 1e-5


def test_causal_decoder_ignores_later_tokens():
    from mononn_b200.models import opt_tiny
    cfg = opt_tiny(batch=1, seq=12)
    w = make_weights(cfg, 8, stress=True)
    inp = make_inputs(cfg, 8)
    base, _ = R.opt_decoder(cfg, w, inp)
    inp2 = {k: v.copy() for k, v in inp.items()}
    inp2["input_ids"][0, 7] = (inp2["input_ids"][0, 7] + 1) % cfg.vocab
    other, _ = R.opt_decoder(cfg, w, inp2)
    assert np.abs(base[:7] - other[:7]).max() == 0.0   # positions before the change are untouched
    assert np.abs(base[7:] - other[7:]).max() > 1e-4


def test_dual_encoder_pools_the_first_largest_id():
    from mononn_b200.models import clip_tiny
    cfg = clip_tiny()
    w = make_weights(cfg, 4, stress=True)
    inp = make_clip_inputs(cfg, 4)
    ids = inp["input_ids"]
    ids[:, :] = 5
    ids[:, 3] = 150
    base = R.clip_dual(cfg, w, inp)[2]
    ids[:, 9] = 150                      # a later tie does not move the pooled row ...
    causal_same = R.clip_dual(cfg, w, inp)[2]
    assert np.abs(base - causal_same).max() < 1e-6   # ... and, being causal, row 3 does not see it
    ids[:, 1] = 150                      # an earlier one does
    assert np.abs(base - R.clip_dual(cfg, w, inp)[2]).max() > 1e-4


def test_layer_norm_eps_and_biased_variance():
    x = np.array([[1.0, 2.0, 3.0, 6.0]], np.float32)
    y = R.layer_norm(x, np.ones(4, np.float32), np.zeros(4, np.float32), 1e-12)
    assert abs(float(y.mean())) < 1e-6
    assert abs(float((y ** 2).mean()) - 1.0) < 1e-5  # biased variance -> unit second moment


def test_gelu_is_the_exact_erf_form():
    x = np.linspace(-4, 4, 33, dtype=np.float32)
    import math
    want = np.array([0.5 * v * (1 + math.erf(v / math.sqrt(2))) for v in x], np.float32)
    assert np.abs(R.gelu_erf(x) - want).max() < 1e-6


def test_weights_are_f16_representable_and_seeded():
    cfg = bert_tiny()
    a, b = make_weights(cfg, 9), make_weights(cfg, 9)
    for k in a:
        assert np.array_equal(a[k], b[k])
        assert np.array_equal(a[k].astype(np.float16).astype(np.float32), a[k])
    assert not np.array_equal(make_weights(cfg, 10)["embeddings.word"], a["embeddings.word"])


@pytest.mark.parametrize("patch,stride,pad,image", [(7, 4, 3, 32), (16, 8, 0, 48), (8, 8, 1, 30), (16, 16, 0, 32)])
def test_window_rows_times_filter_is_the_convolution(patch, stride, pad, image):
    """The oracle writes the patch convolution as window rows times the [out, ky*kx*c] filter;
    pinned here against torch's conv2d (cross-correlation, zero padding) on the same numbers."""
    import torch
    from mononn_b200.models import vit_tiny
    cfg = vit_tiny(batch=2, image=image, patch=patch, patch_stride=stride, patch_pad=pad)
    rng = np.random.default_rng(5)
    px = rng.uniform(-1, 1, (2, 3, image, image)).astype(np.float32)
    wt = rng.normal(0, 0.1, (cfg.hidden, patch, patch, 3)).astype(np.float32)     # [out, ky, kx, in]
    got = R.vit_patches(cfg, px) @ wt.reshape(cfg.hidden, -1).T
    want = torch.nn.functional.conv2d(torch.from_numpy(px), torch.from_numpy(wt).permute(0, 3, 1, 2).contiguous(),
                                      stride=stride, padding=pad)               # [B, out, gy, gx]
    g = cfg.patch_grid
    assert want.shape == (2, cfg.hidden, g, g)
    np.testing.assert_allclose(got, want.permute(0, 2, 3, 1).reshape(-1, cfg.hidden).numpy(), rtol=1e-4, atol=1e-4)
