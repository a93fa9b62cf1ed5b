"""The size points of the five configurations that the smaller cases do not reach (-m gpu):
BERT-large 24 layers at batch 16, ViT-B/16 at batch 64, the OPT-1.3B-shaped prefill at full
depth for batch 1 and batch 8. Each runs as one launch through the C ABI and is compared with the
fp32 CPU oracle (its torch variants, which tests/test_oracle.py pins to the numpy restatement) at
the tolerance of tests/helpers.py; token ids are checked as in test_gpu_parity.check_argmax and the
share of rows whose fp32 top-2 margin is decisive is printed."""
import numpy as np
import pytest

from mononn_b200 import compile_hlo, make_inputs, make_vit_inputs, make_weights, opt_1p3b, vit_base
from mononn_b200.hlo_builder import opt_hlo
from mononn_b200.models import EncoderConfig
from oracle import ref_encoder as R
from tests.helpers import assert_parity
from tests.test_gpu_parity import build, check_argmax, run_module, run_vit

pytestmark = pytest.mark.gpu


def test_bert_large_full_depth_batch16():
    cfg = EncoderConfig(layers=24, hidden=1024, heads=16, ffn=4096, batch=16, seq=384)
    w = make_weights(cfg, 1235)
    inp = make_inputs(cfg, 1235, pad_fraction=0.25)
    mod = build(cfg, w, "hlo")
    got = run_module(mod, cfg, inp)
    mod.close()
    err, cos = assert_parity(got, R.bert_encoder_torch(cfg, w, inp), "BERT-large b16 s384, 24 layers")
    print(f"BERT-large b16: max-abs {err:.5f} cosine {cos:.6f}")


def test_vit_base_batch64():
    cfg = vit_base(batch=64)
    w = make_weights(cfg, 1236, stress=True)
    inp = make_vit_inputs(cfg, 1236)
    err, cos = assert_parity(run_vit(cfg, w, inp), R.vit_encoder_torch(cfg, w, inp), "ViT-B/16 b64")
    print(f"ViT-B/16 b64: max-abs {err:.5f} cosine {cos:.6f}")


@pytest.fixture(scope="module")
def opt_weights():
    return make_weights(opt_1p3b(), 1237)


@pytest.mark.parametrize("batch", [1, 8])
def test_opt_1p3b_full_depth(opt_weights, batch):
    cfg = opt_1p3b(batch=batch)
    inp = make_inputs(cfg, 1237)
    text, names = opt_hlo(cfg)
    mod = compile_hlo(text, barrier_timeout_us=2000000)
    mod.set_weights({names[k]: v for k, v in opt_weights.items()})
    outs = mod.run([inp["input_ids"]])
    mod.close()
    logits = outs[0][: cfg.tokens * cfg.vocab].reshape(cfg.tokens, cfg.vocab).astype(np.float32)
    ids = outs[1].view(np.int32)[: cfg.tokens]
    ref, ref_ids = R.opt_decoder_torch(cfg, opt_weights, inp)
    err, cos = assert_parity(logits, ref, f"OPT-1.3B b{batch} s128, 24 layers")
    check_argmax(logits, ids, ref)
    top2 = np.sort(ref, axis=-1)[:, -2:]
    clear = int(((top2[:, 1] - top2[:, 0]) > 2 * 2e-2).sum())
    agree = int((ids == ref_ids).sum())
    print(f"OPT-1.3B b{batch}: max-abs {err:.5f} cosine {cos:.6f}; rows with a decisive fp32 margin "
          f"{clear}/{cfg.tokens}; ids equal to the fp32 arg-max on {agree}/{cfg.tokens} rows")
