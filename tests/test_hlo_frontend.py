"""HLO text front end (no GPU): parsing, fusion recognition by hypothesis + numeric check,
and rejection of what the path does not support."""
import pytest

from mononn_b200 import bert_tiny, capi
from mononn_b200.hlo_builder import bert_hlo
from mononn_b200.models import EncoderConfig
from mononn_b200.module import describe


def lower(text):
    return describe("hlo", text)["plan"]


@pytest.fixture(scope="module")
def tiny_text(lib_built):
    return bert_hlo(bert_tiny())[0]


def test_module_name_and_arguments(tiny_text):
    p = lower(tiny_text)
    assert p["module"] == "cluster_0"
    names = [a["name"] for a in p["args"]]
    assert names == ["input_ids", "attention_mask", "token_type_ids", "last_hidden_state", "temp_buffer"]
    assert [a["bytes"] for a in p["args"][:4]] == [64, 64, 64, 16 * 64 * 2]


def test_constants_keep_their_hlo_names_and_shapes(tiny_text):
    consts = {c["name"]: c for c in lower(tiny_text)["constants"]}
    assert consts["embeddings.word"]["src_bytes"] == 100 * 64 * 2
    assert consts["layer0.ffn.up.w"]["kind"] == "pack_b" and consts["layer0.ffn.up.w"]["K"] == 64
    assert consts["layer0.ffn.up.b"]["kind"] == "raw"


@pytest.mark.parametrize("act,code", [("gelu_erf", 1), ("relu", 2), ("quick_gelu", 3), ("gelu_tanh", 4)])
def test_activation_is_recognised_from_the_arithmetic(lib_built, act, code):
    cfg = bert_tiny()
    cfg.act = act
    ops = {o["name"]: o for s in lower(bert_hlo(cfg)[0])["stages"] for o in s["ops"]}
    assert ops["gemm_up_0"]["act"] == code


def test_recognition_does_not_depend_on_operand_order(tiny_text):
    # commute the bias add and the GELU product; the numeric check still identifies them
    t = tiny_text.replace("%y = f16[16,256]{1,0} add(f16[16,256]{1,0} %x, f16[16,256]{1,0} %bb)",
                          "%y = f16[16,256]{1,0} add(f16[16,256]{1,0} %bb, f16[16,256]{1,0} %x)")
    t = t.replace("%act = f32[16,256]{1,0} multiply(f32[16,256]{1,0} %g4, f32[16,256]{1,0} %g3)",
                  "%act = f32[16,256]{1,0} multiply(f32[16,256]{1,0} %g3, f32[16,256]{1,0} %g4)")
    assert t != tiny_text
    ops = {o["name"]: o for s in lower(t)["stages"] for o in s["ops"]}
    assert ops["gemm_up_0"]["act"] == 1 and ops["gemm_up_0"]["flags"] & 1


def test_layernorm_eps_is_read_from_the_module(lib_built):
    cfg = bert_tiny()
    cfg.eps = 1e-5
    text = bert_hlo(cfg)[0]
    assert "constant(1e-05)" in text
    lower(text)  # recognised with the other epsilon


def test_wrong_arithmetic_is_rejected_not_guessed(tiny_text):
    # an activation that is none of the supported ones
    bad = tiny_text.replace("%g2 = f32[16,256]{1,0} erf(", "%g2 = f32[16,256]{1,0} tanh(")
    with pytest.raises(capi.MononnError) as e:
        lower(bad)
    assert e.value.code == -3 and "fused_bias_act" in str(e.value)
    # a softmax that forgets to subtract the maximum is still a softmax mathematically, so it
    # is accepted; one that normalises by the maximum instead of the sum is not
    bad = tiny_text.replace("divide(f32[1,1,16,16]{3,2,1,0} %e, f32[1,1,16,16]{3,2,1,0} %esum_b)",
                            "divide(f32[1,1,16,16]{3,2,1,0} %e, f32[1,1,16,16]{3,2,1,0} %zmax_b)")
    with pytest.raises(capi.MononnError) as e:
        lower(bad)
    assert e.value.code == -3 and "softmax" in str(e.value)


def test_unsupported_constructs_name_the_instruction(tiny_text):
    bad = tiny_text.replace('custom_call_target="__cublas$gemm"', 'custom_call_target="__cudnn$convForward"', 1)
    with pytest.raises(capi.MononnError) as e:
        lower(bad)
    assert e.value.code == -3 and "gemm.q.0" in str(e.value)
    bad = tiny_text.replace("s32[1,16]{1,0} parameter(0)", "s32[1,<=16]{1,0} parameter(0)", 1)
    with pytest.raises(capi.MononnError) as e:
        lower(bad)
    assert e.value.code == -2  # dynamic dimension
    with pytest.raises(capi.MononnError) as e:
        lower("HloModule m\n\nENTRY %e () -> f16[1] {\n  ROOT %c = f16[1]{0} constant({...})\n}\n")
    assert e.value.code == -3


def test_parse_errors_carry_the_line(lib_built):
    with pytest.raises(capi.MononnError) as e:
        lower("HloModule m\n\nENTRY %e (p: f16[4]) -> f16[4] {\n  %p = f16[4]{0} parameter(0)\n  ROOT %r = f16[4]{0} add(f16[4]{0} %p, f16[4]{0} %nope)\n}\n")
    assert e.value.code == -2 and "nope" in str(e.value)
    with pytest.raises(capi.MononnError) as e:
        lower("this is not hlo")
    assert e.value.code == -2


def test_padding_mask_and_batches(lib_built):
    cfg = EncoderConfig(layers=1, hidden=128, heads=2, ffn=256, vocab=50, max_pos=40, batch=3, seq=20)
    p = lower(bert_hlo(cfg)[0])
    att = [o for s in p["stages"] for o in s["ops"] if o["kind"] == "attention"][0]
    assert att["n_items"] == 3 * 2 and att["flags"] & 0x10
