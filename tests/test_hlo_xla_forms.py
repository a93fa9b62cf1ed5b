"""The HLO front end on text in the forms XLA's GPU pipeline prints (no GPU except the last test).

tests/hlo/*.hlo hold one BERT layer rewritten by tests/hlo/make_fixtures.py: `erf` as a clamped
rational polynomial, `bitcast` for `reshape`, a layout `copy`, a multi-output fusion read through
get-tuple-element, a compare + select mask, converts moved and operands swapped, a pad / slice
and a dynamic-slice detour. Each must lower to the plan of the text this package authors; random
re-orderings of the instructions of a fused computation must not change the plan either."""
import importlib.util
import os
import re

import numpy as np
import pytest
from hypothesis import HealthCheck, given, settings, strategies as st

from mononn_b200 import bert_tiny, make_inputs, make_weights
from mononn_b200.hlo_builder import bert_hlo
from mononn_b200.module import describe
from tests.helpers import ROOT, assert_parity

HLO_DIR = os.path.join(ROOT, "tests", "hlo")


def _maker():
    spec = importlib.util.spec_from_file_location("make_fixtures", os.path.join(HLO_DIR, "make_fixtures.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def fixture(name):
    with open(os.path.join(HLO_DIR, f"bert_layer_{name}.hlo")) as f:
        return f.read()


def signature(plan):
    """What the device executes: stages, operators with geometry / flags / fused activation, and the
    constants with their packing. Tensor and fusion names (which follow HLO instruction names) are
    left out."""
    ops = [[(o["kind"], o["n_items"], o["flags"], o["act"], o.get("M"), o.get("N"), o.get("K"), o.get("n_tile"),
             o.get("k_split"), o.get("out_mode"), o.get("flag_target")) for o in s["ops"]] for s in plan["stages"]]
    consts = sorted((c["name"], c["kind"], c["src_bytes"]) for c in plan["constants"])
    return ops, consts, [(a["name"], a["bytes"], a["kind"]) for a in plan["args"]]


FORMS = ["erf_polynomial", "bitcast", "copy", "multi_output", "select_mask", "convert_moved", "pad_slice",
         "dynamic_slice", "all"]


def test_committed_fixtures_are_what_the_generator_writes(lib_built):
    made = _maker().fixtures()
    assert sorted(made) == sorted(FORMS + ["builder"])
    for name, text in made.items():
        assert fixture(name) == text, f"tests/hlo/bert_layer_{name}.hlo is stale: run tests/hlo/make_fixtures.py"


@pytest.mark.parametrize("form", FORMS)
def test_xla_forms_lower_to_the_builders_plan(lib_built, form):
    want = signature(describe("hlo", fixture("builder"))["plan"])
    got = signature(describe("hlo", fixture(form))["plan"])
    assert got == want


def test_expanded_erf_is_recognised_as_gelu(lib_built):
    text = fixture("erf_polynomial")
    assert " erf(" not in text and " clamp(" in text and " divide(" in text
    ops = {o["name"]: o for s in describe("hlo", text)["plan"]["stages"] for o in s["ops"]}
    assert ops["gemm_up_0"]["act"] == 1   # exact-erf GELU


def test_a_polynomial_that_is_not_erf_is_rejected(lib_built):
    from mononn_b200 import capi
    text = fixture("erf_polynomial").replace("constant(1.1283788184)", "constant(1.3)")
    with pytest.raises(capi.MononnError) as e:
        describe("hlo", text)
    assert e.value.code == -3 and "epilogue" in str(e.value)


def test_multi_output_fusion_is_split_per_element(lib_built):
    text = fixture("multi_output")
    assert "get-tuple-element" in text and "tuple(" in text
    plan = describe("hlo", text)["plan"]
    att = [o for s in plan["stages"] for o in s["ops"] if o["kind"] == "attention"]
    assert len(att) == 1 and att[0]["flags"] & (1 << 11)   # projections still fused into the attention items


def _reorder(text: str, comp: str, seed_order) -> str:
    """A random topological order of the instruction lines of fused computation `comp`."""
    m = re.search(r"(%" + re.escape(comp) + r" \([^\n]*\{\n)(.*?)(\n\}\n)", text, re.S)
    lines = m.group(2).split("\n")
    names = [re.match(r"\s*(?:ROOT )?%(\S+) =", ln).group(1) for ln in lines]
    deps = []
    for ln in lines:
        rhs = ln.split("=", 1)[1]
        deps.append({n for n in re.findall(r"%([\w.\-]+)", rhs) if n in names})
    done, out, pending = set(), [], list(range(len(lines)))
    prio = {i: seed_order[i % len(seed_order)] + i * 1e-6 for i in pending}
    while pending:
        ready = [i for i in pending if deps[i] <= done]
        pick = min(ready, key=lambda i: prio[i])
        out.append(lines[pick])
        done.add(names[pick])
        pending.remove(pick)
    return text.replace(m.group(0), m.group(1) + "\n".join(out) + m.group(3))


@settings(max_examples=12, deadline=None, derandomize=True, suppress_health_check=[HealthCheck.function_scoped_fixture])
@given(order=st.lists(st.floats(0, 1, allow_nan=False), min_size=8, max_size=40),
       comp=st.sampled_from(["fused_ln", "fused_softmax", "fused_bias_act", "fused_bias_split_qk", "fused_embed"]))
def test_instruction_order_inside_a_fusion_does_not_matter(lib_built, order, comp):
    base = fixture("all")
    want = signature(describe("hlo", base)["plan"])
    shuffled = _reorder(base, comp, order)
    assert signature(describe("hlo", shuffled)["plan"]) == want


@pytest.mark.gpu
def test_xla_style_text_runs_against_the_oracle():
    from mononn_b200 import compile_hlo
    from oracle import ref_encoder as R
    maker = _maker()
    cfg = bert_tiny(**maker.CFG)
    w = make_weights(cfg, 33, stress=True)
    inp = make_inputs(cfg, 33, pad_fraction=0.25)
    from mononn_b200.hlo_builder import bert_hlo
    names = bert_hlo(cfg)[1]   # weight name -> HLO constant name (the rewrites keep the constants)
    mod = compile_hlo(fixture("all"), barrier_timeout_us=500000)
    mod.set_weights({names[k]: v for k, v in w.items()})
    out = mod.run([inp["input_ids"], inp["attention_mask"], inp["token_type_ids"]])[0]
    mod.close()
    got = out[: cfg.tokens * cfg.hidden].reshape(cfg.tokens, cfg.hidden).astype(np.float32)
    assert_parity(got, R.bert_encoder(cfg, w, inp), "XLA-style HLO text")


def test_constants_printed_with_their_values_are_taken_from_the_text(lib_built):
    """XLA prints small constants with their values; `constant({...})` is only the elided form.
    Values are converted to the constant's element type exactly as numpy rounds them (ties to
    even, subnormals, infinities), and the module then needs no set_constant for that name."""
    cfg = bert_tiny(batch=2, seq=16, layers=1, hidden=64, ffn=128)
    text, names = bert_hlo(cfg)
    rng = np.random.default_rng(9)
    vals = np.concatenate([rng.normal(0, 1, 40), [0.0, -0.0, 65504.0, 1e6, -1e6, 6e-8, 3e-8, 2.98e-8, 6.1e-5, 1.0009765625,
                                                  1.00048828125, 1.00146484375, float("inf"), -float("inf")]]).astype(np.float64)
    vals = np.concatenate([vals, rng.normal(0, 1e-3, 64 - len(vals))])
    key = names["layer0.attn.q.b"]
    line = [l for l in text.splitlines() if f"%{key} =" in l][0]
    body = ", ".join("inf" if v == np.inf else "-inf" if v == -np.inf else repr(float(v)) for v in vals)
    d = describe("hlo", text.replace(line, line.replace("constant({...})", "constant({ /*i0=0*/ " + body + " })")))
    assert list(d["literals"]) == [key]
    got = np.frombuffer(bytes.fromhex(d["literals"][key]), dtype=np.float16)
    with np.errstate(over="ignore"):
        want = vals.astype(np.float32).astype(np.float16)
    assert got.tobytes() == want.tobytes()
    # a literal of the wrong length is not taken (the constant stays to be set by the caller)
    short = line.replace("constant({...})", "constant({1, 2, 3})")
    assert describe("hlo", text.replace(line, short))["literals"] == {}


@pytest.mark.gpu
def test_a_module_runs_with_constants_taken_from_the_text():
    """Every bias and LayerNorm vector is printed with its values; only the matrices are set."""
    from mononn_b200 import compile_hlo
    from oracle import ref_encoder as R
    cfg = bert_tiny(batch=2, seq=24, layers=1, hidden=128, ffn=256)
    w = make_weights(cfg, 35, stress=True)
    inp = make_inputs(cfg, 35, pad_fraction=0.25)
    text, names = bert_hlo(cfg)
    printed = [k for k, v in w.items() if v.ndim == 1]
    assert len(printed) >= 10
    for k in printed:
        line = [l for l in text.splitlines() if f"%{names[k]} =" in l][0]
        body = ", ".join(repr(float(x)) for x in w[k].astype(np.float32))
        text = text.replace(line, line.replace("constant({...})", "constant({" + body + "})"))
    mod = compile_hlo(text, barrier_timeout_us=500000)
    for k, v in w.items():
        if k not in printed:
            mod.set_constant(names[k], np.asarray(v).astype(np.float16))
    out = mod.run([inp["input_ids"], inp["attention_mask"], inp["token_type_ids"]])[0]
    mod.close()
    got = out[: cfg.tokens * cfg.hidden].reshape(cfg.tokens, cfg.hidden).astype(np.float32)
    assert_parity(got, R.bert_encoder(cfg, w, inp), "constants from the text")
