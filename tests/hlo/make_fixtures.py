"""Writes tests/hlo/*.hlo: one BERT layer in the forms XLA's GPU pipeline prints it.

    python tests/hlo/make_fixtures.py

No XLA dump of the example models exists offline, so the fixtures are made from the HLO text
this package authors (mononn_b200.hlo_builder.bert_hlo) by rewriting it into the shapes the
reference's parser has to accept (mononn_engine/parser/ir_parser_fused.cc:319-539, op list
mononn_engine/core/op/op_type.h:20-65):

  erf_polynomial   `erf` expanded into a clamped rational polynomial in x^2 (XLA has no erf
                   instruction on the GPU path of that TensorFlow version); the coefficients
                   are a least-squares fit made for this fixture (max error 3e-7), evaluated by
                   Horner's rule with explicit multiply / add / divide / clamp instructions
  bitcast          `reshape` printed as `bitcast`
  copy             a layout `copy` after the head-merge transpose
  multi_output     the Q and K bias + head-split fusions merged into one fusion that returns a
                   tuple, read through get-tuple-element
  select_mask      the additive attention mask built with compare + select instead of (1 - m) * c
  convert_moved    LayerNorm scale / shift converted to f32 after the broadcast, operands of the
                   commutative ops swapped
  pad_slice        the FFN activation padded by eight columns and sliced back (`pad`, `slice`)
  dynamic_slice    the same value taken through a `dynamic-slice` with constant zero offsets
  all              everything above at once
"""
import os
import re
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from mononn_b200 import bert_tiny  # noqa: E402
from mononn_b200.hlo_builder import bert_hlo  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))
CFG = dict(batch=2, seq=24, layers=1, hidden=128, ffn=256)

# erf(x) ~ x * A(x^2) / B(x^2) for |x| <= 4 (clamped outside): weighted linear least squares on
# 4001 points, refitted 20 times with weights 1 / B
ALPHA = [1.1283788184, 0.20619341715, 0.051396516305, 0.003968846111, 0.00014828774811, -1.9773976869e-06,
         1.9659607112e-08]
BETA = [1.0, 0.51606330704, 0.11758625898, 0.014887363477, 0.0010212098438]


def base_text():
    return bert_hlo(bert_tiny(**CFG))[0]


def erf_polynomial(text: str) -> str:
    m = re.search(r"  %g2 = (\S+) erf\(\S+ %g1\)\n", text)
    shp = m.group(1)
    L = []

    def c(name, v):
        L.append(f"  %{name}_s = f32[] constant({v!r})")
        L.append(f"  %{name} = {shp} broadcast(f32[] %{name}_s), dimensions={{}}")

    c("e_lo", -4.0)
    c("e_hi", 4.0)
    L.append(f"  %e_x = {shp} clamp({shp} %e_lo, {shp} %g1, {shp} %e_hi)")
    L.append(f"  %e_u = {shp} multiply({shp} %e_x, {shp} %e_x)")
    for tag, coef in (("ea", ALPHA), ("eb", BETA)):
        c(f"{tag}{len(coef) - 1}", coef[-1])
        acc = f"{tag}{len(coef) - 1}"
        for i in range(len(coef) - 2, -1, -1):
            c(f"{tag}{i}", coef[i])
            L.append(f"  %{tag}m{i} = {shp} multiply({shp} %{acc}, {shp} %e_u)")
            L.append(f"  %{tag}p{i} = {shp} add({shp} %{tag}m{i}, {shp} %{tag}{i})")
            acc = f"{tag}p{i}"
    L.append(f"  %e_num = {shp} multiply({shp} %e_x, {shp} %eap0)")
    L.append(f"  %g2 = {shp} divide({shp} %e_num, {shp} %ebp0)")
    return text.replace(m.group(0), "\n".join(L) + "\n")


def bitcast(text: str) -> str:
    return re.sub(r"\breshape\(", "bitcast(", text)


def copy(text: str) -> str:
    m = re.search(r"  %t = (\S+) transpose\((\S+) %x\), dimensions=\{0,2,1,3\}\n  ROOT %r = (\S+) reshape\(\S+ %t\)", text)
    assert m
    new = (f"  %t = {m.group(1)} transpose({m.group(2)} %x), dimensions={{0,2,1,3}}\n"
           f"  %tc = {m.group(1)} copy({m.group(1)} %t)\n  ROOT %r = {m.group(3)} reshape({m.group(1)} %tc)")
    return text.replace(m.group(0), new)


def multi_output(text: str) -> str:
    m = re.search(r"%fused_bias_split \(p0: (\S+), p1: (\S+)\) -> (\S+) \{\n(.*?)\n\}\n", text, re.S)
    x_s, b_s, out_s = m.group(1), m.group(2), m.group(3)
    body = m.group(4)
    mid = re.search(r"%r = (\S+) reshape", body).group(1)

    def half(tag, px, pb):
        return (f"  %x{tag} = {x_s} parameter({px})\n  %b{tag} = {b_s} parameter({pb})\n"
                f"  %bb{tag} = {x_s} broadcast({b_s} %b{tag}), dimensions={{1}}\n"
                f"  %y{tag} = {x_s} add({x_s} %x{tag}, {x_s} %bb{tag})\n"
                f"  %r{tag} = {mid} reshape({x_s} %y{tag})\n"
                f"  %t{tag} = {out_s} transpose({mid} %r{tag}), dimensions={{0,2,1,3}}\n")
    comp = (f"%fused_bias_split_qk (p0: {x_s}, p1: {b_s}, p2: {x_s}, p3: {b_s}) -> ({out_s}, {out_s}) {{\n"
            + half("q", 0, 1) + half("k", 2, 3) +
            f"  ROOT %qk = ({out_s}, {out_s}) tuple({out_s} %tq, {out_s} %tk)\n}}\n\n")
    text = text.replace("%fused_bias_split (", comp + "%fused_bias_split (", 1)
    q = re.search(r"  %fusion\.q\.0 = \S+ fusion\((\S+ %gemm\.q\.0), (\S+ %layer0\.attn\.q\.b)\), kind=kLoop, calls=%fused_bias_split\n", text)
    k = re.search(r"  %fusion\.k\.0 = \S+ fusion\((\S+ %gemm\.k\.0), (\S+ %layer0\.attn\.k\.b)\), kind=kLoop, calls=%fused_bias_split\n", text)
    text = text.replace(q.group(0), "")
    tup = f"({out_s}, {out_s})"
    text = text.replace(k.group(0),
                        f"  %fusion.qk.0 = {tup} fusion({q.group(1)}, {q.group(2)}, {k.group(1)}, {k.group(2)}), "
                        f"kind=kLoop, calls=%fused_bias_split_qk\n"
                        f"  %fusion.q.0 = {out_s} get-tuple-element({tup} %fusion.qk.0), index=0\n"
                        f"  %fusion.k.0 = {out_s} get-tuple-element({tup} %fusion.qk.0), index=1\n")
    return text


def select_mask(text: str) -> str:
    m = re.search(r"%fused_mask \(p0: (\S+)\) -> (\S+) \{\n.*?\n\}\n", text, re.S)
    i_s, f_s = m.group(1), m.group(2)
    p_s = f_s.replace("f32", "pred")
    new = (f"%fused_mask (p0: {i_s}) -> {f_s} {{\n  %m = {i_s} parameter(0)\n"
           f"  %zero_i_s = s32[] constant(0)\n  %zero_i = {i_s} broadcast(s32[] %zero_i_s), dimensions={{}}\n"
           f"  %is_pad = {p_s} compare({i_s} %m, {i_s} %zero_i), direction=EQ\n"
           f"  %neg_s = f32[] constant(-10000)\n  %neg = {f_s} broadcast(f32[] %neg_s), dimensions={{}}\n"
           f"  %zero_s = f32[] constant(0)\n  %zero = {f_s} broadcast(f32[] %zero_s), dimensions={{}}\n"
           f"  ROOT %bias = {f_s} select({p_s} %is_pad, {f_s} %neg, {f_s} %zero)\n}}\n")
    return text.replace(m.group(0), new)


def convert_moved(text: str) -> str:
    # gamma / beta: broadcast in f16, then convert (the builder converts first)
    def fix(match):
        fv, hv, s2 = match.group(1), match.group(2), match.group(3)
        h2 = s2.replace("f32", "f16")
        return (f"  %gamma_h = {h2} broadcast({hv} %gamma), dimensions={{1}}\n"
                f"  %beta_h = {h2} broadcast({hv} %beta), dimensions={{1}}\n"
                f"  %gamma_b = {s2} convert({h2} %gamma_h)\n  %beta_b = {s2} convert({h2} %beta_h)\n")
    text = re.sub(r"  %gamma32 = (\S+) convert\((\S+) %gamma\)\n  %beta32 = \S+ convert\(\S+ %beta\)\n"
                  r"  %gamma_b = (\S+) broadcast\(\S+ %gamma32\), dimensions=\{1\}\n"
                  r"  %beta_b = \S+ broadcast\(\S+ %beta32\), dimensions=\{1\}\n", fix, text)
    # swap the operands of commutative instructions in the LayerNorm and epilogue fusions
    text = re.sub(r"(%scaled = \S+ multiply)\((\S+ %norm), (\S+ %gamma_b)\)", r"\1(\3, \2)", text)
    text = re.sub(r"(%shifted = \S+ add)\((\S+ %scaled), (\S+ %beta_b)\)", r"\1(\3, \2)", text)
    text = re.sub(r"(ROOT %yr = \S+ add)\((\S+ %y), (\S+ %res)\)", r"\1(\3, \2)", text)
    return text


def _after_act_input(text: str, build) -> str:
    """Replaces `%y32 = convert(%y)` of the bias + activation fusion by a detour through `build`."""
    m = re.search(r"  %y32 = (\S+) convert\((\S+) %y\)\n", text)
    f_s, h_s = m.group(1), m.group(2)
    rows, cols = (int(v) for v in re.match(r"f16\[(\d+),(\d+)\]", h_s).groups())
    return text.replace(m.group(0), build(f_s, h_s, rows, cols) + f"  %y32 = {f_s} convert({h_s} %yd)\n")


def pad_slice(text: str) -> str:
    def build(f_s, h_s, rows, cols):
        wide = f"f16[{rows},{cols + 8}]{{1,0}}"
        return (f"  %pad_v = f16[] constant(0)\n  %yw = {wide} pad({h_s} %y, f16[] %pad_v), padding=0_0x0_8\n"
                f"  %yd = {h_s} slice({wide} %yw), slice={{[0:{rows}], [0:{cols}]}}\n")
    return _after_act_input(text, build)


def dynamic_slice(text: str) -> str:
    def build(f_s, h_s, rows, cols):
        return (f"  %ds_zero = s32[] constant(0)\n"
                f"  %yd = {h_s} dynamic-slice({h_s} %y, s32[] %ds_zero, s32[] %ds_zero), "
                f"dynamic_slice_sizes={{{rows},{cols}}}\n")
    return _after_act_input(text, build)


REWRITES = {"erf_polynomial": erf_polynomial, "bitcast": bitcast, "copy": copy, "multi_output": multi_output,
            "select_mask": select_mask, "convert_moved": convert_moved, "pad_slice": pad_slice,
            "dynamic_slice": dynamic_slice}


def fixtures() -> dict:
    base = base_text()
    out = {"builder": base}
    for name, fn in REWRITES.items():
        out[name] = fn(base)
        assert out[name] != base, name
    allt = base
    for name in ("erf_polynomial", "copy", "multi_output", "select_mask", "convert_moved", "pad_slice", "bitcast"):
        allt = REWRITES[name](allt)
    out["all"] = allt
    return out


if __name__ == "__main__":
    for name, text in fixtures().items():
        with open(os.path.join(HERE, f"bert_layer_{name}.hlo"), "w") as f:
            f.write(text)
        print(name, len(text))
