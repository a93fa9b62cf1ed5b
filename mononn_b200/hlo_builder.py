"""Authors the XLA HLO text of the example encoder graphs.

The reference receives a post-optimisation XLA-GPU module from TensorFlow: an ENTRY
computation made of parameters, constants (the frozen weights), kLoop/kInput fusions and
``__cublas$gemm`` custom-calls (mononn_engine/parser/ir_parser_fused.cc:319-385; example
GEMM HLO in mononn_engine/core/op_impl/gemm_impl.cc:290-316).  No dump of the example models
exists offline and TensorFlow is absent, so this module writes that text for the model
definitions of examples/utils/save_model.py:44-110: same op vocabulary
(mononn_engine/core/op/op_type.h:20-65, plus the newer ``erf`` opcode), same
``backend_config`` JSON keys (gemm_impl.cc:182-231), f16 storage with f32 reductions as
TensorFlow's auto_mixed_precision graph rewrite produces (examples/run_mononn.py:44).

Large constants are written the way XLA prints them when literals are elided:
``constant({...})``; their values are supplied separately through ``mononn_set_constant``.
"""
from __future__ import annotations

import json

from .models import ClipConfig, EncoderConfig


class _Emitter:
    def __init__(self):
        self.comps: list[str] = []
        self.entry: list[str] = []
        self._n = 0

    def uid(self, stem: str) -> str:
        self._n += 1
        return f"{stem}.{self._n}"


def _shape(dtype: str, dims) -> str:
    dims = list(dims)
    layout = ",".join(str(i) for i in reversed(range(len(dims))))
    return f"{dtype}[{','.join(str(d) for d in dims)}]" + ("{" + layout + "}" if dims else "")


def _gemm_config(alpha: float, lhs_c: int, rhs_c: int, batch_dims, batch_size: int, lhs_stride: int,
                 rhs_stride: int) -> str:
    cfg = {
        "alpha_real": alpha, "alpha_imag": 0, "beta": 0,
        "dot_dimension_numbers": {
            "lhs_contracting_dimensions": [str(lhs_c)], "rhs_contracting_dimensions": [str(rhs_c)],
            "lhs_batch_dimensions": [str(d) for d in batch_dims],
            "rhs_batch_dimensions": [str(d) for d in batch_dims]},
        "batch_size": str(batch_size), "lhs_stride": str(lhs_stride), "rhs_stride": str(rhs_stride),
        "selected_algorithm": "-1",
    }
    return json.dumps(json.dumps(cfg, separators=(",", ":")))  # quoted + escaped, as XLA prints it


_REGIONS = """%region_add (a: f32[], b: f32[]) -> f32[] {
  %a = f32[] parameter(0)
  %b = f32[] parameter(1)
  ROOT %add = f32[] add(f32[] %a, f32[] %b)
}

%region_max (a: f32[], b: f32[]) -> f32[] {
  %a = f32[] parameter(0)
  %b = f32[] parameter(1)
  ROOT %max = f32[] maximum(f32[] %a, f32[] %b)
}
"""


def _activation_lines(kind: str, x: str, shp: str) -> tuple[list[str], str]:
    """f32 elementwise activation on value `x` of printed shape `shp`."""
    def c(name, v):
        return [f"  %{name}_s = f32[] constant({v})",
                f"  %{name} = {shp} broadcast(f32[] %{name}_s), dimensions={{}}"]
    L: list[str] = []
    if kind == "gelu_erf":
        L += c("half", 0.5) + c("rsqrt2", 0.70710678118654752) + c("one", 1)
        L += [f"  %g1 = {shp} multiply({shp} %{x}, {shp} %rsqrt2)",
              f"  %g2 = {shp} erf({shp} %g1)",
              f"  %g3 = {shp} add({shp} %g2, {shp} %one)",
              f"  %g4 = {shp} multiply({shp} %{x}, {shp} %half)",
              f"  %act = {shp} multiply({shp} %g4, {shp} %g3)"]
    elif kind == "relu":
        L += c("zero", 0)
        L += [f"  %act = {shp} maximum({shp} %{x}, {shp} %zero)"]
    elif kind == "quick_gelu":
        L += c("k", -1.702) + c("one", 1)
        L += [f"  %q1 = {shp} multiply({shp} %{x}, {shp} %k)",
              f"  %q2 = {shp} exponential({shp} %q1)",
              f"  %q3 = {shp} add({shp} %q2, {shp} %one)",
              f"  %act = {shp} divide({shp} %{x}, {shp} %q3)"]
    elif kind == "gelu_tanh":
        L += c("half", 0.5) + c("one", 1) + c("c0", 0.7978845608028654) + c("c1", 0.044715)
        L += [f"  %t1 = {shp} multiply({shp} %{x}, {shp} %{x})",
              f"  %t2 = {shp} multiply({shp} %t1, {shp} %{x})",
              f"  %t3 = {shp} multiply({shp} %t2, {shp} %c1)",
              f"  %t4 = {shp} add({shp} %{x}, {shp} %t3)",
              f"  %t5 = {shp} multiply({shp} %t4, {shp} %c0)",
              f"  %t6 = {shp} tanh({shp} %t5)",
              f"  %t7 = {shp} add({shp} %t6, {shp} %one)",
              f"  %t8 = {shp} multiply({shp} %{x}, {shp} %half)",
              f"  %act = {shp} multiply({shp} %t8, {shp} %t7)"]
    else:
        raise ValueError(kind)
    return L, "act"


def _ln_body(rows: int, cols: int, eps: float, x32: str) -> list[str]:
    """LayerNorm over the last dim of f32 value `x32` [rows, cols]; result in %ln (f16)."""
    s2, s1 = _shape("f32", [rows, cols]), _shape("f32", [rows])
    h2, hv, fv = _shape("f16", [rows, cols]), _shape("f16", [cols]), _shape("f32", [cols])
    return [
        f"  %zero = f32[] constant(0)",
        f"  %inv_n_s = f32[] constant({1.0 / cols!r})",
        f"  %inv_n = {s1} broadcast(f32[] %inv_n_s), dimensions={{}}",
        f"  %eps_s = f32[] constant({eps!r})",
        f"  %eps = {s1} broadcast(f32[] %eps_s), dimensions={{}}",
        f"  %sum = {s1} reduce({s2} %{x32}, f32[] %zero), dimensions={{1}}, to_apply=%region_add",
        f"  %mean = {s1} multiply({s1} %sum, {s1} %inv_n)",
        f"  %mean_b = {s2} broadcast({s1} %mean), dimensions={{0}}",
        f"  %cent = {s2} subtract({s2} %{x32}, {s2} %mean_b)",
        f"  %sq = {s2} multiply({s2} %cent, {s2} %cent)",
        f"  %sqsum = {s1} reduce({s2} %sq, f32[] %zero), dimensions={{1}}, to_apply=%region_add",
        f"  %var = {s1} multiply({s1} %sqsum, {s1} %inv_n)",
        f"  %var_eps = {s1} add({s1} %var, {s1} %eps)",
        f"  %rstd = {s1} rsqrt({s1} %var_eps)",
        f"  %rstd_b = {s2} broadcast({s1} %rstd), dimensions={{0}}",
        f"  %norm = {s2} multiply({s2} %cent, {s2} %rstd_b)",
        f"  %gamma32 = {fv} convert({hv} %gamma)",
        f"  %beta32 = {fv} convert({hv} %beta)",
        f"  %gamma_b = {s2} broadcast({fv} %gamma32), dimensions={{1}}",
        f"  %beta_b = {s2} broadcast({fv} %beta32), dimensions={{1}}",
        f"  %scaled = {s2} multiply({s2} %norm, {s2} %gamma_b)",
        f"  %shifted = {s2} add({s2} %scaled, {s2} %beta_b)",
        f"  ROOT %ln = {h2} convert({s2} %shifted)",
    ]


def bert_hlo(cfg: EncoderConfig) -> tuple[str, dict[str, str]]:
    """HLO text of the BERT encoder of `cfg` and the map weight name -> HLO constant name."""
    B, S, H, F, NH = cfg.batch, cfg.seq, cfg.hidden, cfg.ffn, cfg.heads
    D = H // NH
    T = B * S
    em = _Emitter()
    comps: list[str] = [_REGIONS]
    entry: list[str] = []
    names: dict[str, str] = {}

    def const(name: str, dims) -> str:
        names[name] = name
        entry.append(f"  %{name} = {_shape('f16', dims)} constant({{...}})")
        return name

    h_TH, h_H = _shape("f16", [T, H]), _shape("f16", [H])
    f_TH = _shape("f32", [T, H])
    i_BS, i_T = _shape("s32", [B, S]), _shape("s32", [T])

    entry.append(f"  %input_ids = {i_BS} parameter(0)")
    entry.append(f"  %attention_mask = {i_BS} parameter(1)")
    entry.append(f"  %token_type_ids = {i_BS} parameter(2)")

    # ---- embeddings: gather + position + type, then LayerNorm
    word = const("embeddings.word", [cfg.vocab, H])
    pos = const("embeddings.position", [cfg.max_pos, H])
    typ = const("embeddings.token_type", [cfg.types, H])
    g0 = const("embeddings.ln.gamma", [H])
    b0 = const("embeddings.ln.beta", [H])
    h_SH, h_BSH = _shape("f16", [S, H]), _shape("f16", [B, S, H])
    comps.append(f"""%fused_embed (p0: {i_BS}, p1: {i_BS}, p2: {_shape('f16', [cfg.vocab, H])}, p3: {_shape('f16', [cfg.max_pos, H])}, p4: {_shape('f16', [cfg.types, H])}) -> {h_TH} {{
  %ids = {i_BS} parameter(0)
  %types = {i_BS} parameter(1)
  %word = {_shape('f16', [cfg.vocab, H])} parameter(2)
  %pos = {_shape('f16', [cfg.max_pos, H])} parameter(3)
  %type = {_shape('f16', [cfg.types, H])} parameter(4)
  %gw = {h_BSH} gather({_shape('f16', [cfg.vocab, H])} %word, {i_BS} %ids), offset_dims={{2}}, collapsed_slice_dims={{0}}, start_index_map={{0}}, index_vector_dim=2, slice_sizes={{1,{H}}}
  %gt = {h_BSH} gather({_shape('f16', [cfg.types, H])} %type, {i_BS} %types), offset_dims={{2}}, collapsed_slice_dims={{0}}, start_index_map={{0}}, index_vector_dim=2, slice_sizes={{1,{H}}}
  %pos_s = {h_SH} slice({_shape('f16', [cfg.max_pos, H])} %pos), slice={{[0:{S}], [0:{H}]}}
  %pos_b = {h_BSH} broadcast({h_SH} %pos_s), dimensions={{1,2}}
  %e1 = {h_BSH} add({h_BSH} %gw, {h_BSH} %pos_b)
  %e2 = {h_BSH} add({h_BSH} %e1, {h_BSH} %gt)
  ROOT %e3 = {h_TH} reshape({h_BSH} %e2)
}}
""")
    entry.append(f"  %fusion.embed = {h_TH} fusion({i_BS} %input_ids, {i_BS} %token_type_ids, "
                 f"{_shape('f16', [cfg.vocab, H])} %{word}, {_shape('f16', [cfg.max_pos, H])} %{pos}, "
                 f"{_shape('f16', [cfg.types, H])} %{typ}), kind=kLoop, calls=%fused_embed")
    comps.append(f"%fused_ln (p0: {h_TH}, p1: {h_H}, p2: {h_H}) -> {h_TH} {{\n"
                 f"  %x = {h_TH} parameter(0)\n  %gamma = {h_H} parameter(1)\n  %beta = {h_H} parameter(2)\n"
                 f"  %x32 = {f_TH} convert({h_TH} %x)\n" + "\n".join(_ln_body(T, H, cfg.eps, "x32")) + "\n}\n")
    entry.append(f"  %fusion.embed_ln = {h_TH} fusion({h_TH} %fusion.embed, {h_H} %{g0}, {h_H} %{b0}), "
                 f"kind=kInput, calls=%fused_ln")
    # ---- additive attention mask (1 - m) * -10000, f32 [B, S]
    f_BS = _shape("f32", [B, S])
    comps.append(f"""%fused_mask (p0: {i_BS}) -> {f_BS} {{
  %m = {i_BS} parameter(0)
  %mf = {f_BS} convert({i_BS} %m)
  %one_s = f32[] constant(1)
  %one = {f_BS} broadcast(f32[] %one_s), dimensions={{}}
  %neg_s = f32[] constant(-10000)
  %neg = {f_BS} broadcast(f32[] %neg_s), dimensions={{}}
  %inv = {f_BS} subtract({f_BS} %one, {f_BS} %mf)
  ROOT %bias = {f_BS} multiply({f_BS} %inv, {f_BS} %neg)
}}
""")
    entry.append(f"  %fusion.mask = {f_BS} fusion({i_BS} %attention_mask), kind=kLoop, calls=%fused_mask")

    # ---- shared fused computations of the layers
    h_heads, h_BShd = _shape("f16", [B, NH, S, D]), _shape("f16", [B, S, NH, D])
    comps.append(f"""%fused_bias_split (p0: {h_TH}, p1: {h_H}) -> {h_heads} {{
  %x = {h_TH} parameter(0)
  %b = {h_H} parameter(1)
  %bb = {h_TH} broadcast({h_H} %b), dimensions={{1}}
  %y = {h_TH} add({h_TH} %x, {h_TH} %bb)
  %r = {h_BShd} reshape({h_TH} %y)
  ROOT %t = {h_heads} transpose({h_BShd} %r), dimensions={{0,2,1,3}}
}}
""")
    h_sc, f_sc, f_row = _shape("f16", [B, NH, S, S]), _shape("f32", [B, NH, S, S]), _shape("f32", [B, NH, S])
    comps.append(f"""%fused_softmax (p0: {h_sc}, p1: {f_BS}) -> {h_sc} {{
  %s = {h_sc} parameter(0)
  %mask = {f_BS} parameter(1)
  %s32 = {f_sc} convert({h_sc} %s)
  %mask_b = {f_sc} broadcast({f_BS} %mask), dimensions={{0,3}}
  %z = {f_sc} add({f_sc} %s32, {f_sc} %mask_b)
  %ninf = f32[] constant(-inf)
  %zmax = {f_row} reduce({f_sc} %z, f32[] %ninf), dimensions={{3}}, to_apply=%region_max
  %zmax_b = {f_sc} broadcast({f_row} %zmax), dimensions={{0,1,2}}
  %zc = {f_sc} subtract({f_sc} %z, {f_sc} %zmax_b)
  %e = {f_sc} exponential({f_sc} %zc)
  %zero = f32[] constant(0)
  %esum = {f_row} reduce({f_sc} %e, f32[] %zero), dimensions={{3}}, to_apply=%region_add
  %esum_b = {f_sc} broadcast({f_row} %esum), dimensions={{0,1,2}}
  %p = {f_sc} divide({f_sc} %e, {f_sc} %esum_b)
  ROOT %p16 = {h_sc} convert({f_sc} %p)
}}
""")
    comps.append(f"""%fused_merge (p0: {h_heads}) -> {h_TH} {{
  %x = {h_heads} parameter(0)
  %t = {h_BShd} transpose({h_heads} %x), dimensions={{0,2,1,3}}
  ROOT %r = {h_TH} reshape({h_BShd} %t)
}}
""")
    comps.append(f"%fused_bias_resid_ln (p0: {h_TH}, p1: {h_H}, p2: {h_TH}, p3: {h_H}, p4: {h_H}) -> {h_TH} {{\n"
                 f"  %x = {h_TH} parameter(0)\n  %b = {h_H} parameter(1)\n  %res = {h_TH} parameter(2)\n"
                 f"  %gamma = {h_H} parameter(3)\n  %beta = {h_H} parameter(4)\n"
                 f"  %bb = {h_TH} broadcast({h_H} %b), dimensions={{1}}\n"
                 f"  %y = {h_TH} add({h_TH} %x, {h_TH} %bb)\n"
                 f"  %yr = {h_TH} add({h_TH} %y, {h_TH} %res)\n"
                 f"  %x32 = {f_TH} convert({h_TH} %yr)\n" + "\n".join(_ln_body(T, H, cfg.eps, "x32")) + "\n}\n")
    h_TF, h_F, f_TF = _shape("f16", [T, F]), _shape("f16", [F]), _shape("f32", [T, F])
    act_lines, act_name = _activation_lines(cfg.act, "y32", f_TF)
    comps.append(f"%fused_bias_act (p0: {h_TF}, p1: {h_F}) -> {h_TF} {{\n"
                 f"  %x = {h_TF} parameter(0)\n  %b = {h_F} parameter(1)\n"
                 f"  %bb = {h_TF} broadcast({h_F} %b), dimensions={{1}}\n"
                 f"  %y = {h_TF} add({h_TF} %x, {h_TF} %bb)\n"
                 f"  %y32 = {f_TF} convert({h_TF} %y)\n" + "\n".join(act_lines) + "\n"
                 f"  ROOT %out = {h_TF} convert({f_TF} %{act_name})\n}}\n")

    def gemm(name: str, a: str, a_shape, w: str, w_shape, out_shape, alpha=1.0, lhs_c=1, rhs_c=0,
             batch_dims=(), batch=1, ls=0, rs=0) -> str:
        entry.append(f"  %{name} = {_shape('f16', out_shape)} custom-call({_shape('f16', a_shape)} %{a}, "
                     f"{_shape('f16', w_shape)} %{w}), custom_call_target=\"__cublas$gemm\", "
                     f"backend_config={_gemm_config(alpha, lhs_c, rhs_c, batch_dims, batch, ls, rs)}")
        return name

    x = "fusion.embed_ln"
    for l in range(cfg.layers):
        p = f"layer{l}."
        heads = {}
        for n in ("q", "k", "v"):
            w = const(p + f"attn.{n}.w", [H, H])
            b = const(p + f"attn.{n}.b", [H])
            gname = gemm(f"gemm.{n}.{l}", x, [T, H], w, [H, H], [T, H], ls=T * H, rs=H * H)
            entry.append(f"  %fusion.{n}.{l} = {h_heads} fusion({h_TH} %{gname}, {h_H} %{b}), kind=kLoop, "
                         f"calls=%fused_bias_split")
            heads[n] = f"fusion.{n}.{l}"
        sc = gemm(f"gemm.scores.{l}", heads["q"], [B, NH, S, D], heads["k"], [B, NH, S, D], [B, NH, S, S],
                  alpha=1.0 / (D ** 0.5), lhs_c=3, rhs_c=3, batch_dims=(0, 1), batch=B * NH, ls=S * D, rs=S * D)
        entry.append(f"  %fusion.softmax.{l} = {h_sc} fusion({h_sc} %{sc}, {f_BS} %fusion.mask), kind=kInput, "
                     f"calls=%fused_softmax")
        pv = gemm(f"gemm.pv.{l}", f"fusion.softmax.{l}", [B, NH, S, S], heads["v"], [B, NH, S, D],
                  [B, NH, S, D], lhs_c=3, rhs_c=2, batch_dims=(0, 1), batch=B * NH, ls=S * S, rs=S * D)
        entry.append(f"  %fusion.ctx.{l} = {h_TH} fusion({h_heads} %{pv}), kind=kLoop, calls=%fused_merge")
        wo, bo = const(p + "attn.o.w", [H, H]), const(p + "attn.o.b", [H])
        g1, be1 = const(p + "attn.ln.gamma", [H]), const(p + "attn.ln.beta", [H])
        go = gemm(f"gemm.o.{l}", f"fusion.ctx.{l}", [T, H], wo, [H, H], [T, H], ls=T * H, rs=H * H)
        entry.append(f"  %fusion.attn_ln.{l} = {h_TH} fusion({h_TH} %{go}, {h_H} %{bo}, {h_TH} %{x}, {h_H} %{g1}, "
                     f"{h_H} %{be1}), kind=kInput, calls=%fused_bias_resid_ln")
        x1 = f"fusion.attn_ln.{l}"
        w1, b1 = const(p + "ffn.up.w", [H, F]), const(p + "ffn.up.b", [F])
        gu = gemm(f"gemm.up.{l}", x1, [T, H], w1, [H, F], [T, F], ls=T * H, rs=H * F)
        entry.append(f"  %fusion.act.{l} = {h_TF} fusion({h_TF} %{gu}, {h_F} %{b1}), kind=kLoop, calls=%fused_bias_act")
        w2, b2 = const(p + "ffn.down.w", [F, H]), const(p + "ffn.down.b", [H])
        g2, be2 = const(p + "ffn.ln.gamma", [H]), const(p + "ffn.ln.beta", [H])
        gd = gemm(f"gemm.down.{l}", f"fusion.act.{l}", [T, F], w2, [F, H], [T, H], ls=T * F, rs=F * H)
        entry.append(f"  %fusion.ffn_ln.{l} = {h_TH} fusion({h_TH} %{gd}, {h_H} %{b2}, {h_TH} %{x1}, {h_H} %{g2}, "
                     f"{h_H} %{be2}), kind=kInput, calls=%fused_bias_resid_ln")
        x = f"fusion.ffn_ln.{l}"
    out_shape = _shape("f16", [B, S, H])
    entry.append(f"  ROOT %last_hidden_state = {out_shape} bitcast({h_TH} %{x})")

    text = (f"HloModule {cfg.name}, entry_computation_layout={{({i_BS}, {i_BS}, {i_BS})->{out_shape}}}\n\n"
            + "\n".join(comps)
            + f"\nENTRY %{cfg.name}_main (input_ids: {i_BS}, attention_mask: {i_BS}, token_type_ids: {i_BS}) "
              f"-> {out_shape} {{\n" + "\n".join(entry) + "\n}\n")
    return text, names


def _preln_blocks(cfg: EncoderConfig, comps: list, entry: list, const, x: str, causal: bool, tag: str = "",
                  final_ln: bool = True) -> str:
    """Appends the fused computations and the entry instructions of `cfg.layers` pre-LN
    transformer blocks plus the final LayerNorm, reading the [tokens, hidden] f16 value `x`;
    returns the name of the final LayerNorm fusion. With `causal` the softmax fusion masks
    keys after the query position (iota/compare/select, as XLA prints a causal mask). `tag`
    prefixes every computation, instruction and constant name (models with two towers); without
    `final_ln` the name of the last residual value is returned instead."""
    B, S, H, F, NH = cfg.batch, cfg.seq, cfg.hidden, cfg.ffn, cfg.heads
    D, T = H // NH, cfg.batch * cfg.seq
    h_TH, h_H, f_TH = _shape("f16", [T, H]), _shape("f16", [H]), _shape("f32", [T, H])
    comps.append(f"%{tag}fused_ln (p0: {h_TH}, p1: {h_H}, p2: {h_H}) -> {h_TH} {{\n"
                 f"  %x = {h_TH} parameter(0)\n  %gamma = {h_H} parameter(1)\n  %beta = {h_H} parameter(2)\n"
                 f"  %x32 = {f_TH} convert({h_TH} %x)\n" + "\n".join(_ln_body(T, H, cfg.eps, "x32")) + "\n}\n")
    h_heads, h_BShd = _shape("f16", [B, NH, S, D]), _shape("f16", [B, S, NH, D])
    comps.append(f"""%{tag}fused_bias_split (p0: {h_TH}, p1: {h_H}) -> {h_heads} {{
  %x = {h_TH} parameter(0)
  %b = {h_H} parameter(1)
  %bb = {h_TH} broadcast({h_H} %b), dimensions={{1}}
  %y = {h_TH} add({h_TH} %x, {h_TH} %bb)
  %r = {h_BShd} reshape({h_TH} %y)
  ROOT %t = {h_heads} transpose({h_BShd} %r), dimensions={{0,2,1,3}}
}}
""")
    h_sc, f_sc, f_row = _shape("f16", [B, NH, S, S]), _shape("f32", [B, NH, S, S]), _shape("f32", [B, NH, S])
    i_sc, p_sc = _shape("s32", [B, NH, S, S]), _shape("pred", [B, NH, S, S])
    if causal:
        causal_lines = (f"  %qi = {i_sc} iota(), iota_dimension=2\n  %ki = {i_sc} iota(), iota_dimension=3\n"
                        f"  %keep = {p_sc} compare({i_sc} %qi, {i_sc} %ki), direction=GE\n"
                        f"  %ninf_b = {f_sc} broadcast(f32[] %ninf), dimensions={{}}\n"
                        f"  %z = {f_sc} select({p_sc} %keep, {f_sc} %z0, {f_sc} %ninf_b)")
    else:
        causal_lines = f"  %z = {f_sc} copy({f_sc} %z0)"
    comps.append(f"""%{tag}fused_softmax (p0: {h_sc}) -> {h_sc} {{
  %s = {h_sc} parameter(0)
  %z0 = {f_sc} convert({h_sc} %s)
  %ninf = f32[] constant(-inf)
{causal_lines}
  %zmax = {f_row} reduce({f_sc} %z, f32[] %ninf), dimensions={{3}}, to_apply=%region_max
  %zmax_b = {f_sc} broadcast({f_row} %zmax), dimensions={{0,1,2}}
  %zc = {f_sc} subtract({f_sc} %z, {f_sc} %zmax_b)
  %e = {f_sc} exponential({f_sc} %zc)
  %zero = f32[] constant(0)
  %esum = {f_row} reduce({f_sc} %e, f32[] %zero), dimensions={{3}}, to_apply=%region_add
  %esum_b = {f_sc} broadcast({f_row} %esum), dimensions={{0,1,2}}
  %p = {f_sc} divide({f_sc} %e, {f_sc} %esum_b)
  ROOT %p16 = {h_sc} convert({f_sc} %p)
}}
""")
    comps.append(f"""%{tag}fused_merge (p0: {h_heads}) -> {h_TH} {{
  %x = {h_heads} parameter(0)
  %t = {h_BShd} transpose({h_heads} %x), dimensions={{0,2,1,3}}
  ROOT %r = {h_TH} reshape({h_BShd} %t)
}}
""")
    comps.append(f"""%{tag}fused_bias_resid (p0: {h_TH}, p1: {h_H}, p2: {h_TH}) -> {h_TH} {{
  %x = {h_TH} parameter(0)
  %b = {h_H} parameter(1)
  %res = {h_TH} parameter(2)
  %bb = {h_TH} broadcast({h_H} %b), dimensions={{1}}
  %y = {h_TH} add({h_TH} %x, {h_TH} %bb)
  ROOT %yr = {h_TH} add({h_TH} %y, {h_TH} %res)
}}
""")
    h_TF, h_F, f_TF = _shape("f16", [T, F]), _shape("f16", [F]), _shape("f32", [T, F])
    act_lines, act_name = _activation_lines(cfg.act, "y32", f_TF)
    comps.append(f"%{tag}fused_bias_act (p0: {h_TF}, p1: {h_F}) -> {h_TF} {{\n"
                 f"  %x = {h_TF} parameter(0)\n  %b = {h_F} parameter(1)\n"
                 f"  %bb = {h_TF} broadcast({h_F} %b), dimensions={{1}}\n"
                 f"  %y = {h_TF} add({h_TF} %x, {h_TF} %bb)\n"
                 f"  %y32 = {f_TF} convert({h_TF} %y)\n" + "\n".join(act_lines) + "\n"
                 f"  ROOT %out = {h_TF} convert({f_TF} %{act_name})\n}}\n")

    def gemm(name, a, a_shape, w, w_shape, out_shape, alpha=1.0, lhs_c=1, rhs_c=0, batch_dims=(), batch=1,
             ls=0, rs=0):
        entry.append(f"  %{name} = {_shape('f16', out_shape)} custom-call({_shape('f16', a_shape)} %{a}, "
                     f"{_shape('f16', w_shape)} %{w}), custom_call_target=\"__cublas$gemm\", "
                     f"backend_config={_gemm_config(alpha, lhs_c, rhs_c, batch_dims, batch, ls, rs)}")
        return name

    for l in range(cfg.layers):
        p = f"{tag}layer{l}."
        g1, b1 = const(p + "ln1.gamma", [H]), const(p + "ln1.beta", [H])
        entry.append(f"  %{tag}fusion.ln1.{l} = {h_TH} fusion({h_TH} %{x}, {h_H} %{g1}, {h_H} %{b1}), kind=kInput, calls=%{tag}fused_ln")
        heads = {}
        for n in ("q", "k", "v"):
            w = const(p + f"attn.{n}.w", [H, H])
            b = const(p + f"attn.{n}.b", [H])
            gname = gemm(f"{tag}gemm.{n}.{l}", f"{tag}fusion.ln1.{l}", [T, H], w, [H, H], [T, H], ls=T * H, rs=H * H)
            entry.append(f"  %{tag}fusion.{n}.{l} = {h_heads} fusion({h_TH} %{gname}, {h_H} %{b}), kind=kLoop, "
                         f"calls=%{tag}fused_bias_split")
            heads[n] = f"{tag}fusion.{n}.{l}"
        sc = gemm(f"{tag}gemm.scores.{l}", heads["q"], [B, NH, S, D], heads["k"], [B, NH, S, D], [B, NH, S, S],
                  alpha=1.0 / (D ** 0.5), lhs_c=3, rhs_c=3, batch_dims=(0, 1), batch=B * NH, ls=S * D, rs=S * D)
        entry.append(f"  %{tag}fusion.softmax.{l} = {h_sc} fusion({h_sc} %{sc}), kind=kInput, calls=%{tag}fused_softmax")
        pv = gemm(f"{tag}gemm.pv.{l}", f"{tag}fusion.softmax.{l}", [B, NH, S, S], heads["v"], [B, NH, S, D], [B, NH, S, D],
                  lhs_c=3, rhs_c=2, batch_dims=(0, 1), batch=B * NH, ls=S * S, rs=S * D)
        entry.append(f"  %{tag}fusion.ctx.{l} = {h_TH} fusion({h_heads} %{pv}), kind=kLoop, calls=%{tag}fused_merge")
        wo, bo = const(p + "attn.o.w", [H, H]), const(p + "attn.o.b", [H])
        go = gemm(f"{tag}gemm.o.{l}", f"{tag}fusion.ctx.{l}", [T, H], wo, [H, H], [T, H], ls=T * H, rs=H * H)
        entry.append(f"  %{tag}fusion.res1.{l} = {h_TH} fusion({h_TH} %{go}, {h_H} %{bo}, {h_TH} %{x}), kind=kLoop, "
                     f"calls=%{tag}fused_bias_resid")
        x = f"{tag}fusion.res1.{l}"
        g2, b2 = const(p + "ln2.gamma", [H]), const(p + "ln2.beta", [H])
        entry.append(f"  %{tag}fusion.ln2.{l} = {h_TH} fusion({h_TH} %{x}, {h_H} %{g2}, {h_H} %{b2}), kind=kInput, calls=%{tag}fused_ln")
        w1, bb1 = const(p + "ffn.up.w", [H, F]), const(p + "ffn.up.b", [F])
        gu = gemm(f"{tag}gemm.up.{l}", f"{tag}fusion.ln2.{l}", [T, H], w1, [H, F], [T, F], ls=T * H, rs=H * F)
        entry.append(f"  %{tag}fusion.act.{l} = {h_TF} fusion({h_TF} %{gu}, {h_F} %{bb1}), kind=kLoop, calls=%{tag}fused_bias_act")
        w2, bb2 = const(p + "ffn.down.w", [F, H]), const(p + "ffn.down.b", [H])
        gd = gemm(f"{tag}gemm.down.{l}", f"{tag}fusion.act.{l}", [T, F], w2, [F, H], [T, H], ls=T * F, rs=F * H)
        entry.append(f"  %{tag}fusion.res2.{l} = {h_TH} fusion({h_TH} %{gd}, {h_H} %{bb2}, {h_TH} %{x}), kind=kLoop, "
                     f"calls=%{tag}fused_bias_resid")
        x = f"{tag}fusion.res2.{l}"
    if not final_ln:
        return x
    gf, bf = const(tag + "ln.gamma", [H]), const(tag + "ln.beta", [H])
    entry.append(f"  %{tag}fusion.lnf = {h_TH} fusion({h_TH} %{x}, {h_H} %{gf}, {h_H} %{bf}), kind=kInput, calls=%{tag}fused_ln")
    return f"{tag}fusion.lnf"


def vit_hlo(cfg: EncoderConfig) -> tuple[str, dict[str, str]]:
    """HLO text of the pre-LN vision encoder (ViT) of `cfg`: NCHW f32 pixels, patch embedding as
    a ``__cudnn$convForward`` custom-call on the NHWC f16 image (window = stride = patch, or an
    overlapping zero-padded window when the configuration sets ``patch_stride`` / ``patch_pad``;
    mononn_engine/parser/ir_parser_fused.cc:749-823), class token + learned positions, pre-LN
    blocks, final LayerNorm (model of examples/utils/save_model.py:76-82)."""
    B, S, H, F, NH = cfg.batch, cfg.seq, cfg.hidden, cfg.ffn, cfg.heads
    D, T, C, IMG, PS = H // NH, cfg.batch * cfg.seq, cfg.channels, cfg.image, cfg.patch
    G = cfg.patch_grid
    P = G * G
    assert S == P + 1
    ST, PAD = cfg.patch_stride or PS, cfg.patch_pad
    window = f"size={PS}x{PS} stride={ST}x{ST}" + (f" pad={PAD}_{PAD}x{PAD}_{PAD}" if PAD else "")
    comps: list[str] = [_REGIONS]
    entry: list[str] = []
    names: dict[str, str] = {}

    def const(name: str, dims) -> str:
        names[name] = name
        entry.append(f"  %{name} = {_shape('f16', dims)} constant({{...}})")
        return name

    h_TH, h_H, f_TH = _shape("f16", [T, H]), _shape("f16", [H]), _shape("f32", [T, H])
    px_s, nhwc_s = _shape("f32", [B, C, IMG, IMG]), _shape("f16", [B, IMG, IMG, C])
    entry.append(f"  %pixel_values = {px_s} parameter(0)")
    comps.append(f"""%fused_nhwc (p0: {px_s}) -> {nhwc_s} {{
  %x = {px_s} parameter(0)
  %t = {_shape('f32', [B, IMG, IMG, C])} transpose({px_s} %x), dimensions={{0,2,3,1}}
  ROOT %c = {nhwc_s} convert({_shape('f32', [B, IMG, IMG, C])} %t)
}}
""")
    entry.append(f"  %fusion.nhwc = {nhwc_s} fusion({px_s} %pixel_values), kind=kLoop, calls=%fused_nhwc")
    wp = const("embeddings.patch.w", [H, PS, PS, C])
    bp = const("embeddings.patch.b", [H])
    cls = const("embeddings.cls", [1, H])
    pos = const("embeddings.position", [S, H])
    conv_s = _shape("f16", [B, G, G, H])
    conv_cfg = json.dumps(json.dumps({"conv_result_scale": 1, "side_input_scale": 0, "activation_mode": "0",
                                      "tensor_ops_enabled": True}, separators=(",", ":")))
    entry.append(f"  %conv.patch = ({conv_s}, u8[0]{{0}}) custom-call({nhwc_s} %fusion.nhwc, "
                 f"{_shape('f16', [H, PS, PS, C])} %{wp}), window={{{window}}}, "
                 f"dim_labels=b01f_o01i->b01f, custom_call_target=\"__cudnn$convForward\", backend_config={conv_cfg}")
    entry.append(f"  %gte.patch = {conv_s} get-tuple-element(({conv_s}, u8[0]{{0}}) %conv.patch), index=0")
    h_BPH, h_BSH, h_B1H, h_SH = (_shape("f16", [B, P, H]), _shape("f16", [B, S, H]), _shape("f16", [B, 1, H]),
                                 _shape("f16", [S, H]))
    comps.append(f"""%fused_tokens (p0: {conv_s}, p1: {h_H}, p2: {_shape('f16', [1, H])}, p3: {h_SH}) -> {h_TH} {{
  %y = {conv_s} parameter(0)
  %b = {h_H} parameter(1)
  %cls = {_shape('f16', [1, H])} parameter(2)
  %pos = {h_SH} parameter(3)
  %yr = {h_BPH} reshape({conv_s} %y)
  %bb = {h_BPH} broadcast({h_H} %b), dimensions={{2}}
  %yb = {h_BPH} add({h_BPH} %yr, {h_BPH} %bb)
  %cls_b = {h_B1H} broadcast({_shape('f16', [1, H])} %cls), dimensions={{1,2}}
  %cat = {h_BSH} concatenate({h_B1H} %cls_b, {h_BPH} %yb), dimensions={{1}}
  %pos_b = {h_BSH} broadcast({h_SH} %pos), dimensions={{1,2}}
  %tok = {h_BSH} add({h_BSH} %cat, {h_BSH} %pos_b)
  ROOT %r = {h_TH} reshape({h_BSH} %tok)
}}
""")
    entry.append(f"  %fusion.tokens = {h_TH} fusion({conv_s} %gte.patch, {h_H} %{bp}, {_shape('f16', [1, H])} %{cls}, "
                 f"{h_SH} %{pos}), kind=kLoop, calls=%fused_tokens")

    lnf = _preln_blocks(cfg, comps, entry, const, "fusion.tokens", causal=False)
    out_shape = _shape("f16", [B, S, H])
    entry.append(f"  ROOT %last_hidden_state = {out_shape} bitcast({h_TH} %{lnf})")
    text = (f"HloModule {cfg.name}, entry_computation_layout={{({px_s})->{out_shape}}}\n\n" + "\n".join(comps)
            + f"\nENTRY %{cfg.name}_main (pixel_values: {px_s}) -> {out_shape} {{\n" + "\n".join(entry) + "\n}\n")
    return text, names


def opt_hlo(cfg: EncoderConfig) -> tuple[str, dict[str, str]]:
    """HLO text of the prefill of a pre-LN causal decoder (OPT) of `cfg`: token gather + learned
    positions (table rows 2..2+S), causal pre-LN blocks with ReLU, final LayerNorm, LM head
    against the transposed token table (tied weights) and the arg-max token per position as
    XLA's (value, index) reduce. Outputs: (logits f16 [B*S, vocab], ids s32 [B*S]); the model of
    examples/utils/save_model.py:55-64 returns the arg-max of the last position only."""
    B, S, H, V = cfg.batch, cfg.seq, cfg.hidden, cfg.vocab
    T = B * S
    comps: list[str] = [_REGIONS]
    entry: list[str] = []
    names: dict[str, str] = {}

    def const(name: str, dims) -> str:
        names[name] = name
        entry.append(f"  %{name} = {_shape('f16', dims)} constant({{...}})")
        return name

    i_BS = _shape("s32", [B, S])
    h_TH, h_BSH, h_SH = _shape("f16", [T, H]), _shape("f16", [B, S, H]), _shape("f16", [S, H])
    entry.append(f"  %input_ids = {i_BS} parameter(0)")
    word = const("embeddings.word", [V, H])
    pos = const("embeddings.position", [cfg.max_pos + 2, H])
    w_s, p_s = _shape("f16", [V, H]), _shape("f16", [cfg.max_pos + 2, H])
    comps.append(f"""%fused_embed (p0: {i_BS}, p1: {w_s}, p2: {p_s}) -> {h_TH} {{
  %ids = {i_BS} parameter(0)
  %word = {w_s} parameter(1)
  %pos = {p_s} parameter(2)
  %tok = {h_BSH} gather({w_s} %word, {i_BS} %ids), offset_dims={{2}}, collapsed_slice_dims={{0}}, start_index_map={{0}}, index_vector_dim=2, slice_sizes={{1,{H}}}
  %pos_s = {h_SH} slice({p_s} %pos), slice={{[2:{2 + S}], [0:{H}]}}
  %pos_b = {h_BSH} broadcast({h_SH} %pos_s), dimensions={{1,2}}
  %sum = {h_BSH} add({h_BSH} %tok, {h_BSH} %pos_b)
  ROOT %r = {h_TH} reshape({h_BSH} %sum)
}}
""")
    entry.append(f"  %fusion.embed = {h_TH} fusion({i_BS} %input_ids, {w_s} %{word}, {p_s} %{pos}), kind=kLoop, "
                 f"calls=%fused_embed")
    lnf = _preln_blocks(cfg, comps, entry, const, "fusion.embed", causal=True)
    h_TV, f_TV, i_TV = _shape("f16", [T, V]), _shape("f32", [T, V]), _shape("s32", [T, V])
    f_T, i_T = _shape("f32", [T]), _shape("s32", [T])
    entry.append(f"  %gemm.lm_head = {h_TV} custom-call({h_TH} %{lnf}, {w_s} %{word}), "
                 f"custom_call_target=\"__cublas$gemm\", "
                 f"backend_config={_gemm_config(1.0, 1, 1, (), 1, T * H, V * H)}")
    comps.append(f"""%region_argmax (a_v: f32[], a_i: s32[], b_v: f32[], b_i: s32[]) -> (f32[], s32[]) {{
  %a_v = f32[] parameter(0)
  %a_i = s32[] parameter(1)
  %b_v = f32[] parameter(2)
  %b_i = s32[] parameter(3)
  %gt = pred[] compare(f32[] %a_v, f32[] %b_v), direction=GT
  %eq = pred[] compare(f32[] %a_v, f32[] %b_v), direction=EQ
  %lt_i = pred[] compare(s32[] %a_i, s32[] %b_i), direction=LT
  %tie = pred[] and(pred[] %eq, pred[] %lt_i)
  %keep = pred[] or(pred[] %gt, pred[] %tie)
  %v = f32[] select(pred[] %keep, f32[] %a_v, f32[] %b_v)
  %i = s32[] select(pred[] %keep, s32[] %a_i, s32[] %b_i)
  ROOT %t = (f32[], s32[]) tuple(f32[] %v, s32[] %i)
}}

%fused_argmax (p0: {h_TV}) -> {i_T} {{
  %x = {h_TV} parameter(0)
  %x32 = {f_TV} convert({h_TV} %x)
  %idx = {i_TV} iota(), iota_dimension=1
  %ninf = f32[] constant(-inf)
  %zero = s32[] constant(0)
  %r = ({f_T}, {i_T}) reduce({f_TV} %x32, {i_TV} %idx, f32[] %ninf, s32[] %zero), dimensions={{1}}, to_apply=%region_argmax
  ROOT %ids = {i_T} get-tuple-element(({f_T}, {i_T}) %r), index=1
}}
""")
    entry.append(f"  %fusion.argmax = {i_T} fusion({h_TV} %gemm.lm_head), kind=kInput, calls=%fused_argmax")
    out_shape = f"({h_TV}, {i_T})"
    entry.append(f"  ROOT %outputs = {out_shape} tuple({h_TV} %gemm.lm_head, {i_T} %fusion.argmax)")
    text = (f"HloModule {cfg.name}, entry_computation_layout={{({i_BS})->{out_shape}}}\n\n" + "\n".join(comps)
            + f"\nENTRY %{cfg.name}_main (input_ids: {i_BS}) -> {out_shape} {{\n" + "\n".join(entry) + "\n}\n")
    return text, names


def clip_hlo(cfg: ClipConfig, towers: str = "both") -> tuple[str, dict[str, str]]:
    """HLO text of a CLIP-shaped dual encoder (model of examples/utils/save_model.py:66-74, which
    returns logits_per_image). Vision tower: bias-free patch convolution, class token +
    positions, LayerNorm, pre-LN blocks, LayerNorm of the class row (slice inside the fusion),
    projection. Text tower: token + position rows, causal pre-LN blocks, final LayerNorm, the row
    at the largest token id (arg-max reduce + gather), projection. Both embeddings are
    L2-normalised; logits = logit_scale * image . text^T as one GEMM of two activations.
    Outputs: (logits_per_image f16 [images, texts], image_embeds, text_embeds). With
    `towers` = "vision" or "text" only that tower is emitted and its normalised embeddings are
    the single output (the get_image_features / get_text_features use of the model)."""
    assert towers in ("both", "vision", "text")
    v, t, P = cfg.vision, cfg.text, cfg.proj
    live = [True]  # False while the tower being written is not part of the module

    class _Sink(list):
        def append(self, item):
            if live[0]:
                super().append(item)

    comps = _Sink([_REGIONS])
    entry = _Sink()
    names: dict[str, str] = {}

    def const(name: str, dims) -> str:
        if live[0]:
            names[name] = name
        entry.append(f"  %{name} = {_shape('f16', dims)} constant({{...}})")
        return name

    def gemm(name, a, a_shape, w, w_shape, out_shape, alpha=1.0, rhs_c=0):
        entry.append(f"  %{name} = {_shape('f16', out_shape)} custom-call({_shape('f16', a_shape)} %{a}, "
                     f"{_shape('f16', w_shape)} %{w}), custom_call_target=\"__cublas$gemm\", "
                     f"backend_config={_gemm_config(alpha, 1, rhs_c, (), 1, 0, 0)}")
        return name

    # ---------------------------------------------------------------- vision tower
    live[0] = towers != "text"
    B, S, H, C, IMG, PS = v.batch, v.seq, v.hidden, v.channels, v.image, v.patch
    G = IMG // PS
    Pn, T = G * G, B * S
    px_s, nhwc_s = _shape("f32", [B, C, IMG, IMG]), _shape("f16", [B, IMG, IMG, C])
    h_TH, h_H, f_TH = _shape("f16", [T, H]), _shape("f16", [H]), _shape("f32", [T, H])
    i_BS = _shape("s32", [t.batch, t.seq])
    live[0] = True
    if towers != "text":
        entry.append(f"  %pixel_values = {px_s} parameter(0)")
    if towers != "vision":
        entry.append(f"  %input_ids = {i_BS} parameter({1 if towers == 'both' else 0})")
    live[0] = towers != "text"
    comps.append(f"""%fused_nhwc (p0: {px_s}) -> {nhwc_s} {{
  %x = {px_s} parameter(0)
  %t = {_shape('f32', [B, IMG, IMG, C])} transpose({px_s} %x), dimensions={{0,2,3,1}}
  ROOT %c = {nhwc_s} convert({_shape('f32', [B, IMG, IMG, C])} %t)
}}
""")
    entry.append(f"  %fusion.nhwc = {nhwc_s} fusion({px_s} %pixel_values), kind=kLoop, calls=%fused_nhwc")
    wp = const("vision.embeddings.patch.w", [H, PS, PS, C])
    cls = const("vision.embeddings.cls", [1, H])
    pos = const("vision.embeddings.position", [S, H])
    conv_s = _shape("f16", [B, G, G, H])
    conv_cfg = json.dumps(json.dumps({"conv_result_scale": 1, "side_input_scale": 0, "activation_mode": "0",
                                      "tensor_ops_enabled": True}, separators=(",", ":")))
    entry.append(f"  %conv.patch = ({conv_s}, u8[0]{{0}}) custom-call({nhwc_s} %fusion.nhwc, "
                 f"{_shape('f16', [H, PS, PS, C])} %{wp}), window={{size={PS}x{PS} stride={PS}x{PS}}}, "
                 f"dim_labels=b01f_o01i->b01f, custom_call_target=\"__cudnn$convForward\", backend_config={conv_cfg}")
    entry.append(f"  %gte.patch = {conv_s} get-tuple-element(({conv_s}, u8[0]{{0}}) %conv.patch), index=0")
    h_BPH, h_BSH, h_B1H, h_SH, h_1H = (_shape("f16", [B, Pn, H]), _shape("f16", [B, S, H]), _shape("f16", [B, 1, H]),
                                       _shape("f16", [S, H]), _shape("f16", [1, H]))
    comps.append(f"""%fused_tokens (p0: {conv_s}, p1: {h_1H}, p2: {h_SH}) -> {h_TH} {{
  %y = {conv_s} parameter(0)
  %cls = {h_1H} parameter(1)
  %pos = {h_SH} parameter(2)
  %yr = {h_BPH} reshape({conv_s} %y)
  %cls_b = {h_B1H} broadcast({h_1H} %cls), dimensions={{1,2}}
  %cat = {h_BSH} concatenate({h_B1H} %cls_b, {h_BPH} %yr), dimensions={{1}}
  %pos_b = {h_BSH} broadcast({h_SH} %pos), dimensions={{1,2}}
  %tok = {h_BSH} add({h_BSH} %cat, {h_BSH} %pos_b)
  ROOT %r = {h_TH} reshape({h_BSH} %tok)
}}
""")
    entry.append(f"  %fusion.tokens = {h_TH} fusion({conv_s} %gte.patch, {h_1H} %{cls}, {h_SH} %{pos}), kind=kLoop, "
                 f"calls=%fused_tokens")
    g0, b0 = const("vision.pre_ln.gamma", [H]), const("vision.pre_ln.beta", [H])
    entry.append(f"  %vision.fusion.pre_ln = {h_TH} fusion({h_TH} %fusion.tokens, {h_H} %{g0}, {h_H} %{b0}), "
                 f"kind=kInput, calls=%vision.fused_ln")
    x = _preln_blocks(v, comps, entry, const, "vision.fusion.pre_ln", causal=False, tag="vision.", final_ln=False)
    h_BH, f_BH = _shape("f16", [B, H]), _shape("f32", [B, H])
    comps.append(f"%fused_cls_ln (p0: {h_TH}, p1: {h_H}, p2: {h_H}) -> {h_BH} {{\n"
                 f"  %xa = {h_TH} parameter(0)\n  %gamma = {h_H} parameter(1)\n  %beta = {h_H} parameter(2)\n"
                 f"  %x3 = {h_BSH} reshape({h_TH} %xa)\n"
                 f"  %xs = {h_B1H} slice({h_BSH} %x3), slice={{[0:{B}], [0:1], [0:{H}]}}\n"
                 f"  %xc = {h_BH} reshape({h_B1H} %xs)\n"
                 f"  %x32 = {f_BH} convert({h_BH} %xc)\n" + "\n".join(_ln_body(B, H, v.eps, "x32")) + "\n}\n")
    g1, b1 = const("vision.ln.gamma", [H]), const("vision.ln.beta", [H])
    entry.append(f"  %fusion.cls_ln = {h_BH} fusion({h_TH} %{x}, {h_H} %{g1}, {h_H} %{b1}), kind=kInput, "
                 f"calls=%fused_cls_ln")
    wv = const("vision.proj.w", [H, P])
    gi = gemm("gemm.image_proj", "fusion.cls_ln", [B, H], wv, [H, P], [B, P])

    def l2norm(tag, rows, src):
        h_s, f_s, f_r = _shape("f16", [rows, P]), _shape("f32", [rows, P]), _shape("f32", [rows])
        comps.append(f"""%fused_l2norm_{tag} (p0: {h_s}) -> {h_s} {{
  %x = {h_s} parameter(0)
  %x32 = {f_s} convert({h_s} %x)
  %sq = {f_s} multiply({f_s} %x32, {f_s} %x32)
  %zero = f32[] constant(0)
  %ss = {f_r} reduce({f_s} %sq, f32[] %zero), dimensions={{1}}, to_apply=%region_add
  %nrm = {f_r} sqrt({f_r} %ss)
  %nrm_b = {f_s} broadcast({f_r} %nrm), dimensions={{0}}
  %y = {f_s} divide({f_s} %x32, {f_s} %nrm_b)
  ROOT %y16 = {h_s} convert({f_s} %y)
}}
""")
        entry.append(f"  %{tag}_embeds = {h_s} fusion({h_s} %{src}), kind=kInput, calls=%fused_l2norm_{tag}")
        return f"{tag}_embeds"

    img = l2norm("image", B, gi)

    # ------------------------------------------------------------------ text tower
    live[0] = towers != "vision"
    Bt, St, Ht, V = t.batch, t.seq, t.hidden, t.vocab
    Tt = Bt * St
    t_TH, t_BSH, t_SH, t_BH = (_shape("f16", [Tt, Ht]), _shape("f16", [Bt, St, Ht]), _shape("f16", [St, Ht]),
                               _shape("f16", [Bt, Ht]))
    word = const("text.embeddings.word", [V, Ht])
    tpos = const("text.embeddings.position", [t.max_pos, Ht])
    w_s, p_s = _shape("f16", [V, Ht]), _shape("f16", [t.max_pos, Ht])
    comps.append(f"""%fused_embed (p0: {i_BS}, p1: {w_s}, p2: {p_s}) -> {t_TH} {{
  %ids = {i_BS} parameter(0)
  %word = {w_s} parameter(1)
  %pos = {p_s} parameter(2)
  %tok = {t_BSH} gather({w_s} %word, {i_BS} %ids), offset_dims={{2}}, collapsed_slice_dims={{0}}, start_index_map={{0}}, index_vector_dim=2, slice_sizes={{1,{Ht}}}
  %pos_s = {t_SH} slice({p_s} %pos), slice={{[0:{St}], [0:{Ht}]}}
  %pos_b = {t_BSH} broadcast({t_SH} %pos_s), dimensions={{1,2}}
  %sum = {t_BSH} add({t_BSH} %tok, {t_BSH} %pos_b)
  ROOT %r = {t_TH} reshape({t_BSH} %sum)
}}
""")
    entry.append(f"  %fusion.embed = {t_TH} fusion({i_BS} %input_ids, {w_s} %{word}, {p_s} %{tpos}), kind=kLoop, "
                 f"calls=%fused_embed")
    lnf = _preln_blocks(t, comps, entry, const, "fusion.embed", causal=True, tag="text.")
    i_B, f_B = _shape("s32", [Bt]), _shape("s32", [Bt])
    comps.append(f"""%region_argmax_s32 (a_v: s32[], a_i: s32[], b_v: s32[], b_i: s32[]) -> (s32[], s32[]) {{
  %a_v = s32[] parameter(0)
  %a_i = s32[] parameter(1)
  %b_v = s32[] parameter(2)
  %b_i = s32[] parameter(3)
  %gt = pred[] compare(s32[] %a_v, s32[] %b_v), direction=GT
  %eq = pred[] compare(s32[] %a_v, s32[] %b_v), direction=EQ
  %lt_i = pred[] compare(s32[] %a_i, s32[] %b_i), direction=LT
  %tie = pred[] and(pred[] %eq, pred[] %lt_i)
  %keep = pred[] or(pred[] %gt, pred[] %tie)
  %v = s32[] select(pred[] %keep, s32[] %a_v, s32[] %b_v)
  %i = s32[] select(pred[] %keep, s32[] %a_i, s32[] %b_i)
  ROOT %t = (s32[], s32[]) tuple(s32[] %v, s32[] %i)
}}

%fused_eos_pool (p0: {t_TH}, p1: {i_BS}) -> {t_BH} {{
  %x = {t_TH} parameter(0)
  %ids = {i_BS} parameter(1)
  %idx = {i_BS} iota(), iota_dimension=1
  %imin = s32[] constant(-2147483648)
  %zero = s32[] constant(0)
  %r = ({i_B}, {i_B}) reduce({i_BS} %ids, {i_BS} %idx, s32[] %imin, s32[] %zero), dimensions={{1}}, to_apply=%region_argmax_s32
  %eos = {i_B} get-tuple-element(({i_B}, {i_B}) %r), index=1
  %b = {i_B} iota(), iota_dimension=0
  %len = s32[] constant({St})
  %len_b = {i_B} broadcast(s32[] %len), dimensions={{}}
  %base = {i_B} multiply({i_B} %b, {i_B} %len_b)
  %flat = {i_B} add({i_B} %base, {i_B} %eos)
  ROOT %rows = {t_BH} gather({t_TH} %x, {i_B} %flat), offset_dims={{1}}, collapsed_slice_dims={{0}}, start_index_map={{0}}, index_vector_dim=1, slice_sizes={{1,{Ht}}}
}}
""")
    entry.append(f"  %fusion.eos_pool = {t_BH} fusion({t_TH} %{lnf}, {i_BS} %input_ids), kind=kInput, "
                 f"calls=%fused_eos_pool")
    wt = const("text.proj.w", [Ht, P])
    gt = gemm("gemm.text_proj", "fusion.eos_pool", [Bt, Ht], wt, [Ht, P], [Bt, P])
    txt = l2norm("text", Bt, gt)
    live[0] = True
    lg_s = _shape("f16", [B, Bt])
    i_s, t_s = _shape("f16", [B, P]), _shape("f16", [Bt, P])
    if towers == "both":
        gemm("logits_per_image", img, [B, P], txt, [Bt, P], [B, Bt], alpha=cfg.logit_scale, rhs_c=1)
        out_shape = f"({lg_s}, {i_s}, {t_s})"
        entry.append(f"  ROOT %outputs = {out_shape} tuple({lg_s} %logits_per_image, {i_s} %{img}, {t_s} %{txt})")
        params, sig = f"{px_s}, {i_BS}", f"pixel_values: {px_s}, input_ids: {i_BS}"
    elif towers == "vision":
        out_shape, params, sig = i_s, px_s, f"pixel_values: {px_s}"
        entry.append(f"  ROOT %outputs = {i_s} bitcast({i_s} %{img})")
    else:
        out_shape, params, sig = t_s, i_BS, f"input_ids: {i_BS}"
        entry.append(f"  ROOT %outputs = {t_s} bitcast({t_s} %{txt})")
    text = (f"HloModule {cfg.name}, entry_computation_layout={{({params})->{out_shape}}}\n\n"
            + "\n".join(comps) + f"\nENTRY %{cfg.name}_main ({sig}) -> {out_shape} "
            f"{{\n" + "\n".join(entry) + "\n}\n")
    return text, names


def t5_hlo(cfg: EncoderConfig) -> tuple[str, dict[str, str]]:
    """HLO text of a T5-shaped encoder-decoder (model of examples/utils/save_model.py:84-92, which
    returns the decoder's last hidden state): token gather from the shared table (no position
    table), pre-norm blocks with RMS LayerNorm (x * rsqrt(mean(x^2) + eps) * scale), bias-free
    projections, un-scaled attention scores plus a constant per-(head, query, key) bias -- the
    stack's relative position bias as the compiler folds it, since the bucket arithmetic has no
    run-time input -- causal self-attention and bias-free cross-attention over the encoder output
    in the decoder, ReLU FFN. Inputs: input_ids, decoder_input_ids s32 [B, S]; output f16
    [B, S, H]. The constants named *.pos_bias are [heads * S, S]
    (mononn_b200.models.t5_device_weights makes them from the learned tables)."""
    B, S, H, F, NH = cfg.batch, cfg.seq, cfg.hidden, cfg.ffn, cfg.heads
    D, T, V = H // NH, cfg.batch * cfg.seq, cfg.vocab
    comps: list[str] = [_REGIONS]
    entry: list[str] = []
    names: dict[str, str] = {}

    def const(name: str, dims) -> str:
        names[name] = name
        entry.append(f"  %{name} = {_shape('f16', dims)} constant({{...}})")
        return name

    def gemm(name, a, a_shape, w, w_shape, out_shape, alpha=1.0, lhs_c=1, rhs_c=0, batch_dims=(), batch=1, ls=0, rs=0):
        entry.append(f"  %{name} = {_shape('f16', out_shape)} custom-call({_shape('f16', a_shape)} %{a}, "
                     f"{_shape('f16', w_shape)} %{w}), custom_call_target=\"__cublas$gemm\", "
                     f"backend_config={_gemm_config(alpha, lhs_c, rhs_c, batch_dims, batch, ls, rs)}")
        return name

    i_BS = _shape("s32", [B, S])
    h_TH, h_BSH, h_H, f_TH, f_T = (_shape("f16", [T, H]), _shape("f16", [B, S, H]), _shape("f16", [H]),
                                   _shape("f32", [T, H]), _shape("f32", [T]))
    w_s = _shape("f16", [V, H])
    entry.append(f"  %input_ids = {i_BS} parameter(0)")
    entry.append(f"  %decoder_input_ids = {i_BS} parameter(1)")
    shared = const("shared", [V, H])
    comps.append(f"""%fused_embed (p0: {i_BS}, p1: {w_s}) -> {h_TH} {{
  %ids = {i_BS} parameter(0)
  %word = {w_s} parameter(1)
  %tok = {h_BSH} gather({w_s} %word, {i_BS} %ids), offset_dims={{2}}, collapsed_slice_dims={{0}}, start_index_map={{0}}, index_vector_dim=2, slice_sizes={{1,{H}}}
  ROOT %r = {h_TH} reshape({h_BSH} %tok)
}}
""")
    f_H = _shape("f32", [H])
    comps.append(f"""%fused_rms (p0: {h_TH}, p1: {h_H}) -> {h_TH} {{
  %x = {h_TH} parameter(0)
  %gamma = {h_H} parameter(1)
  %x32 = {f_TH} convert({h_TH} %x)
  %zero = f32[] constant(0)
  %inv_n_s = f32[] constant({1.0 / H!r})
  %inv_n = {f_T} broadcast(f32[] %inv_n_s), dimensions={{}}
  %eps_s = f32[] constant({cfg.eps!r})
  %eps = {f_T} broadcast(f32[] %eps_s), dimensions={{}}
  %sq = {f_TH} multiply({f_TH} %x32, {f_TH} %x32)
  %sqsum = {f_T} reduce({f_TH} %sq, f32[] %zero), dimensions={{1}}, to_apply=%region_add
  %ms = {f_T} multiply({f_T} %sqsum, {f_T} %inv_n)
  %ms_eps = {f_T} add({f_T} %ms, {f_T} %eps)
  %rstd = {f_T} rsqrt({f_T} %ms_eps)
  %rstd_b = {f_TH} broadcast({f_T} %rstd), dimensions={{0}}
  %norm = {f_TH} multiply({f_TH} %x32, {f_TH} %rstd_b)
  %gamma32 = {f_H} convert({h_H} %gamma)
  %gamma_b = {f_TH} broadcast({f_H} %gamma32), dimensions={{1}}
  %scaled = {f_TH} multiply({f_TH} %norm, {f_TH} %gamma_b)
  ROOT %out = {h_TH} convert({f_TH} %scaled)
}}
""")
    h_heads, h_BShd = _shape("f16", [B, NH, S, D]), _shape("f16", [B, S, NH, D])
    comps.append(f"""%fused_split (p0: {h_TH}) -> {h_heads} {{
  %x = {h_TH} parameter(0)
  %r = {h_BShd} reshape({h_TH} %x)
  ROOT %t = {h_heads} transpose({h_BShd} %r), dimensions={{0,2,1,3}}
}}
""")
    h_sc, f_sc, f_row = _shape("f16", [B, NH, S, S]), _shape("f32", [B, NH, S, S]), _shape("f32", [B, NH, S])
    i_sc, p_sc = _shape("s32", [B, NH, S, S]), _shape("pred", [B, NH, S, S])
    h_pb, f_pb = _shape("f16", [NH * S, S]), _shape("f32", [NH, S, S])
    tail = f"""  %zmax = {f_row} reduce({f_sc} %z, f32[] %ninf), dimensions={{3}}, to_apply=%region_max
  %zmax_b = {f_sc} broadcast({f_row} %zmax), dimensions={{0,1,2}}
  %zc = {f_sc} subtract({f_sc} %z, {f_sc} %zmax_b)
  %e = {f_sc} exponential({f_sc} %zc)
  %zero = f32[] constant(0)
  %esum = {f_row} reduce({f_sc} %e, f32[] %zero), dimensions={{3}}, to_apply=%region_add
  %esum_b = {f_sc} broadcast({f_row} %esum), dimensions={{0,1,2}}
  %p = {f_sc} divide({f_sc} %e, {f_sc} %esum_b)
  ROOT %p16 = {h_sc} convert({f_sc} %p)
}}
"""
    bias_lines = (f"  %pb = {h_pb} parameter(1)\n  %pb3 = {_shape('f16', [NH, S, S])} reshape({h_pb} %pb)\n"
                  f"  %pb32 = {f_pb} convert({_shape('f16', [NH, S, S])} %pb3)\n"
                  f"  %pb_b = {f_sc} broadcast({f_pb} %pb32), dimensions={{1,2,3}}\n"
                  f"  %zb = {f_sc} add({f_sc} %z0, {f_sc} %pb_b)\n")
    head = f"  %s = {h_sc} parameter(0)\n  %z0 = {f_sc} convert({h_sc} %s)\n  %ninf = f32[] constant(-inf)\n"
    comps.append(f"%fused_softmax_enc (p0: {h_sc}, p1: {h_pb}) -> {h_sc} {{\n" + head + bias_lines +
                 f"  %z = {f_sc} copy({f_sc} %zb)\n" + tail)
    comps.append(f"%fused_softmax_dec (p0: {h_sc}, p1: {h_pb}) -> {h_sc} {{\n" + head + bias_lines +
                 f"  %qi = {i_sc} iota(), iota_dimension=2\n  %ki = {i_sc} iota(), iota_dimension=3\n"
                 f"  %keep = {p_sc} compare({i_sc} %qi, {i_sc} %ki), direction=GE\n"
                 f"  %ninf_b = {f_sc} broadcast(f32[] %ninf), dimensions={{}}\n"
                 f"  %z = {f_sc} select({p_sc} %keep, {f_sc} %zb, {f_sc} %ninf_b)\n" + tail)
    comps.append(f"%fused_softmax_x (p0: {h_sc}) -> {h_sc} {{\n" + head + f"  %z = {f_sc} copy({f_sc} %z0)\n" + tail)
    comps.append(f"""%fused_merge (p0: {h_heads}) -> {h_TH} {{
  %x = {h_heads} parameter(0)
  %t = {h_BShd} transpose({h_heads} %x), dimensions={{0,2,1,3}}
  ROOT %r = {h_TH} reshape({h_BShd} %t)
}}
""")
    comps.append(f"""%fused_resid (p0: {h_TH}, p1: {h_TH}) -> {h_TH} {{
  %x = {h_TH} parameter(0)
  %res = {h_TH} parameter(1)
  ROOT %y = {h_TH} add({h_TH} %x, {h_TH} %res)
}}
""")
    h_TF, f_TF = _shape("f16", [T, F]), _shape("f32", [T, F])
    act_lines, act_name = _activation_lines(cfg.act, "y32", f_TF)
    comps.append(f"%fused_act (p0: {h_TF}) -> {h_TF} {{\n  %x = {h_TF} parameter(0)\n"
                 f"  %y32 = {f_TF} convert({h_TF} %x)\n" + "\n".join(act_lines) + "\n"
                 f"  ROOT %out = {h_TF} convert({f_TF} %{act_name})\n}}\n")

    def rms(tag, x, gamma_name):
        g = const(gamma_name, [H])
        entry.append(f"  %{tag} = {h_TH} fusion({h_TH} %{x}, {h_H} %{g}), kind=kInput, calls=%fused_rms")
        return tag

    def heads_of(tag, src, wname):
        w = const(wname, [H, H])
        g = gemm(f"gemm.{tag}", src, [T, H], w, [H, H], [T, H], ls=T * H, rs=H * H)
        entry.append(f"  %fusion.{tag} = {h_heads} fusion({h_TH} %{g}), kind=kLoop, calls=%fused_split")
        return f"fusion.{tag}"

    def attention(tag, q_src, kv_src, prefix, softmax, bias):
        q, k, v = (heads_of(f"{tag}.q", q_src, prefix + "q.w"), heads_of(f"{tag}.k", kv_src, prefix + "k.w"),
                   heads_of(f"{tag}.v", kv_src, prefix + "v.w"))
        sc = gemm(f"gemm.{tag}.scores", q, [B, NH, S, D], k, [B, NH, S, D], [B, NH, S, S], alpha=1.0, lhs_c=3,
                  rhs_c=3, batch_dims=(0, 1), batch=B * NH, ls=S * D, rs=S * D)
        ops = f"{h_sc} %{sc}" + (f", {h_pb} %{bias}" if bias else "")
        entry.append(f"  %fusion.{tag}.softmax = {h_sc} fusion({ops}), kind=kInput, calls=%{softmax}")
        pv = gemm(f"gemm.{tag}.pv", f"fusion.{tag}.softmax", [B, NH, S, S], v, [B, NH, S, D], [B, NH, S, D],
                  lhs_c=3, rhs_c=2, batch_dims=(0, 1), batch=B * NH, ls=S * S, rs=S * D)
        entry.append(f"  %fusion.{tag}.ctx = {h_TH} fusion({h_heads} %{pv}), kind=kLoop, calls=%fused_merge")
        wo = const(prefix + "o.w", [H, H])
        return gemm(f"gemm.{tag}.o", f"fusion.{tag}.ctx", [T, H], wo, [H, H], [T, H], ls=T * H, rs=H * H)

    def resid(tag, g, x):
        entry.append(f"  %{tag} = {h_TH} fusion({h_TH} %{g}, {h_TH} %{x}), kind=kLoop, calls=%fused_resid")
        return tag

    def ffn(tag, y, x, prefix):
        w1, w2 = const(prefix + "ffn.up.w", [H, F]), const(prefix + "ffn.down.w", [F, H])
        gu = gemm(f"gemm.{tag}.up", y, [T, H], w1, [H, F], [T, F], ls=T * H, rs=H * F)
        entry.append(f"  %fusion.{tag}.act = {h_TF} fusion({h_TF} %{gu}), kind=kLoop, calls=%fused_act")
        gd = gemm(f"gemm.{tag}.down", f"fusion.{tag}.act", [T, F], w2, [F, H], [T, H], ls=T * F, rs=F * H)
        return resid(f"fusion.{tag}.res2", gd, x)

    # ---- encoder
    entry.append(f"  %fusion.enc.embed = {h_TH} fusion({i_BS} %input_ids, {w_s} %{shared}), kind=kLoop, calls=%fused_embed")
    enc_pb = const("encoder.pos_bias", [NH * S, S])
    x = "fusion.enc.embed"
    for l in range(cfg.layers):
        p = f"encoder.layer{l}."
        y = rms(f"fusion.enc.ln1.{l}", x, p + "ln1.gamma")
        x = resid(f"fusion.enc.res1.{l}", attention(f"enc.{l}", y, y, p + "attn.", "fused_softmax_enc", enc_pb), x)
        y = rms(f"fusion.enc.ln2.{l}", x, p + "ln2.gamma")
        x = ffn(f"enc.{l}", y, x, p)
    enc_out = rms("fusion.enc.lnf", x, "encoder.ln.gamma")
    # ---- decoder
    entry.append(f"  %fusion.dec.embed = {h_TH} fusion({i_BS} %decoder_input_ids, {w_s} %{shared}), kind=kLoop, calls=%fused_embed")
    dec_pb = const("decoder.pos_bias", [NH * S, S])
    x = "fusion.dec.embed"
    for l in range(cfg.layers):
        p = f"decoder.layer{l}."
        y = rms(f"fusion.dec.ln1.{l}", x, p + "ln1.gamma")
        x = resid(f"fusion.dec.res1.{l}", attention(f"dec.{l}", y, y, p + "attn.", "fused_softmax_dec", dec_pb), x)
        y = rms(f"fusion.dec.lnx.{l}", x, p + "lnx.gamma")
        x = resid(f"fusion.dec.resx.{l}", attention(f"decx.{l}", y, enc_out, p + "xattn.", "fused_softmax_x", None), x)
        y = rms(f"fusion.dec.ln2.{l}", x, p + "ln2.gamma")
        x = ffn(f"dec.{l}", y, x, p)
    dec_out = rms("fusion.dec.lnf", x, "decoder.ln.gamma")
    out_shape = _shape("f16", [B, S, H])
    entry.append(f"  ROOT %last_hidden_state = {out_shape} bitcast({h_TH} %{dec_out})")
    text = (f"HloModule {cfg.name}, entry_computation_layout={{({i_BS}, {i_BS})->{out_shape}}}\n\n" + "\n".join(comps)
            + f"\nENTRY %{cfg.name}_main (input_ids: {i_BS}, decoder_input_ids: {i_BS}) -> {out_shape} {{\n"
            + "\n".join(entry) + "\n}\n")
    return text, names
