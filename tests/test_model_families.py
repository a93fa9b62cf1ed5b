"""Device-free lowering of the pre-LN families (vision encoder, causal decoder): what the
recogniser finds in their HLO and what the scheduler plans for it."""
import pytest

from mononn_b200 import capi
from mononn_b200.hlo_builder import clip_hlo, opt_hlo, vit_hlo
from mononn_b200.models import clip_b32, clip_tiny, opt_1p3b, opt_tiny, vit_tiny
from mononn_b200.module import describe

F_CAUSAL, F_SRC_F32, F_NO_NORM = 1 << 3, 1 << 5, 1 << 9


def plan_of(text):
    return describe("hlo", text)["plan"]


def ops_of(plan, kind):
    return [o for st in plan["stages"] for o in st["ops"] if o["kind"] == kind]


def test_decoder_structure(lib_built):
    cfg = opt_tiny(batch=2, seq=24, layers=2, hidden=128, vocab=160)
    plan = plan_of(opt_hlo(cfg)[0])
    # embed, first LN | per layer: projections + attention + out-proj + LN, up, down + next LN | LM head, arg-max
    # (every LayerNorm but the first shares the stage of the split-K GEMM that feeds the stream, and
    # the out-projection the stage of the attention it reads)
    assert len(plan["stages"]) == 2 + 3 * cfg.layers + 2
    embed = ops_of(plan, "embed")
    assert len(embed) == 1 and embed[0]["flags"] & F_NO_NORM          # the sum is the residual stream
    assert embed[0]["p"][0]["space"] == "none"                          # no f16 copy of it is written
    att = ops_of(plan, "attention")
    assert len(att) == cfg.layers and all(o["flags"] & F_CAUSAL for o in att)
    assert all(o["flags"] & F_SRC_F32 for o in ops_of(plan, "layernorm"))
    assert len(ops_of(plan, "argmax")) == 1 and ops_of(plan, "argmax")[0]["n_items"] == cfg.tokens
    # residual updates accumulate into the stream: out-proj and FFN-down write f32 reductions
    red = [o for o in ops_of(plan, "gemm") if o["out_mode"] == 2]
    assert len(red) == 2 * cfg.layers
    assert len({(o["p"][0]["space"], o["p"][0]["offset"]) for o in red}) == 1


def test_decoder_arguments_and_tied_head(lib_built):
    cfg = opt_tiny(batch=2, seq=24, layers=1, hidden=128, vocab=160)
    plan = plan_of(opt_hlo(cfg)[0])
    args = plan["args"]
    assert [(a["name"], a["kind"]) for a in args] == [("input_ids", 0), ("gemm.lm_head", 1), ("fusion.argmax", 1),
                                                     ("temp_buffer", 2)]
    assert args[1]["bytes"] == cfg.tokens * cfg.vocab * 2 and args[2]["bytes"] == cfg.tokens * 4
    # the token table is bound twice: raw rows for the gather, packed tiles for the LM head
    kinds = sorted(c["kind"] for c in plan["constants"] if c["name"] == "embeddings.word")
    assert len(kinds) == 2 and kinds[0] != kinds[1]
    head = [o for o in ops_of(plan, "gemm") if o["name"] == "gemm_lm_head"][0]
    assert (head["N"], head["K"]) == (cfg.vocab, cfg.hidden)


def test_position_rows_start_at_the_slice_offset(lib_built):
    cfg = opt_tiny(seq=16)
    text, _ = opt_hlo(cfg)
    # a slice that would run past the table is refused rather than read out of bounds
    bad = text.replace(f"slice={{[2:{2 + cfg.seq}]", f"slice={{[{cfg.max_pos}:{cfg.max_pos + cfg.seq}]")
    lib = capi.lib()
    import ctypes as C
    out = C.c_void_p()
    rc = lib.mononn_describe(b"hlo", bad.encode(), len(bad.encode()), None, 148, C.byref(out))
    assert rc != 0


def test_non_causal_softmax_is_not_flagged_causal(lib_built):
    plan = plan_of(vit_hlo(vit_tiny())[0])
    assert all(not (o["flags"] & F_CAUSAL) for o in ops_of(plan, "attention"))
    assert len(ops_of(plan, "patchify")) == 1 and len(ops_of(plan, "assemble")) == 1


def test_argmax_with_another_tie_rule_is_rejected(lib_built):
    text, _ = opt_hlo(opt_tiny())
    # prefer the later index on ties: not the arg-max the kernel computes
    bad = text.replace("%lt_i = pred[] compare(s32[] %a_i, s32[] %b_i), direction=LT",
                       "%lt_i = pred[] compare(s32[] %a_i, s32[] %b_i), direction=GT")
    assert bad != text
    with pytest.raises(capi.MononnError) as e:
        plan_of(bad)
    assert "arg-max" in str(e.value)


def test_full_size_decoder_cost(lib_built):
    """OPT-1.3B prefill b1/s128: every weight once (token table: rows gathered + the whole
    table for the tied head), 338.8 GFLOP."""
    cfg = opt_1p3b()
    plan = plan_of(opt_hlo(cfg)[0])
    h, f, v = cfg.hidden, cfg.ffn, cfg.vocab
    per_layer = 4 * h * h + 2 * h * f
    flops = 2.0 * cfg.tokens * (cfg.layers * per_layer + h * v) + cfg.layers * 4.0 * cfg.seq * cfg.seq * h
    assert abs(plan["algorithmic_flops"] - flops) / flops < 1e-6
    weights = 2.0 * (cfg.layers * (per_layer + 9 * h + f) + 2 * h + h * v)
    assert abs(plan["algorithmic_bytes"] - weights) / weights < 0.01
    # (hidden 2048: the projections stay a stage of their own, see the fusion rule)
    assert len(plan["stages"]) == 2 + 5 * cfg.layers + 2


def _f32_regions(plan):
    """(offset, bytes, first stage, last stage, first write accumulates) of every f32 scratch tensor."""
    out = []
    for t in plan["tensors"]:
        if t["kind"] != "acc_f32":
            continue
        off = t["at"]["offset"]
        first = None
        for si, st in enumerate(plan["stages"]):
            for o in st["ops"]:
                writes_red = o["kind"] == "gemm" and o["out_mode"] == 2 and o["p"][0] == t["at"]
                writes_plain = o["q"][2] == t["at"]
                if first is None and (writes_red or writes_plain):
                    first = "red" if writes_red else "plain"
        out.append((off, t["rows"] * t["cols"] * 4, t["def_stage"], t["last_stage"], first == "red", t["name"]))
    return out


@pytest.mark.parametrize("towers", ["both", "vision", "text"])
def test_accumulators_never_inherit_a_dirty_buffer(lib_built, towers):
    """A GEMM accumulator whose first write is a reduction starts from zeros: it may reuse the
    memory of an accumulator that its reader cleared, never that of a residual stream."""
    plan = plan_of(clip_hlo(clip_tiny(layers=2), towers)[0])
    regions = _f32_regions(plan)
    assert any(r[4] for r in regions) and any(not r[4] for r in regions)
    for a in regions:
        for b in regions:
            if a[4] and not b[4]:
                overlap = not (a[0] + a[1] <= b[0] or b[0] + b[1] <= a[0])
                assert not overlap, (a[5], b[5])


def test_dual_encoder_structure(lib_built):
    cfg = clip_tiny(layers=2)
    plan = plan_of(clip_hlo(cfg)[0])
    assert [a["name"] for a in plan["args"]] == ["pixel_values", "input_ids", "logits_per_image", "image_embeds",
                                                 "text_embeds", "temp_buffer"]
    att = ops_of(plan, "attention")
    assert len(att) == 2 * cfg.vision.layers
    assert sum(1 for o in att if o["flags"] & F_CAUSAL) == cfg.text.layers     # the text tower only
    assert len(ops_of(plan, "rowsel")) == 1 and len(ops_of(plan, "pairdot")) == 1
    l2 = [o for o in ops_of(plan, "layernorm") if o["flags"] & (1 << 10)]
    assert len(l2) == 2
    # both towers share stages: fewer stages than the two towers one after the other
    alone = sum(len(plan_of(clip_hlo(cfg, t)[0])["stages"]) for t in ("vision", "text"))
    assert len(plan["stages"]) < alone


def test_full_size_dual_encoder_cost(lib_built):
    plan = plan_of(clip_hlo(clip_b32())[0])
    assert abs(plan["algorithmic_flops"] / 1e9 - 472.87) < 5.0
    # every weight once, gathered token rows, the f32 pixels (19.27 MB) and the outputs
    assert abs(plan["algorithmic_bytes"] / 1e6 - 273.8) < 1.0


def test_encoder_decoder_structure(lib_built):
    """T5: two token gathers without a position table, RMS LayerNorm everywhere, a position bias
    on self-attention only, decoder self-attention causal; the cross-attention K / V projections
    of all layers depend on the encoder output alone and are spread over stages of at most
    eight operators."""
    from mononn_b200.hlo_builder import t5_hlo
    from mononn_b200.models import t5_small, t5_tiny
    cfg = t5_tiny(batch=2, seq=32, layers=2, hidden=128, ffn=256)
    plan = plan_of(t5_hlo(cfg)[0])
    assert [a["name"] for a in plan["args"]] == ["input_ids", "decoder_input_ids", "last_hidden_state", "temp_buffer"]
    embed = ops_of(plan, "embed")
    assert len(embed) == 2 and all(o["p"][4]["space"] == "none" for o in embed)      # no position table
    F_POS_BIAS, F_RMSNORM = 1 << 12, 1 << 13
    ln = ops_of(plan, "layernorm")
    assert len(ln) == 2 * cfg.layers + 1 + 3 * cfg.layers + 1 and all(o["flags"] & F_RMSNORM for o in ln)
    att = ops_of(plan, "attention")
    assert len(att) == 3 * cfg.layers
    assert sum(1 for o in att if o["flags"] & F_POS_BIAS) == 2 * cfg.layers            # not on cross-attention
    assert sum(1 for o in att if o["flags"] & F_CAUSAL) == cfg.layers                  # decoder self-attention
    assert all(bool(o["flags"] & F_CAUSAL) <= bool(o["flags"] & F_POS_BIAS) for o in att)
    full = plan_of(t5_hlo(t5_small())[0])
    assert all(len(st["ops"]) <= 8 for st in full["stages"])
    kv = [i for i, st in enumerate(full["stages"]) for o in st["ops"] if o["name"].startswith("gemm_decx_") and
          o["name"].endswith(("_k", "_v"))]
    assert len(kv) == 12 and len(set(kv)) >= 2     # twelve projections, more than one stage
    assert abs(full["algorithmic_flops"] / 1e9 - 11.88) < 0.1


def test_overlapping_padded_patch_convolution_lowers_to_windows_and_a_gemm(lib_built):
    """A 7x7 window moved by 4 with 3 pixels of zero padding (an overlapping patch stem): the
    window rows are 147 elements, written as 192 (whole 64-element k blocks) with zeros behind
    them, and the filter constant keeps its own 147-element rows (zero-extended when packed)."""
    cfg = vit_tiny(batch=2, image=32, patch=7, patch_stride=4, patch_pad=3, hidden=128)
    assert cfg.patch_grid == 8 and cfg.seq == 65
    text = vit_hlo(cfg)[0]
    assert "window={size=7x7 stride=4x4 pad=3_3x3_3}" in text
    plan = plan_of(text)
    (win,) = ops_of(plan, "patchify")
    assert (win["rows"], win["cols"], win["window_elements"]) == (2 * 64, 192, 147)
    assert (win["window"], win["stride"], win["pad"]) == (7, 4, 3)
    gemm = [o for o in ops_of(plan, "gemm") if o["name"] == "conv_patch"][0]
    assert (gemm["M"], gemm["N"], gemm["K"]) == (128, 128, 192)
    with pytest.raises(capi.MononnError, match="dilated"):
        describe("hlo", text.replace("pad=3_3x3_3", "pad=3_3x3_3 rhs_dilate=2x2"))
    with pytest.raises(capi.MononnError, match="inconsistent"):
        describe("hlo", text.replace("stride=4x4", "stride=3x3"))
