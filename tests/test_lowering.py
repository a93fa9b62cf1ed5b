"""Host-side lowering (no GPU): stage structure, tile choice, buffer assignment, spec I/O."""
import json
import os

import pytest

from mononn_b200 import bert_base, bert_tiny, capi
from mononn_b200.hlo_builder import bert_hlo
from mononn_b200.module import describe


@pytest.fixture(scope="module")
def base_plan(lib_built):
    return describe("encoder", bert_base().to_json())


def test_bert_base_stage_structure(base_plan):
    p = base_plan["plan"]
    assert p["grid"] == 148 and p["block"] == 384
    assert p["smem_bytes"] <= 232448
    stages = p["stages"]
    # 12 (batch, head) pairs cannot fill 148 CTAs: the Q/K/V projections run inside the attention items,
    # the out-projection shares their stage behind the attention's arrival counter, and each
    # LayerNorm shares the stage of the split-K GEMM that feeds it: three stages a layer
    assert len(stages) == 1 + 12 * 3
    kinds = [tuple(o["kind"] for o in s["ops"]) for s in stages[:4]]
    assert kinds == [("embed",), ("attention", "gemm", "layernorm"), ("gemm",), ("gemm", "layernorm")]
    assert stages[1]["ops"][0]["flags"] & (1 << 11)
    # the out-projection waits for exactly the attention items, on a counter of its own
    att, o, ln = stages[1]["ops"]
    assert o["wait_flag"] == att["flag"] and o["wait_target"] == att["n_items"] == 12 and not att["waits"]
    assert o["flag"] == ln["flag"] != att["flag"] and o["n_items"] + att["n_items"] <= 148
    # the row items wait for exactly the GEMM items dealt before them
    for s in stages:
        if [x["kind"] for x in s["ops"]][-2:] == ["gemm", "layernorm"]:
            g, ln = s["ops"][-2:]
            assert g["flag"] == ln["flag"] and not g["waits"] and ln["waits"] and ln["flag_target"] == g["n_items"]
    # with out_fusion off the out-projection keeps a stage of its own: four stages a layer
    four = describe("encoder", bert_base().to_json(), spec=dict(base_plan["spec"], out_fusion="off"))["plan"]
    assert len(four["stages"]) == 1 + 12 * 4 and base_plan["spec"]["out_fusion"] == "fused_qkv"
    assert [tuple(o["kind"] for o in s["ops"]) for s in four["stages"][1:3]] == [("attention",), ("gemm", "layernorm")]
    # every GEMM / attention operator fits one wave of the 148 CTAs at b1/s128
    assert all(o["n_items"] <= 148 for s in stages for o in s["ops"])


def test_row_fusion_off_keeps_layernorm_stages(base_plan):
    off = dict(base_plan["spec"], row_fusion="off", out_fusion="off")
    p = describe("encoder", bert_base().to_json(), spec=off)["plan"]
    assert len(p["stages"]) == 1 + 12 * 6
    assert all("flag" not in o and "wait_flag" not in o for s in p["stages"] for o in s["ops"])
    # the two choices are independent: the out-projection can still share the attention's stage
    p = describe("encoder", bert_base().to_json(), spec=dict(off, out_fusion="on"))["plan"]
    assert len(p["stages"]) == 1 + 12 * 5
    assert [o["kind"] for o in p["stages"][1]["ops"]] == ["attention", "gemm"]
    assert p["spec_echo"]["row_fusion"] == "off" if "spec_echo" in p else True


def test_layernorm_rows_are_shared_by_four_warps_when_there_are_few_rows(base_plan):
    """128 rows dealt eight to an item occupy 16 CTAs with one row per warp; two rows per item,
    four warps each, spread the same rows over 64 CTAs. Many rows keep the row-per-warp form."""
    lns = [o for s in base_plan["plan"]["stages"] for o in s["ops"] if o["kind"] == "layernorm"]
    assert lns and all(o["flags"] & (1 << 14) and o["n_items"] == 64 for o in lns)
    off = describe("encoder", bert_base().to_json(), spec=dict(base_plan["spec"], row_split="off"))
    assert off["spec"]["row_split"] == "off"
    lns = [o for s in off["plan"]["stages"] for o in s["ops"] if o["kind"] == "layernorm"]
    assert all(not (o["flags"] & (1 << 14)) and o["n_items"] == 16 for o in lns)
    big = describe("encoder", bert_base(batch=16).to_json())["plan"]
    lns = [o for s in big["stages"] for o in s["ops"] if o["kind"] == "layernorm"]
    assert all(not (o["flags"] & (1 << 14)) and o["n_items"] == 16 * 128 // 8 for o in lns)


def test_projections_stay_a_stage_of_their_own_when_attention_fills_the_gpu(lib_built, base_plan):
    """Fusing costs every (batch, head) item a pass over its head's weights: it is done only
    when the attention stage leaves CTAs idle (or on request), never for long sequences."""
    off = dict(base_plan["spec"], qkv_fusion="off")
    p = describe("encoder", bert_base().to_json(), spec=off)["plan"]
    assert len(p["stages"]) == 1 + 12 * 5
    assert [o["kind"] for o in p["stages"][1]["ops"]] == ["gemm", "gemm", "gemm"]
    # (an attention without its own projections is short: the out-projection stays behind a barrier)
    assert [o["kind"] for o in p["stages"][2]["ops"]] == ["attention"]
    assert abs(p["algorithmic_flops"] - base_plan["plan"]["algorithmic_flops"]) < 1e6
    many = describe("encoder", bert_tiny(batch=160, seq=16, layers=1).to_json())["plan"]   # 160 pairs > 148 CTAs
    assert [o["kind"] for o in many["stages"][1]["ops"]] == ["gemm", "gemm", "gemm"]
    forced = describe("encoder", bert_tiny(batch=160, seq=16, layers=1).to_json(),
                      spec=dict(describe("encoder", bert_tiny(batch=160, seq=16, layers=1).to_json())["spec"],
                                qkv_fusion="on"))["plan"]
    assert [o["kind"] for o in forced["stages"][1]["ops"]][0] == "attention"
    long_seq = describe("encoder", bert_tiny(batch=1, seq=200, layers=1).to_json())["plan"]
    assert [o["kind"] for o in long_seq["stages"][1]["ops"]] == ["gemm", "gemm", "gemm"]


def test_algorithmic_cost_matches_the_model(base_plan):
    p = base_plan["plan"]
    # 85 054 464 encoder parameters in f16 + gathered rows + ids + output
    assert abs(p["algorithmic_bytes"] - 170.70e6) < 0.05e6
    assert abs(p["algorithmic_flops"] - 22.35e9) < 0.02e9


def test_residual_and_bias_are_preloaded_by_the_row_stage(base_plan):
    """The split-K GEMMs accumulate into an f32 buffer that the preceding LayerNorm /
    embedding stage fills with residual + bias, so their epilogue flags are empty."""
    ops = {o["name"]: o for s in base_plan["plan"]["stages"] for o in s["ops"]}
    for name in ("layer0.attn.o", "layer3.ffn.down"):
        assert ops[name]["flags"] & 0x3 == 0 and ops[name]["out_mode"] == 2
    assert ops["layer0.ffn.up"]["flags"] & 0x1 and ops["layer0.ffn.up"]["act"] == 1


def _live_ranges_do_not_overlap(plan):
    tensors = [t for t in plan["tensors"] if t["kind"] in ("act_f16", "act_f16_t", "acc_f32", "vec_f32")]

    def size(t):
        if t["kind"] == "act_f16":
            return t["rows"] * t["ld"] * 2
        if t["kind"] == "act_f16_t":
            return t["batches"] * t["cols"] * t["ld"] * 2
        if t["kind"] == "acc_f32":
            return t["rows"] * t["cols"] * 4
        return t["rows"] * 4
    for i, a in enumerate(tensors):
        for b in tensors[i + 1:]:
            if a["at"]["space"] != b["at"]["space"] or a["at"]["index"] != b["at"]["index"]:
                continue
            live = not (a["last_stage"] < b["def_stage"] or b["last_stage"] < a["def_stage"])
            mem = not (a["at"]["offset"] + size(a) <= b["at"]["offset"] or
                       b["at"]["offset"] + size(b) <= a["at"]["offset"])
            assert not (live and mem), (a["name"], b["name"])
    for t in tensors:
        if t["at"]["space"] == "arg":
            assert t["at"]["offset"] + size(t) <= plan["temp_bytes"]
        assert t["at"]["offset"] % 256 == 0


def test_buffers_with_overlapping_lifetimes_never_share_memory(base_plan):
    _live_ranges_do_not_overlap(base_plan["plan"])
    _live_ranges_do_not_overlap(describe("encoder", bert_tiny(batch=3, seq=20, layers=3).to_json())["plan"])


def test_temp_arena_reuses_memory_across_layers(base_plan):
    # 12 layers of activations fit in the footprint of about one layer
    assert base_plan["plan"]["temp_bytes"] < 2 * (128 * 3072 * 2 + 4 * 128 * 768 * 2)


def test_tensor_maps_obey_the_tma_rules(base_plan):
    for tm in base_plan["plan"]["tensor_maps"]:
        assert tm["stride1_bytes"] % 16 == 0
        assert tm["box0"] * 2 % 16 == 0 and tm["box0"] * 2 <= 128  # 128-byte swizzle span
        assert 1 <= tm["box1"] <= 256
        assert tm["base"]["offset"] % 16 == 0


def test_spec_controls_the_tiles_and_round_trips(lib_built, tmp_path):
    cfg = bert_tiny(layers=1, hidden=128, ffn=512, seq=32)
    d = describe("encoder", cfg.to_json())
    spec = d["spec"]
    assert set(spec) >= {"cuda_context", "gemm_spec_list", "cluster_elewise_spec", "cluster_reduce_spec",
                         "conv_spec_list", "codegen_allow_list", "codegen_reject_list"}
    rt = spec["cuda_context"]["cuda_runtime_context"]
    assert rt["grid_dim"] == {"x": 148, "y": 1, "z": 1} and rt["block_dim"]["x"] == 384
    spec["gemm_spec_list"]["layer0.ffn.down"]["sm100_config"].update(mma_n=64, k_split=2)
    d2 = describe("encoder", cfg.to_json(), spec=spec)
    ops = {o["name"]: o for s in d2["plan"]["stages"] for o in s["ops"]}
    assert ops["layer0.ffn.down"]["n_tile"] == 64 and ops["layer0.ffn.down"]["k_split"] == 2
    # an illegal request (K split on a GEMM whose activation needs the full sum) falls back
    spec["gemm_spec_list"]["layer0.ffn.up"]["sm100_config"].update(mma_n=32, k_split=2)
    d3 = describe("encoder", cfg.to_json(), spec=spec)
    ops = {o["name"]: o for s in d3["plan"]["stages"] for o in s["ops"]}
    assert ops["layer0.ffn.up"]["k_split"] == 1
    # a spec in the reference's layout (cutlass_config only) parses and is ignored
    ref_style = {"cuda_context": spec["cuda_context"],
                 "gemm_spec_list": {"layer0.ffn.down": {"cutlass_config": {"ThreadBlockShape": {"m": 128, "n": 64, "k": 32}}}}}
    describe("encoder", cfg.to_json(), spec=ref_style)


def test_tiles_wider_than_a_ring_slot_are_never_planned(lib_built):
    # a 16-CTA grid once made the heuristic pick a tile whose weight slab overflowed its ring
    # slot; a spec asking for one (320 columns = 40 KB for a 32 KB slot) is not honoured either
    cfg = bert_base()
    spec = describe("encoder", cfg.to_json())["spec"]
    spec["cuda_context"]["cuda_runtime_context"]["grid_dim"]["x"] = 16
    spec["gemm_spec_list"] = {"layer0.ffn.up": {"sm100_config": {"mma_n": 320, "k_split": 1}}}
    p = describe("encoder", cfg.to_json(), spec=spec)["plan"]
    widest = 0
    for st in p["stages"]:
        for o in st["ops"]:
            if o["kind"] == "gemm":
                assert o["n_tile"] * o["kb_per_bslot"] * 128 <= 32768 and o["n_tile"] <= 256
                widest = max(widest, o["n_tile"])
    assert widest > 128   # with 16 CTAs the wide tiles are what the heuristic wants


def test_long_sequences_and_large_batches_lower(lib_built):
    from mononn_b200.models import EncoderConfig
    cfg = EncoderConfig(layers=2, hidden=1024, heads=16, ffn=4096, batch=16, seq=384)
    p = describe("encoder", cfg.to_json())["plan"]
    att = [o for s in p["stages"] for o in s["ops"] if o["kind"] == "attention"][0]
    assert att["n_items"] == 16 * 16 * 3
    _live_ranges_do_not_overlap(p)
    cfg.seq, cfg.max_pos = 512, 512
    with pytest.raises(capi.MononnError) as e:
        describe("encoder", cfg.to_json())
    assert e.value.code == -3 and "384" in str(e.value)


def test_allow_list_isolates_one_node(lib_built):
    cfg = bert_tiny(layers=1)
    spec = describe("encoder", cfg.to_json())["spec"]
    spec["codegen_allow_list"] = ["layer0.ffn.up"]
    d = describe("encoder", cfg.to_json(), spec=spec)
    assert [s["name"] for s in d["plan"]["stages"]] == ["layer0.ffn.up"]


def test_malformed_inputs_give_error_codes_not_aborts(lib_built):
    with pytest.raises(capi.MononnError) as e:
        describe("encoder", "{not json")
    assert e.value.code == -2
    with pytest.raises(capi.MononnError) as e:
        describe("encoder", json.dumps({"model": "bert", "hidden": 100, "heads": 2}))
    assert e.value.code == -3
    with pytest.raises(capi.MononnError) as e:
        describe("encoder", bert_tiny().to_json(), spec={"gemm_spec_list": 3})
    assert e.value.code == -2


def test_hlo_and_builder_paths_agree(lib_built):
    for cfg in (bert_tiny(), bert_tiny(batch=2, seq=24, layers=2, hidden=128, ffn=512)):
        text, _ = bert_hlo(cfg)
        a = describe("hlo", text)["plan"]
        b = describe("encoder", cfg.to_json())["plan"]
        assert len(a["stages"]) == len(b["stages"])
        for sa, sb in zip(a["stages"], b["stages"]):
            ka = [(o["kind"], o.get("M"), o.get("N"), o.get("K"), o.get("n_tile"), o.get("k_split"), o["flags"], o["act"]) for o in sa["ops"]]
            kb = [(o["kind"], o.get("M"), o.get("N"), o.get("K"), o.get("n_tile"), o.get("k_split"), o["flags"], o["act"]) for o in sb["ops"]]
            assert ka == kb
        assert a["temp_bytes"] == b["temp_bytes"] and a["algorithmic_bytes"] == b["algorithmic_bytes"]
        assert [x["kind"] for x in a["args"]] == [0, 0, 0, 1, 2]


def test_structure_choices_left_to_the_scheduler_follow_the_row_count(base_plan):
    """With few rows the LayerNorms join their GEMMs' stage and the weight stream is marked
    evict-first; with thousands of rows (48 row tiles re-reading every weight tile, 768 row items
    that would wait for a whole GEMM) both are off. An explicit spec wins either way."""
    assert (base_plan["spec"]["row_fusion"], base_plan["spec"]["l2_hints"]) == ("on", "on")
    big = describe("encoder", bert_base(batch=16).to_json())
    assert (big["spec"]["row_fusion"], big["spec"]["l2_hints"]) == ("off", "off")
    assert all(len(s["ops"]) == 1 for s in big["plan"]["stages"] if s["ops"][0]["kind"] == "layernorm")
    forced = describe("encoder", bert_base(batch=16).to_json(), spec=dict(big["spec"], row_fusion="on", l2_hints="on"))
    assert (forced["spec"]["row_fusion"], forced["spec"]["l2_hints"]) == ("on", "on")
    assert len(forced["plan"]["stages"]) < len(big["plan"]["stages"])


def test_chain_fusion_puts_both_ffn_gemms_in_one_stage(base_plan):
    """With chain_fusion a GEMM whose A operand is written by another GEMM joins that GEMM's stage
    and waits for its counter: FFN-up -> FFN-down -> LayerNorm in one stage, every operator behind
    the ones it waits for, every target the item count of what it waits for. Off by default."""
    assert base_plan["spec"]["chain_fusion"] == "off"
    spec = dict(base_plan["spec"], chain_fusion="on")
    spec.pop("gemm_spec_list")          # tiles are chosen anew for the new structure
    d = describe("encoder", bert_base().to_json(), spec=spec)
    stages = d["plan"]["stages"]
    assert len(stages) == 1 + 12 * 2
    assert [x["kind"] for x in stages[1]["ops"]] == ["attention", "gemm", "layernorm"]
    up, down, ln2 = stages[2]["ops"]
    assert [x["kind"] for x in stages[2]["ops"]] == ["gemm", "gemm", "layernorm"]
    assert "wait_flag" not in up and down["wait_flag"] == up["flag"] and down["wait_target"] == up["n_items"]
    assert ln2["waits"] and ln2["flag"] == down["flag"] != up["flag"] and ln2["flag_target"] == down["n_items"]
    # chained GEMMs run one after another: each may use all the CTAs
    assert up["n_items"] <= 148 and down["n_items"] <= 148
