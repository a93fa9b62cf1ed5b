"""Runtime behaviour on the device (-m gpu): launch geometry, one launch per inference,
status reporting when a bounded wait expires, per-stage profile, spec dump and reload."""
import json
import os

import numpy as np
import pytest

from mononn_b200 import bert_tiny, capi, compile_encoder, compile_hlo, make_inputs, make_weights
from mononn_b200.hlo_builder import bert_hlo
from oracle import ref_encoder as R
from tests.helpers import assert_parity

pytestmark = pytest.mark.gpu


def small():
    cfg = bert_tiny(batch=2, seq=24, layers=2, hidden=128, ffn=512)
    w = make_weights(cfg, 4, stress=True)
    inp = make_inputs(cfg, 4)
    return cfg, w, inp


def run(mod, cfg, inp):
    out = mod.run([inp["input_ids"], inp["attention_mask"], inp["token_type_ids"]])[0]
    return out[: cfg.tokens * cfg.hidden].reshape(cfg.tokens, cfg.hidden).astype(np.float32)


def test_launch_configuration_and_arguments():
    cfg, w, inp = small()
    mod = compile_encoder(cfg)
    lc = mod.launch_config()
    import torch
    assert lc["grid"][0] == torch.cuda.get_device_properties(0).multi_processor_count
    assert lc["block"] == (384, 1, 1) and lc["smem_bytes"] <= 232448
    kinds = [a["kind"] for a in mod.args()]
    assert kinds == [0, 0, 0, 1, 2]
    mod.close()


def test_launch_before_constants_is_an_error():
    cfg, w, inp = small()
    mod = compile_encoder(cfg)
    with pytest.raises(capi.MononnError) as e:
        mod.launch()
    assert e.value.code == -9
    with pytest.raises(capi.MononnError) as e:
        mod.set_constant("no.such.constant", np.zeros(4, np.float16))
    assert e.value.code == -7
    with pytest.raises(capi.MononnError) as e:
        mod.set_constant("embeddings.ln.gamma", np.zeros(3, np.float16))
    assert e.value.code == -7
    mod.close()


def test_expired_wait_is_reported_and_the_module_recovers():
    """Host-side fault injection: the launch is told to wait for arrivals nobody makes. The
    kernel's bounded wait gives up after the (short) timeout, the status word says where, and
    the next launch on the same module works."""
    cfg, w, inp = small()
    mod = compile_encoder(cfg, barrier_timeout_us=20000)
    mod.set_weights(w)
    want = R.bert_encoder(cfg, w, inp)
    assert_parity(run(mod, cfg, inp), want, "before")
    mod.debug_skew_barrier(7)
    mod.launch()
    with pytest.raises(capi.MononnError) as e:
        mod.status()
    assert e.value.code == -6 and "stage" in str(e.value)
    assert_parity(run(mod, cfg, inp), want, "after recovery")
    mod.close()


def test_stage_profile_and_trace():
    cfg, w, inp = small()
    mod = compile_encoder(cfg)
    mod.set_weights(w)
    run(mod, cfg, inp)
    prof = mod.profile_stages()
    assert len(prof) == len(mod.plan()["stages"]) and all(t > 0 for _, t in prof)
    tr = mod.trace()
    assert tr.shape[1] == len(prof) and tr.shape[2] == 16
    # every CTA arrives at every stage's barrier (event 2)
    assert (tr[:, :, 2] > 0).all()
    mod.close()


def test_single_stage_isolation_matches_full_run():
    cfg, w, inp = small()
    mod = compile_encoder(cfg)
    mod.set_weights(w)
    full = run(mod, cfg, inp)
    n = len(mod.plan()["stages"])
    for s in range(n):
        mod.launch_stages(s, s + 1)
    mod.status()
    descs = mod.args()
    out_idx = [d["index"] for d in descs if d["kind"] == 1][0]
    step = mod.buffers[out_idx].cpu().numpy().view(np.float16)[: full.size].reshape(full.shape).astype(np.float32)
    assert np.abs(step - full).max() <= 4e-3
    mod.close()


def test_spec_dump_and_reload(tmp_path):
    cfg, w, inp = small()
    text, names = bert_hlo(cfg)
    mod = compile_hlo(text)
    mod.set_weights({names[k]: v for k, v in w.items()})
    run(mod, cfg, inp)
    mod.profile_stages()
    mod.save_spec(str(tmp_path))
    cdir = tmp_path / "cluster_0"
    assert (cdir / "best_tuning_spec.json").exists() and (cdir / "performance_report.csv").exists()
    spec = json.loads((cdir / "best_tuning_spec.json").read_text())
    grid = spec["cuda_context"]["cuda_runtime_context"]["grid_dim"]["x"]
    assert (cdir / f"{grid}_1_1__384_1_1.json").exists()
    rows = (cdir / "performance_report.csv").read_text().strip().splitlines()
    assert len(rows) == len(mod.plan()["stages"]) and rows[0].split(",")[0] == f"{grid}_1_1__384_1_1"
    # change a tile in the saved spec, reload through TF_MONONN_EXISTING_TUNING_SPEC_DIR semantics
    spec["gemm_spec_list"]["gemm_down_0"]["sm100_config"].update(mma_n=32, k_split=2)
    (cdir / "best_tuning_spec.json").write_text(json.dumps(spec))
    mod2 = compile_hlo(text, spec_dir=str(tmp_path))
    mod2.set_weights({names[k]: v for k, v in w.items()})
    ops = {o["name"]: o for s in mod2.plan()["stages"] for o in s["ops"]}
    assert ops["gemm_down_0"]["n_tile"] == 32 and ops["gemm_down_0"]["k_split"] == 2
    assert_parity(run(mod2, cfg, inp), R.bert_encoder(cfg, w, inp), "reloaded spec")
    mod.close()
    mod2.close()


def test_tuner_keeps_parity(tmp_path):
    cfg, w, inp = small()
    mod = compile_encoder(cfg, tuning_level=1, dump_dir=str(tmp_path))
    mod.set_weights(w)
    mod.tune()
    assert_parity(run(mod, cfg, inp), R.bert_encoder(cfg, w, inp), "after tuning")
    assert (tmp_path / "cluster_0" / "tuning_log.log").exists()
    mod.close()


def test_interrupted_tuning_resumes_from_its_journal(tmp_path):
    """Every timed candidate is journalled as it is measured; a later tune of the same module
    replays the journal (all of it, or the part an interrupted run got to) instead of
    measuring again, and ends with the same spec."""
    cfg, w, inp = small()
    journal = tmp_path / "cluster_0" / "tuning_progress.log"

    def tune_once():
        mod = compile_encoder(cfg, tuning_level=1, dump_dir=str(tmp_path))
        mod.set_weights(w)
        mod.tune()
        spec = mod.spec()["gemm_spec_list"]
        log = (tmp_path / "cluster_0" / "tuning_log.log").read_text()
        mod.close()
        return spec, log

    spec1, log1 = tune_once()
    lines = journal.read_text().splitlines()
    assert len(lines) > 3 and lines[0].startswith("default\t") and "reused" not in log1
    spec2, log2 = tune_once()                                  # complete journal: nothing is timed twice
    assert f"reused {len(lines)} measurements" in log2 and spec2 == spec1
    journal.write_text("\n".join(lines[: len(lines) // 2]) + "\nM128 N1 K1 torn li")   # an interrupted run
    spec3, log3 = tune_once()
    assert f"reused {len(lines) // 2} measurements" in log3
    assert len(journal.read_text().splitlines()) == len(lines)


def test_infer_host_matches_run_and_reports_timeouts():
    """The host-buffer entry point (copies + launch + status in one call) gives the result of
    the separate calls, twice in a row, and surfaces an expired wait as an error code."""
    import torch
    from mononn_b200 import capi
    cfg = bert_tiny(batch=2, seq=24, layers=2, hidden=128, ffn=512)
    w = make_weights(cfg, 21, stress=True)
    inp = make_inputs(cfg, 21, pad_fraction=0.25)
    mod = compile_encoder(cfg, barrier_timeout_us=20000)
    mod.set_weights(w)
    want = mod.run([inp["input_ids"], inp["attention_mask"], inp["token_type_ids"]])[0].copy()
    hin = [torch.from_numpy(inp[k]).contiguous().view(torch.uint8).reshape(-1).pin_memory()
           for k in ("input_ids", "attention_mask", "token_type_ids")]
    out_bytes = [a["bytes"] for a in mod.args() if a["kind"] == 1][0]
    hout = torch.zeros(out_bytes, dtype=torch.uint8).pin_memory()
    for _ in range(2):
        hout.zero_()
        mod.infer_host(hin, [hout])
        got = hout.numpy().view(np.float16)
        # (split-K partial sums are added with atomics: two runs agree to rounding, not bit for bit)
        assert np.abs(got[: want.size].astype(np.float32) - want[: got.size].astype(np.float32)).max() < 5e-3
    with pytest.raises(capi.MononnError):
        mod.infer_host(hin[:2], [hout])          # wrong number of host buffers
    mod.debug_skew_barrier(1)
    with pytest.raises(capi.MononnError) as e:
        mod.infer_host(hin, [hout])
    assert e.value.code == -6  # MONONN_ERR_BARRIER_TIMEOUT
    mod.infer_host(hin, [hout])                   # usable again
    got = hout.numpy().view(np.float16)
    assert np.abs(got[: want.size].astype(np.float32) - want[: got.size].astype(np.float32)).max() < 5e-3
    # the prepared form of the same call (pointer arrays and stream handle built once)
    step = mod.host_runner(hin, [hout])
    for _ in range(2):
        hout.zero_()
        step()
        got = hout.numpy().view(np.float16)
        assert np.abs(got[: want.size].astype(np.float32) - want[: got.size].astype(np.float32)).max() < 5e-3
    mod.debug_skew_barrier(1)
    with pytest.raises(capi.MononnError) as e:
        step()
    assert e.value.code == -6
    step()
    mod.close()


def test_mma_issue_probe_reports_cycles_per_instruction():
    """The tile menu rests on what one tcgen05.mma costs in isolation: the probe issues 256
    instructions back to back from resident operands and reports cycles per instruction. A
    wide instruction cannot beat the pipe (128 x 256 x 16 needs >= 100 cycles); a narrow one
    must not cost more than a wide one."""
    import ctypes as C
    from mononn_b200 import capi
    l = capi.lib()
    table = {}
    for n in (16, 64, 128, 256):
        cyc, iss, ns = C.c_double(), C.c_double(), C.c_double()
        capi.check(l.mononn_debug_mma_issue(0, n, 256, 1, 0, 148, C.byref(cyc), C.byref(iss), C.byref(ns)))
        table[n] = cyc.value
        assert 1.0 < cyc.value < 2000.0 and ns.value > 0
    print("cycles per tcgen05.mma 128xNx16:", {n: round(v, 1) for n, v in table.items()})
    assert table[256] >= 100.0
    assert table[16] <= table[256] * 1.1
    with pytest.raises(capi.MononnError):
        capi.check(l.mononn_debug_mma_issue(0, 24, 256, 1, 0, 1, None, None, None))


@pytest.mark.parametrize("cluster", [2, 4])
def test_cluster_scoped_barrier_arrival_keeps_parity(cluster, tmp_path):
    """Launched as thread-block clusters, the CTAs of a cluster arrive at the grid barrier through
    an mbarrier in the first CTA's shared memory and only that CTA touches the global counter.
    Same results; a shape that cannot be co-resident is refused when the plan is loaded."""
    from mononn_b200.module import describe
    cfg, w, inp = small()
    text, names = bert_hlo(cfg)
    spec = describe("hlo", text)["spec"]
    spec["cuda_context"]["cuda_runtime_context"]["cluster_dim"] = {"x": cluster, "y": 1, "z": 1}
    (tmp_path / "cluster_0").mkdir()
    (tmp_path / "cluster_0" / "best_tuning_spec.json").write_text(json.dumps(spec))
    try:
        mod = compile_hlo(text, spec_dir=str(tmp_path), barrier_timeout_us=500000)
    except capi.MononnError as e:
        assert e.code == -1 and "co-resident" in str(e)
        pytest.skip(str(e))
    assert mod.plan()["cluster"] == cluster
    mod.set_weights({names[k]: v for k, v in w.items()})
    assert_parity(run(mod, cfg, inp), R.bert_encoder(cfg, w, inp), f"clusters of {cluster}")
    for _ in range(3):
        mod.launch()
    mod.status()
    assert_parity(run(mod, cfg, inp), R.bert_encoder(cfg, w, inp), f"clusters of {cluster}, relaunched")
    mod.close()


def test_row_per_warp_layernorm_keeps_parity_when_the_split_is_switched_off(tmp_path):
    """Few rows are normalised by four warps each (the default here); `row_split: off` in the
    spec deals whole rows to single warps, the form large batches always use. Same results."""
    from mononn_b200.module import describe
    cfg, w, inp = small()
    text, names = bert_hlo(cfg)
    spec = describe("hlo", text)["spec"]
    assert spec["row_split"] == "on"
    spec["row_split"] = "off"
    (tmp_path / "cluster_0").mkdir()
    (tmp_path / "cluster_0" / "best_tuning_spec.json").write_text(json.dumps(spec))
    mod = compile_hlo(text, spec_dir=str(tmp_path), barrier_timeout_us=500000)
    lns = [o for s in mod.plan()["stages"] for o in s["ops"] if o["kind"] == "layernorm"]
    assert lns and all(not (o["flags"] & (1 << 14)) for o in lns)
    mod.set_weights({names[k]: v for k, v in w.items()})
    assert_parity(run(mod, cfg, inp), R.bert_encoder(cfg, w, inp), "row per warp")
    mod.close()


def test_out_projection_in_a_stage_of_its_own_keeps_parity(tmp_path):
    """By default the out-projection shares the attention's stage and waits on its arrival
    counter; `out_fusion: off` gives it a stage behind a grid barrier. Same results."""
    from mononn_b200.module import describe
    cfg, w, inp = small()
    text, names = bert_hlo(cfg)
    spec = describe("hlo", text)["spec"]
    assert spec["out_fusion"] == "fused_qkv"
    spec["out_fusion"] = "off"
    (tmp_path / "cluster_0").mkdir()
    (tmp_path / "cluster_0" / "best_tuning_spec.json").write_text(json.dumps(spec))
    mod = compile_hlo(text, spec_dir=str(tmp_path), barrier_timeout_us=500000)
    assert all("wait_flag" not in o for s in mod.plan()["stages"] for o in s["ops"])
    mod.set_weights({names[k]: v for k, v in w.items()})
    assert_parity(run(mod, cfg, inp), R.bert_encoder(cfg, w, inp), "out-projection behind a grid barrier")
    mod.close()


def test_ffn_gemms_chained_in_one_stage_keep_parity(tmp_path):
    """`chain_fusion: on`: FFN-down waits on FFN-up's arrival counter instead of a grid barrier;
    launched repeatedly (the counters grow from launch to launch) and after a launch of a stage
    sub-range (which clears them)."""
    from mononn_b200.module import describe
    cfg, w, inp = small()
    text, names = bert_hlo(cfg)
    spec = dict(describe("hlo", text)["spec"], chain_fusion="on")
    (tmp_path / "cluster_0").mkdir()
    (tmp_path / "cluster_0" / "best_tuning_spec.json").write_text(json.dumps(spec))
    mod = compile_hlo(text, spec_dir=str(tmp_path), barrier_timeout_us=500000)
    assert len(mod.plan()["stages"]) == 1 + 2 * cfg.layers
    mod.set_weights({names[k]: v for k, v in w.items()})
    ref = R.bert_encoder(cfg, w, inp)
    assert_parity(run(mod, cfg, inp), ref, "FFN in one stage")
    for _ in range(3):
        mod.launch()
    mod.launch_stages(0, 1)
    mod.status()
    assert_parity(run(mod, cfg, inp), ref, "FFN in one stage, relaunched")
    mod.close()
