"""The allocation-free attention entry point (-m gpu), collected last on purpose.

Some hosts cannot let this library allocate device memory (a framework allocator that owns
the whole GPU, or a serving thread that must not hit cudaMalloc's device synchronisation).
`mononn_attention_noalloc` runs the persistent kernel's attention stage with all of its
internal state in a static device array.  Here it is called through the C ABI on the Q, K,
V^T tensors a regular module produced, twice in a row, and must reproduce the regular entry
point's attention output.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _tensor(plan, name):
    return next(t for t in plan["tensors"] if t["name"] == name)


def test_noalloc_attention_matches_the_module_path_twice(tmp_path):
    import json
    import torch
    from mononn_b200 import bert_tiny, capi, compile_encoder, make_inputs, make_weights
    from mononn_b200.module import attention_noalloc, describe

    cfg = bert_tiny(batch=3, seq=40, layers=1, hidden=128, ffn=256)
    w = make_weights(cfg, 31, stress=True)
    inp = make_inputs(cfg, 31, pad_fraction=0.25)
    # the regular module with the Q/K/V projections as a stage of their own, so that its Q, K
    # and V^T tensors exist in the temp buffer for the stand-alone call to read
    spec = dict(describe("encoder", cfg.to_json())["spec"], qkv_fusion="off", out_fusion="off")
    (tmp_path / "cluster_0").mkdir()
    (tmp_path / "cluster_0" / "best_tuning_spec.json").write_text(json.dumps(spec))
    mod = compile_encoder(cfg, spec_dir=str(tmp_path))
    mod.set_weights(w)
    bufs = mod.allocate()
    descs = mod.args()
    for d, key in zip(descs[:3], ("input_ids", "attention_mask", "token_type_ids")):
        src = torch.from_numpy(inp[key]).view(torch.uint8).reshape(-1)
        bufs[d["index"]][: src.numel()].copy_(src)
    plan = mod.plan()
    names = [s["name"] for s in plan["stages"]]
    att_stage = next(i for i, s in enumerate(plan["stages"]) if s["ops"][0]["kind"] == "attention")
    assert names[att_stage] == "layer0.attn.core"
    # existing entry point: embeddings, Q/K/V projections, then the attention stage
    mod.launch_stages(0, att_stage + 1)
    mod.status()
    temp = bufs[[d["index"] for d in descs if d["kind"] == 2][0]]
    q, k, vt, ctx = (_tensor(plan, "layer0." + n) for n in ("q", "k", "v_t", "ctx"))
    T, H = cfg.tokens, cfg.hidden

    def view(t):
        raw = temp.cpu().numpy()[t["at"]["offset"]: t["at"]["offset"] + T * H * 2]
        return raw.view(np.float16).reshape(T, H).astype(np.float32)

    want = view(ctx)
    assert np.isfinite(want).all() and np.abs(want).max() > 0
    base = temp.data_ptr()
    mask_dev = bufs[descs[1]["index"]]
    out = torch.zeros(T * H, dtype=torch.float16, device="cuda")
    free_before = torch.cuda.mem_get_info()[0]
    for call in range(2):  # the static scratch keeps the previous call's contents
        out.zero_()
        attention_noalloc(base + q["at"]["offset"], base + k["at"]["offset"], base + vt["at"]["offset"],
                          mask_dev.data_ptr(), out.data_ptr(), cfg.batch, cfg.heads, cfg.seq,
                          q["ld"], vt["ld"], H, 1.0 / 8.0)
        torch.cuda.synchronize()
        got = out.cpu().numpy().reshape(T, H).astype(np.float32)
        # same kernel code on the same inputs: the two paths agree to f16 rounding
        assert np.abs(got - want).max() <= 1e-3, f"call {call}: {np.abs(got - want).max()}"
    assert torch.cuda.mem_get_info()[0] >= free_before  # nothing was allocated on the device

    # sizes beyond the static array are refused with a clear error
    with pytest.raises(capi.MononnError) as e:
        attention_noalloc(base, base, base, None, out.data_ptr(), 1024, 2, 128, 128, 128, 128, 0.125)
    assert e.value.code == -10 and "16384" in str(e.value)
    with pytest.raises(capi.MononnError) as e:
        attention_noalloc(base, base, base, None, out.data_ptr(), 1, 2, 200, 128, 200, 128, 0.125)
    assert e.value.code == -10
    mod.close()


def _oracle_case(rng, batches, heads, seq, with_mask, causal):
    """Random f16 Q, K, V for the stand-alone call and the fp32 oracle's context for them."""
    import torch
    from oracle import ref_encoder as R
    H = heads * 64
    q, k, v = (rng.standard_normal((batches, seq, H)).astype(np.float16) for _ in range(3))
    mask = None
    if with_mask:
        mask = np.ones((batches, seq), np.int32)
        mask[:, seq - max(1, seq // 4):] = 0
    bias = None if mask is None else ((1.0 - mask.astype(np.float32)) * np.float32(-10000.0))
    want = R.attention(q.astype(np.float32), k.astype(np.float32), v.astype(np.float32), bias, heads,
                       causal=causal).reshape(batches * seq, H)
    ld_vt = (seq + 7) // 8 * 8  # V^T rows need a 16-byte pitch
    vt = np.zeros((batches * H, ld_vt), np.float16)
    vt[:, :seq] = v.reshape(batches, seq, H).transpose(0, 2, 1).reshape(batches * H, seq)
    dev = lambda a: torch.from_numpy(a).cuda()
    return dict(q=dev(q.reshape(-1, H)), k=dev(k.reshape(-1, H)), vt=dev(vt), ld_vt=ld_vt,
                mask=None if mask is None else dev(mask), want=want, H=H,
                out=torch.zeros(batches * seq, H, dtype=torch.float16, device="cuda"),
                geom=(batches, heads, seq), causal=causal)


def _run_case(c):
    import torch
    from mononn_b200.module import attention_noalloc, attention_noalloc_status
    from tests.helpers import assert_parity
    b, h, s = c["geom"]
    c["out"].zero_()
    attention_noalloc(c["q"].data_ptr(), c["k"].data_ptr(), c["vt"].data_ptr(),
                      None if c["mask"] is None else c["mask"].data_ptr(), c["out"].data_ptr(), b, h, s,
                      c["H"], c["ld_vt"], c["H"], 1.0 / 8.0, causal=c["causal"])
    attention_noalloc_status()  # raises when a bounded wait expired in the kernel
    got = c["out"].cpu().numpy().astype(np.float32)
    rows = np.ones(b * s, bool)
    if c["mask"] is not None and not c["causal"]:
        pass  # padded queries still attend to the valid keys: every row is defined
    assert_parity(got[rows], c["want"][rows], f"noalloc attention {c['geom']} causal={c['causal']}")


def test_noalloc_attention_matches_the_oracle_across_changing_problems():
    """Consecutive calls rewrite the shared static array (tensor maps, descriptor, mask) with a
    different problem on other buffers each time; every result is checked against the fp32
    oracle softmax(scale QK^T + mask [+ causal]) V at the path's tolerance."""
    rng = np.random.default_rng(77)
    cases = [
        _oracle_case(rng, 3, 2, 40, with_mask=True, causal=False),
        _oracle_case(rng, 2, 1, 77, with_mask=False, causal=True),    # no mask operand, causal
        _oracle_case(rng, 80, 2, 16, with_mask=True, causal=True),    # 160 tiles: more than the SMs
        _oracle_case(rng, 1, 4, 128, with_mask=False, causal=False),
    ]
    for c in cases + cases[:1]:  # and the first problem again after the others
        _run_case(c)


def test_noalloc_attention_refuses_a_misaligned_output():
    """`out` is written with 16-byte vector stores: an address that is not 16-byte aligned is
    refused on the host (nothing is launched, the context stays usable)."""
    import torch
    from mononn_b200 import capi
    from mononn_b200.module import attention_noalloc
    rng = np.random.default_rng(5)
    c = _oracle_case(rng, 1, 1, 16, with_mask=False, causal=False)
    with pytest.raises(capi.MononnError) as e:
        attention_noalloc(c["q"].data_ptr(), c["k"].data_ptr(), c["vt"].data_ptr(), None,
                          c["out"].data_ptr() + 4, 1, 1, 16, 64, c["ld_vt"], 64, 0.125)
    assert e.value.code == -1 and "16" in str(e.value)
    with pytest.raises(capi.MononnError) as e:  # a row pitch that is not a multiple of 8 halves
        attention_noalloc(c["q"].data_ptr(), c["k"].data_ptr(), c["vt"].data_ptr(), None,
                          c["out"].data_ptr(), 1, 1, 16, 64, c["ld_vt"], 68, 0.125)
    assert e.value.code == -1
    torch.cuda.synchronize()
    _run_case(c)  # the device is still fine
