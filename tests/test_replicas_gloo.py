"""The N>1 path of bench.py is 'replicas only': each rank lowers its own module, runs its own
inferences on its own inputs, and the ranks only agree on the slowest time.  Checked here with
two gloo ranks on CPU (lowering needs no device; the launches are covered on the GPU box)."""
import os
import subprocess
import sys
import textwrap

from tests.helpers import ROOT

WORKER = textwrap.dedent("""
    import os, sys, json
    sys.path.insert(0, {root!r})
    import torch, torch.distributed as dist
    import bench
    dist.init_process_group("gloo")
    rank, world, local = bench.dist_env()
    assert world == 2 and rank == int(os.environ["RANK"])
    # every replica lowers the module on its own (no device is needed to lower) and draws its own
    # inputs; the stage tables must be identical, the inputs must not
    import hashlib
    from mononn_b200 import bert_tiny, make_inputs
    from mononn_b200.hlo_builder import bert_hlo
    from mononn_b200.module import describe
    cfg = bert_tiny(batch=2, seq=24, layers=2, hidden=128, ffn=512)
    plan = describe("hlo", bert_hlo(cfg)[0])["plan"]
    digest = hashlib.sha256(json.dumps(plan, sort_keys=True).encode()).digest()[:8]
    ids = make_inputs(cfg, 1234 + rank)["input_ids"]
    mine = torch.tensor(list(digest) + [int(ids.sum())], dtype=torch.int64)
    both = [torch.zeros_like(mine) for _ in range(world)]
    dist.all_gather(both, mine)
    assert torch.equal(both[0][:8], both[1][:8]), "replicas lowered different plans"
    assert both[0][8] != both[1][8], "replicas drew the same inputs"
    # every rank 'measures' its own time; the job time is the maximum over ranks
    t = torch.tensor([0.5 if rank == 0 else 0.8], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    value = bench.replica_throughput(world, 100, float(t))
    if rank == 0:
        print(json.dumps({{"value": value, "max_s": float(t), "stages": len(plan["stages"])}}))
    dist.barrier()
    dist.destroy_process_group()
""")


def test_two_replicas_report_whole_job_throughput(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER.format(root=ROOT))
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29731")
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                          "--master-addr", "127.0.0.1", "--master-port", "29731", str(script)],
                         capture_output=True, text=True, env=env, timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    line = [l for l in out.stdout.splitlines() if l.startswith("{")][-1]
    import json
    r = json.loads(line)
    assert r["max_s"] == 0.8 and r["stages"] == 1 + 2 * 3
    assert abs(r["value"] - 2 * 100 / 0.8) < 1e-9


def test_reference_arm_runs_on_cpu_and_prints_the_contract_line():
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1",
                          "--warmup", "0"], capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    import json
    r = json.loads([l for l in out.stdout.splitlines() if l.startswith("{")][-1])
    assert r["impl"] == "reference" and r["unit"] == "samples/s" and r["value"] > 0
    assert r["cpu_baseline"]["kind"] == "port" and r["e2e"]["h2d_bytes_per_step"] == 0
