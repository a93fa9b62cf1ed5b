"""The N>1 path of bench.py is 'replicas only': each rank runs its own inferences and the
ranks only agree on the slowest time.  Checked here with two gloo ranks on CPU."""
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
    # every rank 'measures' its own time; the job time is the maximum over ranks
    t = torch.tensor([0.5 if rank == 0 else 0.8], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    value = bench.replica_throughput(world, 100, float(t))
    if rank == 0:
        print(json.dumps({{"value": value, "max_s": float(t)}}))
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
    assert r["max_s"] == 0.8
    assert abs(r["value"] - 2 * 100 / 0.8) < 1e-9


def test_reference_arm_runs_on_cpu_and_prints_the_contract_line():
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1",
                          "--warmup", "0"], capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    import json
    r = json.loads([l for l in out.stdout.splitlines() if l.startswith("{")][-1])
    assert r["impl"] == "reference" and r["unit"] == "samples/s" and r["value"] > 0
    assert r["cpu_baseline"]["kind"] == "port" and r["e2e"]["h2d_bytes_per_step"] == 0
