#!/usr/bin/env python
"""Benchmark of the hot path: BERT-base b1/s128, one persistent-kernel launch per inference.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

A step is one inference (batch 1, 128 tokens) on every participating GPU; the GPUs run
independent replicas (the path does not shard beyond batch, so there is no collective on
the data path -- torch.distributed is used only for the barrier and the max-over-ranks of
the measured time).  Rank 0 prints one JSON line.

  value      samples/s of the whole job, inputs resident in HBM, device time (CUDA events)
  e2e        the same through the public API with pinned HOST buffers: H2D of the three id
             tensors, the launch, D2H of the hidden state, per step, wall clock
  roofline   algorithmic bytes of one inference / measured kernel time vs the measured HBM peak
  cpu_baseline  the fp32 CPU restatement (oracle/) timed on this box's host cores

`--impl reference` times the reference's CPU path.  The reference's own TF-XLA CPU execution
cannot run here (no TensorFlow), so the arm runs the CPU restatement under oracle/ with all
host threads.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "bert_base_b1_s128_samples_per_s"
UNIT = "samples/s"
FALLBACK_HBM_GBS = 6650.0
# dram__bytes_read.sum + dram__bytes_write.sum of one launch, from the ncu capture summarised
# in profiles/ (None until a capture exists)
NCU_TRAFFIC_BYTES = 175083520  # 170.77 MB read + 4.32 MB written


def measured_hbm_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap,utilization.gpu")

    def __init__(self, device_index: int):
        self.proc = None
        self.index = device_index
        self.thread = None
        self.rows = []

    def _nvml_loop(self, nv, handle):
        # read-only NVML queries every 2 ms: a timed region of ten milliseconds still gets samples
        # (one nvidia-smi query takes longer than that region)
        bits = {"hw_slowdown": nv.nvmlClocksThrottleReasonHwSlowdown,
                "hw_thermal_slowdown": nv.nvmlClocksThrottleReasonHwThermalSlowdown,
                "sw_thermal_slowdown": nv.nvmlClocksThrottleReasonSwThermalSlowdown,
                "sw_power_cap": nv.nvmlClocksThrottleReasonSwPowerCap}
        while not self.stop_flag:
            try:
                sm = nv.nvmlDeviceGetClockInfo(handle, nv.NVML_CLOCK_SM)
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(handle)
                util = nv.nvmlDeviceGetUtilizationRates(handle).gpu
                self.rows.append((float(sm), [n for n, b in bits.items() if mask & b], util > 0))
            except Exception:
                pass
            time.sleep(0.002)

    def start(self):
        try:
            import threading
            import pynvml as nv
            nv.nvmlInit()
            uuid = None
            try:
                import torch
                uuid = str(torch.cuda.get_device_properties(self.index).uuid)
            except Exception:
                pass
            handle = None
            if uuid:
                try:
                    handle = nv.nvmlDeviceGetHandleByUUID(("GPU-" + uuid) if not uuid.startswith("GPU-") else uuid)
                except Exception:
                    handle = None
            if handle is None:
                handle = nv.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = float(nv.nvmlDeviceGetMaxClockInfo(handle, nv.NVML_CLOCK_SM))
            self.stop_flag = False
            self.thread = threading.Thread(target=self._nvml_loop, args=(nv, handle), daemon=True)
            self.thread.start()
            return
        except Exception:
            self.thread = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "20"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            # nvidia-smi needs about a second before its first sample: wait for that line, so that
            # the samples that follow fall into the timed region and not behind it
            self.first = self.proc.stdout.readline()
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        if self.thread is not None:
            self.stop_flag = True
            self.thread.join(timeout=2)
            sm = [r[0] for r in self.rows]
            loaded = [r[0] for r in self.rows if r[2]]
            reasons = sorted({n for r in self.rows for n in r[1]})
            return {"sm_mhz": float(np.median(loaded or sm)) if sm else None, "sm_max_mhz": self.max_mhz,
                    "samples": len(sm), "samples_under_load": len(loaded), "reasons": reasons, "source": "nvml",
                    "window": "from before the warm-up launches to after the end-to-end leg"}
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except Exception:
            self.proc.kill()
            out = ""
        out = getattr(self, "first", "") + out
        sm, mx, busy, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 8:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
                busy.append(float(f[7]) > 0.0)
            except ValueError:
                continue
            for n, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        loaded = [c for c, b in zip(sm, busy) if b]
        return {"sm_mhz": float(np.median(loaded or sm)) if sm else None,
                "sm_max_mhz": float(max(mx)) if mx else None,
                "samples": len(sm), "samples_under_load": len(loaded), "reasons": sorted(reasons),
                "window": "from before the warm-up launches to after the end-to-end leg"}


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


def replica_throughput(n_gpus: int, steps: int, max_seconds: float) -> float:
    """Whole-job samples/s of `n_gpus` replicas that each ran `steps` inferences."""
    return n_gpus * steps / max_seconds if max_seconds > 0 else 0.0


def physical_cores() -> int:
    """Physical cores of the host (distinct (package, core) pairs), else the logical count."""
    try:
        pairs, phys, core = set(), None, None
        for line in open("/proc/cpuinfo"):
            if line.startswith("physical id"):
                phys = line.split(":")[1].strip()
            elif line.startswith("core id"):
                core = line.split(":")[1].strip()
            elif not line.strip():
                if phys is not None and core is not None:
                    pairs.add((phys, core))
                phys = core = None
        if pairs:
            return len(pairs)
    except OSError:
        pass
    return os.cpu_count() or 1


def time_cpu_restatement(cfg, weights, inputs, budget_s: float = 15.0, max_iters: int = 100,
                         warmup: int = 3, threads: int = 0):
    """Bounded timing of the fp32 CPU restatement on `threads` host threads (0: one per
    physical core)."""
    import torch
    from oracle import ref_encoder
    cores = threads or physical_cores()
    torch.set_num_threads(cores)
    for _ in range(warmup):
        ref_encoder.bert_encoder_torch(cfg, weights, inputs)
    t0 = time.perf_counter()
    n = 0
    while n < max_iters and time.perf_counter() - t0 < budget_s:
        ref_encoder.bert_encoder_torch(cfg, weights, inputs)
        n += 1
    dt = time.perf_counter() - t0
    return n / dt, cores, n, dt


def run_reference(args):
    """The reference's CPU path on the host cores: rank 0 only."""
    rank, world, _ = dist_env()
    if rank != 0:
        return
    from mononn_b200 import bert_base, make_inputs, make_weights
    cfg = bert_base()
    w = make_weights(cfg, 1234)
    inp = make_inputs(cfg, 1234)
    per_step = max(1, min(20, int(100 / max(1, args.steps))))  # inferences per step (bounded)
    import torch
    from oracle import ref_encoder
    cores = physical_cores()
    torch.set_num_threads(cores)
    for _ in range(args.warmup):
        ref_encoder.bert_encoder_torch(cfg, w, inp)
    t0 = time.perf_counter()
    for _ in range(args.steps * per_step):
        ref_encoder.bert_encoder_torch(cfg, w, inp)
    dt = time.perf_counter() - t0
    value = args.steps * per_step / dt
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": "BERT-base encoder b1 s128, random-init N(0,0.02), ids uniform",
                   "note": "TF-XLA CPU is not installable here; this is the fp32 CPU restatement "
                           "(torch CPU ops) of the same graph"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port",
                         "logical_cpus": os.cpu_count(),
                         "sample": f"{per_step} inferences per step x {args.steps} steps, "
                                   f"one thread per physical core"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def spec_override_dir(overrides: str, text: str, kind: str):
    """Diagnostic A/B switch: `--spec row_fusion=off,qkv_fusion=off` writes the heuristic spec
    with those fields changed into a temporary spec directory and returns it (else None)."""
    if not overrides:
        return None
    import tempfile
    from mononn_b200.module import describe
    d = describe(kind, text)
    spec = d["spec"]
    for kv in overrides.split(","):
        k, v = kv.split("=")
        if k == "grid":
            spec["cuda_context"]["cuda_runtime_context"]["grid_dim"]["x"] = int(v)
            spec["gemm_spec_list"] = {}
        elif k == "cluster":
            spec["cuda_context"]["cuda_runtime_context"]["cluster_dim"] = {"x": int(v), "y": 1, "z": 1}
        else:
            spec[k] = v
            if k in ("qkv_fusion", "row_fusion"):
                spec["gemm_spec_list"] = {}
    name = d["plan"]["module"]
    root = tempfile.mkdtemp(prefix="mononn_spec_")
    from mononn_b200.module import cluster_dir
    os.makedirs(os.path.join(root, cluster_dir(name)), exist_ok=True)
    with open(os.path.join(root, cluster_dir(name), "best_tuning_spec.json"), "w") as f:
        json.dump(spec, f)
    return root


def run_ours(args):
    import torch
    rank, world, local = dist_env()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the backend has no CPU path")
    torch.cuda.set_device(local)
    use_dist = world > 1
    if use_dist:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    from mononn_b200 import bert_base, compile_encoder, make_inputs, make_weights
    from mononn_b200.hlo_builder import bert_hlo
    from mononn_b200 import compile_hlo

    cfg = bert_base()
    w = make_weights(cfg, 1234)
    inp = make_inputs(cfg, 1234 + rank)
    opts = dict(device=local, tuning_level=args.tuning_level)
    spec_dir = spec_override_dir(args.spec, bert_hlo(cfg)[0] if args.frontend == "hlo" else cfg.to_json(),
                                 "hlo" if args.frontend == "hlo" else "encoder")
    if spec_dir:
        opts["spec_dir"] = spec_dir
    if args.frontend == "hlo":
        text, names = bert_hlo(cfg)
        mod = compile_hlo(text, **opts)
        mod.set_weights({names[k]: v for k, v in w.items()})
    else:
        mod = compile_encoder(cfg, **opts)
        mod.set_weights(w)
    if args.tune:
        mod.tune()
    bufs = mod.allocate()
    descs = mod.args()
    params = sorted([d for d in descs if d["kind"] == 0], key=lambda d: d["param_number"])
    out_desc = [d for d in descs if d["kind"] == 1][0]
    host_in = [torch.from_numpy(inp[k]).contiguous().view(torch.uint8).reshape(-1).pin_memory()
               for k in ("input_ids", "attention_mask", "token_type_ids")]
    host_out = torch.empty(out_desc["bytes"], dtype=torch.uint8).pin_memory()
    for d, h in zip(params, host_in):
        bufs[d["index"]][: h.numel()].copy_(h)
    flush = None if args.no_flush else torch.empty(256 << 20, dtype=torch.uint8, device="cuda")

    def barrier():
        torch.cuda.synchronize()
        if use_dist:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing: K steps, each bracketed by its own event pair so that the
    # L2 flush between steps stays outside the measured time
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    for _ in range(max(args.warmup, 3)):
        mod.launch()
    mod.status()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
          for _ in range(args.steps)]
    barrier()
    for e0, e1 in ev:
        if flush is not None:
            flush.zero_()
        e0.record()
        mod.launch()
        e1.record()
    barrier()
    mod.status()
    dev_s = sum(e0.elapsed_time(e1) for e0, e1 in ev) * 1e-3

    # ---- end to end through the public API with host buffers
    # (mononn_infer_host: pinned host inputs -> device, one launch, live-out -> pinned host,
    # status word checked, stream synchronised)
    if args.e2e_io == "zero_copy":
        # the parameters and the live-out are bound to the pinned host buffers themselves: the
        # kernel pulls the ids over PCIe and writes the hidden states to host memory
        mod.bind_host_io(host_in, [host_out])

    # (a prepared call: same library entry point, pointer arrays and stream handle built once)
    e2e_step = mod.host_runner(host_in, [host_out])

    for _ in range(3):
        e2e_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        e2e_step()
    e2e_s = time.perf_counter() - t0
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    mod.status()

    times = torch.tensor([dev_s, e2e_s], dtype=torch.float64, device="cuda")
    if use_dist:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    dev_s, e2e_s = times.tolist()

    if rank == 0:
        alg_bytes, alg_flops = mod.cost()
        peak, peak_kind = measured_hbm_peak()
        us = dev_s / args.steps * 1e6
        achieved = alg_bytes / (us * 1e-6) / 1e9
        cpu = None
        if world == 1 and not args.no_cpu:
            v, cores, n, dt = time_cpu_restatement(cfg, w, inp)
            v1, _, n1, dt1 = time_cpu_restatement(cfg, w, inp, budget_s=6.0, max_iters=20, warmup=1, threads=1)
            cpu = {"value": v, "unit": UNIT, "cores": cores, "kind": "port",
                   "logical_cpus": os.cpu_count(), "single_thread": v1,
                   "sample": f"{n} inferences of the same workload in {dt:.1f} s on {cores} threads (one per "
                             f"physical core) and {n1} in {dt1:.1f} s on one thread (torch CPU fp32)"}
        h2d = sum(h.numel() for h in host_in)
        line = {
            "metric": METRIC, "value": replica_throughput(world, args.steps, dev_s), "unit": UNIT,
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": dev_s / args.steps * 1e3, "latency_us": us,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16",
            "data": "synthetic",
            "config": {"workload": "BERT-base encoder b1 s128 (12 layers, hidden 768, FFN 3072), "
                                   "random-init N(0,0.02), ids uniform, one launch per inference",
                       "parallelism": f"replicas x{world} (no collective on the data path)",
                       "frontend": args.frontend,
                       "e2e_io": "kernel reads/writes mapped pinned host buffers (no copy calls)"
                                 if args.e2e_io == "zero_copy" else "cudaMemcpyAsync from/to pinned host buffers",
                       "l2": "256 MiB device write between timed steps" if flush is not None
                             else "no flush; 170 MB of weights per step exceed the 126 MB L2",
                       "grid": mod.launch_config()["grid"][0], "stages": len(mod.plan()["stages"])},
            "e2e": {"value": replica_throughput(world, args.steps, e2e_s), "unit": UNIT,
                    "latency_us": e2e_s / args.steps * 1e6,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": int(host_out.numel())},
            "gpu_launches": 2 * args.steps + max(args.warmup, 3) + 3,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "traffic": NCU_TRAFFIC_BYTES,
                         "peak_source": peak_kind, "algorithmic_bytes": alg_bytes,
                         "kernel_us": us},
            "cpu_baseline": cpu,
            "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    mod.close()
    if use_dist:
        dist.destroy_process_group()


def stage_class(stage: dict) -> str:
    """Operator class of a stage, e.g. 'gemm N2304 K768', 'attention', 'layernorm'."""
    kinds = sorted({o["kind"] for o in stage["ops"]})
    gemms = [o for o in stage["ops"] if o["kind"] == "gemm"]
    if gemms:
        n = sum(o["N"] for o in gemms)
        return f"gemm N{n} K{gemms[0]['K']} split{gemms[0]['k_split']}" + ("" if kinds == ["gemm"] else " +" + "+".join(
            k for k in kinds if k != "gemm"))
    return "+".join(kinds)


def stage_report(mod):
    """Per operator class, the time from the in-kernel event trace of one launch, and the share of
    the kernel between the last CTA finishing a stage's work and the first CTA past the barrier."""
    import numpy as np
    plan = mod.plan()
    for _ in range(5):
        mod.launch()
    mod.trace()
    tr = mod.trace()
    tr = np.where(tr == 0, np.nan, tr)
    n_st = tr.shape[1]
    ready = np.nanmin(tr[:, :, 0], axis=0)            # first CTA past the barrier
    done = np.nanmax(tr[:, :, 1], axis=0)             # last CTA finished the stage's work
    total = float(np.nanmax(tr[:, :, 2]) - ready[0])
    per_class: dict[str, list[float]] = {}
    sync = 0.0
    for s_ in range(n_st):
        end = ready[s_ + 1] if s_ + 1 < n_st else np.nanmax(tr[:, s_, 2])
        sync += float(end - done[s_])
        acc = per_class.setdefault(stage_class(plan["stages"][s_]), [0, 0.0, 0.0])
        acc[0] += 1
        acc[1] += float(end - ready[s_])
        acc[2] += float(end - done[s_])
    classes = {k: {"stages": v[0], "us_per_stage": v[1] / v[0] / 1e3, "share": v[1] / total,
                   "barrier_us_per_stage": v[2] / v[0] / 1e3} for k, v in per_class.items()}
    return {"diagnostic": "stage_report", "kernel_us": total / 1e3, "stages": n_st,
            "barrier_share": sync / total, "classes": classes}


def run_diagnostics(args):
    """Not a bench line. `--stages A:B` launches only stages [A, B) of the headline workload
    `--steps` times (so that a profiler can capture one operator class alone) and prints their
    time; `--stage-report` prints, per operator class, the time from the in-kernel event trace
    and the share of the kernel spent between the last CTA finishing a stage's work and the
    first CTA observing the barrier (release fence + arrive + propagation)."""
    import numpy as np
    import torch
    from mononn_b200 import bert_base, compile_hlo, make_inputs, make_weights
    from mononn_b200.hlo_builder import bert_hlo
    torch.cuda.set_device(0)
    cfg = bert_base()
    w = make_weights(cfg, 1234)
    inp = make_inputs(cfg, 1234)
    text, names = bert_hlo(cfg)
    mod = compile_hlo(text, device=0)
    mod.set_weights({names[k]: v for k, v in w.items()})
    mod.run([inp["input_ids"], inp["attention_mask"], inp["token_type_ids"]])
    plan = mod.plan()
    if args.stages:
        a, b = (int(x) for x in args.stages.split(":"))
        for _ in range(max(args.warmup, 1)):
            mod.launch_stages(a, b)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            mod.launch_stages(a, b)
        e1.record()
        torch.cuda.synchronize()
        mod.status()
        print(json.dumps({"diagnostic": "stage_range", "stages": [a, b],
                          "classes": [stage_class(st) for st in plan["stages"][a:b]],
                          "us_per_launch": e0.elapsed_time(e1) * 1e3 / args.steps, "launches": args.steps}))
    else:
        print(json.dumps(stage_report(mod)))
    mod.close()


def run_config(args):
    """Not a bench line: one launch per inference of another configuration at full size, device
    time by CUDA events with an L2 flush between launches, against the slower of algorithmic
    bytes at the measured HBM peak and FLOPs at the measured dense tensor peak."""
    import torch
    from mononn_b200 import (clip_b32, compile_hlo, make_clip_inputs, make_inputs, make_t5_inputs, make_vit_inputs,
                             make_weights, opt_1p3b, t5_device_weights, t5_small, vit_base)
    from mononn_b200.hlo_builder import bert_hlo, clip_hlo, opt_hlo, t5_hlo, vit_hlo
    from mononn_b200.models import EncoderConfig
    torch.cuda.set_device(0)
    name = args.config
    large = lambda b: EncoderConfig(layers=24, hidden=1024, heads=16, ffn=4096, batch=b, seq=384)
    table = {
        "bert_large_b1": (large(1), bert_hlo, 1235, "bert"), "bert_large_b16": (large(16), bert_hlo, 1235, "bert"),
        "vit_b1": (vit_base(1), vit_hlo, 1236, "vit"), "vit_b64": (vit_base(64), vit_hlo, 1236, "vit"),
        "opt_b1": (opt_1p3b(1), opt_hlo, 1237, "opt"), "opt_b8": (opt_1p3b(8), opt_hlo, 1237, "opt"),
        "clip": (clip_b32(), clip_hlo, 1238, "clip"),
        "t5_small": (t5_small(1), t5_hlo, 1239, "t5"),
    }
    cfg, hlo, seed, family = table[name]
    w = make_weights(cfg, seed)
    if family == "t5":
        w = t5_device_weights(cfg, w)
    text, names = hlo(cfg)
    mod = compile_hlo(text, device=0, barrier_timeout_us=2000000, tuning_level=args.tuning_level,
                      dump_dir=(args.dump_dir or None) if args.tune else None)
    mod.set_weights({names[k]: v for k, v in w.items()})
    if family == "bert":
        inp = make_inputs(cfg, seed, pad_fraction=0.25)
        ins = [inp["input_ids"], inp["attention_mask"], inp["token_type_ids"]]
    elif family == "vit":
        ins = [make_vit_inputs(cfg, seed)["pixel_values"]]
    elif family == "opt":
        ins = [make_inputs(cfg, seed)["input_ids"]]
    elif family == "t5":
        inp = make_t5_inputs(cfg, seed)
        ins = [inp["input_ids"], inp["decoder_input_ids"]]
    else:
        inp = make_clip_inputs(cfg, seed)
        ins = [inp["pixel_values"], inp["input_ids"]]
    mod.run(ins)
    if args.tune:
        mod.tune()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(max(args.warmup, 3)):
        mod.launch()
    steps = min(args.steps, 50)
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    for e0, e1 in ev:
        flush.zero_()
        e0.record()
        mod.launch()
        e1.record()
    torch.cuda.synchronize()
    mod.status()
    us = sum(e0.elapsed_time(e1) for e0, e1 in ev) * 1e3 / steps
    if args.stage_report:
        print(json.dumps(dict(stage_report(mod), config=name)))
    alg_bytes, alg_flops = mod.cost()
    peak_gbs, kind = measured_hbm_peak()
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            peak_tf = float(json.load(f)["bf16_tflops"])
    except Exception:
        peak_tf = 1590.0
    t_hbm = alg_bytes / (peak_gbs * 1e9) * 1e6
    t_tc = alg_flops / (peak_tf * 1e12) * 1e6
    print(json.dumps({"diagnostic": "config", "config": name, "us_per_launch": us, "launches": steps,
                      "stages": len(mod.plan()["stages"]), "algorithmic_bytes": alg_bytes,
                      "algorithmic_flops": alg_flops, "roofline_us": max(t_hbm, t_tc),
                      "bound": "hbm" if t_hbm >= t_tc else "tensor", "frac": max(t_hbm, t_tc) / us,
                      "peaks": {"hbm_gbs": peak_gbs, "tensor_tflops": peak_tf, "source": kind}}))
    mod.close()


def run_mma_probe(args):
    """Not a bench line: the issue-cost table of tcgen05.mma (128 x N x 16, f16 in, f32 accumulate)
    from operands resident in shared memory, one issuing thread per CTA on every SM."""
    import ctypes as C
    import torch
    from mononn_b200 import capi
    l = capi.lib()
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    rows = []
    for mode, what in ((16, "back to back, one lane"),
                       (16 + 64, "+ descriptors rebuilt per four from a ring slot"),
                       (16 + 64 + 3, "+ commit, satisfied wait and fence per four (a main loop), one lane"),
                       (16 + 64 + 3 + 32, "the same main loop, warp converged with an elected issuer"),
                       (16 + 32 + 4, "back to back, M = 64"),
                       (32 + 8, "back to back, A from tensor memory")):
        for n in (16, 32, 64, 128, 192, 256):
            cyc, iss, ns = C.c_double(), C.c_double(), C.c_double()
            capi.check(l.mononn_debug_mma_issue(0, n, 1024, 1, mode, sms, C.byref(cyc), C.byref(iss), C.byref(ns)))
            rows.append({"n": n, "mode": what, "cycles_per_mma": round(cyc.value, 1),
                         "issue_cycles_per_mma": round(iss.value, 1), "ns_per_mma": round(ns.value, 1)})
    print(json.dumps({"diagnostic": "mma_issue_probe", "ctas": sms, "instructions": 1024, "table": rows}))


def run_torch_baseline(args):
    """Not a bench line and not the product path: BERT-base b1/s128 forward written with plain
    torch fp16 ops (library GEMMs, one kernel per operator) on the same GPU, eager and replayed
    from a CUDA graph, so that the single persistent launch can be compared with the path every
    user already has."""
    import math
    import torch
    import torch.nn.functional as F
    from mononn_b200 import bert_base, make_inputs, make_weights
    torch.cuda.set_device(0)
    cfg = bert_base()
    w = {k: torch.from_numpy(v).cuda().half() for k, v in make_weights(cfg, 1234).items()}
    inp = make_inputs(cfg, 1234)
    ids = torch.from_numpy(inp["input_ids"]).long().cuda()
    types = torch.from_numpy(inp["token_type_ids"]).long().cuda()
    mask_bias = ((1.0 - torch.from_numpy(inp["attention_mask"]).float()) * -10000.0).cuda().half()
    b, s_, h, nh = cfg.batch, cfg.seq, cfg.hidden, cfg.heads

    def forward():
        x = w["embeddings.word"][ids] + w["embeddings.position"][:s_][None] + w["embeddings.token_type"][types]
        x = F.layer_norm(x, (h,), w["embeddings.ln.gamma"], w["embeddings.ln.beta"], cfg.eps)
        for l in range(cfg.layers):
            p = f"layer{l}."
            lin = lambda t, n: torch.addmm(w[p + n + ".b"], t.reshape(-1, t.shape[-1]), w[p + n + ".w"]).view(b, s_, -1)
            split = lambda t: t.view(b, s_, nh, h // nh).transpose(1, 2)
            q, k, v = split(lin(x, "attn.q")), split(lin(x, "attn.k")), split(lin(x, "attn.v"))
            sc = q @ k.transpose(-1, -2) / math.sqrt(h // nh) + mask_bias[:, None, None, :]
            ctx = (torch.softmax(sc, -1) @ v).transpose(1, 2).reshape(b, s_, h)
            x = F.layer_norm(lin(ctx, "attn.o") + x, (h,), w[p + "attn.ln.gamma"], w[p + "attn.ln.beta"], cfg.eps)
            y = F.gelu(lin(x, "ffn.up"))
            x = F.layer_norm(lin(y, "ffn.down") + x, (h,), w[p + "ffn.ln.gamma"], w[p + "ffn.ln.beta"], cfg.eps)
        return x

    def timed(fn, n):
        for _ in range(5):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e3 / n

    with torch.no_grad():
        eager = timed(forward, args.steps)
        g = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            forward()
            with torch.cuda.graph(g, stream=side):
                forward()
        torch.cuda.synchronize()
        replay = timed(g.replay, args.steps)
    print(json.dumps({"diagnostic": "torch_fp16_baseline", "workload": "BERT-base b1 s128",
                      "eager_us": eager, "cuda_graph_replay_us": replay, "launches": args.steps,
                      "note": "plain torch fp16 ops with library GEMMs; weights stay L2/HBM resident between "
                              "launches (no flush)"}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--frontend", default="hlo", choices=["hlo", "builder"],
                    help="lower from authored HLO text (the hook path) or the config builder")
    ap.add_argument("--tune", action="store_true", help="run the on-device schedule search first")
    ap.add_argument("--dump-dir", default="", help="with --config --tune: where the tuner writes its spec and logs")
    ap.add_argument("--tuning-level", type=int, default=1, help="what --tune searches (see include/mononn.h)")
    ap.add_argument("--spec", default="", help="diagnostic: spec fields to override, e.g. row_fusion=off,grid=128")
    ap.add_argument("--config", default="", help="diagnostic: time another configuration (bert_large_b1, "
                    "bert_large_b16, vit_b1, vit_b64, opt_b1, opt_b8, clip, t5_small) and print its roofline fraction")
    ap.add_argument("--mma-probe", action="store_true",
                    help="diagnostic: cycles per tcgen05.mma by tile width (mononn_debug_mma_issue)")
    ap.add_argument("--torch-baseline", action="store_true",
                    help="diagnostic: the same BERT-base forward in plain torch fp16 on this GPU (eager and graph replay)")
    ap.add_argument("--no-flush", action="store_true", help="do not flush L2 between timed steps")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--e2e-io", default="copy", choices=["copy", "zero_copy"],
                    help="end-to-end leg: explicit copies, or parameters/live-out bound to pinned host memory")
    ap.add_argument("--stages", default="", help="diagnostic: launch only stages A:B of the workload")
    ap.add_argument("--stage-report", action="store_true",
                    help="diagnostic: per operator class time and the barrier's share, from the event trace")
    args = ap.parse_args()
    if args.mma_probe:
        run_mma_probe(args)
    elif args.config:
        run_config(args)
    elif args.torch_baseline:
        run_torch_baseline(args)
    elif args.stages or args.stage_report:
        run_diagnostics(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
