"""Host-side mirror of the reference's module interface on top of the C ABI.

``Module`` corresponds to MonoNNModule (mononn_engine/module/mononn_module.h:31-87):
arguments in the order (parameters.., live-outs.., temp), launch configuration from the
tuning spec, one launch per inference.  PyTorch is used only as the owner of device
memory and streams.
"""
from __future__ import annotations

import ctypes as C
import json
import os

import numpy as np

from . import capi
from .capi import ArgDesc, Options, check, lib


def _options(device=0, dump_dir=None, spec_dir=None, threadpool_size=0, tuning_level=0,
             barrier_timeout_us=0) -> Options:
    o = Options()
    o.device = device
    o.dump_dir = dump_dir.encode() if dump_dir else None
    o.spec_dir = spec_dir.encode() if spec_dir else None
    o.threadpool_size = threadpool_size
    o.tuning_level = tuning_level
    o.barrier_timeout_us = barrier_timeout_us
    return o


class Module:
    def __init__(self, handle: C.c_void_p, device: int = 0):
        self._h = handle
        self.device = device
        self._bufs = None
        self._ptrs = None

    # ------------------------------------------------------------------ metadata
    def args(self) -> list[dict]:
        descs = C.POINTER(ArgDesc)()
        n = C.c_int()
        check(lib().mononn_module_args(self._h, C.byref(descs), C.byref(n)))
        return [dict(index=descs[i].index, bytes=descs[i].bytes, kind=descs[i].kind,
                     param_number=descs[i].param_number) for i in range(n.value)]

    def launch_config(self) -> dict:
        g, b, s = (C.c_uint * 3)(), (C.c_uint * 3)(), C.c_uint()
        check(lib().mononn_module_launch_config(self._h, C.byref(g), C.byref(b), C.byref(s)))
        return dict(grid=tuple(g), block=tuple(b), smem_bytes=s.value)

    def constants(self) -> dict[str, int]:
        n = C.c_int()
        check(lib().mononn_constant_count(self._h, C.byref(n)))
        out = {}
        for i in range(n.value):
            name, size = C.c_char_p(), C.c_size_t()
            check(lib().mononn_constant_info(self._h, i, C.byref(name), C.byref(size)))
            out[name.value.decode()] = size.value
        return out

    def cost(self) -> tuple[float, float]:
        b, f = C.c_double(), C.c_double()
        check(lib().mononn_module_cost(self._h, C.byref(b), C.byref(f)))
        return b.value, f.value

    def spec(self) -> dict:
        p = C.c_char_p()
        check(lib().mononn_spec_json(self._h, C.byref(p)))
        return json.loads(p.value.decode())

    def plan(self) -> dict:
        p = C.c_char_p()
        check(lib().mononn_plan_json(self._h, C.byref(p)))
        return json.loads(p.value.decode())

    def launch_stages(self, begin: int, end: int, stream=None) -> None:
        """Single-stage isolation: run stages [begin, end) in one launch."""
        if self._ptrs is None:
            self.allocate()
        check(lib().mononn_launch_stages(self._h, self._ptrs, len(self._bufs), self._stream(stream), begin, end))

    def debug_skew_barrier(self, missing_arrivals: int) -> None:
        check(lib().mononn_debug_skew_barrier(self._h, missing_arrivals))

    def save_spec(self, directory: str) -> None:
        check(lib().mononn_save_spec(self._h, directory.encode()))

    # ----------------------------------------------------------------- constants
    def set_constant(self, name: str, array: np.ndarray) -> None:
        a = np.ascontiguousarray(array)
        check(lib().mononn_set_constant(self._h, name.encode(), a.ctypes.data_as(C.c_void_p), a.nbytes))

    def set_weights(self, weights: dict[str, np.ndarray]) -> None:
        """fp32 weight dict -> fp16 constants, by name."""
        for name in self.constants():
            self.set_constant(name, np.asarray(weights[name]).astype(np.float16))

    # ------------------------------------------------------------------- buffers
    def allocate(self):
        """Device buffers for every kernel argument (torch owns the memory)."""
        import torch
        dev = torch.device("cuda", self.device)
        self._bufs = [torch.zeros(max(a["bytes"], 16), dtype=torch.uint8, device=dev) for a in self.args()]
        self._ptrs = (C.c_void_p * len(self._bufs))(*[b.data_ptr() for b in self._bufs])
        return self._bufs

    @property
    def buffers(self):
        if self._bufs is None:
            self.allocate()
        return self._bufs

    def _stream(self, stream) -> C.c_void_p:
        import torch
        s = stream if stream is not None else torch.cuda.current_stream(self.device)
        return C.c_void_p(s.cuda_stream)

    def launch(self, stream=None) -> None:
        """Exactly one kernel launch on `stream` (default: torch's current stream)."""
        if self._ptrs is None:
            self.allocate()
        check(lib().mononn_launch(self._h, self._ptrs, len(self._bufs), self._stream(stream)))

    def status(self) -> None:
        st, cta = C.c_int(), C.c_int()
        check(lib().mononn_last_status(self._h, C.byref(st), C.byref(cta)))

    def tune(self, stream=None) -> None:
        if self._ptrs is None:
            self.allocate()
        check(lib().mononn_tune(self._h, self._ptrs, len(self._bufs), self._stream(stream)))

    def profile_stages(self, stream=None) -> list[tuple[str, float]]:
        if self._ptrs is None:
            self.allocate()
        cap = 4096
        us = (C.c_double * cap)()
        names = (C.c_char_p * cap)()
        n = C.c_int()
        check(lib().mononn_profile_stages(self._h, self._ptrs, len(self._bufs), self._stream(stream),
                                          us, names, cap, C.byref(n)))
        return [(names[i].decode(), us[i]) for i in range(min(n.value, cap))]

    def trace(self, stream=None) -> np.ndarray:
        """Per-CTA event trace of one launch: array [grid, stages, 16] in ns (0 = no event)."""
        if self._ptrs is None:
            self.allocate()
        cfg = self.launch_config()
        n_st = len(self.plan()["stages"])
        out = np.zeros(cfg["grid"][0] * n_st * 16, np.float64)
        g, s = C.c_int(), C.c_int()
        check(lib().mononn_trace_stages(self._h, self._ptrs, len(self._bufs), self._stream(stream),
                                        out.ctypes.data_as(C.POINTER(C.c_double)), out.size, C.byref(g), C.byref(s)))
        return out.reshape(g.value, s.value, 16)

    # ---------------------------------------------------------------- inference
    def run(self, inputs: list[np.ndarray]) -> list[np.ndarray]:
        """Host arrays in (by parameter number) -> host arrays out (live-outs, raw bytes
        viewed as fp16).  Copies are on torch's current stream around the single launch."""
        import torch
        bufs = self.buffers
        descs = self.args()
        params = [d for d in descs if d["kind"] == 0]
        for d, x in zip(sorted(params, key=lambda d: d["param_number"]), inputs):
            src = torch.from_numpy(np.ascontiguousarray(x)).view(torch.uint8).reshape(-1)
            bufs[d["index"]][: src.numel()].copy_(src, non_blocking=True)
        self.launch()
        outs = [bufs[d["index"]].cpu().numpy().view(np.float16) for d in descs if d["kind"] == 1]
        self.status()
        return outs

    def bind_host_io(self, host_inputs, host_outputs) -> None:
        """Zero-copy I/O: bind the parameters and live-outs to PINNED host tensors (inputs by
        parameter number, outputs by live-out order), so that the kernel reads and writes host
        memory itself and `infer_host` on the same tensors issues no copies."""
        if self._ptrs is None:
            self.allocate()
        descs = self.args()
        for d in descs:
            if d["kind"] == 0:
                self._ptrs[d["index"]] = host_inputs[d["param_number"]].data_ptr()
            elif d["kind"] == 1:
                self._ptrs[d["index"]] = host_outputs[d["param_number"]].data_ptr()

    def infer_host(self, host_inputs, host_outputs, stream=None) -> None:
        """One inference between host buffers (torch CPU tensors, pinned for asynchronous
        copies; inputs by parameter number, outputs by live-out order): H2D copies, one
        launch, D2H copies, status check and stream synchronisation, all inside the library."""
        if self._ptrs is None:
            self.allocate()
        key = tuple(t.data_ptr() for t in host_inputs) + tuple(t.data_ptr() for t in host_outputs)
        if getattr(self, "_host_key", None) != key:  # pointer arrays are rebuilt only when the buffers change
            self._host_key = key
            self._host_in = (C.c_void_p * len(host_inputs))(*key[: len(host_inputs)])
            self._host_out = (C.c_void_p * len(host_outputs))(*key[len(host_inputs):])
        check(lib().mononn_infer_host(self._h, self._host_in, len(host_inputs), self._host_out, len(host_outputs),
                                      self._ptrs, len(self._bufs), self._stream(stream)))

    def host_runner(self, host_inputs, host_outputs, stream=None):
        """A prepared `infer_host`: the pointer arrays and the stream handle are built once, and the
        returned zero-argument callable does nothing but the library call (for serving loops that
        reuse their pinned buffers; the Python bookkeeping of `infer_host` is several microseconds
        per call). The stream is the one given, or torch's current stream at preparation time."""
        if self._ptrs is None:
            self.allocate()
        keep = (list(host_inputs), list(host_outputs))   # the buffers must outlive the runner
        h_in = (C.c_void_p * len(host_inputs))(*[t.data_ptr() for t in host_inputs])
        h_out = (C.c_void_p * len(host_outputs))(*[t.data_ptr() for t in host_outputs])
        fn, args = lib().mononn_infer_host, (self._h, h_in, len(host_inputs), h_out, len(host_outputs),
                                             self._ptrs, len(self._bufs), self._stream(stream))

        def run(_keep=keep):
            rc = fn(*args)
            if rc:
                check(rc)
        return run

    def close(self) -> None:
        if self._h:
            lib().mononn_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def compile_encoder(cfg, kernel_name: str | None = None, **opts) -> Module:
    """Standalone path: fused graph from an encoder configuration."""
    h = C.c_void_p()
    o = _options(**opts)
    check(lib().mononn_compile_encoder_json(cfg.to_json().encode(), kernel_name.encode() if kernel_name else None,
                                            C.byref(o), C.byref(h)))
    return Module(h, o.device)


def compile_hlo(hlo_text: str, kernel_name: str | None = None, **opts) -> Module:
    """Hook path: post-optimisation XLA HLO text of a cluster -> module."""
    h = C.c_void_p()
    o = _options(**opts)
    data = hlo_text.encode()
    check(lib().mononn_compile_hlo_text(data, len(data), kernel_name.encode() if kernel_name else None,
                                        C.byref(o), C.byref(h)))
    return Module(h, o.device)


def describe(kind: str, text: str, spec: dict | None = None, sm_count: int = 148) -> dict:
    """Lower without a device: {"plan": ..., "spec": ...} for an HLO text or encoder JSON."""
    out = C.c_void_p()
    data = text.encode()
    check(lib().mononn_describe(kind.encode(), data, len(data), json.dumps(spec).encode() if spec else None,
                                sm_count, C.byref(out)))
    try:
        return json.loads(C.string_at(out).decode())
    finally:
        lib().mononn_free_string(out)


def cluster_dir(module_name: str) -> str:
    """Directory name of a module inside a spec / dump directory: "cluster_<digits>" taken from the
    module name (mononn_engine/helpers/string_helpers.cc:34-46), else the sanitised name."""
    import re
    m = re.match(r"cluster_(\d+)", module_name)
    if m:
        return f"cluster_{m.group(1)}"
    return re.sub(r"[^0-9A-Za-z]", "_", module_name) or "cluster_0"


def attention_noalloc(q_ptr: int, k_ptr: int, vt_ptr: int, mask_ptr: int | None, out_ptr: int, batches: int,
                      heads: int, seq: int, ld_qk: int, ld_vt: int, ld_out: int, scale: float,
                      mask_scale: float = -10000.0, causal: bool = False, stream=None) -> None:
    """Allocation-free attention on caller-owned device buffers (raw device pointers): for
    hosts whose allocator owns the GPU and where this library must not cudaMalloc.  Calls on
    one device share a static scratch array and must not overlap on the GPU."""
    import torch
    st = stream if stream is not None else torch.cuda.current_stream()
    check(lib().mononn_attention_noalloc(C.c_void_p(q_ptr), C.c_void_p(k_ptr), C.c_void_p(vt_ptr),
                                         C.c_void_p(mask_ptr) if mask_ptr else None, C.c_void_p(out_ptr),
                                         batches, heads, seq, ld_qk, ld_vt, ld_out, scale, mask_scale,
                                         1 if causal else 0, C.c_void_p(st.cuda_stream)))


def attention_noalloc_status(stream=None) -> None:
    """Waits for the stream and raises MononnError(-6) when a bounded wait expired in the last
    allocation-free attention call on this device (its output is then incomplete)."""
    import torch
    st = stream if stream is not None else torch.cuda.current_stream()
    check(lib().mononn_attention_noalloc_status(C.c_void_p(st.cuda_stream)))


def enabled() -> bool:
    """TF_MONONN_ENABLED truthiness (True / true / 1)."""
    return bool(lib().mononn_enabled())
