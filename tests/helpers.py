"""Shared helpers of the test-suite (not collected as tests)."""
import importlib.util
import os

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLDEN = os.path.join(ROOT, "tests", "golden")

# Tolerance of the path: the device computes in f16 with fp32 accumulation, the oracle in
# fp32; the final hidden states must agree to cosine >= 0.999 and max-abs <= 2e-2.
COS_MIN = 0.999
MAX_ABS = 2e-2


def golden_cases():
    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(GOLDEN, "make_golden.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.CASES


def load_golden(name):
    return np.load(os.path.join(GOLDEN, name + ".npz"))


def cosine(a, b):
    a, b = a.astype(np.float64).ravel(), b.astype(np.float64).ravel()
    return float(a @ b / (np.linalg.norm(a) * np.linalg.norm(b) + 1e-30))


def assert_parity(got, ref, what=""):
    got = np.asarray(got, np.float32)
    ref = np.asarray(ref, np.float32)
    assert got.shape == ref.shape, (what, got.shape, ref.shape)
    assert np.isfinite(got).all(), what
    err = float(np.abs(got - ref).max())
    cos = cosine(got, ref)
    assert cos >= COS_MIN and err <= MAX_ABS, f"{what}: cosine {cos:.6f}, max-abs {err:.5f}"
    return err, cos


def reference_fixture_inputs():
    """The reference's only fixture, examples/data/bert_bs1.npy: int32 [1,128] tensors
    input_ids = 101, 7592 x 126, 102; attention_mask all ones; token_type_ids all zero."""
    ids = np.full((1, 128), 7592, np.int32)
    ids[0, 0], ids[0, -1] = 101, 102
    return {"input_ids": ids, "attention_mask": np.ones((1, 128), np.int32),
            "token_type_ids": np.zeros((1, 128), np.int32)}
