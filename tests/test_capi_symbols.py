"""The C-ABI library loads on a machine without a GPU, exports every function the header
declares, and fails loudly (no CPU fallback) when asked to compile without a device."""
import ctypes
import os
import re

import pytest

from mononn_b200 import capi
from tests.helpers import ROOT


def declared_functions():
    text = open(os.path.join(ROOT, "include", "mononn.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(mononn_[a-z_0-9]+)\s*\(", text)))


def test_header_declares_the_boundary():
    names = declared_functions()
    for must in ("mononn_compile_hlo_text", "mononn_module_args", "mononn_module_launch_config",
                 "mononn_set_constant", "mononn_launch", "mononn_last_status", "mononn_save_spec",
                 "mononn_destroy", "mononn_strerror"):
        assert must in names


def test_library_exports_every_declared_symbol(lib_built):
    lib = ctypes.CDLL(lib_built)
    for name in declared_functions():
        assert hasattr(lib, name), f"{name} is declared in include/mononn.h but not exported"


def test_python_binding_lists_the_same_symbols(lib_built):
    assert sorted(capi.EXPORTS) == declared_functions()


def test_strerror_and_enabled(lib_built, monkeypatch):
    l = capi.lib()
    assert l.mononn_strerror(0) == b"ok"
    assert b"kernel" in l.mononn_strerror(-6)
    for v, want in (("True", 1), ("true", 1), ("1", 1), ("yes", 0), ("0", 0), ("TRUE", 0)):
        monkeypatch.setenv("TF_MONONN_ENABLED", v)
        assert l.mononn_enabled() == want  # helpers/env_variable.cc:20-26
    monkeypatch.delenv("TF_MONONN_ENABLED")
    assert l.mononn_enabled() == 0


def test_no_cpu_fallback(lib_built):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from mononn_b200 import bert_tiny, compile_encoder
    with pytest.raises(capi.MononnError) as e:
        compile_encoder(bert_tiny())
    assert e.value.code == -5  # MONONN_ERR_NO_DEVICE
