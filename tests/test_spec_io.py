"""Dump-directory layout of TF_MONONN_DUMP_DIR / TF_MONONN_EXISTING_TUNING_SPEC_DIR."""
import ctypes as C
import json
import os

from mononn_b200 import bert_tiny, capi
from mononn_b200.module import describe


def test_cluster_directory_name_follows_the_module_name(lib_built):
    # get_hlo_module_short_name: "cluster_<digits>" prefix (helpers/string_helpers.cc:34-46)
    cfg = bert_tiny()
    cfg.name = "cluster_12__XlaCompiledKernel_true"
    d = describe("encoder", cfg.to_json())
    assert d["plan"]["module"] == cfg.name
    assert d["spec"]["hlo_module_name"] == cfg.name


def test_spec_json_is_plain_json_with_original_field_names(lib_built):
    d = describe("encoder", bert_tiny().to_json())["spec"]
    text = json.dumps(d)
    back = json.loads(text)
    assert back["cuda_context"]["cuda_device_context"]["cuda_arch"] == "1000"
    g = back["gemm_spec_list"]["layer0.attn.o"]
    assert set(g["sm100_config"]) >= {"mma_m", "mma_n", "k_split", "cluster_x", "cluster_y", "cta_group", "epilogue_fusion"}
    assert g["problem"] == {"m": 16, "n": 64, "k": 64}
    assert back["qkv_fusion"] == "auto" and "layer0.attn.q" not in back["gemm_spec_list"]   # computed inside attention
