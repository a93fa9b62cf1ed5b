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


def test_structure_fields_round_trip_through_the_spec(lib_built):
    """Cluster shape, LayerNorm placement and projection fusion are spec fields: a spec that sets
    them lowers to a plan that carries them, and a shape that does not divide the grid is refused."""
    cfg = bert_tiny(batch=2, seq=24, layers=2, hidden=128, ffn=512)
    base = describe("encoder", cfg.to_json())
    assert base["plan"]["cluster"] == 1 and base["spec"]["row_fusion"] == "on"
    spec = dict(base["spec"], row_fusion="off")
    spec["cuda_context"]["cuda_runtime_context"]["cluster_dim"] = {"x": 4, "y": 1, "z": 1}
    d = describe("encoder", cfg.to_json(), spec=spec)
    assert d["plan"]["cluster"] == 4 and d["spec"]["row_fusion"] == "off"
    assert d["spec"]["cuda_context"]["cuda_runtime_context"]["cluster_dim"]["x"] == 4
    assert len(d["plan"]["stages"]) > len(base["plan"]["stages"])
    assert all(g["sm100_config"]["cluster_x"] == 4 for g in d["spec"]["gemm_spec_list"].values())
    spec["cuda_context"]["cuda_runtime_context"]["cluster_dim"]["x"] = 3
    import pytest
    with pytest.raises(capi.MononnError):
        describe("encoder", cfg.to_json(), spec=spec)
