"""CPU checks of the drop-in boundary: the library loads without a GPU and exports every symbol
the headers declare; the Python mirror refuses CPU tensors (no fallback path)."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    names = set()
    for h in ("bonsai_p40.h", "bonsai_b200_ext.h", "bonsai_kv.h"):
        text = open(os.path.join(ROOT, "include", h)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names |= set(re.findall(r"\b(?:int|int64_t|void|float \*|bonsai_kv_cache \*)\s*(bonsai_\w+)\s*\(", text))
    return names


def test_library_exports_every_declared_symbol():
    import bonsai_b200
    names = declared_symbols()
    assert {"bonsai_p40_gemv", "bonsai_p40_quant_activations", "bonsai_p40_gemm", "bonsai_p40_repack",
            "bonsai_p40_gemv_repack", "bonsai_p40_fwht", "bonsai_p40_rmsnorm", "bonsai_p40_gdn_step",
            "bonsai_p40_attn"} <= names
    handle = ctypes.CDLL(bonsai_b200.LIB_PATH)
    for n in names:
        assert hasattr(handle, n), n
    assert names == set(bonsai_b200.SIGNATURES), names ^ set(bonsai_b200.SIGNATURES)


def test_version_and_options_without_gpu():
    import bonsai_b200
    assert bonsai_b200.version() >= 100
    assert bonsai_b200.set_option("pdl", 0) == 0
    assert bonsai_b200.set_option("gemv_variant", -1) == 0
    assert bonsai_b200.set_option("gemv_order", 0) == 0
    assert bonsai_b200.set_option("no_such_key", 1) == 1


def test_python_mirror_refuses_cpu_tensors():
    import torch
    import bonsai_b200
    x = torch.zeros(1024)
    with pytest.raises(RuntimeError, match="no CPU path"):
        bonsai_b200.quant_activations(x, torch.zeros(1152, dtype=torch.uint8), 1024)


def test_shape_rejections_need_no_gpu():
    # argument validation happens before any CUDA call (reference wrappers: gemv_p40.cu:201,212;
    # gemm_p40.cu:145; gemv_repack_p40.cu:198-200; elementwise_p40.cu:76)
    import bonsai_b200
    L = bonsai_b200.lib()
    assert L.bonsai_p40_gemv(None, None, None, 8, 100, None) == 1
    assert L.bonsai_p40_gemv(None, None, None, 8, 0, None) == 1
    assert L.bonsai_p40_gemv(None, None, None, 0, 128, None) == 0
    assert L.bonsai_p40_quant_activations(None, None, 33, None) == 1
    assert L.bonsai_p40_quant_activations(None, None, 0, None) == 1
    assert L.bonsai_p40_gemm(None, None, None, 8, 130, 4, None) == 1
    assert L.bonsai_p40_gemm(None, None, None, 0, 128, 4, None) == 0
    assert L.bonsai_p40_gemm(None, None, None, 8, 128, 0, None) == 0
    assert L.bonsai_p40_repack(None, None, 8, 128, None) == 1          # 1 block: not a multiple of 8
    assert L.bonsai_p40_repack(None, None, 0, 1024, None) == 1
    assert L.bonsai_p40_gemv_repack(None, None, None, 8, 640, None) == 1
    assert L.bonsai_p40_fwht(None, None, 1000, None) == 1
    assert L.bonsai_p40_fwht(None, None, 0, None) == 1
    # the operators beside the path (reference: elementwise_p40.cu:82-84, attn_p40.cu:121-124, 134-136)
    assert L.bonsai_p40_rmsnorm(None, None, None, 1, 0, 1e-6, None) == 1
    assert L.bonsai_p40_rmsnorm(None, None, None, 0, 8, 1e-6, None) == 0
    assert L.bonsai_p40_gdn_step(None, None, None, None, None, None, None, 4, 8, 128, 33, None) == 1
    assert L.bonsai_p40_gdn_step(None, None, None, None, None, None, None, 4, 8, 129, 128, None) == 1
    assert L.bonsai_p40_gdn_step(None, None, None, None, None, None, None, 3, 8, 128, 128, None) == 1
    assert L.bonsai_p40_attn(None, None, None, None, 4, 24, 4, 128, 0.1, None) == 1
    assert L.bonsai_p40_attn(None, None, None, None, 4, 24, 5, 256, 0.1, None) == 1
    assert L.bonsai_p40_attn(None, None, None, None, 0, 24, 4, 256, 0.1, None) == 0
