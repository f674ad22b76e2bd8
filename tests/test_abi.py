"""CPU-only: the C-ABI library builds, loads and exports what include/moe_b200.h declares."""
import ctypes as C
import os
import re

import numpy as np
import pytest

from moe_infer_b200 import _lib

INCLUDE = os.path.join(os.path.dirname(__file__), "..", "include")
HEADER = os.path.join(INCLUDE, "moe_b200.h")


def declared_functions():
    """Every function any header under include/ declares (the product ABI and the bench tooling header)."""
    names = set()
    for f in sorted(os.listdir(INCLUDE)):
        if not f.endswith(".h"):
            continue
        src = open(os.path.join(INCLUDE, f)).read()
        src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
        names.update(re.findall(r"\b(moe_[a-z0-9_]+)\s*\(", src))
    return sorted(n for n in names if not n.endswith("_fn"))


def test_header_functions_are_exported(native_lib):
    names = declared_functions()
    assert len(names) >= 40
    for n in names:
        assert hasattr(native_lib, n), f"{n} declared in moe_b200.h but not exported"


def test_binding_covers_header():
    assert set(declared_functions()) == set(_lib.SIGNATURES)


def test_every_entry_point_cites_the_reference_or_says_none():
    src = open(HEADER).read()
    assert src.count("src/") >= 20
    assert "No counterpart in the reference" in src


def test_layout_through_abi(native_lib):
    lay = _lib.expert_layout(2048, 512, 64)
    assert lay["expert_size"] == 1769472
    assert (lay["gate_s"], lay["up_w"], lay["down_w"], lay["down_b"]) == (524288, 589824, 1179648, 1736704)
    with pytest.raises(ValueError):
        _lib.expert_layout(2048, 500, 64)


def test_no_cpu_fallback(native_lib):
    """Without a CUDA device, creating an engine fails loudly instead of computing on the CPU."""
    n = C.c_int(0)
    try:
        cudart = C.CDLL("libcudart.so")
        has_gpu = cudart.cudaGetDeviceCount(C.byref(n)) == 0 and n.value > 0
    except OSError:
        has_gpu = os.path.exists("/dev/nvidia0")
    if has_gpu:
        pytest.skip("a GPU is present")
    from moe_infer_b200.native import Dims, NativeEngine
    with pytest.raises(_lib.MoeError) as ei:
        NativeEngine(Dims(num_experts=4, top_k=4, num_layers=1))
    assert ei.value.status == _lib.ERR_CUDA


def test_dims_validation_happens_before_cuda(native_lib):
    from moe_infer_b200.native import Dims, NativeEngine
    with pytest.raises(ValueError, match="num_active_experts"):
        NativeEngine(Dims(top_k=9))
    with pytest.raises(ValueError, match="group"):
        NativeEngine(Dims(group=32))


def test_product_does_not_import_the_oracle():
    pkg = os.path.join(os.path.dirname(__file__), "..", "moe_infer_b200")
    for root, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(root, f)).read()
                assert "import oracle" not in text and "from oracle" not in text, f
                assert "moe_oracle" not in text, f
