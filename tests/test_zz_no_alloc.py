"""The allocation-free decode entry point (moe_layer_decode_noalloc), through the C ABI.

Some hosts cannot let this library allocate device memory (their HBM is owned by
their own pool, or cudaMalloc is banned after start-up).  For them one decode
entry point keeps its work areas in a fixed array inside the library image.
This test gives it tensors that live in buffers the *test* owns, runs it twice
in a row (the array is shared between calls and keeps the previous call's
contents), and checks both results against the ordinary engine entry point,
with the tolerance the decode tests use.  The file name sorts last so that a run
that stops at the first failure has already run every other test.
"""
import ctypes as C

import numpy as np
import pytest

from moe_infer_b200 import _lib
from benchmarks import synth
from moe_infer_b200.native import Dims, NativeEngine
from tests.util import make_layer, rel_l2, upload_layer

pytestmark = pytest.mark.gpu
TIGHT = 2e-4


def _shared_blob(lw):
    lay = _lib.expert_layout(lw.hidden, lw.shared_inter, 64)
    blob = np.zeros(lay["expert_size"], np.uint8)
    for name, t in (("gate", lw.sh_gate), ("up", lw.sh_up), ("down", lw.sh_down)):
        for suffix, arr in zip(("_w", "_s", "_b"), t):
            raw = np.ascontiguousarray(arr).view(np.uint8).ravel()
            blob[lay[name + suffix]:lay[name + suffix] + raw.size] = raw
    return blob


def test_noalloc_decode_matches_engine_entry_point_twice():
    dims = Dims(num_experts=16, top_k=8, num_layers=1)
    lw = make_layer(31, 0, num_experts=16)
    eng = NativeEngine(dims)
    upload_layer(eng, 0, lw)
    lib = eng.lib

    # the caller's own buffers (allocated by the test, not by the entry point)
    bufs = {
        "experts": eng.alloc(lw.experts.nbytes).upload(lw.experts),
        "post_norm": eng.alloc(lw.post_norm_w.nbytes).upload(lw.post_norm_w),
        "router_bf16": eng.alloc(lw.router_bf16.nbytes).upload(lw.router_bf16),
        "shared": eng.alloc(_shared_blob(lw).nbytes).upload(_shared_blob(lw)),
        "sgate_w": eng.alloc(lw.sgate[0].nbytes).upload(lw.sgate[0]),
        "sgate_s": eng.alloc(256).upload(lw.sgate[1]),
        "sgate_b": eng.alloc(256).upload(lw.sgate[2]),
    }
    ptrs = _lib.LayerPtrs(bufs["experts"].ptr, bufs["post_norm"].ptr, bufs["router_bf16"].ptr, None, None, None,
                          bufs["shared"].ptr, bufs["sgate_w"].ptr, bufs["sgate_s"].ptr, bufs["sgate_b"].ptr)
    h = synth.hidden_states(31, 2, 2, 2048)
    d_in = eng.alloc(h.nbytes).upload(h)
    d_out = eng.alloc(h.nbytes)
    d_idx = eng.alloc(2 * 8 * 4)
    d_w = eng.alloc(2 * 8 * 4)
    cd = dims.to_c()
    eng.sync()
    for t in range(2):  # two calls in a row on the shared scratch array
        _lib.check(lib.moe_layer_decode_noalloc(C.byref(cd), 0, C.byref(ptrs), C.c_void_p(d_in.ptr + t * 8192),
                                                C.c_void_p(d_out.ptr + t * 8192), C.c_void_p(d_idx.ptr + t * 32),
                                                C.c_void_p(d_w.ptr + t * 32), None, 1))
    got = d_out.download(np.float32, (2, 2048))
    got_idx = d_idx.download(np.int32, (2, 8))
    got_w = d_w.download(np.float32, (2, 8))
    for t in range(2):
        want, idx, wts = eng.layer_forward(0, h[t])
        assert np.array_equal(got_idx[t], idx[0])
        assert np.allclose(got_w[t], wts[0], rtol=1e-6)
        assert rel_l2(got[t] - h[t], want[0] - h[t]) < TIGHT
        assert rel_l2(got[t], want[0]) < TIGHT

    # sizes beyond the fixed scratch are refused with a clear message, before any device work
    big = Dims(num_experts=1024, top_k=8, num_layers=1).to_c()
    rc = lib.moe_layer_decode_noalloc(C.byref(big), 0, C.byref(ptrs), C.c_void_p(d_in.ptr), C.c_void_p(d_out.ptr),
                                      None, None, None, 1)
    assert rc == _lib.ERR_INVALID and "at most 512 experts" in _lib.last_error()
    for b in list(bufs.values()) + [d_in, d_out, d_idx, d_w]:
        b.free()
    eng.close()
