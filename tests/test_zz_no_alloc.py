"""The allocation-free decode entry point (moe_layer_decode_noalloc), through the C ABI.

Some hosts cannot let this library allocate device memory (their HBM is owned by
their own pool, or cudaMalloc is banned after start-up).  For them one decode
entry point keeps its work areas in a fixed array inside the library image.
These tests give it tensors that live in buffers the *test* owns, run it twice
in a row (the array is shared between calls and keeps the previous call's
contents), and check both results against the ordinary engine entry point and
against the CPU oracle, with the tolerance the decode tests use.  They also
cover the 4-bit router pointers, the model's full expert count, a call that is
only enqueued (wait == 0) on a stream of its own followed by the status call,
output written over the input, and that the free device memory does not move
across a call.  The file name sorts last so that a run that stops at the first
failure has already run every other test.
"""
import ctypes as C

import numpy as np
import pytest

import oracle
from benchmarks import synth
from moe_infer_b200 import _lib
from moe_infer_b200.native import Dims, NativeEngine
from tests.util import make_layer, rel_l2, routing_maps, upload_layer

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


def _caller_buffers(eng, lw):
    """The caller's own device buffers (allocated by the test, not by the entry point) and the pointer struct."""
    bufs = {
        "experts": eng.alloc(lw.experts.nbytes).upload(lw.experts),
        "post_norm": eng.alloc(lw.post_norm_w.nbytes).upload(lw.post_norm_w),
        "shared": eng.alloc(_shared_blob(lw).nbytes).upload(_shared_blob(lw)),
        "sgate_w": eng.alloc(lw.sgate[0].nbytes).upload(lw.sgate[0]),
        "sgate_s": eng.alloc(256).upload(lw.sgate[1]),
        "sgate_b": eng.alloc(256).upload(lw.sgate[2]),
    }
    rb = rw = rs = rbi = None
    if lw.router_bf16 is not None:
        bufs["router_bf16"] = eng.alloc(lw.router_bf16.nbytes).upload(lw.router_bf16)
        rb = bufs["router_bf16"].ptr
    else:
        for k, a in zip(("router_w", "router_s", "router_b"), lw.router_q4):
            bufs[k] = eng.alloc(max(a.nbytes, 256)).upload(a)
        rw, rs, rbi = bufs["router_w"].ptr, bufs["router_s"].ptr, bufs["router_b"].ptr
    ptrs = _lib.LayerPtrs(bufs["experts"].ptr, bufs["post_norm"].ptr, rb, rw, rs, rbi, bufs["shared"].ptr,
                          bufs["sgate_w"].ptr, bufs["sgate_s"].ptr, bufs["sgate_b"].ptr)
    return bufs, ptrs


def _cudart():
    return C.CDLL("libcudart.so")


def _free_bytes(cudart) -> int:
    free, total = C.c_size_t(), C.c_size_t()
    assert cudart.cudaMemGetInfo(C.byref(free), C.byref(total)) == 0
    return free.value


def _run_case(num_experts, scheme, seed):
    int4 = scheme == "int4"
    dims = Dims(num_experts=num_experts, top_k=8, num_layers=1, scheme=_lib.SCHEME_INT4 if int4 else _lib.SCHEME_BQ4)
    lw = make_layer(seed, 0, num_experts=num_experts, scheme=scheme)
    eng = NativeEngine(dims)
    upload_layer(eng, 0, lw)
    lib = eng.lib
    bufs, ptrs = _caller_buffers(eng, lw)
    h = synth.hidden_states(seed, 2, 2, 2048)
    d_in = eng.alloc(h.nbytes).upload(h)
    d_out = eng.alloc(h.nbytes)
    d_idx = eng.alloc(2 * 8 * 4)
    d_w = eng.alloc(2 * 8 * 4)
    cd = dims.to_c()
    eng.sync()
    cudart = _cudart()
    free_before = None
    for t in range(2):  # two calls in a row on the shared scratch array
        if t == 1:
            free_before = _free_bytes(cudart)  # the first call on a device does the one-time set-up; the second must allocate nothing
        _lib.check(lib.moe_layer_decode_noalloc(C.byref(cd), 0, C.byref(ptrs), C.c_void_p(d_in.ptr + t * 8192),
                                                C.c_void_p(d_out.ptr + t * 8192), C.c_void_p(d_idx.ptr + t * 32),
                                                C.c_void_p(d_w.ptr + t * 32), None, 1))
    assert _free_bytes(cudart) == free_before
    got = d_out.download(np.float32, (2, 2048))
    got_idx = d_idx.download(np.int32, (2, 8))
    got_w = d_w.download(np.float32, (2, 8))
    for t in range(2):
        want, idx, wts = eng.layer_forward(0, h[t])
        assert np.array_equal(np.sort(got_idx[t]), np.sort(idx[0]))
        assert rel_l2(got[t] - h[t], want[0] - h[t]) < TIGHT
        assert rel_l2(got[t], want[0]) < TIGHT
        ref, idx_r, wts_r = oracle.moe_layer(lw, h[t], 8)
        (i, w), (ir, wr) = routing_maps(got_idx[t], got_w[t])[0], routing_maps(idx_r, wts_r)[0]
        assert np.array_equal(i, ir) and np.allclose(w, wr, rtol=1e-4, atol=1e-6)
        assert rel_l2(got[t] - h[t], ref[0] - h[t]) < TIGHT
    return eng, lib, cd, ptrs, bufs, (d_in, d_out, d_idx, d_w), h, got


def _cleanup(eng, bufs, extra):
    for b in list(bufs.values()) + list(extra):
        b.free()
    eng.close()


def test_noalloc_decode_matches_engine_entry_point_twice():
    eng, lib, cd, ptrs, bufs, (d_in, d_out, d_idx, d_w), h, _ = _run_case(16, "bq4", 31)
    # sizes beyond the fixed scratch are refused with a clear message, before any device work
    big = Dims(num_experts=1024, top_k=8, num_layers=1).to_c()
    rc = lib.moe_layer_decode_noalloc(C.byref(big), 0, C.byref(ptrs), C.c_void_p(d_in.ptr), C.c_void_p(d_out.ptr),
                                      None, None, None, 1)
    assert rc == _lib.ERR_INVALID and "at most 512 experts" in _lib.last_error()
    _cleanup(eng, bufs, (d_in, d_out, d_idx, d_w))


def test_noalloc_decode_full_expert_count():
    eng, *_rest = _run_case(256, "bq4", 32)
    _lib_, cd, ptrs, bufs, extra, h, got = _rest
    _cleanup(eng, bufs, extra)


def test_noalloc_decode_four_bit_router():
    eng, *_rest = _run_case(32, "int4", 33)
    _lib_, cd, ptrs, bufs, extra, h, got = _rest
    _cleanup(eng, bufs, extra)


def test_noalloc_decode_enqueue_only_own_stream_in_place():
    eng, lib, cd, ptrs, bufs, (d_in, d_out, d_idx, d_w), h, got = _run_case(16, "bq4", 34)
    cudart = _cudart()
    stream = C.c_void_p()
    assert cudart.cudaStreamCreate(C.byref(stream)) == 0
    # enqueue only (wait == 0), output over the input, then ask for the status before looking at the result
    d_io = eng.alloc(8192).upload(h[0])
    eng.sync()
    _lib.check(lib.moe_layer_decode_noalloc(C.byref(cd), 0, C.byref(ptrs), C.c_void_p(d_io.ptr), C.c_void_p(d_io.ptr),
                                            None, None, stream, 0))
    code = C.c_uint(7)
    _lib.check(lib.moe_layer_decode_noalloc_status(0, stream, C.byref(code)))
    assert code.value == 0
    in_place = d_io.download(np.float32, (2048,))
    assert np.array_equal(in_place, got[0])  # same kernel, same inputs: bit-identical to the separate-buffer call
    assert cudart.cudaStreamDestroy(stream) == 0
    _cleanup(eng, bufs, (d_in, d_out, d_idx, d_w, d_io))
