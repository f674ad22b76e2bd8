"""GPU parity of the batched (grouped tensor-core GEMM) path of the MoE block.

The grouped path rounds activations and dequantised weights to bf16 before the
tensor-core contraction (f32 accumulate), so it is held to the contract's
tolerance, 1e-2 relative L2 against the CPU oracle (over the batch and for every
single token), not to the tighter bound of the decode path.  The router runs in f32, so the expert choices must match
the oracle's exactly (no ties occur with these seeds).
"""
import numpy as np
import pytest

import oracle
from moe_infer_b200 import _lib
from benchmarks import synth
from moe_infer_b200.native import Dims, NativeEngine
from tests.util import make_layer, rel_l2, routing_maps, upload_layer

pytestmark = pytest.mark.gpu
TOL = 1e-2


def _check(eng, lw, h, k, **kw):
    out, idx, wts = eng.layer_forward(0, h, **kw)
    ref, idx_r, wts_r = oracle.moe_layer(lw, h, k, threads=8, **kw)
    for (i, w), (ir, wr) in zip(routing_maps(idx, wts), routing_maps(idx_r, wts_r)):
        assert np.array_equal(i, ir)
        assert np.allclose(w, wr, rtol=1e-4, atol=1e-6)
    assert rel_l2(out, ref) < TOL
    upd = rel_l2(out - h, ref - h)
    assert upd < TOL, upd
    per_token = np.linalg.norm((out - ref), axis=1) / np.linalg.norm(ref - h, axis=1)
    assert per_token.max() < TOL, per_token.max()  # measured: about 6e-3 for the worst token, 4.5e-3 over a batch
    return upd


@pytest.fixture(scope="module")
def small():
    lw = make_layer(21, 0, num_experts=16)
    eng = NativeEngine(Dims(num_experts=16, top_k=8, num_layers=1))
    upload_layer(eng, 0, lw)
    yield eng, lw
    eng.close()


@pytest.mark.parametrize("n", [2, 5, 37, 48, 49, 128, 130, 300])  # up to 48 tokens: the slot-wise expert FFN; beyond: the grouped GEMMs
def test_batched_layer_small(small, n):
    eng, lw = small
    _check(eng, lw, synth.hidden_states(n, 3, n, 2048), 8)


def test_batched_matches_decode_path(small):
    eng, lw = small
    h = synth.hidden_states(77, 3, 9, 2048)
    out_b, idx_b, _ = eng.layer_forward(0, h)
    for t in range(9):
        out_d, idx_d, _ = eng.layer_forward(0, h[t])
        assert set(idx_b[t].tolist()) == set(idx_d[0].tolist())
        assert rel_l2(out_b[t] - h[t], out_d[0] - h[t]) < TOL


def test_batched_forced_and_bias(small):
    eng, lw = small
    n = 40
    h = synth.hidden_states(5, 3, n, 2048)
    rng = np.random.default_rng(5)
    forced = np.stack([rng.choice(16, size=8, replace=False) for _ in range(n)]).astype(np.int32)
    _check(eng, lw, h, 8, forced_idx=forced)
    bias = np.zeros(16, np.float32)
    bias[[3, 9]] = 4.0
    _check(eng, lw, h, 8, logit_bias=bias)


def test_batched_all_tokens_one_expert_set():
    """Maximum skew: every token picks the same experts (one tile list entry per expert, M = n)."""
    lw = make_layer(22, 0, num_experts=8)
    eng = NativeEngine(Dims(num_experts=8, top_k=2, num_layers=1))
    upload_layer(eng, 0, lw)
    n = 200
    h = synth.hidden_states(6, 3, n, 2048)
    forced = np.tile(np.array([[5, 1]], np.int32), (n, 1))
    _check(eng, lw, h, 2, forced_idx=forced)
    _check(eng, lw, h[:20], 2, forced_idx=forced[:20])  # the same skew through the slot-wise path: 20 slots per expert in a row
    eng.close()


def test_batched_config3_zipf_256_experts():
    """Config 3: 64 tokens, 256 experts, top-8, Zipf(1.1)-skewed routing."""
    lw = make_layer(0, 0, num_experts=256)
    eng = NativeEngine(Dims(num_experts=256, top_k=8, num_layers=1))
    upload_layer(eng, 0, lw)
    h = synth.hidden_states(3, 3, 64, 2048)
    bias = synth.zipf_logit_bias(0, 256, alpha=1.1, strength=1.0)
    _check(eng, lw, h, 8, logit_bias=bias)
    _, idx, _ = eng.layer_forward(0, h, logit_bias=bias)
    counts = np.bincount(idx.ravel(), minlength=256)
    assert counts.max() >= 10 and (counts == 0).sum() > 20  # skewed: some experts hot, many idle
    eng.close()


def test_batched_int4_scheme_router():
    lw = make_layer(23, 0, num_experts=32, scheme="int4")
    eng = NativeEngine(Dims(num_experts=32, top_k=8, num_layers=1, scheme=_lib.SCHEME_INT4))
    upload_layer(eng, 0, lw)
    _check(eng, lw, synth.hidden_states(8, 3, 70, 2048), 8)
    eng.close()
