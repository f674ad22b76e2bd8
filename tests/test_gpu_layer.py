"""GPU parity of the MoE block and the layer stack (decode path), through the C ABI.

Tolerance: <= 1e-2 relative L2 against the CPU oracle (f32 accumulate), as the
contract states; the decode path keeps activations to 23 bits relative to each
32-element chunk's maximum and sums exactly, so the tests also hold a much
tighter bound.  Expert choices must match exactly except where two
probabilities tie to the last bit (none occur with these seeds).
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
TIGHT = 2e-4


def _check_routing(idx, wts, idx_ref, wts_ref):
    for (i, w), (ir, wr) in zip(routing_maps(idx, wts), routing_maps(idx_ref, wts_ref)):
        assert np.array_equal(i, ir)
        assert np.allclose(w, wr, rtol=1e-4, atol=1e-6)


@pytest.fixture(scope="module")
def full_layer():
    """Config 2: 256 experts, top-8, BQ4 (bf16 router)."""
    lw = make_layer(0, 0, num_experts=256, scheme="bq4")
    eng = NativeEngine(Dims(num_experts=256, top_k=8, num_layers=1))
    upload_layer(eng, 0, lw)
    yield eng, lw
    eng.close()


def test_decode_layer_config2(full_layer):
    eng, lw = full_layer
    h = synth.hidden_states(0, 2, 1, 2048)
    out, idx, wts = eng.layer_forward(0, h)
    ref, idx_r, wts_r = oracle.moe_layer(lw, h, 8)
    _check_routing(idx, wts, idx_r, wts_r)
    assert rel_l2(out, ref) < TOL and rel_l2(out, ref) < TIGHT
    assert rel_l2(out - h, ref - h) < TOL  # the MoE update itself, without the residual


def test_decode_layer_many_tokens_serial(full_layer):
    eng, lw = full_layer
    h = synth.hidden_states(1, 2, 6, 2048)
    for t in range(6):
        out, idx, wts = eng.layer_forward(0, h[t])
        ref, idx_r, wts_r = oracle.moe_layer(lw, h[t], 8)
        _check_routing(idx, wts, idx_r, wts_r)
        assert rel_l2(out - h[t], ref - h[t]) < TIGHT


def test_decode_layer_repeatable(full_layer):
    eng, _ = full_layer
    h = synth.hidden_states(2, 2, 1, 2048)
    a = eng.layer_forward(0, h)[0]
    b = eng.layer_forward(0, h)[0]
    assert np.array_equal(a, b)


def test_forced_indices_and_logit_bias(full_layer):
    eng, lw = full_layer
    h = synth.hidden_states(3, 2, 1, 2048)
    forced = np.array([[3, 200, 17, 255, 0, 64, 128, 99]], np.int32)
    out, idx, wts = eng.layer_forward(0, h, forced_idx=forced)
    ref, idx_r, wts_r = oracle.moe_layer(lw, h, 8, forced_idx=forced)
    _check_routing(idx, wts, idx_r, wts_r)
    assert rel_l2(out - h, ref - h) < TIGHT
    bias = synth.zipf_logit_bias(0, 256, strength=2.0)
    out, idx, wts = eng.layer_forward(0, h, logit_bias=bias)
    ref, idx_r, wts_r = oracle.moe_layer(lw, h, 8, logit_bias=bias)
    _check_routing(idx, wts, idx_r, wts_r)
    assert rel_l2(out - h, ref - h) < TIGHT


@pytest.mark.parametrize("scale", [1e-3, 1.0, 1e3])
def test_decode_layer_activation_scale(full_layer, scale):
    """The decode router sums exact products in fixed point, scaled by the running 1/rms: expert choices
    and outputs must not depend on the magnitude of the residual stream."""
    eng, lw = full_layer
    h = (synth.hidden_states(4, 2, 1, 2048) * np.float32(scale)).astype(np.float32)
    out, idx, wts = eng.layer_forward(0, h)
    ref, idx_r, wts_r = oracle.moe_layer(lw, h, 8)
    _check_routing(idx, wts, idx_r, wts_r)
    # out = h + update is rounded to f32 at the magnitude of h: that rounding bounds how well the update
    # can be recovered by subtracting h again
    floor = np.finfo(np.float32).eps * np.linalg.norm(h) / np.linalg.norm(ref - h)
    assert rel_l2(out - h, ref - h) < TIGHT + 2.0 * floor
    assert rel_l2(out, ref) < TIGHT


def test_decode_layer_outlier_activations(full_layer):
    """A few elements hundreds of times the rms (as in real residual streams): the integer dot products keep
    23 bits relative to each 32-element chunk's maximum, so the rest of the chunk must not lose accuracy."""
    eng, lw = full_layer
    h = synth.hidden_states(5, 2, 1, 2048).copy()
    h[0, [7, 300, 1029, 2047]] *= np.float32(300.0)
    out, idx, wts = eng.layer_forward(0, h)
    ref, idx_r, wts_r = oracle.moe_layer(lw, h, 8)
    _check_routing(idx, wts, idx_r, wts_r)
    assert rel_l2(out - h, ref - h) < TIGHT


def test_stripped_model_shape_int4_router():
    """The reference's test model: 4 experts, top-4; INT4 scheme (4-bit router)."""
    lw = make_layer(5, 0, num_experts=4, scheme="int4")
    eng = NativeEngine(Dims(num_experts=4, top_k=4, num_layers=1, scheme=_lib.SCHEME_INT4))
    upload_layer(eng, 0, lw)
    h = synth.hidden_states(5, 2, 3, 2048)
    for t in range(3):
        out, idx, wts = eng.layer_forward(0, h[t])
        ref, idx_r, wts_r = oracle.moe_layer(lw, h[t], 4)
        _check_routing(idx, wts, idx_r, wts_r)
        assert rel_l2(out - h[t], ref - h[t]) < TIGHT
    eng.close()


def test_top_k_smaller_than_model_default():
    lw = make_layer(6, 0, num_experts=16)
    eng = NativeEngine(Dims(num_experts=16, top_k=2, num_layers=1))
    upload_layer(eng, 0, lw)
    h = synth.hidden_states(6, 2, 1, 2048)
    out, idx, wts = eng.layer_forward(0, h)
    ref, idx_r, wts_r = oracle.moe_layer(lw, h, 2)
    _check_routing(idx, wts, idx_r, wts_r)
    assert rel_l2(out - h, ref - h) < TIGHT
    eng.close()


@pytest.fixture(scope="module")
def small_stack():
    layers = [make_layer(9, l, num_experts=16) for l in range(5)]
    eng = NativeEngine(Dims(num_experts=16, top_k=8, num_layers=4, num_mtp_layers=1))
    for l, lw in enumerate(layers):
        upload_layer(eng, l, lw)
    yield eng, layers
    eng.close()


def test_stack_decode(small_stack):
    eng, layers = small_stack
    emb = synth.hidden_states(9, 2, 3, 2048)
    out = eng.forward_hidden(emb)
    ref = oracle.moe_stack(layers[:4], emb, 8)
    assert rel_l2(out, ref) < TOL and rel_l2(out, ref) < 1e-3
    assert np.array_equal(eng.last_h_pre_norm(), out[-1])
    # batched flag gives the same hidden states (tolerance: the grouped path computes in bf16)
    out_b = eng.forward_hidden(emb, batched=True)
    assert rel_l2(out_b, ref) < TOL


def test_stack_decode_growing_residual(small_stack):
    """Inside a stack the next layer's logits are accumulated with the previous layer's 1/rms as scale: a
    residual stream that starts tiny and one that starts huge must both route like the oracle."""
    eng, layers = small_stack
    for scale in (1e-4, 50.0):
        emb = (synth.hidden_states(11, 2, 2, 2048) * np.float32(scale)).astype(np.float32)
        out = eng.forward_hidden(emb)
        ref = oracle.moe_stack(layers[:4], emb, 8)
        floor = np.finfo(np.float32).eps * np.linalg.norm(emb) / np.linalg.norm(ref - emb)
        assert rel_l2(out - emb, ref - emb) < 1e-3 + 2.0 * floor


def test_stack_interrupt(small_stack):
    eng, _ = small_stack
    emb = synth.hidden_states(9, 2, 4, 2048)
    calls = {"n": 0}

    def check():
        calls["n"] += 1
        return calls["n"] > 2

    with pytest.raises(_lib.MoeError) as ei:
        eng.forward_hidden(emb, check=check)
    assert ei.value.status == _lib.ERR_INTERRUPTED and "interrupted" in str(ei.value)
    # the engine stays usable
    out = eng.forward_hidden(emb[:1])
    assert np.isfinite(out).all()


def test_mtp_block_uses_layer_index_num_layers(small_stack):
    eng, layers = small_stack
    h = synth.hidden_states(10, 2, 1, 2048)[0]
    eng.mtp_reset()
    out = eng.mtp_forward(h)
    ref, _, _ = oracle.moe_layer(layers[4], h, 8)
    assert rel_l2(out - h, ref[0] - h) < TIGHT
    assert eng.mtp_pos() == 1
    eng.mtp_rollback(0)
    assert eng.mtp_pos() == 0


def test_missing_tensors_fail_loudly():
    eng = NativeEngine(Dims(num_experts=4, top_k=4, num_layers=1))
    with pytest.raises(_lib.MoeError) as ei:
        eng.layer_forward(0, np.zeros(2048, np.float32))
    assert ei.value.status == _lib.ERR_STATE
    with pytest.raises(ValueError):
        eng.load_layer(0, np.zeros(100, np.uint8))  # short blob (src/model/expert.rs:36-41)
    with pytest.raises(ValueError):
        eng.load_layer(3, np.zeros(4 * 1769472, np.uint8))  # layer out of range
    eng.close()


def test_telemetry_keys(small_stack):
    eng, _ = small_stack
    eng.lib.moe_set_record_telemetry(1)
    eng.forward_hidden(synth.hidden_states(11, 2, 2, 2048))
    tel = eng.telemetry()
    eng.lib.moe_set_record_telemetry(0)
    assert tel["engine.total_ms"] > 0 and tel["engine.tokens"] >= 2
    assert "engine.expert_io_ms" in tel
    # the reference's per-phase keys (src/engine/qwen35_moe/fused_exp5.rs:170-176, 249, 378, 401, 412)
    for key in ("phase.op2_encode_ms", "phase.hidden_wait_ms", "phase.lm_head_ms", "phase.route_cpu_ms"):
        assert key in tel and tel[key] >= 0.0
    assert tel["phase.op2_encode_ms"] + tel["phase.hidden_wait_ms"] > 0.0


def test_nan_hidden_state_selects_valid_experts(full_layer):
    """A NaN hidden state must never turn into an expert index outside [0, E).

    With NaN logits every comparison is false; the reference's heap then keeps its first K entries
    (src/math_util.rs:89-99: experts 0..K-1, NaN weights) and the output is NaN.  Here: the same expert set, an
    output that still carries NaN, no error, and the other tokens of the batch are untouched.
    """
    eng, lw = full_layer
    h = synth.hidden_states(12, 2, 6, 2048)
    clean, idx_clean, _ = eng.layer_forward(0, h)
    bad = h.copy()
    bad[2, 100] = np.nan
    # batched path: token 2 is NaN, the others must come out exactly as before
    out, idx, wts = eng.layer_forward(0, bad)
    assert idx.min() >= 0 and idx.max() < 256
    assert np.array_equal(np.sort(idx[2]), np.arange(8))
    assert np.isnan(out[2]).any()  # the caller can see that this token is invalid
    keep = [0, 1, 3, 4, 5]
    assert np.array_equal(out[keep], clean[keep]) and np.array_equal(idx[keep], idx_clean[keep])
    # decode path, one token
    out1, idx1, _ = eng.layer_forward(0, bad[2])
    assert np.array_equal(np.sort(idx1[0]), np.arange(8)) and np.isnan(out1).any()
    # the engine is still usable and still right
    again, idx_again, _ = eng.layer_forward(0, h[0])
    assert np.array_equal(again[0], eng.layer_forward(0, h[0])[0][0]) and np.isfinite(again).all()


def test_same_expert_prefetch_option_changes_nothing_but_the_statistics(monkeypatch):
    """MOE_B200_DECODE_PREFETCH=1: the decode kernel asks for the next layer's copy of each chosen expert ahead of time
    (the reference's predictor, src/engine/qwen35_moe/expert_prefetch.rs:95-135).  A prefetch moves no data the kernel
    computes with: results are bit-identical; the telemetry counts predictions and hits."""
    layers = [make_layer(14, l, num_experts=16) for l in range(4)]
    h = synth.hidden_states(14, 2, 3, 2048)

    def run(flag):
        if flag:
            monkeypatch.setenv("MOE_B200_DECODE_PREFETCH", "1")
        else:
            monkeypatch.delenv("MOE_B200_DECODE_PREFETCH", raising=False)
        eng = NativeEngine(Dims(num_experts=16, top_k=8, num_layers=4))
        for l, lw in enumerate(layers):
            upload_layer(eng, l, lw)
        out = eng.forward_hidden(h)
        tel = eng.telemetry()
        eng.close()
        return out, tel

    base, tel0 = run(False)
    pre, tel1 = run(True)
    assert np.array_equal(base, pre)
    assert "prefetch.checks" not in tel0
    assert tel1["prefetch.checks"] == 3 * (4 - 1) * 8          # tokens x layer transitions x routed slots
    assert 0 <= tel1["prefetch.hits"] <= tel1["prefetch.checks"]
    print(f"same-expert predictor: {int(tel1['prefetch.hits'])} of {int(tel1['prefetch.checks'])} right (16 experts, top-8)")
