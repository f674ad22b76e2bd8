"""GPU parity of the model head (embedding rows, final norm, lm_head, INT8 codec), through the C ABI."""
import numpy as np
import pytest

import oracle
from benchmarks import synth
from moe_infer_b200 import _lib
from moe_infer_b200.native import Dims, NativeEngine
from tests.util import rel_l2

pytestmark = pytest.mark.gpu
H = 2048


def _q4_random(rng, rows, cols):
    """Random packed words with plausible bf16 scales and biases (values do not need a float source)."""
    w = rng.integers(0, 2**32, size=(rows, cols // 8), dtype=np.uint64).astype(np.uint32)
    s = oracle.f32_to_bf16(rng.uniform(0.002, 0.01, (rows, cols // 64)).astype(np.float32))
    b = oracle.f32_to_bf16(rng.uniform(-0.08, -0.02, (rows, cols // 64)).astype(np.float32))
    return w, s, b


def test_int8_codec_bit_exact():
    eng = NativeEngine(Dims(num_experts=4, top_k=4, num_layers=1))
    rng = np.random.default_rng(0)
    W = synth.normal_weights(rng, (1000, H), outlier_frac=0.001)
    W[17] = 0.0                      # all-zero row: scale 1/127
    W[18, 5] = np.float32(3.0)       # a dominant element
    q, s = eng.pack_int8(W)
    q_ref, s_ref = oracle.quant_int8(W)
    assert np.array_equal(q, q_ref) and np.array_equal(s.view(np.uint32), s_ref.view(np.uint32))
    Wb = synth.to_bf16_rne(W)        # bf16 source, widened exactly
    q, s = eng.pack_int8(Wb)
    q_ref, s_ref = oracle.quant_int8(synth.bf16_to_f32(Wb))
    assert np.array_equal(q, q_ref) and np.array_equal(s.view(np.uint32), s_ref.view(np.uint32))
    eng.close()


@pytest.mark.parametrize("vocab,kind", [(1000, "int8"), (1000, "int4"), (248320, "int8"), (248320, "int4")])
def test_head_logits(vocab, kind):
    """vocab 248,320 is the model's lm_head: the streaming kernels; 1,000 rows take the generic ones."""
    dims = Dims(num_experts=4, top_k=4, num_layers=1, vocab=vocab)
    eng = NativeEngine(dims)
    rng = np.random.default_rng(vocab + len(kind))
    norm = oracle.f32_to_bf16(rng.uniform(0.8, 1.2, H).astype(np.float32))
    eng.load_final_norm(norm)
    if kind == "int8":
        q = rng.integers(-127, 128, size=(vocab, H), dtype=np.int8)
        sc = rng.uniform(1e-4, 4e-4, vocab).astype(np.float32)
        eng.load_lm_head_int8(q, sc)
    else:
        t = _q4_random(rng, vocab, H)
        eng.load_lm_head_q4(t)
    h = (synth.hidden_states(vocab, 2, 2, H) * np.float32(3.0)).astype(np.float32)
    got = eng.logits(h)
    x = oracle.final_norm(h, norm)
    for t_ in range(2):
        want = oracle.matvec_int8(q, sc, x[t_], threads=8) if kind == "int8" else oracle.matvec_int4(*t, x[t_], threads=8)
        assert rel_l2(got[t_], want) < 1e-4
        assert int(got[t_].argmax()) == int(want.argmax())
    eng.close()


def test_embed_rows_and_missing_head():
    vocab = 5000
    dims = Dims(num_experts=4, top_k=4, num_layers=1, vocab=vocab)
    eng = NativeEngine(dims)
    with pytest.raises(_lib.MoeError) as ei:
        eng.embed_lookup(np.array([1], np.int64))
    assert ei.value.status == _lib.ERR_STATE and "embed_tokens" in str(ei.value)
    with pytest.raises(_lib.MoeError) as ei:
        eng.logits(np.zeros(H, np.float32))
    assert ei.value.status == _lib.ERR_STATE
    rng = np.random.default_rng(3)
    t = _q4_random(rng, vocab, H)
    eng.load_embed(t)
    ids = np.array([0, 4999, 17, 17, 2500], np.int64)
    assert np.array_equal(eng.embed_lookup(ids), oracle.embed_lookup(*t, ids))
    with pytest.raises(ValueError, match="token id"):
        eng.embed_lookup(np.array([5000], np.int64))
    assert np.isfinite(eng.embed_lookup(ids[:1])).all()  # the engine stays usable
    eng.close()
