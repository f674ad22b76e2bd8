"""GPU parity of the packer and the single dequant-matvec, through the C ABI."""
import os

import numpy as np
import pytest

import oracle
from benchmarks import synth
from moe_infer_b200.native import Dims, NativeEngine
from tests.util import rel_l2

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")


@pytest.fixture(scope="module")
def eng():
    e = NativeEngine(Dims(num_experts=4, top_k=4, num_layers=1))
    yield e
    e.close()


def _same(a, b):
    return all(np.array_equal(x, y) for x, y in zip(a, b))


def test_packer_known_answers_bit_exact(eng):
    kat = np.load(os.path.join(GOLD, "packer_kat.npz"))
    names = sorted({k.rsplit(".", 1)[0] for k in kat.files})
    for n in names:
        w, s, b = eng.pack_int4(kat[n + ".in"])
        assert np.array_equal(w, kat[n + ".w"]), n
        assert np.array_equal(s, kat[n + ".s"]), n
        assert np.array_equal(b, kat[n + ".b"]), n


@pytest.mark.parametrize("rows,cols", [(1, 64), (3, 192), (512, 2048), (2048, 512), (37, 4096)])
def test_packer_random_f32_bit_exact(eng, rows, cols):
    rng = np.random.default_rng(rows * 7919 + cols)
    v = synth.normal_weights(rng, (rows, cols), outlier_frac=0.001)
    assert _same(eng.pack_int4(v), oracle.quant_int4(v))


def test_packer_bf16_source_bit_exact(eng):
    rng = np.random.default_rng(11)
    u = synth.to_bf16_rne(synth.normal_weights(rng, (512, 2048), outlier_frac=0.001))
    assert _same(eng.pack_int4(u), oracle.quant_int4_bf16(u))


def test_packer_wide_dynamic_range_bit_exact(eng):
    rng = np.random.default_rng(12)
    v = (rng.standard_normal((64, 256)) * np.exp(rng.uniform(-40, 40, size=(64, 1)))).astype(np.float32)
    assert _same(eng.pack_int4(v), oracle.quant_int4(v))


def test_packer_device_pointers_any_word_alignment(eng):
    """Device entry point: a destination that is only 4-byte aligned takes the narrow stores; a source that is
    not 16-byte aligned is refused before any device work."""
    from moe_infer_b200 import _lib
    rng = np.random.default_rng(13)
    rows, cols = 70, 192  # 210 groups: six full warps of 32 groups and a ragged one
    v = synth.normal_weights(rng, (rows, cols), outlier_frac=0.001)
    want = oracle.quant_int4(v)
    d_src = eng.alloc(v.nbytes + 16).upload(v)
    d_w = eng.alloc(rows * cols // 2 + 16)
    d_s = eng.alloc(rows * cols // 64 * 2 + 16)
    d_b = eng.alloc(rows * cols // 64 * 2 + 16)
    for off in (0, 4):
        eng.pack_int4_dev(d_src.ptr, _lib.DT_F32, rows, cols, d_w.ptr + off, d_s.ptr + 2, d_b.ptr + 2)
        eng.sync()
        w = d_w.download(np.uint8, (rows * cols // 2 + 16,))[off:off + rows * cols // 2].view(np.uint32).reshape(rows, cols // 8)
        s = d_s.download(np.uint8, (rows * cols // 64 * 2 + 16,))[2:2 + rows * cols // 32].view(np.uint16).reshape(rows, cols // 64)
        b = d_b.download(np.uint8, (rows * cols // 64 * 2 + 16,))[2:2 + rows * cols // 32].view(np.uint16).reshape(rows, cols // 64)
        assert _same((w, s, b), want), off
    with pytest.raises(ValueError, match="16-byte aligned"):
        eng.pack_int4_dev(d_src.ptr + 4, _lib.DT_F32, rows, cols, d_w.ptr, d_s.ptr, d_b.ptr)
    for d in (d_src, d_w, d_s, d_b):
        d.free()


def test_packer_empty_and_ragged(eng):
    w, s, b = eng.pack_int4(np.zeros((0, 64), np.float32))
    assert w.shape == (0, 8) and s.shape == (0, 1)
    with pytest.raises(ValueError):
        eng.pack_int4(np.zeros((2, 100), np.float32))


def test_pack_experts_blob_bit_exact(eng):
    """process_experts_common layout: 4 experts of the reference shape, f32 and bf16 sources."""
    t = synth.layer_tensors(0, 5, 0, hidden=2048, inter=512, shared_inter=512, num_experts=4,
                            bf16_source=True, outlier_frac=0.001)
    want = oracle.pack_experts_layer(t["gate_up"], t["down"])
    got = eng.pack_experts(t["gate_up"], t["down"])
    assert np.array_equal(got, want)
    got16 = eng.pack_experts(synth.to_bf16_rne(t["gate_up"]), synth.to_bf16_rne(t["down"]))
    assert np.array_equal(got16, want)


def test_packer_idempotent_on_its_own_output(eng):
    """Packing the dequantised output again keeps every nibble (a size-independent property)."""
    rng = np.random.default_rng(13)
    v = synth.normal_weights(rng, (256, 1024))
    w, s, b = eng.pack_int4(v)
    deq = oracle.dequant_int4(w, s, b)
    w2, _, _ = eng.pack_int4(deq)
    nib = lambda a: np.stack([(a >> (4 * n)) & 0xF for n in range(8)], -1)
    assert (np.abs(nib(w).astype(int) - nib(w2).astype(int)) <= 1).all()


def test_matvec_config1(eng):
    """512x2048 gate_proj ~ N(0, 0.02^2) from seed 0, x ~ N(0,1) bf16; <= 1e-2 relative L2."""
    rng = np.random.Generator(np.random.PCG64(0))
    W = (rng.standard_normal((512, 2048), dtype=np.float32) * np.float32(0.02))
    x = synth.hidden_states(0, 1, 1, 2048)[0]
    w, s, b = oracle.quant_int4(W)
    y_ref = oracle.matvec_int4(w, s, b, x)
    y_deq = oracle.dequant_int4(w, s, b) @ x  # the dequantise-then-f32-matvec path
    y = eng.matvec_int4(w, s, b, x)
    assert rel_l2(y, y_ref) < 1e-2 and rel_l2(y, y_deq) < 1e-2
    assert rel_l2(y, y_ref) < 1e-4  # f32 accumulate: far inside the contract tolerance
    # GPU-packed weights give the same bytes, hence the same product
    assert _same(eng.pack_int4(W), (w, s, b))


@pytest.mark.parametrize("rows,cols", [(1, 2048), (2048, 512), (5, 64), (300, 4096), (64, 16384), (4099, 2048), (9000, 2048)])
def test_matvec_shapes(eng, rows, cols):
    rng = np.random.default_rng(rows + cols)
    w, s, b = oracle.quant_int4(synth.normal_weights(rng, (rows, cols)))
    x = rng.standard_normal(cols).astype(np.float32)
    assert rel_l2(eng.matvec_int4(w, s, b, x), oracle.matvec_int4(w, s, b, x)) < 1e-4


def test_matvec_linearity(eng):
    rng = np.random.default_rng(21)
    w, s, b = oracle.quant_int4(synth.normal_weights(rng, (512, 2048)))
    x1 = rng.standard_normal(2048).astype(np.float32)
    x2 = rng.standard_normal(2048).astype(np.float32)
    y = eng.matvec_int4(w, s, b, x1 + 2 * x2)
    assert rel_l2(y, eng.matvec_int4(w, s, b, x1) + 2 * eng.matvec_int4(w, s, b, x2)) < 1e-4


def test_matvec_rejects_bad_shapes(eng):
    with pytest.raises(ValueError):
        eng.matvec_int4(np.zeros((4, 9), np.uint32), np.zeros((4, 1), np.uint16), np.zeros((4, 1), np.uint16),
                        np.zeros(72, np.float32))
