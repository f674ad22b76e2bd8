"""CPU-only: the oracle against the committed golden vectors and its own properties."""
import os

import numpy as np
import pytest

import oracle
from tests.util import make_layer, rel_l2

GOLD = os.path.join(os.path.dirname(__file__), "golden")


@pytest.fixture(scope="module")
def ref():
    return np.load(os.path.join(GOLD, "ref_codec.npz"))


@pytest.fixture(scope="module")
def kat():
    return np.load(os.path.join(GOLD, "packer_kat.npz"))


def test_bf16_rounding_matches_reference_python(ref):
    got = oracle.f32_to_bf16(ref["bf16_in"].view(np.float32))
    assert np.array_equal(got, ref["bf16_out"])


def test_bf16_rounding_is_not_rne():
    # bit15 = 1, bit16 = 0, bit0 = 0, other low bits set: the reference rounds DOWN
    v = np.array([0x3F808002], np.uint32).view(np.float32)
    assert oracle.f32_to_bf16(v)[0] == 0x3F80
    v = np.array([0x3F808001], np.uint32).view(np.float32)  # bit0 = 1 -> up
    assert oracle.f32_to_bf16(v)[0] == 0x3F81
    v = np.array([0x3F818000], np.uint32).view(np.float32)  # bit16 = 1 -> up
    assert oracle.f32_to_bf16(v)[0] == 0x3F82


def test_dequant_matches_reference_python(ref):
    got = oracle.dequant_int4(ref["dq_w"], ref["dq_s"], ref["dq_b"])
    assert np.array_equal(got, ref["dq_out"])


def test_layout_matches_reference_python(ref):
    keys = ["gate_w", "gate_s", "gate_b", "up_w", "up_s", "up_b", "down_w", "down_s", "down_b", "expert_size"]
    for (h, m, g), want in zip(ref["layouts_in"], ref["layouts_out"]):
        lay = oracle.expert_layout(int(h), int(m), int(g))
        assert [lay[k] for k in keys] == list(want)
    assert oracle.expert_layout(2048, 512)["expert_size"] == 1769472


def test_blob_sections_decoded_by_reference(ref):
    """The reference's blob reader finds gate/up/down where the oracle's packer put them."""
    blob = oracle.pack_experts_layer(ref["blob_gate_up"], ref["blob_down"])
    assert np.array_equal(blob, ref["blob_bytes"])
    E, two_i, hd = ref["blob_gate_up"].shape
    mi = two_i // 2
    for e in range(E):
        g = oracle.dequant_int4(*oracle.quant_int4(ref["blob_gate_up"][e, :mi]))
        u = oracle.dequant_int4(*oracle.quant_int4(ref["blob_gate_up"][e, mi:]))
        d = oracle.dequant_int4(*oracle.quant_int4(ref["blob_down"][e]))
        assert np.array_equal(g, ref["blob_sec_gate"][e])
        assert np.array_equal(u, ref["blob_sec_up"][e])
        assert np.array_equal(d, ref["blob_sec_down"][e])


def test_packer_known_answers(kat):
    names = sorted({k.rsplit(".", 1)[0] for k in kat.files})
    assert len(names) >= 12
    for n in names:
        w, s, b = oracle.quant_int4(kat[n + ".in"])
        assert np.array_equal(w, kat[n + ".w"]), n
        assert np.array_equal(s, kat[n + ".s"]), n
        assert np.array_equal(b, kat[n + ".b"]), n


def test_packer_constant_group(kat):
    # max = min + 1, scale = 1/15, every nibble 0
    assert not kat["constant_group.w"].any()
    assert oracle.bf16_to_f32(kat["constant_group.s"])[0, 0] == oracle.bf16_to_f32(
        oracle.f32_to_bf16(np.array([1.0 / 15.0], np.float32)))[0]


def test_packer_half_rounds_up(kat):
    w = kat["half_way_levels.w"][0]
    nib = np.array([(int(w[i // 8]) >> (4 * (i % 8))) & 0xF for i in range(64)])
    assert list(nib[:16]) == list(range(16))
    assert list(nib[16:31]) == list(range(1, 16))  # k + 0.5 -> k + 1, not half-even


def test_packer_min_is_0_max_is_15():
    rng = np.random.default_rng(1)
    v = (rng.standard_normal((64, 512)) * 0.02).astype(np.float32)
    w, s, b = oracle.quant_int4(v)
    nib = np.stack([(w >> (4 * n)) & 0xF for n in range(8)], axis=-1).reshape(64, 512)
    g = nib.reshape(64, 8, 64)
    assert (g.min(axis=2) == 0).all() and (g.max(axis=2) == 15).all()
    # nibble n of word g*8+p is column g*64 + p*8 + n
    col = 3 * 64 + 5 * 8 + 6
    assert nib[7, col] == (int(w[7, 3 * 8 + 5]) >> 24) & 0xF


def test_packer_roundtrip_property_of_reference_test():
    """src/dtype.rs:483-499 restated: max error / range < 0.1 per group on sin(i)."""
    v = np.sin(np.arange(2 * 128, dtype=np.float32)).reshape(2, 128)
    r = oracle.dequant_int4(*oracle.quant_int4(v))
    for row in range(2):
        for g in range(2):
            a, b = v[row, g * 64:(g + 1) * 64], r[row, g * 64:(g + 1) * 64]
            rng_ = a.max() - a.min()
            if rng_ > 0.001:
                assert np.abs(a - b).max() / rng_ < 0.1


def _np_bf16_ref(v: np.ndarray) -> np.ndarray:
    """The reference's f32 -> bf16 rounding (src/dtype.rs:85-89), in numpy integer arithmetic."""
    bits = v.astype(np.float32).view(np.uint32).astype(np.uint64)
    # the reference ANDs a one-bit value with an unnormalised word: only bit 0 of (low 15 bits | bit 16) counts
    round_up = ((bits >> 15) & 1) & ((bits & 0x7FFF) | ((bits >> 16) & 1))
    return (((bits + (round_up << 16)) >> 16) & 0xFFFF).astype(np.uint16)


def _np_quant_int4(v: np.ndarray):
    """quant_f32_to_int4 (src/dtype.rs:102-135) written a second time, in numpy float32 arithmetic: every
    numpy f32 operation rounds once, like the Rust expression it stands for."""
    v = v.astype(np.float32)
    rows, cols = v.shape
    g = v.reshape(rows, cols // 64, 64)
    vmin = g.min(axis=2)
    vmax = g.max(axis=2)
    vmax = np.where(vmax == vmin, vmin + np.float32(1.0), vmax).astype(np.float32)
    scale = ((vmax - vmin) / np.float32(15.0)).astype(np.float32)
    inv = (np.float32(1.0) / scale).astype(np.float32)
    t = ((g - vmin[..., None]).astype(np.float32) * inv[..., None]).astype(np.float32) + np.float32(0.5)
    q = np.clip(np.trunc(t.astype(np.float32)), 0, 15).astype(np.uint32).reshape(rows, cols // 8, 8)
    w = np.zeros((rows, cols // 8), np.uint32)
    for n in range(8):
        w |= q[:, :, n] << np.uint32(4 * n)
    return w, _np_bf16_ref(scale), _np_bf16_ref(vmin)


@pytest.mark.parametrize("seed,shape,spread", [(3, (16, 256), 0.0), (4, (7, 128), 30.0), (5, (33, 2048), 0.0)])
def test_packer_matches_numpy_restatement(seed, shape, spread):
    """The C packer against a second, independent statement of the same arithmetic (numpy f32), bit for bit;
    spread > 0 scales rows over many decades."""
    rng = np.random.default_rng(seed)
    v = (rng.standard_normal(shape) * 0.02).astype(np.float32)
    if spread:
        v = (v * np.exp(rng.uniform(-spread, spread, size=(shape[0], 1)))).astype(np.float32)
    v[0, :64] = 0.25  # a constant group
    got = oracle.quant_int4(v)
    want = _np_quant_int4(v)
    for a, b in zip(got, want):
        assert np.array_equal(a, b)


def test_bf16_source_equals_widened_f32():
    rng = np.random.default_rng(2)
    u = oracle.f32_to_bf16((rng.standard_normal((8, 128)) * 0.02).astype(np.float32))
    a = oracle.quant_int4_bf16(u)
    b = oracle.quant_int4(oracle.bf16_to_f32(u))
    assert all(np.array_equal(x, y) for x, y in zip(a, b))


def test_matvec_against_dequantise_then_f32():
    rng = np.random.default_rng(0)
    W = (rng.standard_normal((512, 2048)) * 0.02).astype(np.float32)
    x = oracle.bf16_to_f32(oracle.f32_to_bf16(rng.standard_normal(2048).astype(np.float32)))
    w, s, b = oracle.quant_int4(W)
    y = oracle.matvec_int4(w, s, b, x)
    y2 = oracle.dequant_int4(w, s, b).astype(np.float64) @ x.astype(np.float64)
    assert rel_l2(y, y2) < 1e-5
    assert np.array_equal(oracle.matvec_int4(w, s, b, x, threads=4), y)


def test_topk_semantics():
    scores = np.array([0.1, 0.5, 0.5, 0.2, 0.9, 0.05, 0.3, 0.5], np.float32)
    idx, wts, probs = oracle.route_experts(np.log(scores), 3)
    assert set(idx.tolist()) == {4, 1, 2}  # strict '>' keeps the earlier of equal scores
    assert abs(wts.sum() - 1.0) < 1e-6
    rng = np.random.default_rng(3)
    logits = rng.standard_normal(256).astype(np.float32)
    idx, wts, probs = oracle.route_experts(logits, 8)
    assert set(idx.tolist()) == set(np.argsort(-logits)[:8].tolist())
    want = probs[idx] / probs[idx].sum()
    assert np.allclose(wts, want, rtol=1e-6)


def test_layer_matches_numpy_restatement():
    """The C layer function against an independent numpy statement of the same block."""
    lw = make_layer(0, 0, num_experts=8)
    rng = np.random.default_rng(5)
    h = rng.standard_normal((3, 2048)).astype(np.float32)
    out, idx, wts = oracle.moe_layer(lw, h, 4)
    lay = oracle.expert_layout(2048, 512)
    for t in range(3):
        x = oracle.rms_norm_bf16(h[t], lw.post_norm_w)
        logits = oracle.bf16_to_f32(lw.router_bf16).astype(np.float64) @ x
        p = np.exp(logits - logits.max())
        p /= p.sum()
        top = np.argsort(-p)[:4]
        assert set(top.tolist()) == set(idx[t].tolist())
        acc = h[t].astype(np.float64).copy()
        for e in top:
            blob = lw.experts[e * lay["expert_size"]:(e + 1) * lay["expert_size"]]

            def sec(off, rows, cols):
                wb = rows * cols // 2
                sb = rows * (cols // 64) * 2
                w = blob[off:off + wb].view(np.uint32).reshape(rows, cols // 8)
                s = blob[off + wb:off + wb + sb].view(np.uint16).reshape(rows, cols // 64)
                b = blob[off + wb + sb:off + wb + 2 * sb].view(np.uint16).reshape(rows, cols // 64)
                return oracle.dequant_int4(w, s, b).astype(np.float64)

            g = sec(lay["gate_w"], 512, 2048) @ x
            u = sec(lay["up_w"], 512, 2048) @ x
            a = g / (1 + np.exp(-g)) * u
            acc += (p[e] / p[top].sum()) * (sec(lay["down_w"], 2048, 512) @ a)
        g = oracle.dequant_int4(*lw.sh_gate).astype(np.float64) @ x
        u = oracle.dequant_int4(*lw.sh_up).astype(np.float64) @ x
        a = g / (1 + np.exp(-g)) * u
        sg = float((oracle.dequant_int4(*lw.sgate).astype(np.float64) @ x)[0])
        acc += 1 / (1 + np.exp(-sg)) * (oracle.dequant_int4(*lw.sh_down).astype(np.float64) @ a)
        assert rel_l2(out[t], acc) < 1e-5
    out_mt, _, _ = oracle.moe_layer(lw, h, 4, threads=3)
    assert np.array_equal(out, out_mt)
    o1, i1, w1 = oracle.moe_layer_decode_mt(lw, h[0], 4)
    assert np.array_equal(o1, out[0])


def test_forced_indices_and_bias():
    lw = make_layer(0, 1, num_experts=8)
    h = np.random.default_rng(6).standard_normal((2, 2048)).astype(np.float32)
    forced = np.array([[0, 1, 2, 3], [7, 6, 5, 4]], np.int32)
    out, idx, wts = oracle.moe_layer(lw, h, 4, forced_idx=forced)
    assert np.array_equal(idx, forced)
    assert np.allclose(wts.sum(axis=1), 1.0, atol=1e-6)
    bias = np.zeros(8, np.float32)
    bias[5] = 100.0
    _, idx2, wts2 = oracle.moe_layer(lw, h, 4, logit_bias=bias)
    assert (idx2 == 5).any(axis=1).all() and wts2.max() > 0.99
