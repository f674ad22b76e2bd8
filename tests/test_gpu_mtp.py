"""GPU parity of the whole MTP step (token embedding, pre-fc norms, fc, gated full attention with per-head norm,
RoPE and KV cache, MoE half, output norm, lm_head) against the CPU oracle's restatement of
src/engine/qwen35_moe/mtp.rs:58-225, through the C ABI.

Both storage variants of the projections (bf16 matrices as in the BQ4 scheme, 4-bit triples as in the INT4 scheme),
several positions in a row so that the cache is attended over, rollback, and the error paths.
Tolerance: 1e-2 relative L2 on the logits, as for every floating-point path here; the achieved values are printed.
"""
import numpy as np
import pytest

import oracle
from benchmarks import synth
from moe_infer_b200 import _lib as L
from moe_infer_b200.native import Dims, NativeEngine
from tests.util import make_layer, rel_l2, upload_layer

pytestmark = pytest.mark.gpu
H, V, E, K = 2048, 300, 16, 8
NH, NKV, HD, ROPE, THETA = 4, 2, 64, 16, 1.0e7


def _weights(seed, scheme):
    rng = np.random.default_rng(seed)
    bf = lambda a: oracle.f32_to_bf16(np.asarray(a, np.float32))
    f = oracle.bf16_to_f32
    norm = lambda n: bf(rng.uniform(0.8, 1.2, n))
    q_dim, kv_dim = NH * HD, NKV * HD

    def proj(rows, cols):
        m = f(bf(synth.normal_weights(rng, (rows, cols)) * 2.0))
        return oracle.quant_int4(m) if scheme == "int4" else bf(m)

    mw = oracle.MtpWeights(hnorm=norm(H), enorm=norm(H), fc=oracle.quant_int4(f(bf(synth.normal_weights(rng, (H, 2 * H))))),
                           attn_norm=norm(H), q_proj=proj(2 * q_dim, H), k_proj=proj(kv_dim, H), v_proj=proj(kv_dim, H),
                           q_norm=norm(HD), k_norm=norm(HD), o_proj=proj(H, q_dim), out_norm=norm(H),
                           num_heads=NH, num_kv_heads=NKV, head_dim=HD, rope_dim=ROPE, rope_theta=THETA)
    embed = oracle.quant_int4(f(bf(synth.normal_weights(rng, (V, H)) * 30.0)))
    lm = f(bf(synth.normal_weights(rng, (V, H))))
    lm_head = oracle.quant_int4(lm) if scheme == "int4" else oracle.quant_int8(lm)
    return mw, embed, lm_head, norm(H)


def _engine(scheme, mw, embed, lm_head, final_norm, moe, *, max_seq=16, out_norm=True):
    eng = NativeEngine(Dims(num_experts=E, top_k=K, num_layers=1, num_mtp_layers=1, vocab=V,
                            scheme=L.SCHEME_INT4 if scheme == "int4" else L.SCHEME_BQ4))
    upload_layer(eng, 1, moe)  # the MTP block's MoE half is layer index num_layers
    eng.load_embed(embed)
    eng.load_final_norm(final_norm)
    if scheme == "int4":
        eng.load_lm_head_q4(lm_head)
    else:
        eng.load_lm_head_int8(*lm_head)
    eng.mtp_configure(NH, NKV, HD, ROPE, THETA, max_seq=max_seq)
    for which, w in ((L.M_PRE_FC_NORM_HIDDEN, mw.hnorm), (L.M_PRE_FC_NORM_EMBEDDING, mw.enorm), (L.M_INPUT_NORM, mw.attn_norm),
                     (L.M_Q_NORM, mw.q_norm), (L.M_K_NORM, mw.k_norm)):
        eng.mtp_load_norm(which, w)
    if out_norm:
        eng.mtp_load_norm(L.M_OUT_NORM, mw.out_norm)
    for which, t in ((L.M_FC, mw.fc), (L.M_Q_PROJ, mw.q_proj), (L.M_K_PROJ, mw.k_proj), (L.M_V_PROJ, mw.v_proj),
                     (L.M_O_PROJ, mw.o_proj)):
        eng.mtp_load_proj(which, t)
    return eng


@pytest.mark.parametrize("scheme", ["bq4", "int4"])
def test_mtp_step_matches_oracle_over_positions(scheme):
    mw, embed, lm_head, final_norm = _weights(41, scheme)
    moe = make_layer(41, 1, num_experts=E, scheme=scheme)
    eng = _engine(scheme, mw, embed, lm_head, final_norm, moe)
    kc = np.zeros((16, NKV * HD), np.float32)
    vc = np.zeros((16, NKV * HD), np.float32)
    hs = synth.hidden_states(41, 2, 5, H)
    toks = [7, 299, 0, 123, 42]
    worst = 0.0
    for pos in range(4):
        got = eng.mtp_step(hs[pos], toks[pos])
        want = oracle.mtp_step(mw, moe, K, embed, lm_head, hs[pos], toks[pos], pos, kc, vc)
        err = rel_l2(got, want)
        worst = max(worst, err)
        assert got.shape == (V,) and err < 1e-2, (pos, err)
        assert eng.mtp_pos() == pos + 1
    print(f"MTP step, {scheme} projections: worst rel-L2 over 4 positions {worst:.2e}")
    # roll back to position 2 and take another token there: the cache entries behind it are replaced
    eng.mtp_rollback(2)
    got = eng.mtp_step(hs[4], toks[4])
    want = oracle.mtp_step(mw, moe, K, embed, lm_head, hs[4], toks[4], 2, kc, vc)
    assert rel_l2(got, want) < 1e-2 and eng.mtp_pos() == 3
    # reset starts a new sequence: position 0 attends to itself only
    eng.mtp_reset()
    kc[:] = 0
    vc[:] = 0
    got = eng.mtp_step(hs[1], toks[1])
    want = oracle.mtp_step(mw, moe, K, embed, lm_head, hs[1], toks[1], 0, kc, vc)
    assert rel_l2(got, want) < 1e-2
    eng.close()


def test_mtp_step_without_its_own_output_norm_uses_the_final_norm():
    mw, embed, lm_head, final_norm = _weights(43, "bq4")
    moe = make_layer(43, 1, num_experts=E)
    eng = _engine("bq4", mw, embed, lm_head, final_norm, moe, out_norm=False)
    mw.out_norm = final_norm  # mtp.rs:209-216
    kc = np.zeros((4, NKV * HD), np.float32)
    vc = np.zeros((4, NKV * HD), np.float32)
    h = synth.hidden_states(43, 2, 1, H)[0]
    assert rel_l2(eng.mtp_step(h, 5), oracle.mtp_step(mw, moe, K, embed, lm_head, h, 5, 0, kc, vc)) < 1e-2
    eng.close()


def test_mtp_step_error_paths():
    mw, embed, lm_head, final_norm = _weights(44, "bq4")
    moe = make_layer(44, 1, num_experts=E)
    eng = _engine("bq4", mw, embed, lm_head, final_norm, moe, max_seq=2)
    h = synth.hidden_states(44, 2, 1, H)[0]
    with pytest.raises(ValueError, match="token id"):
        eng.mtp_step(h, V)
    eng.mtp_step(h, 1)
    eng.mtp_step(h, 2)
    with pytest.raises(L.MoeError, match="KV cache is full") as ei:
        eng.mtp_step(h, 3)
    assert ei.value.status == L.ERR_STATE and eng.mtp_pos() == 2
    eng.close()
    # a block whose tensors are incomplete says which one is missing; an engine without an MTP layer refuses
    eng = NativeEngine(Dims(num_experts=E, top_k=K, num_layers=1, num_mtp_layers=1, vocab=V))
    eng.mtp_configure(NH, NKV, HD, ROPE, THETA, max_seq=4)
    with pytest.raises(L.MoeError, match="mtp.pre_fc_norm_hidden missing"):
        eng.mtp_step(h, 1)
    eng.close()
    eng = NativeEngine(Dims(num_experts=E, top_k=K, num_layers=1, vocab=V))
    with pytest.raises(L.MoeError, match="no MTP block"):
        eng.mtp_configure(NH, NKV, HD, ROPE, THETA)
    eng.close()
