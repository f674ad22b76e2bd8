"""GPU parity of the main layers' attention halves (gated full attention and Gated DeltaNet, batch-1 decode) with the
MoE half behind each, against the CPU oracle's restatement of src/engine/qwen35_moe/cpu.rs:87-347 and
src/math_util.rs:149-168, 401-597, through the C ABI.

A 4-layer stack (three linear-attention layers and one full-attention layer, as the model's interval of 4 arranges
them) is stepped over several tokens so that the KV cache, the conv state and the recurrence state all carry over;
both storage variants of the projections; reset; error paths.  Tolerance 1e-2 relative L2 (achieved values printed).
"""
import numpy as np
import pytest

import oracle
from benchmarks import synth
from moe_infer_b200 import _lib as L
from moe_infer_b200 import _moe_infer_rs as rs
from moe_infer_b200.native import Dims, NativeEngine
from tests.util import make_layer, rel_l2, upload_layer

pytestmark = pytest.mark.gpu
H, V, E, K = 2048, 200, 16, 8
AD = dict(num_heads=4, num_kv_heads=2, head_dim=64, rotary_dim=16, rope_theta=1.0e7, lin_num_k_heads=2, lin_num_v_heads=4,
          lin_key_dim=32, lin_value_dim=64, conv_kernel=4, full_attn_interval=4)


def _attn_weights(seed, scheme, layers, dims=None):
    ad = oracle.AttnDims(**(dims or AD))
    rng = np.random.default_rng(seed)
    bf = lambda a: oracle.f32_to_bf16(np.asarray(a, np.float32))
    f = oracle.bf16_to_f32
    norm = lambda n: bf(rng.uniform(0.8, 1.2, n))
    q4 = lambda r, c, gain=2.0: oracle.quant_int4(f(bf(synth.normal_weights(rng, (r, c)) * gain)))

    def attn_proj(r, c):  # bf16 in the BQ4 scheme, 4-bit in the INT4 scheme (bq4.rs:25-32)
        m = f(bf(synth.normal_weights(rng, (r, c)) * 2.0))
        return oracle.quant_int4(m) if scheme == "int4" else bf(m)

    q_dim, kv_dim = ad.num_heads * ad.head_dim, ad.num_kv_heads * ad.head_dim
    out = []
    for l in range(layers):
        if (l + 1) % ad.full_attn_interval == 0:
            out.append(oracle.FullAttnWeights(input_norm=norm(H), q_proj=attn_proj(2 * q_dim, H), k_proj=attn_proj(kv_dim, H),
                                              v_proj=attn_proj(kv_dim, H), q_norm=norm(ad.head_dim), k_norm=norm(ad.head_dim),
                                              o_proj=attn_proj(H, q_dim)))
        else:
            out.append(oracle.LinAttnWeights(
                input_norm=norm(H), in_proj_qkv=q4(ad.conv_dim, H), in_proj_z=q4(ad.total_value, H), in_proj_b=q4(ad.lin_num_v_heads, H),
                in_proj_a=q4(ad.lin_num_v_heads, H), conv1d=bf(rng.standard_normal((ad.conv_dim, ad.conv_kernel)) * 0.5),
                a_log=rng.uniform(-1.0, 1.0, ad.lin_num_v_heads).astype(np.float32), dt_bias=bf(rng.uniform(-1.0, 1.0, ad.lin_num_v_heads)),
                norm=norm(ad.lin_value_dim), out_proj=q4(H, ad.total_value)))
    return ad, out


def _upload_attn(eng, attn_layers, max_seq=16, dims=None):
    eng.attn_configure(max_seq=max_seq, **(dims or AD))
    for l, w in enumerate(attn_layers):
        eng.attn_load_vec(l, L.A_INPUT_NORM, w.input_norm)
        if isinstance(w, oracle.FullAttnWeights):
            eng.attn_load_vec(l, L.A_Q_NORM, w.q_norm)
            eng.attn_load_vec(l, L.A_K_NORM, w.k_norm)
            for which, t in ((L.A_Q_PROJ, w.q_proj), (L.A_K_PROJ, w.k_proj), (L.A_V_PROJ, w.v_proj), (L.A_O_PROJ, w.o_proj)):
                eng.attn_load_proj(l, which, t)
        else:
            for which, v in ((L.A_CONV1D, w.conv1d), (L.A_A_LOG, w.a_log), (L.A_DT_BIAS, w.dt_bias), (L.A_LIN_NORM, w.norm)):
                eng.attn_load_vec(l, which, v)
            for which, t in ((L.A_IN_PROJ_QKV, w.in_proj_qkv), (L.A_IN_PROJ_Z, w.in_proj_z), (L.A_IN_PROJ_B, w.in_proj_b),
                             (L.A_IN_PROJ_A, w.in_proj_a), (L.A_OUT_PROJ, w.out_proj)):
                eng.attn_load_proj(l, which, t)


@pytest.mark.parametrize("scheme", ["bq4", "int4"])
def test_decode_with_attention_matches_oracle(scheme):
    layers = 4
    ad, attn = _attn_weights(51, scheme, layers)
    moe = [make_layer(51, l, num_experts=E, scheme=scheme) for l in range(layers)]
    eng = NativeEngine(Dims(num_experts=E, top_k=K, num_layers=layers, vocab=V, scheme=L.SCHEME_INT4 if scheme == "int4" else L.SCHEME_BQ4))
    for l in range(layers):
        upload_layer(eng, l, moe[l])
    _upload_attn(eng, attn)
    emb = synth.hidden_states(51, 2, 6, H)
    state = oracle.ModelState(ad, layers, 16)
    want = np.stack([oracle.model_decode_token(attn, moe, ad, state, emb[t], K) for t in range(6)])
    got = np.concatenate([eng.model_forward_hidden(emb[:1]), eng.model_forward_hidden(emb[1:4]), eng.model_forward_hidden(emb[4:])])
    errs = [rel_l2(got[t], want[t]) for t in range(6)]
    print(f"decode with attention, {scheme}: rel-L2 per token {['%.1e' % x for x in errs]}")
    assert max(errs) < 1e-2 and eng.model_pos() == 6
    assert rel_l2(got - emb, want - emb) < 1e-2     # the layers' updates themselves, without the residual stream
    # the state itself, tensor by tensor, in the layout the reference's cache file uses (src/cache.rs:140-160)
    kv_dim = ad.num_kv_heads * ad.head_dim
    for l in range(layers):
        if l in state.kv:
            for which, ref in ((L.ST_K_CACHE, state.kv[l][0]), (L.ST_V_CACHE, state.kv[l][1])):
                assert rel_l2(eng.model_state_download(l, which, 6 * kv_dim).reshape(6, kv_dim), ref[:6]) < 1e-2
        else:
            ring = eng.model_state_download(l, L.ST_CONV, ad.conv_kernel * ad.conv_dim).reshape(ad.conv_kernel, ad.conv_dim)
            assert rel_l2(rs._shifted_from_ring(ring, 6), state.lin[l][0]) < 1e-2
            ssm = eng.model_state_download(l, L.ST_SSM, state.lin[l][1].size)
            assert rel_l2(ssm, state.lin[l][1].ravel()) < 1e-2
    with pytest.raises(ValueError, match="no KV cache"):
        eng.model_state_download(0, L.ST_K_CACHE, kv_dim)
    with pytest.raises(ValueError, match="holds"):
        eng.model_state_download(0, L.ST_SSM, 5)
    # snapshot, run ahead, roll back: the same tokens give the same result again (speculative decoding's reject path)
    snap = eng.model_snapshot()
    ahead = eng.model_forward_hidden(emb[:2])
    eng.model_restore(snap)
    assert eng.model_pos() == 6
    assert np.array_equal(eng.model_forward_hidden(emb[:2]), ahead)
    snap.free()
    # a new sequence: the caches and recurrence states start from zero again
    eng.model_reset()
    state = oracle.ModelState(ad, layers, 16)
    again = eng.model_forward_hidden(emb[2:4])
    want2 = np.stack([oracle.model_decode_token(attn, moe, ad, state, emb[t], K) for t in (2, 3)])
    assert rel_l2(again, want2) < 1e-2 and eng.model_pos() == 2
    eng.close()


def test_decode_with_attention_at_the_model_own_head_counts():
    """The shapes the kernels are tuned for (Qwen3.6-35B-A3B: 16 query / 2 KV heads of 256 with 64 rotary dimensions; 16 key
    and 32 value heads of 128, conv over 8,192 channels): the streaming 4-bit matvec with the input norm folded in
    (12,352 stacked rows), four CTAs per DeltaNet head with the norm's 1/rms folded into the 4,096-column output
    projection, the bf16 projections of 9,216 and 2,048 rows, attention over 256-wide heads.  Four layers (three DeltaNet,
    one full attention), five tokens so that the conv ring wraps and the cache is attended over."""
    dims = dict(num_heads=16, num_kv_heads=2, head_dim=256, rotary_dim=64, rope_theta=1.0e7, lin_num_k_heads=16, lin_num_v_heads=32,
                lin_key_dim=128, lin_value_dim=128, conv_kernel=4, full_attn_interval=4)
    layers = 4
    ad, attn = _attn_weights(57, "bq4", layers, dims)
    moe = [make_layer(57, l, num_experts=E) for l in range(layers)]
    eng = NativeEngine(Dims(num_experts=E, top_k=K, num_layers=layers, vocab=V))
    for l in range(layers):
        upload_layer(eng, l, moe[l])
    _upload_attn(eng, attn, dims=dims)
    emb = synth.hidden_states(57, 2, 5, H)
    state = oracle.ModelState(ad, layers, 16)
    want = np.stack([oracle.model_decode_token(attn, moe, ad, state, emb[t], K) for t in range(5)])
    got = np.concatenate([eng.model_forward_hidden(emb[:2]), eng.model_forward_hidden(emb[2:])])
    errs = [rel_l2(got[t], want[t]) for t in range(5)]
    print(f"decode with attention at the model's head counts: rel-L2 per token {['%.1e' % x for x in errs]}")
    assert max(errs) < 1e-2 and rel_l2(got - emb, want - emb) < 1e-2
    ssm = eng.model_state_download(0, L.ST_SSM, state.lin[0][1].size)
    assert rel_l2(ssm, state.lin[0][1].ravel()) < 1e-2
    # the same shapes as a prompt: nine tokens in one call run layer by layer, every projection over the nine tokens in one launch
    eng.model_reset()
    emb9 = synth.hidden_states(58, 2, 9, H)
    state = oracle.ModelState(ad, layers, 16)
    want9 = np.stack([oracle.model_decode_token(attn, moe, ad, state, emb9[t], K) for t in range(9)])
    got9 = eng.model_forward_hidden(emb9)
    print(f"the same as a 9-token prompt: rel-L2 {rel_l2(got9, want9):.1e}, on the updates {rel_l2(got9 - emb9, want9 - emb9):.1e}")
    assert rel_l2(got9, want9) < 1e-2 and rel_l2(got9 - emb9, want9 - emb9) < 1e-2 and eng.model_pos() == 9
    # what the prompt left behind: the recurrence state and conv inputs of a DeltaNet layer (kept in registers across the nine
    # tokens by one launch), and a tenth token decoded from there
    ssm = eng.model_state_download(1, L.ST_SSM, state.lin[1][1].size)
    ring = eng.model_state_download(1, L.ST_CONV, ad.conv_kernel * ad.conv_dim).reshape(ad.conv_kernel, ad.conv_dim)
    assert rel_l2(ssm, state.lin[1][1].ravel()) < 1e-2 and rel_l2(rs._shifted_from_ring(ring, 9), state.lin[1][0]) < 1e-2
    nxt = synth.hidden_states(60, 2, 1, H)
    want10 = oracle.model_decode_token(attn, moe, ad, state, nxt[0], K)
    assert rel_l2(eng.model_forward_hidden(nxt)[0], want10) < 1e-2
    eng.close()


@pytest.mark.parametrize("n", [8, 60])
def test_prompt_runs_layer_by_layer_and_matches_the_oracle(n):
    """A call of 4 tokens or more goes layer by layer: a layer's attention half token after token, its MoE half over all
    the tokens in one batched call (the slot-wise FFN up to 48 tokens, the grouped GEMMs on bf16 operands beyond).
    Against the oracle's token-by-token decode, then the sequence goes on token by token from the state it left."""
    layers = 4
    ad, attn = _attn_weights(59, "bq4", layers)
    moe = [make_layer(59, l, num_experts=E) for l in range(layers)]
    eng = NativeEngine(Dims(num_experts=E, top_k=K, num_layers=layers, vocab=V))
    for l in range(layers):
        upload_layer(eng, l, moe[l])
    _upload_attn(eng, attn, max_seq=80)
    emb = synth.hidden_states(59, 2, n + 2, H)
    state = oracle.ModelState(ad, layers, 80)
    want = np.stack([oracle.model_decode_token(attn, moe, ad, state, emb[t], K) for t in range(n + 2)])
    got = eng.model_forward_hidden(emb[:n])
    assert eng.model_pos() == n
    errs = [rel_l2(got[t], want[t]) for t in range(n)]
    print(f"prompt of {n} tokens, layer by layer: worst rel-L2 {max(errs):.1e}, on the layers' updates {rel_l2(got - emb[:n], want[:n] - emb[:n]):.1e}")
    # the whole output to the contract's 1e-2; a single token of the 60-token case (bf16 operands in the grouped GEMMs, four
    # layers deep) is allowed twice that: measured 1.0e-2 for the worst token, 2.3e-3 over the batch, 5e-4 at 8 tokens
    assert rel_l2(got, want[:n]) < 1e-2 and rel_l2(got - emb[:n], want[:n] - emb[:n]) < 1e-2
    assert max(errs) < (1e-2 if n <= 48 else 2e-2)
    tail = eng.model_forward_hidden(emb[n:])          # two tokens: token by token, from the caches the prompt filled
    assert max(rel_l2(tail[i], want[n + i]) for i in range(2)) < 2e-2
    eng.close()


def test_launch_modes_agree(monkeypatch):
    """The ways of launching a token's kernels (every kernel a programmatic dependent of the one before it, the default;
    one CUDA graph per attention half; plain launches; ordinary dependencies) change scheduling only: bit-identical
    results.  The one-CTA-per-head DeltaNet kernel sums in another order than the split one: equal to rounding."""
    layers = 4
    ad, attn = _attn_weights(53, "bq4", layers)
    moe = [make_layer(53, l, num_experts=E) for l in range(layers)]
    emb = synth.hidden_states(53, 2, 5, H)

    def run(env):
        for k in ("MOE_B200_ATTN_CHAIN", "MOE_B200_ATTN_GRAPHS", "MOE_B200_ATTN_PDL", "MOE_B200_LIN_SPLIT"):
            monkeypatch.delenv(k, raising=False)
        for k, v in env.items():
            monkeypatch.setenv(k, v)
        eng = NativeEngine(Dims(num_experts=E, top_k=K, num_layers=layers, vocab=V))   # the switches are read at the first step
        for l in range(layers):
            upload_layer(eng, l, moe[l])
        _upload_attn(eng, attn)
        out = np.concatenate([eng.model_forward_hidden(emb[:2]), eng.model_forward_hidden(emb[2:])])
        eng.close()
        return out

    base = run({})
    for env in ({"MOE_B200_ATTN_CHAIN": "0"}, {"MOE_B200_ATTN_CHAIN": "0", "MOE_B200_ATTN_GRAPHS": "0"}, {"MOE_B200_ATTN_PDL": "0"},
                {"MOE_B200_ATTN_PDL": "0", "MOE_B200_ATTN_GRAPHS": "0"}):
        assert np.array_equal(run(env), base), env
    other = run({"MOE_B200_LIN_SPLIT": "0"})
    assert rel_l2(other, base) < 1e-5
    assert np.array_equal(run({"MOE_B200_LIN_SPLIT": "0", "MOE_B200_ATTN_CHAIN": "0"}), other)


def test_attention_error_paths():
    layers = 4
    ad, attn = _attn_weights(52, "bq4", layers)
    eng = NativeEngine(Dims(num_experts=E, top_k=K, num_layers=layers, vocab=V))
    emb = synth.hidden_states(52, 2, 3, H)
    with pytest.raises(L.MoeError, match="not configured"):
        eng.model_forward_hidden(emb)
    with pytest.raises(L.MoeError, match="must come before"):
        eng.attn_load_vec(0, L.A_INPUT_NORM, attn[0].input_norm)
    eng.attn_configure(max_seq=2, **AD)
    with pytest.raises(ValueError, match="full-attention layer"):
        eng.attn_load_vec(3, L.A_CONV1D, attn[0].conv1d)      # layer 3 is the full-attention one
    with pytest.raises(ValueError, match="linear-attention layer"):
        eng.attn_load_proj(0, L.A_Q_PROJ, attn[3].q_proj)
    with pytest.raises(L.MoeError, match="input_layernorm missing"):
        eng.model_forward_hidden(emb[:1])
    assert eng.model_pos() == 0
    with pytest.raises(L.MoeError, match="do not fit"):
        eng.model_forward_hidden(emb)                           # three tokens, two positions
    eng.close()
