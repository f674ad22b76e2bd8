"""GPU: the callers on the far side of the binding, run against the mirror on a synthetic checkpoint that has every
tensor of the model (attention halves, MoE halves, MTP block, head): speculative decoding with the MTP drafter is
lossless, and the per-sequence state survives `download_cache` -> `Cache.save` -> `Cache.load` -> `upload_cache`
(src/engine.rs:64-79, src/cache.rs:133-233)."""
import json
import os

import numpy as np
import pytest

from benchmarks import synth
from moe_infer_b200 import _moe_infer_rs as rs
from moe_infer_b200.speculative import greedy_decode, speculative_decode
from tests.test_gpu_shim import H, V, _hf_checkpoint, _write_safetensors

pytestmark = pytest.mark.gpu
LAYERS = 4
AD = {"num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 64, "linear_num_key_heads": 2, "linear_num_value_heads": 4,
      "linear_key_head_dim": 32, "linear_value_head_dim": 64, "linear_conv_kernel_dim": 4, "full_attention_interval": 4}


@pytest.fixture(scope="module")
def model_dir(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("gen")
    src, dst = str(tmp / "hf"), str(tmp / "out")
    _hf_checkpoint(src, layers=LAYERS, mtp=1)
    cfg = json.load(open(os.path.join(src, "config.json")))
    cfg["text_config"].update(AD)
    json.dump(cfg, open(os.path.join(src, "config.json"), "w"))
    rng = np.random.default_rng(31)
    bf = lambda a: synth.to_bf16_rne(np.asarray(a, np.float32))
    zc = lambda n: bf(rng.uniform(-0.2, 0.2, n))
    mat = lambda r, c: bf(synth.normal_weights(rng, (r, c)) * 2.0)
    q_dim, kv_dim, conv_dim, total_value = 256, 128, 2 * 64 + 256, 256

    def full_attn(p):
        return {p + "self_attn.q_proj.weight": mat(2 * q_dim, H), p + "self_attn.k_proj.weight": mat(kv_dim, H),
                p + "self_attn.v_proj.weight": mat(kv_dim, H), p + "self_attn.o_proj.weight": mat(H, q_dim),
                p + "self_attn.q_norm.weight": zc(64), p + "self_attn.k_norm.weight": zc(64)}

    t = {}
    for l in range(LAYERS):
        p = f"model.language_model.layers.{l}."
        t[p + "input_layernorm.weight"] = zc(H)
        if (l + 1) % 4 == 0:
            t.update(full_attn(p))
        else:
            t.update({p + "linear_attn.in_proj_qkv.weight": mat(conv_dim, H), p + "linear_attn.in_proj_z.weight": mat(total_value, H),
                      p + "linear_attn.in_proj_b.weight": mat(4, H), p + "linear_attn.in_proj_a.weight": mat(4, H),
                      p + "linear_attn.conv1d.weight": bf(rng.standard_normal((conv_dim, 1, 4)) * 0.5),
                      p + "linear_attn.A_log": rng.uniform(-1, 1, 4).astype(np.float32), p + "linear_attn.dt_bias": bf(rng.uniform(-1, 1, 4)),
                      p + "linear_attn.norm.weight": bf(rng.uniform(0.8, 1.2, 64)), p + "linear_attn.out_proj.weight": mat(H, total_value)})
    t.update({"mtp.pre_fc_norm_hidden.weight": zc(H), "mtp.pre_fc_norm_embedding.weight": zc(H), "mtp.fc.weight": mat(H, 2 * H),
              "mtp.layers.0.input_layernorm.weight": zc(H), "mtp.norm.weight": zc(H)})
    t.update(full_attn("mtp.layers.0."))
    _write_safetensors(os.path.join(src, "model-00002-of-00002.safetensors"), t)
    rs.qwen35_moe_quantize(src, dst, version="3.6", scheme="bq4")
    return dst


def _prefill(model):
    eng = rs.Engine(model, "Qwen35MoEFusedExp2")
    assert not eng._missing_attn and not eng._missing_mtp and not eng._missing_head
    cache = rs.Cache(model)
    first = eng.forward(np.array([5, 17, 3], np.int64), cache, mtp=True)
    eng.mtp_reset()
    return eng, cache, first


def test_speculative_decoding_is_lossless_with_the_real_drafter_and_with_a_perfect_one(model_dir):
    model = rs.Model(model_dir)
    eng, cache, first = _prefill(model)
    want, gs = greedy_decode(first, eng, cache, max_tokens=10, mtp=True)
    eng.native.close()
    assert len(want) == 10 and gs["forwards"] == 10

    eng, cache, first2 = _prefill(model)
    assert np.array_equal(first, first2)
    got, st = speculative_decode(first2, eng, cache, max_tokens=10)
    print(f"MTP drafter on random weights: {st['accepted']} of {st['drafted']} drafts accepted, {st['forwards']} forwards")
    assert got == want and st["tokens"] == 10 and st["mtp_steps"] == st["drafted"] > 0
    assert cache.pos == eng.native.model_pos() and cache.pos >= 3 + 9
    eng.native.close()

    # a drafter that is always right (it reads the greedy run): every draft is accepted, two tokens per forward
    eng, cache, first3 = _prefill(model)
    real_mtp, calls = eng.mtp_forward, []

    def perfect(token_id):
        real_mtp(token_id)  # the real block still runs (its cache advances as it would)
        calls.append(int(token_id))
        out = np.zeros(V, np.float32)
        out[want[2 * len(calls) - 1]] = 1.0              # call i drafts for the token after want[2 i - 2]
        return out

    eng.mtp_forward = perfect
    got, st = speculative_decode(first3, eng, cache, max_tokens=10)
    assert got == want and st["accepted"] == st["drafted"] == 5 and st["forwards"] == 5 and st["forward_tokens"] == 10
    eng.native.close()


def test_cache_download_save_load_upload_continues_the_sequence(model_dir, tmp_path):
    model = rs.Model(model_dir)
    eng = rs.Engine(model, "Qwen35MoEFusedExp2")
    cache = rs.Cache(model)
    ids = np.array([5, 17, 3, 99, 42, 7], np.int64)   # 6 tokens: the conv ring has wrapped
    eng.forward(ids, cache)
    assert cache.gpu_dirty and cache.pos == 6
    eng.download_cache(cache)
    assert not cache.gpu_dirty and len(cache.states) == LAYERS
    assert cache.states[3]["k_cache"].shape == (6, 128) and cache.states[0]["conv_state"].shape == (3, 384)
    assert cache.states[0]["ssm_state"].shape == (4 * 64 * 32,) and np.abs(cache.states[0]["ssm_state"]).max() > 0
    b, j = str(tmp_path / "cache.bin"), str(tmp_path / "cache.json")
    cache.save(b, j)
    nxt = np.array([11, 23], np.int64)
    want = eng.forward(nxt, cache)                     # the sequence goes on: positions 6, 7
    # a second engine picks the sequence up from the file
    eng2 = rs.Engine(model, "Qwen35MoEFusedExp2")
    loaded = rs.Cache.load(b, j)
    assert loaded.pos == 6 and loaded.cpu_dirty
    got = eng2.forward(nxt, loaded)
    assert np.array_equal(got, want) and loaded.pos == 8 and not loaded.cpu_dirty
    # the first engine can go back to the saved point too (upload replaces its newer state)
    again = rs.Cache.load(b, j)
    assert np.array_equal(eng.forward(nxt, again), want)
    # a cache that claims a position but carries no state is refused
    stale = rs.Cache(model)
    stale.pos = 3
    with pytest.raises(RuntimeError, match="carries no state"):
        eng.forward(nxt[:1], stale)
    # reset: a new sequence from zero state gives the first run's logits again
    fresh = rs.Cache(model)
    a0 = eng.forward(ids[:2], fresh)
    cache.reset()
    assert cache.cpu_dirty and cache.states is None
    assert np.array_equal(eng.forward(ids[:2], cache), a0)
    eng.native.close()
    eng2.native.close()
