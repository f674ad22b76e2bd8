"""GPU: the `_moe_infer_rs` mirror end to end — quantise a synthetic HF-style checkpoint,
load it through Model/Engine and compare the forward with the CPU oracle."""
import json
import os
import struct

import numpy as np
import pytest

import oracle
from moe_infer_b200 import _moe_infer_rs as rs
from benchmarks import synth
from tests.util import rel_l2

pytestmark = pytest.mark.gpu
E, K, H, I, V = 4, 4, 2048, 512, 100


def _write_safetensors(path, tensors):
    hdr, blobs, off = {}, [], 0
    for name, arr in tensors.items():
        raw = np.ascontiguousarray(arr).tobytes()
        hdr[name] = {"dtype": "F32" if arr.dtype == np.float32 else "BF16", "shape": list(arr.shape),
                     "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    h = json.dumps(hdr).encode()
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(h)))
        f.write(h)
        for b in blobs:
            f.write(b)


def _hf_checkpoint(tmp, layers, mtp):
    cfg = {"architectures": ["Qwen3_5MoeForConditionalGeneration_Stripped"],
           "text_config": {"hidden_size": H, "num_hidden_layers": layers, "mtp_num_hidden_layers": mtp, "vocab_size": 100,
                           "num_experts": E, "num_experts_per_tok": K, "moe_intermediate_size": I,
                           "shared_expert_intermediate_size": I, "num_key_value_heads": 2, "head_dim": 256}}
    os.makedirs(tmp, exist_ok=True)
    json.dump(cfg, open(os.path.join(tmp, "config.json"), "w"))
    raw, ts = [], {}
    for l in range(layers + mtp):
        t = synth.layer_tensors(7, 5, l, hidden=H, inter=I, shared_inter=I, num_experts=E, bf16_source=True)
        t["post_norm"] = synth.bf16_to_f32(synth.to_bf16_rne(
            np.random.default_rng(l).uniform(-0.1, 0.1, H).astype(np.float32)))  # zero-centred, as in Qwen3.6
        raw.append(t)
        p = f"model.language_model.layers.{l}." if l < layers else f"mtp.layers.{l - layers}."
        b = synth.to_bf16_rne
        ts.update({p + "mlp.experts.gate_up_proj": b(t["gate_up"]), p + "mlp.experts.down_proj": b(t["down"]),
                   p + "mlp.gate.weight": b(t["router"]), p + "mlp.shared_expert.gate_proj.weight": b(t["shared_gate"]),
                   p + "mlp.shared_expert.up_proj.weight": b(t["shared_up"]),
                   p + "mlp.shared_expert.down_proj.weight": b(t["shared_down"]),
                   p + "mlp.shared_expert_gate.weight": b(t["shared_sgate"]),
                   p + "post_attention_layernorm.weight": b(t["post_norm"])})
    rng = np.random.default_rng(99)
    head = {"embed": synth.bf16_to_f32(synth.to_bf16_rne(synth.normal_weights(rng, (V, H)))),
            "norm": synth.bf16_to_f32(synth.to_bf16_rne(rng.uniform(-0.1, 0.1, H).astype(np.float32))),
            "lm_head": synth.bf16_to_f32(synth.to_bf16_rne(synth.normal_weights(rng, (V, H))))}
    ts.update({"model.language_model.embed_tokens.weight": synth.to_bf16_rne(head["embed"]),
               "model.language_model.norm.weight": synth.to_bf16_rne(head["norm"]),
               "lm_head.weight": synth.to_bf16_rne(head["lm_head"])})
    _write_safetensors(os.path.join(tmp, "model-00001-of-00001.safetensors"), ts)
    return raw, head


def _oracle_logits(head, scheme, hidden):
    x = oracle.final_norm(hidden, oracle.f32_to_bf16(head["norm"] + np.float32(1.0)))
    if scheme == "bq4":
        q, sc = oracle.quant_int8(head["lm_head"])
        return np.stack([oracle.matvec_int8(q, sc, xi) for xi in x])
    w, s, b = oracle.quant_int4(head["lm_head"])
    return np.stack([oracle.matvec_int4(w, s, b, xi) for xi in x])


def _oracle_layers(raw, scheme):
    out = []
    for t in raw:
        out.append(oracle.LayerWeights(
            hidden=H, inter=I, shared_inter=I, num_experts=E, post_norm_w=oracle.f32_to_bf16(t["post_norm"] + np.float32(1.0)),
            router_bf16=oracle.f32_to_bf16(t["router"]) if scheme == "bq4" else None,
            router_q4=None if scheme == "bq4" else oracle.quant_int4(t["router"]),
            sh_gate=oracle.quant_int4(t["shared_gate"]), sh_up=oracle.quant_int4(t["shared_up"]),
            sh_down=oracle.quant_int4(t["shared_down"]), sgate=oracle.quant_int4(t["shared_sgate"]),
            experts=oracle.pack_experts_layer(t["gate_up"], t["down"])))
    return out


@pytest.mark.parametrize("scheme", ["bq4", "int4"])
def test_quantize_load_forward(tmp_path, scheme):
    src, dst = str(tmp_path / "hf"), str(tmp_path / "out")
    raw, head = _hf_checkpoint(src, layers=2, mtp=1)
    rs.qwen35_moe_quantize(src, dst, version="3.6", scheme=scheme)
    ref_layers = _oracle_layers(raw, scheme)
    for l, lw in enumerate(ref_layers):  # packed bytes identical to the reference packer's
        assert np.array_equal(np.fromfile(os.path.join(dst, "packed_experts", f"layer_{l:02d}.bin"), np.uint8), lw.experts)
    model = rs.Model(dst)
    eng = rs.Engine(model, "Qwen35MoEFusedExp3")
    cache = rs.Cache(model)
    emb = synth.hidden_states(3, 2, 5, H)
    rs.record_engine_telemetry(True)
    out = eng.forward_hidden_states(emb, cache)
    rs.record_engine_telemetry(False)
    ref = oracle.moe_stack(ref_layers[:2], emb, K)
    assert out.shape == (5, H) and rel_l2(out, ref) < 1e-2
    assert cache.pos == 5 and cache.gpu_dirty and eng.telemetry()["engine.total_ms"] > 0
    assert np.array_equal(eng.last_h_pre_norm(), out[-1])
    # the reference surface: logits [n, vocab] from embeddings and from token ids
    logits = eng.forward_hidden(emb, cache)
    assert logits.shape == (5, V) and rel_l2(logits, _oracle_logits(head, scheme, ref)) < 1e-2
    ids = np.array([3, 99, 0], np.int64)
    ew, es, eb = oracle.quant_int4(head["embed"])
    emb_ref = oracle.embed_lookup(ew, es, eb, ids)
    assert np.array_equal(eng.embed_lookup(ids), emb_ref)                  # row dequantisation is exact
    want = _oracle_logits(head, scheme, oracle.moe_stack(ref_layers[:2], emb_ref, K))
    got = eng.forward(ids, cache)
    assert got.shape == (3, V) and rel_l2(got, want) < 1e-2
    got_b = eng.forward_batched(ids, cache)                                # grouped path: bf16 operands
    assert got_b.shape == (3, V) and rel_l2(got_b, want) < 2e-2 and cache.pos == 16
    assert np.array_equal(got.argmax(axis=1), want.argmax(axis=1))
    assert eng.forward(np.zeros(0, np.int64), cache).shape == (0, V)
    with pytest.raises(ValueError, match="token id"):
        eng.forward(np.array([V], np.int64), cache)
    snap = eng.snapshot_state()
    m = eng.mtp_forward(0)                                                 # MoE half of the MTP block (layer index 2)
    ref_m, _, _ = oracle.moe_layer(ref_layers[2], eng.last_h_pre_norm(), K)
    assert rel_l2(m, ref_m[0]) < 1e-2
    with pytest.raises(ValueError):
        eng.mtp_forward(V)
    eng.forward_hidden_states(emb[:1], cache)
    eng.restore_snapshot(snap)
    assert eng.pos == 16
    eng.native.close()


@pytest.mark.parametrize("scheme", ["bq4", "int4"])
def test_quantize_whole_checkpoint_names_types_values(tmp_path, scheme):
    """Every tensor of a checkpoint goes through the reference's pipeline (src/quantize.rs:171-291): manifest name,
    storage type by scheme, +1 on zero-centred norms (Qwen3.6), conv1d axes, inner-dimension padding, config block."""
    from moe_infer_b200.modeldir import ModelDir
    src, dst = str(tmp_path / "hf"), str(tmp_path / "out")
    _hf_checkpoint(src, layers=1, mtp=0)
    rng = np.random.default_rng(5)
    bf = lambda a: synth.to_bf16_rne(a.astype(np.float32))
    f = lambda bits: synth.bf16_to_f32(bits)
    p = "model.language_model.layers.0."
    extra = {
        p + "input_layernorm.weight": bf(rng.uniform(-0.1, 0.1, H)),
        p + "self_attn.q_proj.weight": bf(synth.normal_weights(rng, (64, H))),
        p + "self_attn.q_norm.weight": bf(rng.uniform(-0.1, 0.1, 256)),
        p + "linear_attn.conv1d.weight": bf(rng.standard_normal((8, 1, 4))),
        p + "linear_attn.A_log": rng.standard_normal(16).astype(np.float32),
        p + "linear_attn.dt_bias": bf(rng.standard_normal(16)),
        p + "linear_attn.norm.weight": bf(rng.uniform(0.9, 1.1, 128)),
        p + "linear_attn.in_proj_a.weight": bf(synth.normal_weights(rng, (16, H))),
        p + "linear_attn.out_proj.weight": bf(synth.normal_weights(rng, (32, 96))),
        "model.visual.blocks.0.attn.qkv.weight": bf(synth.normal_weights(rng, (8, 64))),
    }
    _write_safetensors(os.path.join(src, "model-00002-of-00002.safetensors"), extra)
    from moe_infer_b200.quantize import quantize_moe_checkpoint
    summary = quantize_moe_checkpoint(src, dst, version="3.6", scheme=scheme)
    md = ModelDir(dst)
    L0 = "language_model.model.layers.0."
    assert not any(k.startswith("vision_tower") or "visual" in k for k in md.tensors)
    # zero-centred norms are stored as w + 1; the gated norm of the linear-attention block is not
    for name, shifted in (("input_layernorm.weight", True), ("self_attn.q_norm.weight", True), ("linear_attn.norm.weight", False)):
        want = f(extra[p + name]) + (np.float32(1.0) if shifted else np.float32(0.0))
        info = md.tensors[L0 + name]
        assert info["dtype"] == "bf16" and info["shape"] == [want.size]
        assert np.array_equal(md.tensor(L0 + name), oracle.f32_to_bf16(want))
    # conv1d [C, K, S] -> [C, S, K], bf16, flat
    conv = md.tensor(L0 + "linear_attn.conv1d.weight")
    assert np.array_equal(conv, np.moveaxis(extra[p + "linear_attn.conv1d.weight"], 2, 1).reshape(-1))
    assert md.tensors[L0 + "linear_attn.A_log"]["dtype"] == "f32"
    assert np.array_equal(md.tensor(L0 + "linear_attn.A_log"), extra[p + "linear_attn.A_log"])
    assert np.array_equal(md.tensor(L0 + "linear_attn.dt_bias"), extra[p + "linear_attn.dt_bias"])
    # attention projections: bf16 in BQ4 (under their full name), 4-bit triple in INT4 (".weight" stripped from the base)
    q = f(extra[p + "self_attn.q_proj.weight"])
    if scheme == "bq4":
        assert md.tensors[L0 + "self_attn.q_proj.weight"]["dtype"] == "bf16"
        assert np.array_equal(md.tensor(L0 + "self_attn.q_proj.weight"), extra[p + "self_attn.q_proj.weight"].reshape(-1))
    else:
        got = md.q4(L0 + "self_attn.q_proj")
        assert md.tensors[L0 + "self_attn.q_proj.weight"]["dtype"] == "u32"
        assert all(np.array_equal(a, b) for a, b in zip(got, oracle.quant_int4(q)))
    got = md.q4(L0 + "linear_attn.in_proj_a")
    assert all(np.array_equal(a, b) for a, b in zip(got, oracle.quant_int4(f(extra[p + "linear_attn.in_proj_a.weight"]))))
    # inner dimension 96 is zero-padded to 128 before packing
    padded = np.zeros((32, 128), np.float32)
    padded[:, :96] = f(extra[p + "linear_attn.out_proj.weight"])
    got = md.q4(L0 + "linear_attn.out_proj")
    assert got[0].shape == (32, 16) and all(np.array_equal(a, b) for a, b in zip(got, oracle.quant_int4(padded)))
    # the manifest's config block
    cfg = json.load(open(os.path.join(dst, "model_weights.json")))["config"]
    assert cfg["hidden_size"] == H and cfg["num_hidden_layers"] == 1 and cfg["num_experts"] == E
    assert cfg["layer_types"] == ["linear_attention"] and cfg["full_attention_interval"] == 4
    assert cfg["rope_theta"] == 10_000_000.0 and cfg["partial_rotary_factor"] == 0.25 and cfg["linear_conv_kernel_dim"] == 4
    assert summary["f32"] == 1 and summary.get("int8", 0) == (1 if scheme == "bq4" else 0)


@pytest.mark.parametrize("scheme", ["bq4", "int4"])
def test_mtp_forward_returns_logits_when_the_block_is_complete(tmp_path, scheme):
    """A checkpoint that carries the MTP block's attention tensors: quantise, load, and `mtp_forward(token)` is the
    reference's draft step (src/python_bindings.rs:283-291, src/engine/qwen35_moe/mtp.rs:58-225): logits [vocab]."""
    NH, NKV, HD = 4, 2, 64
    src, dst = str(tmp_path / "hf"), str(tmp_path / "out")
    raw, head = _hf_checkpoint(src, layers=1, mtp=1)
    cfg = json.load(open(os.path.join(src, "config.json")))
    cfg["text_config"].update({"num_attention_heads": NH, "num_key_value_heads": NKV, "head_dim": HD})
    json.dump(cfg, open(os.path.join(src, "config.json"), "w"))
    rng = np.random.default_rng(17)
    bf = lambda a: synth.to_bf16_rne(np.asarray(a, np.float32))
    f = synth.bf16_to_f32
    zc = lambda n: bf(rng.uniform(-0.2, 0.2, n))            # zero-centred norm weights, as stored by Qwen3.6
    mat = lambda r, c: bf(synth.normal_weights(rng, (r, c)) * 2.0)
    q_dim, kv_dim = NH * HD, NKV * HD
    t = {"mtp.pre_fc_norm_hidden.weight": zc(H), "mtp.pre_fc_norm_embedding.weight": zc(H), "mtp.fc.weight": mat(H, 2 * H),
         "mtp.layers.0.input_layernorm.weight": zc(H), "mtp.layers.0.self_attn.q_proj.weight": mat(2 * q_dim, H),
         "mtp.layers.0.self_attn.k_proj.weight": mat(kv_dim, H), "mtp.layers.0.self_attn.v_proj.weight": mat(kv_dim, H),
         "mtp.layers.0.self_attn.q_norm.weight": zc(HD), "mtp.layers.0.self_attn.k_norm.weight": zc(HD),
         "mtp.layers.0.self_attn.o_proj.weight": mat(H, q_dim), "mtp.norm.weight": zc(H)}
    _write_safetensors(os.path.join(src, "model-00002-of-00002.safetensors"), t)
    rs.qwen35_moe_quantize(src, dst, version="3.6", scheme=scheme)
    one = np.float32(1.0)
    nw = lambda k: oracle.f32_to_bf16(f(t[k]) + one)
    pj = lambda k: oracle.quant_int4(f(t[k])) if scheme == "int4" else t[k]
    mw = oracle.MtpWeights(hnorm=nw("mtp.pre_fc_norm_hidden.weight"), enorm=nw("mtp.pre_fc_norm_embedding.weight"),
                           fc=oracle.quant_int4(f(t["mtp.fc.weight"])), attn_norm=nw("mtp.layers.0.input_layernorm.weight"),
                           q_proj=pj("mtp.layers.0.self_attn.q_proj.weight"), k_proj=pj("mtp.layers.0.self_attn.k_proj.weight"),
                           v_proj=pj("mtp.layers.0.self_attn.v_proj.weight"), q_norm=nw("mtp.layers.0.self_attn.q_norm.weight"),
                           k_norm=nw("mtp.layers.0.self_attn.k_norm.weight"), o_proj=pj("mtp.layers.0.self_attn.o_proj.weight"),
                           out_norm=nw("mtp.norm.weight"), num_heads=NH, num_kv_heads=NKV, head_dim=HD, rope_dim=HD // 4,
                           rope_theta=1.0e7)
    layers = _oracle_layers(raw, scheme)
    lm = oracle.quant_int8(head["lm_head"]) if scheme == "bq4" else oracle.quant_int4(head["lm_head"])
    embed = oracle.quant_int4(head["embed"])
    model = rs.Model(dst)
    eng = rs.Engine(model, "Qwen35MoEFusedExp5")
    cache = rs.Cache(model)
    eng.forward(np.array([3, 9], np.int64), cache)       # leaves last_h_pre_norm behind
    h = eng.last_h_pre_norm().copy()
    kc = np.zeros((8, kv_dim), np.float32)
    vc = np.zeros((8, kv_dim), np.float32)
    for pos, tok in enumerate([11, 12]):
        got = eng.mtp_forward(tok)
        want = oracle.mtp_step(mw, layers[1], K, embed, lm, h, tok, pos, kc, vc)
        assert got.shape == (V,) and rel_l2(got, want) < 1e-2
    eng.mtp_reset()
    eng.native.close()


@pytest.mark.parametrize("scheme", ["bq4", "int4"])
def test_forward_runs_attention_when_the_checkpoint_has_it(tmp_path, scheme):
    """A checkpoint with the attention tensors of every layer: quantise, load, and `forward(ids)` is the whole decoder
    (attention half + MoE half per layer, final norm, lm_head), token by token, against the oracle."""
    layers = 4
    adk = dict(num_heads=4, num_kv_heads=2, head_dim=64, rotary_dim=16, rope_theta=1.0e7, lin_num_k_heads=2, lin_num_v_heads=4,
               lin_key_dim=32, lin_value_dim=64, conv_kernel=4, full_attn_interval=4)
    ad = oracle.AttnDims(**adk)
    src, dst = str(tmp_path / "hf"), str(tmp_path / "out")
    raw, head = _hf_checkpoint(src, layers=layers, mtp=0)
    cfg = json.load(open(os.path.join(src, "config.json")))
    cfg["text_config"].update({"num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 64, "linear_num_key_heads": 2,
                               "linear_num_value_heads": 4, "linear_key_head_dim": 32, "linear_value_head_dim": 64,
                               "linear_conv_kernel_dim": 4, "full_attention_interval": 4})
    json.dump(cfg, open(os.path.join(src, "config.json"), "w"))
    rng = np.random.default_rng(23)
    bf = lambda a: synth.to_bf16_rne(np.asarray(a, np.float32))
    f = synth.bf16_to_f32
    zc = lambda n: bf(rng.uniform(-0.2, 0.2, n))
    mat = lambda r, c: bf(synth.normal_weights(rng, (r, c)) * 2.0)
    q_dim, kv_dim = 256, 128
    t, attn = {}, []
    one = np.float32(1.0)
    nw = lambda bits: oracle.f32_to_bf16(f(bits) + one)                       # zero-centred norms are stored as w + 1
    q4 = lambda bits: oracle.quant_int4(f(bits))
    pj = lambda bits: q4(bits) if scheme == "int4" else bits                  # attention projections: bf16 in BQ4
    for l in range(layers):
        p = f"model.language_model.layers.{l}."
        t[p + "input_layernorm.weight"] = zc(H)
        if l == 3:
            w = {"q": mat(2 * q_dim, H), "k": mat(kv_dim, H), "v": mat(kv_dim, H), "o": mat(H, q_dim), "qn": zc(64), "kn": zc(64)}
            t.update({p + "self_attn.q_proj.weight": w["q"], p + "self_attn.k_proj.weight": w["k"], p + "self_attn.v_proj.weight": w["v"],
                      p + "self_attn.o_proj.weight": w["o"], p + "self_attn.q_norm.weight": w["qn"], p + "self_attn.k_norm.weight": w["kn"]})
            attn.append(oracle.FullAttnWeights(input_norm=nw(t[p + "input_layernorm.weight"]), q_proj=pj(w["q"]), k_proj=pj(w["k"]),
                                               v_proj=pj(w["v"]), q_norm=nw(w["qn"]), k_norm=nw(w["kn"]), o_proj=pj(w["o"])))
        else:
            w = {"qkv": mat(ad.conv_dim, H), "z": mat(ad.total_value, H), "b": mat(4, H), "a": mat(4, H),
                 "conv": bf(rng.standard_normal((ad.conv_dim, 1, 4)) * 0.5), "alog": rng.uniform(-1, 1, 4).astype(np.float32),
                 "dt": bf(rng.uniform(-1, 1, 4)), "norm": bf(rng.uniform(0.8, 1.2, 64)), "out": mat(H, ad.total_value)}
            t.update({p + "linear_attn.in_proj_qkv.weight": w["qkv"], p + "linear_attn.in_proj_z.weight": w["z"],
                      p + "linear_attn.in_proj_b.weight": w["b"], p + "linear_attn.in_proj_a.weight": w["a"],
                      p + "linear_attn.conv1d.weight": w["conv"], p + "linear_attn.A_log": w["alog"], p + "linear_attn.dt_bias": w["dt"],
                      p + "linear_attn.norm.weight": w["norm"], p + "linear_attn.out_proj.weight": w["out"]})
            attn.append(oracle.LinAttnWeights(input_norm=nw(t[p + "input_layernorm.weight"]), in_proj_qkv=q4(w["qkv"]), in_proj_z=q4(w["z"]),
                                              in_proj_b=q4(w["b"]), in_proj_a=q4(w["a"]), conv1d=w["conv"].reshape(ad.conv_dim, 4),
                                              a_log=w["alog"], dt_bias=w["dt"], norm=w["norm"], out_proj=q4(w["out"])))
    _write_safetensors(os.path.join(src, "model-00002-of-00002.safetensors"), t)
    rs.qwen35_moe_quantize(src, dst, version="3.6", scheme=scheme)
    moe = _oracle_layers(raw, scheme)
    model = rs.Model(dst)
    eng = rs.Engine(model, "Qwen35MoEFusedExp5")
    cache = rs.Cache(model)
    ids = np.array([5, 17, 3, 99, 42], np.int64)
    got = np.concatenate([eng.forward(ids[:2], cache), eng.forward(ids[2:], cache)])
    emb = oracle.embed_lookup(*oracle.quant_int4(head["embed"]), ids)
    state = oracle.ModelState(ad, layers, 16)
    hid = np.stack([oracle.model_decode_token(attn, moe, ad, state, emb[i], K) for i in range(ids.size)])
    want = _oracle_logits(head, scheme, hid)
    assert got.shape == (5, V) and rel_l2(got, want) < 1e-2 and cache.pos == 5
    assert np.array_equal(got.argmax(axis=1), want.argmax(axis=1))
    # a fresh cache starts a new sequence on the device; a stale position is refused
    again = eng.forward(ids[:1], rs.Cache(model))
    assert rel_l2(again, want[:1]) < 1e-2
    stale = rs.Cache(model)
    stale.pos = 3
    with pytest.raises(RuntimeError, match="carries no state"):
        eng.forward(ids[:1], stale)
    eng.native.close()


def test_top_level_module_alias_runs_a_forward(tmp_path):
    """The reference's Python does `import _moe_infer_rs as _rs` (moe_infer/_core.py:14, pipeline.py:16): with the mirror
    registered under that name, the call sequence of pipeline.py:250-254 and :361-367 runs on the GPU."""
    import sys
    sys.modules["_moe_infer_rs"] = rs
    import _moe_infer_rs as _rs
    src, dst = str(tmp_path / "hf"), str(tmp_path / "out")
    _hf_checkpoint(src, layers=1, mtp=0)
    _rs.qwen35_moe_quantize(src, dst, version="3.6", scheme="bq4")
    model = _rs.Model(dst)
    engine = _rs.Engine(model, "Qwen35MoEFusedExp2", 0, expert_cache_count=0)
    cache = _rs.Cache(model)
    ids = np.array([1, 2, 3], np.int64)
    emb = engine.embed_lookup(ids)
    logits = engine.forward_hidden(emb, cache)
    assert logits.shape == (3, V) and np.isfinite(logits).all()
    again = engine.forward(ids, cache)
    assert np.allclose(again, logits, rtol=1e-5, atol=1e-6) and cache.pos == 6
    cache.reset()
    assert isinstance(engine.telemetry(), dict)
    engine.native.close()
