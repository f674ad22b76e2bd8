"""ctypes front end of the CPU oracle (``moe_oracle.c``).  TEST INFRASTRUCTURE ONLY.

Only the test-suite, the smoke check and the CPU-baseline leg of the benchmark
may import this package; the product (``moe_infer_b200``) never does.

Parity status: bf16 rounding, dequantiser and blob layout are pinned against the
reference's own Python by the fixtures in ``tests/golden``; the packed nibbles of
``quant_int4`` are pinned by source text only (the reference ships no
known-answer vector for them).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from dataclasses import dataclass
from typing import Optional, Tuple

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libmoe_oracle.so")
GROUP = 64


def build(force: bool = False) -> str:
    """Compile ``moe_oracle.c`` with gcc (see the Makefile) and return the .so path."""
    src = os.path.join(_HERE, "moe_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-s", "-C", _HERE, "libmoe_oracle.so"])
    return _SO


_lib = None


class _Layout(C.Structure):
    _fields_ = [(n, C.c_int64) for n in
                ("gate_w", "gate_s", "gate_b", "up_w", "up_s", "up_b",
                 "down_w", "down_s", "down_b", "expert_size")]


class _Dims(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("hidden", "inter", "shared_inter", "num_experts", "top_k")]


class _Q4(C.Structure):
    _fields_ = [("w", C.c_void_p), ("s", C.c_void_p), ("b", C.c_void_p)]


class _Layer(C.Structure):
    _fields_ = [("post_norm_w", C.c_void_p), ("router_bf16", C.c_void_p), ("router_q4", _Q4),
                ("sh_gate", _Q4), ("sh_up", _Q4), ("sh_down", _Q4), ("sgate", _Q4),
                ("experts", C.c_void_p)]


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            build()
        _lib = C.CDLL(_SO)
        _lib.orc_f32_to_bf16.restype = C.c_uint16
        _lib.orc_f32_to_bf16.argtypes = [C.c_float]
        _lib.orc_sigmoid.restype = C.c_float
        _lib.orc_sigmoid.argtypes = [C.c_float]
        _lib.orc_num_threads.restype = C.c_int
    return _lib


def _p(a: Optional[np.ndarray]):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _c(a, dtype):
    a = np.ascontiguousarray(a, dtype=dtype)
    return a


# ─── bf16 ────────────────────────────────────────────────────────────────────

def f32_to_bf16(x: np.ndarray) -> np.ndarray:
    x = _c(x, np.float32)
    out = np.empty(x.shape, np.uint16)
    lib().orc_f32_to_bf16_n(_p(x), _p(out), C.c_size_t(x.size))
    return out


def bf16_to_f32(x: np.ndarray) -> np.ndarray:
    x = _c(x, np.uint16)
    return (x.astype(np.uint32) << 16).view(np.float32)


# ─── codec ───────────────────────────────────────────────────────────────────

def quant_int4(vals: np.ndarray) -> Tuple[np.ndarray, np.ndarray, np.ndarray]:
    """f32 [out, in] -> (u32 [out, in/8], bf16 scales [out, in/64], bf16 biases)."""
    vals = _c(vals, np.float32)
    out_dim, in_dim = vals.shape
    assert in_dim % GROUP == 0
    w = np.empty((out_dim, in_dim // 8), np.uint32)
    s = np.empty((out_dim, in_dim // GROUP), np.uint16)
    b = np.empty((out_dim, in_dim // GROUP), np.uint16)
    lib().orc_quant_int4(_p(vals), out_dim, in_dim, _p(w), _p(s), _p(b))
    return w, s, b


def quant_int4_bf16(vals_u16: np.ndarray):
    """bf16 bit patterns [out, in] widened exactly to f32, then ``quant_int4``."""
    return quant_int4(bf16_to_f32(vals_u16))


def dequant_int4(w, s, b) -> np.ndarray:
    w = _c(w, np.uint32)
    s = _c(s, np.uint16)
    b = _c(b, np.uint16)
    out_dim, wpr = w.shape
    in_dim = wpr * 8
    out = np.empty((out_dim, in_dim), np.float32)
    lib().orc_dequant_int4(_p(w), _p(s), _p(b), out_dim, in_dim, _p(out))
    return out


def expert_layout(hd: int, mi: int, gs: int = GROUP) -> dict:
    L = _Layout()
    lib().orc_expert_layout(hd, mi, gs, C.byref(L))
    return {n: getattr(L, n) for n, _ in _Layout._fields_}


def pack_experts_layer(gate_up: np.ndarray, down: np.ndarray) -> np.ndarray:
    """gate_up f32 [E, 2I, H], down f32 [E, H, I] -> uint8 blob [E * expert_size]."""
    gate_up = _c(gate_up, np.float32)
    down = _c(down, np.float32)
    E, two_i, H = gate_up.shape
    inter = two_i // 2
    assert down.shape == (E, H, inter)
    size = expert_layout(H, inter)["expert_size"]
    blob = np.empty(E * size, np.uint8)
    lib().orc_pack_experts_layer(_p(gate_up), _p(down), E, inter, H, _p(blob))
    return blob


# ─── matvec and small math ───────────────────────────────────────────────────

def matvec_int4(w, s, b, x, threads: int = 1) -> np.ndarray:
    w = _c(w, np.uint32)
    s = _c(s, np.uint16)
    b = _c(b, np.uint16)
    x = _c(x, np.float32)
    out_dim, wpr = w.shape
    out = np.empty(out_dim, np.float32)
    fn = lib().orc_matvec_int4_mt if threads > 1 else lib().orc_matvec_int4
    fn(_p(w), _p(s), _p(b), _p(x), _p(out), out_dim, wpr * 8)
    return out


def matvec_bf16(w_u16, x) -> np.ndarray:
    w_u16 = _c(w_u16, np.uint16)
    x = _c(x, np.float32)
    out = np.empty(w_u16.shape[0], np.float32)
    lib().orc_matvec_bf16(_p(w_u16), _p(x), _p(out), w_u16.shape[0], w_u16.shape[1])
    return out


def route_experts(scores: np.ndarray, k: int):
    """Returns (indices int32 [k] in heap order, weights f32 [k], probabilities [E])."""
    probs = _c(scores, np.float32).copy()
    idx = np.zeros(k, np.int32)
    wts = np.zeros(k, np.float32)
    lib().orc_route_experts(_p(probs), probs.size, k, _p(idx), _p(wts))
    return idx, wts, probs


def swiglu(gate, up) -> np.ndarray:
    gate = _c(gate, np.float32)
    up = _c(up, np.float32)
    out = np.empty_like(gate)
    lib().orc_swiglu(_p(gate), _p(up), _p(out), gate.size)
    return out


def rms_norm_bf16(x, w_u16, eps: float = 1e-6) -> np.ndarray:
    x = _c(x, np.float32)
    w_u16 = _c(w_u16, np.uint16)
    out = np.empty_like(x)
    lib().orc_rms_norm_bf16(_p(x), _p(w_u16), _p(out), x.size, C.c_float(eps))
    return out


def sigmoid(x: float) -> float:
    return float(lib().orc_sigmoid(C.c_float(x)))


def num_threads() -> int:
    return int(lib().orc_num_threads())


# ─── one MoE block ───────────────────────────────────────────────────────────

Q4 = Tuple[np.ndarray, np.ndarray, np.ndarray]


@dataclass
class LayerWeights:
    """Host copy of one MoE block's tensors in the reference's byte layout."""
    hidden: int
    inter: int
    shared_inter: int
    num_experts: int
    post_norm_w: np.ndarray            # bf16 bits [H]
    router_bf16: Optional[np.ndarray]  # bf16 bits [E, H] (BQ4 scheme) or None
    router_q4: Optional[Q4]            # INT4 scheme
    sh_gate: Q4
    sh_up: Q4
    sh_down: Q4
    sgate: Q4
    experts: np.ndarray                # uint8 [E * expert_size]


def _q4(t: Optional[Q4]) -> _Q4:
    if t is None:
        return _Q4(None, None, None)
    return _Q4(_p(t[0]), _p(t[1]), _p(t[2]))


def moe_layer(lw: LayerWeights, h_mid: np.ndarray, top_k: int, *, logit_bias=None,
              forced_idx=None, threads: int = 1):
    """h_mid f32 [n, H] -> (h_out [n, H], idx int32 [n, k] heap order, weights f32 [n, k])."""
    h_mid = _c(h_mid, np.float32).reshape(-1, lw.hidden)
    n = h_mid.shape[0]
    d = _Dims(lw.hidden, lw.inter, lw.shared_inter, lw.num_experts, top_k)
    ly = _Layer(_p(lw.post_norm_w), _p(lw.router_bf16), _q4(lw.router_q4), _q4(lw.sh_gate),
                _q4(lw.sh_up), _q4(lw.sh_down), _q4(lw.sgate), _p(lw.experts))
    h_out = np.empty_like(h_mid)
    idx = np.empty((n, top_k), np.int32)
    wts = np.empty((n, top_k), np.float32)
    lb = None if logit_bias is None else _c(logit_bias, np.float32)
    fi = None if forced_idx is None else _c(forced_idx, np.int32)
    lib().orc_moe_layer(C.byref(d), C.byref(ly), _p(h_mid), n, _p(h_out), _p(idx), _p(wts),
                        _p(lb), _p(fi), threads)
    return h_out, idx, wts


def moe_layer_decode_mt(lw: LayerWeights, h_mid: np.ndarray, top_k: int):
    """One token, matvec rows split over all OpenMP threads; same result as ``moe_layer``."""
    h_mid = _c(h_mid, np.float32).reshape(lw.hidden)
    d = _Dims(lw.hidden, lw.inter, lw.shared_inter, lw.num_experts, top_k)
    ly = _Layer(_p(lw.post_norm_w), _p(lw.router_bf16), _q4(lw.router_q4), _q4(lw.sh_gate),
                _q4(lw.sh_up), _q4(lw.sh_down), _q4(lw.sgate), _p(lw.experts))
    h_out = np.empty_like(h_mid)
    idx = np.empty(top_k, np.int32)
    wts = np.empty(top_k, np.float32)
    lib().orc_moe_layer_decode_mt(C.byref(d), C.byref(ly), _p(h_mid), _p(h_out), _p(idx), _p(wts))
    return h_out, idx, wts


def moe_stack(layers, h: np.ndarray, top_k: int, threads: int = 1) -> np.ndarray:
    """Residual stack with attention omitted: h <- moe_layer_l(h) for each layer."""
    h = _c(h, np.float32).reshape(-1, layers[0].hidden)
    for lw in layers:
        h, _, _ = moe_layer(lw, h, top_k, threads=threads)
    return h


# ─── the model head: embedding rows, final norm, lm_head ─────────────────────

def quant_int8(vals: np.ndarray):
    """f32 [out, in] -> (int8 [out, in], f32 scales [out]); reference src/dtype.rs:164-179."""
    vals = _c(vals, np.float32)
    out_dim, in_dim = vals.shape
    q = np.empty((out_dim, in_dim), np.int8)
    s = np.empty(out_dim, np.float32)
    lib().orc_quant_int8(_p(vals), out_dim, in_dim, _p(q), _p(s))
    return q, s


def matvec_int8(w, scales, x, threads: int = 1) -> np.ndarray:
    w = _c(w, np.int8)
    scales = _c(scales, np.float32)
    x = _c(x, np.float32)
    out = np.empty(w.shape[0], np.float32)
    lib().orc_matvec_int8(_p(w), _p(scales), _p(x), _p(out), w.shape[0], w.shape[1], threads)
    return out


def embed_lookup(w, s, b, token_ids) -> np.ndarray:
    """Rows of a 4-bit table; reference src/math_util.rs:205-236."""
    w = _c(w, np.uint32)
    s = _c(s, np.uint16)
    b = _c(b, np.uint16)
    ids = np.ascontiguousarray(token_ids, np.int64).reshape(-1)
    hidden = w.shape[1] * 8
    out = np.empty((ids.size, hidden), np.float32)
    for i, t in enumerate(ids):
        lib().orc_embed_lookup(_p(w), _p(s), _p(b), C.c_int64(int(t)), hidden, _p(out[i]))
    return out


def final_norm(h, w_u16, eps: float = 1e-6) -> np.ndarray:
    """Reference src/math_util.rs:240-247, on a copy."""
    h = _c(h, np.float32).copy()
    w_u16 = _c(w_u16, np.uint16)
    flat = h.reshape(-1, w_u16.size)
    for i in range(flat.shape[0]):
        lib().orc_final_norm(_p(flat[i]), _p(w_u16), w_u16.size, C.c_float(eps))
    return h


# ── the MTP block (reference src/engine/qwen35_moe/mtp.rs:58-225) ─────────────

def rope(x, num_heads: int, head_dim: int, rope_dim: int, pos: int, theta: float) -> np.ndarray:
    x = _c(x, np.float32)
    out = np.empty_like(x)
    lib().orc_rope(_p(x), _p(out), num_heads, head_dim, rope_dim, pos, C.c_float(theta))
    return out


def attention(q, k_cache, v_cache, num_heads: int, num_kv_heads: int, head_dim: int, seq_len: int) -> np.ndarray:
    q = _c(q, np.float32)
    k_cache = _c(k_cache, np.float32)
    v_cache = _c(v_cache, np.float32)
    out = np.empty(num_heads * head_dim, np.float32)
    lib().orc_attention(_p(q), _p(k_cache), _p(v_cache), num_heads, num_kv_heads, head_dim, seq_len,
                        C.c_float(1.0 / np.sqrt(np.float32(head_dim))), _p(out))
    return out


class MtpWeights:
    """Tensors of the MTP block besides its MoE half.  Norm weights are bf16 bit patterns; a projection is either
    bf16 bit patterns [out, in] or a 4-bit triple (w, s, b)."""

    def __init__(self, *, hnorm, enorm, fc, attn_norm, q_proj, k_proj, v_proj, q_norm, k_norm, o_proj, out_norm,
                 num_heads, num_kv_heads, head_dim, rope_dim, rope_theta):
        self.__dict__.update(locals())


def _project(w, x) -> np.ndarray:
    return matvec_int4(*w, x) if isinstance(w, tuple) else matvec_bf16(w, x)


def mtp_step(mw: "MtpWeights", moe: "LayerWeights", top_k: int, embed_q4, lm_head, h, token_id: int, pos: int,
             k_cache: np.ndarray, v_cache: np.ndarray) -> np.ndarray:
    """(h, token) -> logits; appends this position's K and V to the caches (mtp.rs:85-225)."""
    H = h.size
    tok = embed_lookup(*embed_q4, [token_id])[0]
    concat = np.concatenate([final_norm(tok, mw.enorm), final_norm(h, mw.hnorm)])  # embedding first (mtp.rs:103-105)
    cur = matvec_int4(*mw.fc, concat)
    x = final_norm(cur, mw.attn_norm)
    q_dim, kv_dim = mw.num_heads * mw.head_dim, mw.num_kv_heads * mw.head_dim
    q = _project(mw.q_proj, x)
    k = _project(mw.k_proj, x)
    v = _project(mw.v_proj, x)
    q_head, gate = q[:q_dim], q[q_dim:]
    qn = final_norm(q_head.reshape(mw.num_heads, mw.head_dim), mw.q_norm).reshape(-1)   # per head (mtp.rs:268-276)
    kn = final_norm(k.reshape(mw.num_kv_heads, mw.head_dim), mw.k_norm).reshape(-1)
    qr = rope(qn, mw.num_heads, mw.head_dim, mw.rope_dim, pos, mw.rope_theta)
    kr = rope(kn, mw.num_kv_heads, mw.head_dim, mw.rope_dim, pos, mw.rope_theta)
    k_cache[pos] = kr
    v_cache[pos] = v
    att = attention(qr, k_cache, v_cache, mw.num_heads, mw.num_kv_heads, mw.head_dim, pos + 1)
    gated = (att * (np.float32(1.0) / (np.float32(1.0) + np.exp(-gate)))).astype(np.float32)
    cur = (_project(mw.o_proj, gated) + cur).astype(np.float32)
    cur, _, _ = moe_layer(moe, cur, top_k)                                   # post-attention norm, MoE, residual
    out = final_norm(cur[0], mw.out_norm)
    if isinstance(lm_head, tuple) and len(lm_head) == 2:
        return matvec_int8(lm_head[0], lm_head[1], out)
    return matvec_int4(*lm_head, out)


# ── the main model's attention layers (reference src/engine/qwen35_moe/cpu.rs:87-347) ──────────────────────────

class AttnDims:
    def __init__(self, *, num_heads, num_kv_heads, head_dim, rotary_dim, rope_theta, lin_num_k_heads, lin_num_v_heads,
                 lin_key_dim, lin_value_dim, conv_kernel=4, full_attn_interval=4):
        self.__dict__.update(locals())

    @property
    def total_key(self):
        return self.lin_num_k_heads * self.lin_key_dim

    @property
    def total_value(self):
        return self.lin_num_v_heads * self.lin_value_dim

    @property
    def conv_dim(self):
        return 2 * self.total_key + self.total_value


class FullAttnWeights:
    """input_norm / q_norm / k_norm: bf16 bits; projections: bf16 bits [out, in] or 4-bit triples."""

    def __init__(self, *, input_norm, q_proj, k_proj, v_proj, q_norm, k_norm, o_proj):
        self.__dict__.update(locals())


class LinAttnWeights:
    """input_norm, dt_bias, norm: bf16 bits; conv1d: bf16 bits [channels, kernel]; a_log: f32; projections as above."""

    def __init__(self, *, input_norm, in_proj_qkv, in_proj_z, in_proj_b, in_proj_a, conv1d, a_log, dt_bias, norm, out_proj):
        self.__dict__.update(locals())


def full_attn_block(w: FullAttnWeights, ad: AttnDims, hidden, pos: int, k_cache, v_cache) -> np.ndarray:
    """pre_expert_full up to the residual (cpu.rs:87-183): returns h_mid = o_proj(...) + hidden."""
    hidden = _c(hidden, np.float32)
    nh, nkv, hd = ad.num_heads, ad.num_kv_heads, ad.head_dim
    x = final_norm(hidden, w.input_norm)
    q = _project(w.q_proj, x)          # [head, gate] per head
    k = _project(w.k_proj, x)
    v = _project(w.v_proj, x)
    q_out = np.empty(nh * hd, np.float32)
    k_out = np.empty(nkv * hd, np.float32)
    lib().orc_head_norm_rope_split(_p(q), 2 * hd, _p(_c(w.q_norm, np.uint16)), _p(q_out), nh, hd, ad.rotary_dim,
                                   C.c_float(ad.rope_theta), pos, C.c_float(1e-6))
    lib().orc_head_norm_rope_split(_p(k), hd, _p(_c(w.k_norm, np.uint16)), _p(k_out), nkv, hd, ad.rotary_dim,
                                   C.c_float(ad.rope_theta), pos, C.c_float(1e-6))
    gate = q.reshape(nh, 2 * hd)[:, hd:].reshape(-1)
    k_cache[pos] = k_out
    v_cache[pos] = v
    att = attention(q_out, k_cache, v_cache, nh, nkv, hd, pos + 1)
    gated = (att * (np.float32(1.0) / (np.float32(1.0) + np.exp(-gate)))).astype(np.float32)
    return (_project(w.o_proj, gated) + hidden).astype(np.float32)


def linear_attn_block(w: LinAttnWeights, ad: AttnDims, hidden, conv_state, ssm_state) -> np.ndarray:
    """pre_expert_linear up to the residual (cpu.rs:218-347); conv_state [kernel - 1, channels] and
    ssm_state [v_heads, value_dim, key_dim] are updated in place."""
    hidden = _c(hidden, np.float32)
    x = final_norm(hidden, w.input_norm)
    qkv = _project(w.in_proj_qkv, x)
    z = _project(w.in_proj_z, x)
    beta = _project(w.in_proj_b, x)
    alpha = _project(w.in_proj_a, x)
    conv_out = np.empty_like(qkv)
    conv_w = _c(w.conv1d, np.uint16)
    lib().orc_conv1d_step(_p(conv_state), _p(qkv), _p(conv_w), _p(conv_out), ad.conv_dim, ad.conv_kernel)
    lib().orc_lin_qk_norm(_p(conv_out), ad.total_key, ad.lin_num_k_heads, ad.lin_key_dim)
    out = np.empty(ad.total_value, np.float32)
    a_log = _c(w.a_log, np.float32)
    dt_bias = _c(w.dt_bias, np.uint16)
    qn, kn, vv = conv_out[:ad.total_key], conv_out[ad.total_key:2 * ad.total_key], conv_out[2 * ad.total_key:]
    lib().orc_delta_step(_p(ssm_state), _p(_c(qn, np.float32)), _p(_c(kn, np.float32)), _p(_c(vv, np.float32)), _p(alpha), _p(beta),
                         _p(a_log), _p(dt_bias), _p(out), ad.lin_num_v_heads, ad.lin_num_v_heads // ad.lin_num_k_heads,
                         ad.lin_key_dim, ad.lin_value_dim)
    normed = np.empty_like(out)
    lib().orc_gated_rms_norm(_p(out), _p(z), _p(_c(w.norm, np.uint16)), _p(normed), ad.lin_num_v_heads, ad.lin_value_dim,
                             C.c_float(1e-6))
    return (_project(w.out_proj, normed) + hidden).astype(np.float32)


class ModelState:
    """Per-layer caches of a decode: KV for the full-attention layers, conv + recurrence state for the others."""

    def __init__(self, ad: AttnDims, num_layers: int, max_seq: int):
        self.pos = 0
        self.kv, self.lin = {}, {}
        for l in range(num_layers):
            if (l + 1) % ad.full_attn_interval == 0:
                self.kv[l] = (np.zeros((max_seq, ad.num_kv_heads * ad.head_dim), np.float32),
                              np.zeros((max_seq, ad.num_kv_heads * ad.head_dim), np.float32))
            else:
                self.lin[l] = (np.zeros((ad.conv_kernel - 1, ad.conv_dim), np.float32),
                               np.zeros((ad.lin_num_v_heads, ad.lin_value_dim, ad.lin_key_dim), np.float32))


def model_decode_token(attn_layers, moe_layers, ad: AttnDims, state: ModelState, h, top_k: int) -> np.ndarray:
    """One token through every layer: attention half (full or linear by position in the stack), then the MoE half
    (cpu.rs:398-483); advances the state's position."""
    h = _c(h, np.float32)
    for l, (aw, mw) in enumerate(zip(attn_layers, moe_layers)):
        if l in state.kv:
            h_mid = full_attn_block(aw, ad, h, state.pos, *state.kv[l])
        else:
            h_mid = linear_attn_block(aw, ad, h, *state.lin[l])
        h = moe_layer(mw, h_mid, top_k)[0][0]
    state.pos += 1
    return h
