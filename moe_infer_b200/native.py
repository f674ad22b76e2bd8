"""Thin object wrapper over the C ABI handle (``moe_engine_t``).

Every method is one C-ABI call (plus numpy buffer management); the arithmetic
runs in the CUDA library.  Host arrays go through the ``*_host`` entry points,
``DevBuf`` objects through the ``*_dev`` ones.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional, Sequence, Tuple

import numpy as np

from . import _lib as L


@dataclass
class Dims:
    hidden: int = 2048
    inter: int = 512
    shared_inter: int = 512
    num_experts: int = 256
    top_k: int = 8
    num_layers: int = 40
    num_mtp_layers: int = 0
    group: int = 64
    vocab: int = 248320
    scheme: int = L.SCHEME_BQ4

    def to_c(self) -> L.MoeDims:
        return L.MoeDims(self.hidden, self.inter, self.shared_inter, self.num_experts, self.top_k,
                         self.num_layers, self.num_mtp_layers, self.group, self.vocab, self.scheme)


class DevBuf:
    """A device allocation owned by Python (freed on ``free()`` or engine close)."""

    def __init__(self, eng: "NativeEngine", nbytes: int):
        p = C.c_void_p()
        L.check(eng.lib.moe_dev_alloc(eng.h, nbytes, C.byref(p)))
        self.eng, self.ptr, self.nbytes = eng, p.value, nbytes

    def upload(self, a: np.ndarray, offset: int = 0) -> "DevBuf":
        a = np.ascontiguousarray(a)
        assert offset + a.nbytes <= self.nbytes
        L.check(self.eng.lib.moe_dev_upload(self.eng.h, C.c_void_p(self.ptr + offset), L.ptr(a), a.nbytes))
        return self

    def download(self, dtype, shape, offset: int = 0) -> np.ndarray:
        out = np.empty(shape, dtype)
        assert offset + out.nbytes <= self.nbytes
        L.check(self.eng.lib.moe_dev_download(self.eng.h, L.ptr(out), C.c_void_p(self.ptr + offset), out.nbytes))
        return out

    def at(self, offset: int = 0) -> C.c_void_p:
        return C.c_void_p(self.ptr + offset)

    def free(self) -> None:
        if self.ptr:
            L.check(self.eng.lib.moe_dev_free(self.eng.h, C.c_void_p(self.ptr)))
            self.ptr = 0


class PinnedArray:
    """A numpy view over page-locked host memory from ``moe_host_alloc_pinned``."""

    def __init__(self, shape, dtype):
        self.lib = L.load()
        n = int(np.prod(shape)) * np.dtype(dtype).itemsize
        p = C.c_void_p()
        L.check(self.lib.moe_host_alloc_pinned(max(n, 1), C.byref(p)))
        self.ptr = p.value
        buf = (C.c_char * max(n, 1)).from_address(self.ptr)
        self.array = np.frombuffer(buf, dtype=dtype, count=int(np.prod(shape))).reshape(shape)

    def free(self) -> None:
        if self.ptr:
            self.array = None
            L.check(self.lib.moe_host_free_pinned(C.c_void_p(self.ptr)))
            self.ptr = 0


Q4 = Tuple[np.ndarray, np.ndarray, np.ndarray]


class ModelSnapshot:
    """Device-side copy of what a speculative decode rolls back to (moe_model_snapshot); freed with the object."""

    def __init__(self, eng: "NativeEngine", handle):
        self.eng, self.handle = eng, handle

    def free(self) -> None:
        if self.handle is not None and self.eng.h is not None:
            self.eng.lib.moe_model_snapshot_free(self.handle)
        self.handle = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class NativeEngine:
    def __init__(self, dims: Dims, device: int = 0):
        self.lib = L.load()
        self.dims = dims
        h = C.c_void_p()
        cd = dims.to_c()
        L.check(self.lib.moe_engine_create(C.byref(cd), device, C.byref(h)))
        self.h = h
        self.layout = L.expert_layout(dims.hidden, dims.inter, dims.group)

    def close(self) -> None:
        if getattr(self, "h", None):
            self.lib.moe_engine_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def sync(self) -> None:
        L.check(self.lib.moe_engine_sync(self.h))

    # ── store ────────────────────────────────────────────────────────────
    def load_layer(self, layer: int, blob: np.ndarray) -> None:
        blob = np.ascontiguousarray(blob).view(np.uint8).reshape(-1)
        L.check(self.lib.moe_store_load_layer(self.h, layer, L.ptr(blob), blob.nbytes))

    def layer_dev(self, layer: int) -> int:
        p = C.c_void_p()
        L.check(self.lib.moe_store_layer_dev(self.h, layer, C.byref(p)))
        return p.value

    def mark_loaded(self, layer: int) -> None:
        L.check(self.lib.moe_store_mark_loaded(self.h, layer))

    def load_bf16(self, layer: int, role: int, w: np.ndarray) -> None:
        w = np.ascontiguousarray(w, np.uint16)
        L.check(self.lib.moe_store_load_tensor(self.h, layer, role, L.ptr(w), None, None, L.DT_BF16))

    def load_q4(self, layer: int, role: int, t: Q4) -> None:
        w, s, b = (np.ascontiguousarray(t[0], np.uint32), np.ascontiguousarray(t[1], np.uint16),
                   np.ascontiguousarray(t[2], np.uint16))
        L.check(self.lib.moe_store_load_tensor(self.h, layer, role, L.ptr(w), L.ptr(s), L.ptr(b), L.DT_INT4))

    def resident_bytes(self) -> int:
        n = C.c_size_t()
        L.check(self.lib.moe_store_bytes(self.h, C.byref(n)))
        return n.value

    # ── packer ───────────────────────────────────────────────────────────
    @staticmethod
    def _src(a: np.ndarray):
        if a.dtype == np.float32:
            return np.ascontiguousarray(a), L.DT_F32
        if a.dtype == np.uint16:
            return np.ascontiguousarray(a), L.DT_BF16
        raise ValueError("source must be float32 or bf16 bit patterns (uint16)")

    def pack_int4(self, src: np.ndarray) -> Q4:
        src, dt = self._src(src)
        rows, cols = src.shape
        if cols <= 0 or cols % 64:
            raise ValueError(f"cols ({cols}) must be a positive multiple of 64")
        w = np.empty((rows, cols // 8), np.uint32)
        s = np.empty((rows, cols // 64), np.uint16)
        b = np.empty((rows, cols // 64), np.uint16)
        L.check(self.lib.moe_pack_int4_host(self.h, L.ptr(src), dt, rows, cols, L.ptr(w), L.ptr(s), L.ptr(b)))
        return w, s, b

    def pack_int8(self, src: np.ndarray):
        """f32 / bf16 [rows, cols] -> (int8 [rows, cols], f32 scales [rows]): the INT8 lm_head codec."""
        src, dt = self._src(src)
        rows, cols = src.shape
        q = np.empty((rows, cols), np.int8)
        s = np.empty(rows, np.float32)
        L.check(self.lib.moe_pack_int8_host(self.h, L.ptr(src), dt, rows, cols, L.ptr(q), L.ptr(s)))
        return q, s

    def pack_experts(self, gate_up: np.ndarray, down: np.ndarray) -> np.ndarray:
        gate_up, dt = self._src(gate_up)
        down, dt2 = self._src(down)
        assert dt == dt2
        n = gate_up.shape[0]
        d = self.dims
        assert gate_up.shape == (n, 2 * d.inter, d.hidden) and down.shape == (n, d.hidden, d.inter)
        blob = np.empty(n * self.layout["expert_size"], np.uint8)
        L.check(self.lib.moe_pack_experts_host(self.h, L.ptr(gate_up), L.ptr(down), dt, n, L.ptr(blob)))
        return blob

    def pack_experts_dev(self, gate_up_dev: int, down_dev: int, dtype: int, n_experts: int, blob_dev: int) -> None:
        L.check(self.lib.moe_pack_experts_dev(self.h, C.c_void_p(gate_up_dev), C.c_void_p(down_dev), dtype,
                                              n_experts, C.c_void_p(blob_dev)))

    def pack_int4_dev(self, src_dev: int, dtype: int, rows: int, cols: int, w_dev: int, s_dev: int, b_dev: int):
        L.check(self.lib.moe_pack_int4_dev(self.h, C.c_void_p(src_dev), dtype, rows, cols, C.c_void_p(w_dev),
                                           C.c_void_p(s_dev), C.c_void_p(b_dev)))

    # ── matvec ───────────────────────────────────────────────────────────
    def matvec_int4(self, w: np.ndarray, s: np.ndarray, b: np.ndarray, x: np.ndarray) -> np.ndarray:
        w = np.ascontiguousarray(w, np.uint32)
        s = np.ascontiguousarray(s, np.uint16)
        b = np.ascontiguousarray(b, np.uint16)
        x = np.ascontiguousarray(x, np.float32)
        rows, cols = w.shape[0], w.shape[1] * 8
        y = np.empty(rows, np.float32)
        L.check(self.lib.moe_matvec_int4_host(self.h, L.ptr(w), L.ptr(s), L.ptr(b), L.ptr(x), L.ptr(y), rows, cols))
        return y

    def matvec_int4_dev(self, w: int, s: int, b: int, x: int, y: int, rows: int, cols: int) -> None:
        L.check(self.lib.moe_matvec_int4_dev(self.h, C.c_void_p(w), C.c_void_p(s), C.c_void_p(b), C.c_void_p(x),
                                             C.c_void_p(y), rows, cols))

    # ── MoE block and stack ──────────────────────────────────────────────
    def layer_forward(self, layer: int, h_in: np.ndarray, *, logit_bias=None, forced_idx=None):
        d = self.dims
        h_in = np.ascontiguousarray(h_in, np.float32).reshape(-1, d.hidden)
        n = h_in.shape[0]
        h_out = np.empty_like(h_in)
        idx = np.empty((n, d.top_k), np.int32)
        wts = np.empty((n, d.top_k), np.float32)
        lb = None if logit_bias is None else np.ascontiguousarray(logit_bias, np.float32)
        fi = None if forced_idx is None else np.ascontiguousarray(forced_idx, np.int32)
        L.check(self.lib.moe_layer_forward_host(self.h, layer, L.ptr(h_in), n, L.ptr(h_out), L.ptr(lb), L.ptr(fi),
                                                L.ptr(idx), L.ptr(wts)))
        return h_out, idx, wts

    def forward_hidden(self, emb: np.ndarray, *, batched: bool = False, mtp: bool = False, check=None,
                       out: Optional[np.ndarray] = None) -> np.ndarray:
        d = self.dims
        emb = np.ascontiguousarray(emb, np.float32).reshape(-1, d.hidden)
        n = emb.shape[0]
        if out is None:
            out = np.empty_like(emb)
        cb = L.CHECK_FN(lambda _ctx: 1 if check() else 0) if check else C.cast(None, L.CHECK_FN)
        L.check(self.lib.moe_forward_hidden_host(self.h, L.ptr(emb), n, int(batched), int(mtp), cb, None, L.ptr(out)))
        return out

    def forward_hidden_dev(self, emb_dev: int, n: int, batched: bool, out_dev: int) -> None:
        L.check(self.lib.moe_forward_hidden_dev(self.h, C.c_void_p(emb_dev), n, int(batched), C.c_void_p(out_dev)))

    def layer_forward_dev(self, layer: int, h_in: int, n: int, h_out: int, out_idx: int = 0, out_w: int = 0,
                          logit_bias: int = 0, forced_idx: int = 0) -> None:
        L.check(self.lib.moe_layer_forward_dev(self.h, layer, C.c_void_p(h_in), n, C.c_void_p(h_out),
                                               C.c_void_p(logit_bias or None), C.c_void_p(forced_idx or None),
                                               C.c_void_p(out_idx or None), C.c_void_p(out_w or None)))

    # ── the model head ───────────────────────────────────────────────────
    def load_embed(self, t: Q4) -> None:
        w, s, b = (np.ascontiguousarray(t[0], np.uint32), np.ascontiguousarray(t[1], np.uint16),
                   np.ascontiguousarray(t[2], np.uint16))
        L.check(self.lib.moe_head_load_tensor(self.h, L.H_EMBED, L.ptr(w), L.ptr(s), L.ptr(b), L.DT_INT4))

    def load_final_norm(self, w: np.ndarray) -> None:
        w = np.ascontiguousarray(w, np.uint16)
        L.check(self.lib.moe_head_load_tensor(self.h, L.H_FINAL_NORM, L.ptr(w), None, None, L.DT_BF16))

    def load_lm_head_int8(self, q: np.ndarray, scales: np.ndarray) -> None:
        q = np.ascontiguousarray(q).view(np.int8)
        scales = np.ascontiguousarray(scales, np.float32)
        L.check(self.lib.moe_head_load_tensor(self.h, L.H_LM_HEAD, L.ptr(q), L.ptr(scales), None, L.DT_INT8))

    def load_lm_head_q4(self, t: Q4) -> None:
        w, s, b = (np.ascontiguousarray(t[0], np.uint32), np.ascontiguousarray(t[1], np.uint16),
                   np.ascontiguousarray(t[2], np.uint16))
        L.check(self.lib.moe_head_load_tensor(self.h, L.H_LM_HEAD, L.ptr(w), L.ptr(s), L.ptr(b), L.DT_INT4))

    def embed_lookup(self, ids: np.ndarray) -> np.ndarray:
        ids = np.ascontiguousarray(ids, np.int64).reshape(-1)
        out = np.empty((ids.size, self.dims.hidden), np.float32)
        L.check(self.lib.moe_embed_lookup_host(self.h, L.ptr(ids), ids.size, L.ptr(out)))
        return out

    def logits(self, hidden: np.ndarray) -> np.ndarray:
        hidden = np.ascontiguousarray(hidden, np.float32).reshape(-1, self.dims.hidden)
        out = np.empty((hidden.shape[0], self.dims.vocab), np.float32)
        L.check(self.lib.moe_logits_host(self.h, L.ptr(hidden), hidden.shape[0], L.ptr(out)))
        return out

    def forward(self, ids: np.ndarray, *, batched: bool = False, mtp: bool = False, check=None) -> np.ndarray:
        """Token ids -> logits [n, vocab]: embedding rows, the layer stack, final norm, lm_head."""
        ids = np.ascontiguousarray(ids, np.int64).reshape(-1)
        out = np.empty((ids.size, self.dims.vocab), np.float32)
        cb = L.CHECK_FN(lambda _ctx: 1 if check() else 0) if check else C.cast(None, L.CHECK_FN)
        L.check(self.lib.moe_forward_host(self.h, L.ptr(ids), ids.size, int(batched), int(mtp), cb, None, L.ptr(out)))
        return out

    def last_h_pre_norm(self) -> np.ndarray:
        out = np.empty(self.dims.hidden, np.float32)
        L.check(self.lib.moe_last_h_pre_norm(self.h, L.ptr(out)))
        return out

    def mtp_forward(self, h_in: np.ndarray) -> np.ndarray:
        h_in = np.ascontiguousarray(h_in, np.float32).reshape(self.dims.hidden)
        out = np.empty_like(h_in)
        L.check(self.lib.moe_mtp_forward_host(self.h, L.ptr(h_in), L.ptr(out)))
        return out

    # ── attention halves of the main layers (batch-1 decode) ─────────────
    def attn_configure(self, *, num_heads: int, num_kv_heads: int, head_dim: int, rotary_dim: int, rope_theta: float,
                       lin_num_k_heads: int, lin_num_v_heads: int, lin_key_dim: int, lin_value_dim: int, conv_kernel: int = 4,
                       full_attn_interval: int = 4, max_seq: int = 4096) -> None:
        d = L.ModelAttnDims(L.AttnDims(num_heads, num_kv_heads, head_dim, rotary_dim, max_seq, rope_theta), lin_num_k_heads,
                            lin_num_v_heads, lin_key_dim, lin_value_dim, conv_kernel, full_attn_interval)
        L.check(self.lib.moe_attn_configure(self.h, C.byref(d)))

    def attn_load_vec(self, layer: int, which: int, w: np.ndarray) -> None:
        """A norm weight, conv1d [channels, kernel] or dt_bias (bf16 bit patterns), or A_log (float32)."""
        if which == L.A_A_LOG:
            w = np.ascontiguousarray(w, np.float32)
            L.check(self.lib.moe_attn_load_tensor(self.h, layer, which, L.ptr(w), None, None, L.DT_F32))
        else:
            w = np.ascontiguousarray(w, np.uint16)
            L.check(self.lib.moe_attn_load_tensor(self.h, layer, which, L.ptr(w), None, None, L.DT_BF16))

    def attn_load_proj(self, layer: int, which: int, t) -> None:
        if isinstance(t, tuple):
            w, s, b = (np.ascontiguousarray(t[0], np.uint32), np.ascontiguousarray(t[1], np.uint16),
                       np.ascontiguousarray(t[2], np.uint16))
            L.check(self.lib.moe_attn_load_tensor(self.h, layer, which, L.ptr(w), L.ptr(s), L.ptr(b), L.DT_INT4))
        else:
            w = np.ascontiguousarray(t, np.uint16)
            L.check(self.lib.moe_attn_load_tensor(self.h, layer, which, L.ptr(w), None, None, L.DT_BF16))

    def model_forward_hidden(self, emb: np.ndarray) -> np.ndarray:
        """Embeddings [n, hidden] through attention + MoE of every layer: one decode step per token, or, from four tokens
        on, layer by layer with projections, attention, recurrence and MoE halves batched over the tokens."""
        emb = np.ascontiguousarray(emb, np.float32).reshape(-1, self.dims.hidden)
        out = np.empty_like(emb)
        L.check(self.lib.moe_model_forward_hidden_host(self.h, L.ptr(emb), emb.shape[0], L.ptr(out)))
        return out

    def model_forward(self, ids: np.ndarray) -> np.ndarray:
        ids = np.ascontiguousarray(ids, np.int64).reshape(-1)
        out = np.empty((ids.size, self.dims.vocab), np.float32)
        L.check(self.lib.moe_model_forward_host(self.h, L.ptr(ids), ids.size, L.ptr(out)))
        return out

    def model_snapshot(self) -> "ModelSnapshot":
        h = C.c_void_p()
        L.check(self.lib.moe_model_snapshot(self.h, C.byref(h)))
        return ModelSnapshot(self, h)

    def model_restore(self, snap: "ModelSnapshot") -> None:
        L.check(self.lib.moe_model_restore(self.h, snap.handle))

    def model_reset(self) -> None:
        L.check(self.lib.moe_model_reset(self.h))

    def model_pos(self) -> int:
        p = C.c_int64()
        L.check(self.lib.moe_model_pos(self.h, C.byref(p)))
        return p.value

    def model_set_pos(self, pos: int) -> None:
        L.check(self.lib.moe_model_set_pos(self.h, int(pos)))

    def model_state_download(self, layer: int, which: int, floats: int) -> np.ndarray:
        """One state tensor of one layer (L.ST_*) as float32 [floats]."""
        out = np.empty(int(floats), np.float32)
        L.check(self.lib.moe_model_state_host(self.h, layer, which, L.ptr(out) if out.size else None, out.size, 0))
        return out

    def model_state_upload(self, layer: int, which: int, data: np.ndarray) -> None:
        data = np.ascontiguousarray(data, np.float32).reshape(-1)
        L.check(self.lib.moe_model_state_host(self.h, layer, which, L.ptr(data) if data.size else None, data.size, 1))

    # ── MTP block, whole step (attention + MoE + head) ───────────────────
    def mtp_configure(self, num_heads: int, num_kv_heads: int, head_dim: int, rotary_dim: int, rope_theta: float,
                      max_seq: int = 4096) -> None:
        ad = L.AttnDims(num_heads, num_kv_heads, head_dim, rotary_dim, max_seq, rope_theta)
        L.check(self.lib.moe_mtp_configure(self.h, C.byref(ad)))

    def mtp_load_norm(self, which: int, w: np.ndarray) -> None:
        w = np.ascontiguousarray(w, np.uint16)
        L.check(self.lib.moe_mtp_load_tensor(self.h, which, L.ptr(w), None, None, L.DT_BF16))

    def mtp_load_proj(self, which: int, t) -> None:
        """A projection: bf16 bit patterns [out, in] or a 4-bit triple."""
        if isinstance(t, tuple):
            w, s, b = (np.ascontiguousarray(t[0], np.uint32), np.ascontiguousarray(t[1], np.uint16),
                       np.ascontiguousarray(t[2], np.uint16))
            L.check(self.lib.moe_mtp_load_tensor(self.h, which, L.ptr(w), L.ptr(s), L.ptr(b), L.DT_INT4))
        else:
            w = np.ascontiguousarray(t, np.uint16)
            L.check(self.lib.moe_mtp_load_tensor(self.h, which, L.ptr(w), None, None, L.DT_BF16))

    def mtp_step(self, h: np.ndarray, token_id: int) -> np.ndarray:
        """(hidden state before the final norm, previous token) -> logits [vocab]; advances the block's position."""
        h = np.ascontiguousarray(h, np.float32).reshape(self.dims.hidden)
        out = np.empty(self.dims.vocab, np.float32)
        L.check(self.lib.moe_mtp_step_host(self.h, L.ptr(h), int(token_id), L.ptr(out)))
        return out

    def mtp_reset(self) -> None:
        L.check(self.lib.moe_mtp_reset(self.h))

    def mtp_rollback(self, pos: int) -> None:
        L.check(self.lib.moe_mtp_rollback(self.h, pos))

    def mtp_pos(self) -> int:
        p = C.c_int64()
        L.check(self.lib.moe_mtp_pos(self.h, C.byref(p)))
        return p.value

    def telemetry(self) -> dict:
        n = C.c_int(0)
        L.check(self.lib.moe_telemetry_get(self.h, None, None, C.byref(n)))
        if n.value == 0:
            return {}
        keys = (C.c_char_p * n.value)()
        vals = (C.c_double * n.value)()
        L.check(self.lib.moe_telemetry_get(self.h, keys, vals, C.byref(n)))
        return {keys[i].decode(): vals[i] for i in range(n.value)}

    # ── expert parallelism ───────────────────────────────────────────────
    def ep_export(self, rank: int, world: int, max_tokens_per_rank: int) -> bytes:
        buf = C.create_string_buffer(L.EP_HANDLE_BYTES)
        L.check(self.lib.moe_ep_export(self.h, rank, world, max_tokens_per_rank, buf))
        return buf.raw

    def ep_init(self, all_handles: bytes) -> None:
        L.check(self.lib.moe_ep_init(self.h, C.create_string_buffer(all_handles, len(all_handles))))

    def ep_finalize(self) -> None:
        L.check(self.lib.moe_ep_finalize(self.h))

    def ep_layer_forward_dev(self, layer: int, h_in: int, n_local: int, h_out: int) -> None:
        L.check(self.lib.moe_ep_layer_forward_dev(self.h, layer, C.c_void_p(h_in), n_local, C.c_void_p(h_out)))

    def ep_forward_hidden_dev(self, emb: int, n_local: int, out: int) -> None:
        L.check(self.lib.moe_ep_forward_hidden_dev(self.h, C.c_void_p(emb), n_local, C.c_void_p(out)))

    def decode_profile(self, enable: Optional[bool] = None) -> Optional[np.ndarray]:
        """enable=True/False switches phase stamping; None returns stamps [layers, points]."""
        if enable is not None:
            L.check(self.lib.moe_decode_profile(self.h, int(enable), None, 0, None))
            return None
        n = self.dims.num_layers + self.dims.num_mtp_layers
        buf = np.zeros((n, 16), np.int64)
        pts = C.c_int(0)
        tmp = np.zeros(n * 16, np.int64)
        L.check(self.lib.moe_decode_profile(self.h, 1, tmp.ctypes.data_as(C.POINTER(C.c_int64)), n, C.byref(pts)))
        return tmp[: n * pts.value].reshape(n, pts.value)

    def alloc(self, nbytes: int) -> DevBuf:
        return DevBuf(self, nbytes)


def load_layer_weights(eng: NativeEngine, layer: int, *, post_norm_w, router_bf16=None, router_q4=None,
                       sh_gate: Q4, sh_up: Q4, sh_down: Q4, sgate: Q4, experts: Optional[np.ndarray]) -> None:
    """Uploads every tensor of one MoE block (host arrays in the reference's byte layout)."""
    if experts is not None:
        eng.load_layer(layer, experts)
    eng.load_bf16(layer, L.T_POST_NORM, post_norm_w)
    if router_bf16 is not None:
        eng.load_bf16(layer, L.T_ROUTER, router_bf16)
    else:
        eng.load_q4(layer, L.T_ROUTER, router_q4)
    eng.load_q4(layer, L.T_SHARED_GATE, sh_gate)
    eng.load_q4(layer, L.T_SHARED_UP, sh_up)
    eng.load_q4(layer, L.T_SHARED_DOWN, sh_down)
    eng.load_q4(layer, L.T_SHARED_SGATE, sgate)
