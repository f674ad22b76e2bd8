"""Mirror of the reference's PyO3 module ``_moe_infer_rs`` (src/python_bindings.rs, src/lib.rs:33-49)
for the Qwen3.5/3.6 MoE path, on top of the C ABI of ``libmoe_b200.so``.

Same class and function names, argument meaning and exception classes as the
reference binding: ``Model``, ``Cache``, ``Engine``, ``PyEngineSnapshot``,
``record_engine_telemetry``, ``qwen35_moe_quantize``.  Every forward goes through the
CUDA library; nothing here computes the MoE path on the CPU.

Where this surface departs from the reference, and how the calls behave:
  * a model directory that has the attention tensors of every layer runs the whole decoder (gated full attention /
    Gated DeltaNet half + MoE half per layer) on the GPU: one decode step per token for calls of up to three tokens, layer
    by layer with every stage batched over the call's tokens beyond (``forward`` and ``forward_batched`` alike);
    a directory with the MoE tensors only is still accepted and then each block is h <- h + moe(rmsnorm(h));
  * ``forward`` / ``forward_batched`` / ``forward_hidden`` return logits float32 [n, vocab] like the reference
    (embedding rows, stack, final norm and lm_head all on the GPU).  They raise ``RuntimeError`` naming the missing
    tensor when the model directory has no embedding table, final norm or lm_head, instead of returning zeros
    (the reference's ``embed_lookup`` silently fills zeros, src/math_util.rs:211-214);
  * ``forward_hidden_states`` (not in the reference) returns the hidden states before the final norm,
    float32 [n, hidden], and needs no head tensors;
  * ``mtp_forward(token_id)`` is the reference's draft step (logits float32 [vocab]) when the directory has the MTP
    block's tensors and the head; without them only the block's MoE half runs on ``last_h_pre_norm`` and the result
    is float32 [hidden] (an empty array when the model has no MTP block, like the reference);
  * ``Cache`` holds the per-sequence state in the reference's layout and file format (src/cache.rs:133-233); while a
    sequence runs the state lives on the device and ``download_cache`` / ``upload_cache`` move it.  A cache whose
    position is not 0 but which carries no state is refused (the reference would run on zeros).
"""
from __future__ import annotations

import json
import os
import sys
from typing import Optional

import numpy as np

from . import _lib as L
from .modeldir import ARCHS, ModelDir, ModelDirWriter
from .native import Dims, NativeEngine

_MODES = tuple(f"Qwen35MoEFusedExp{i}" for i in range(1, 7))


def record_engine_telemetry(on: bool) -> None:
    """src/python_bindings.rs:29-32"""
    L.load().moe_set_record_telemetry(1 if on else 0)


class Model:
    """src/python_bindings.rs:41-55: loads a converted model directory; RuntimeError on failure."""

    def __init__(self, model_path: str):
        try:
            self.inner = ModelDir(model_path)
        except (OSError, KeyError, ValueError) as e:
            raise RuntimeError(str(e)) from e

    def __repr__(self) -> str:
        return f"Model({self.inner.get('num_hidden_layers', 0)} layers, hidden={self.inner.get('hidden_size', 0)})"


MAX_SEQ = 4096  # src/constants.rs:12: positions a KV cache holds, and the row count of the cache tensors on disk


def _shifted_from_ring(ring: np.ndarray, pos: int) -> np.ndarray:
    """The device keeps the last conv inputs as a ring (input of step s in row s % kernel); the reference keeps the
    last kernel - 1 inputs oldest first (src/math_util.rs:149-168).  Row k of that layout is the input of step
    pos - (kernel - 1) + k."""
    ks = ring.shape[0]
    return np.stack([ring[(pos - (ks - 1) + k) % ks] for k in range(ks - 1)]) if ks > 1 else ring[:0].copy()


def _ring_from_shifted(shifted: np.ndarray, pos: int) -> np.ndarray:
    ks = shifted.shape[0] + 1
    ring = np.zeros((ks, shifted.shape[1]), np.float32)
    for k in range(ks - 1):
        ring[(pos - (ks - 1) + k) % ks] = shifted[k]
    return ring


class Cache:
    """src/python_bindings.rs:64-100, src/cache.rs:32-233: the per-sequence state on the host side.  Full-attention
    layers: K and V rows of the positions so far; linear-attention layers: the last conv inputs and the recurrence
    state; and the position.  The state itself lives on the device while a sequence runs (``gpu_dirty``);
    ``Engine.download_cache`` brings it here, ``save`` / ``load`` use the reference's file format (a flat binary of
    float32 tensors plus a JSON manifest ``{"tensors": {name: {offset, size, shape, dtype}}}``), so a file written by
    either implementation loads in the other.  ``states is None`` means the all-zero state of a new sequence.
    A model directory without the attention keys in its config (MoE halves only) has no state beyond ``pos``."""

    def __init__(self, model: Model):
        self.pos = 0
        self.cpu_dirty = True   # the device has nothing of this cache yet (src/cache.rs:75)
        self.gpu_dirty = False
        self.states: Optional[list] = None
        self.layout = self._layout_of(model.inner)

    @staticmethod
    def _layout_of(m) -> Optional[dict]:
        need = ("num_hidden_layers", "num_key_value_heads", "head_dim")
        if any(not m.get(k) for k in need):
            return None
        vh, kh = int(m.get("linear_num_value_heads", 0) or 0), int(m.get("linear_num_key_heads", 0) or 0)
        kd, vd = int(m.get("linear_key_head_dim", 0) or 0), int(m.get("linear_value_head_dim", 0) or 0)
        return dict(layers=int(m.get("num_hidden_layers")), kv_dim=int(m.get("num_key_value_heads")) * int(m.get("head_dim")),
                    v_heads=vh, key_dim=kd, value_dim=vd, conv_dim=2 * kh * kd + vh * vd, has_linear=vh > 0 and kh > 0,
                    conv_kernel=int(m.get("linear_conv_kernel_dim", 4)), interval=int(m.get("full_attention_interval", 4)))

    def is_full(self, layer: int) -> bool:
        lay = self.layout
        return not lay["has_linear"] or (layer + 1) % lay["interval"] == 0   # src/cache.rs:63-65

    def reset(self) -> None:
        """src/cache.rs:84-94: position 0, zero conv and recurrence states."""
        self.pos = 0
        self.states = None
        self.cpu_dirty = True
        self.gpu_dirty = False

    def _zero_states(self) -> list:
        lay, out = self.layout, []
        for l in range(lay["layers"]):
            if self.is_full(l):
                out.append({"k_cache": np.zeros((0, lay["kv_dim"]), np.float32), "v_cache": np.zeros((0, lay["kv_dim"]), np.float32)})
            else:
                out.append({"conv_state": np.zeros((lay["conv_kernel"] - 1, lay["conv_dim"]), np.float32),
                            "ssm_state": np.zeros(lay["v_heads"] * lay["value_dim"] * lay["key_dim"], np.float32)})
        return out

    def save(self, bin_path: str, json_path: str) -> None:
        """src/cache.rs:133-175.  K / V tensors are written with MAX_SEQ rows like the reference's."""
        if self.gpu_dirty:
            print("[cache] WARNING: saving cache with gpu_dirty=true", file=sys.stderr)
        tensors, offset = {}, 0
        try:
            with open(bin_path, "wb") as f:
                def put(name, arr, shape, dtype="float32"):
                    nonlocal offset
                    raw = arr.tobytes()
                    f.write(raw)
                    tensors[name] = {"offset": offset, "size": len(raw), "shape": list(shape), "dtype": dtype}
                    offset += len(raw)

                if self.layout is not None:
                    states = self.states if self.states is not None else self._zero_states()
                    kv_dim = self.layout["kv_dim"]
                    for l, st in enumerate(states):
                        if "k_cache" in st:
                            for key in ("k_cache", "v_cache"):
                                full = np.zeros((MAX_SEQ, kv_dim), np.float32)
                                full[:st[key].shape[0]] = st[key]
                                put(f"cache.layer_{l}.{key}", full, (MAX_SEQ, kv_dim))
                            put(f"cache.layer_{l}.len", np.uint32(self.pos), (), "uint32")
                        else:
                            put(f"cache.layer_{l}.conv_state", st["conv_state"], st["conv_state"].shape)
                            put(f"cache.layer_{l}.ssm_state", st["ssm_state"], (st["ssm_state"].size,))
                put("cache.pos", np.uint32(self.pos), (), "uint32")
            with open(json_path, "w") as f:
                json.dump({"tensors": tensors}, f, indent=2)
        except OSError as e:
            raise IOError(str(e)) from e

    @staticmethod
    def load(bin_path: str, json_path: str) -> "Cache":
        """src/cache.rs:177-233: the layer kinds are read off the manifest's tensor names."""
        try:
            with open(json_path) as f:
                tensors = json.load(f)["tensors"]
            raw = np.fromfile(bin_path, np.uint8)
        except (OSError, ValueError, KeyError) as e:
            raise IOError(str(e)) from e

        def get(name, dtype):
            if name not in tensors:
                raise IOError(f"missing tensor: {name}")
            t = tensors[name]
            return raw[int(t["offset"]):int(t["offset"]) + int(t["size"])].view(dtype)

        c = Cache.__new__(Cache)
        c.pos = int(get("cache.pos", np.uint32)[0])
        c.cpu_dirty, c.gpu_dirty, c.states, c.layout = True, False, None, None
        states, l = [], 0
        while f"cache.layer_{l}.k_cache" in tensors or f"cache.layer_{l}.conv_state" in tensors:
            if f"cache.layer_{l}.k_cache" in tensors:
                n = int(get(f"cache.layer_{l}.len", np.uint32)[0])
                shape = tensors[f"cache.layer_{l}.k_cache"]["shape"]
                states.append({key: get(f"cache.layer_{l}.{key}", np.float32).reshape(shape)[:n].copy() for key in ("k_cache", "v_cache")})
            else:
                shape = tensors[f"cache.layer_{l}.conv_state"]["shape"]
                states.append({"conv_state": get(f"cache.layer_{l}.conv_state", np.float32).reshape(shape).copy(),
                               "ssm_state": get(f"cache.layer_{l}.ssm_state", np.float32).copy()})
            l += 1
        if states:
            c.states = states
            c.layout = {"layers": len(states), "from_file": True}
        return c

    def __repr__(self) -> str:
        return f"Cache(pos={self.pos})"


class PyEngineSnapshot:
    """src/python_bindings.rs:21-24, src/engine.rs:98-109"""

    def __init__(self, pos: int, mtp_pos: int, last_h: np.ndarray, device_state=None):
        self.pos, self.mtp_pos, self.last_h_pre_norm = pos, mtp_pos, last_h.copy()
        self.device_state = device_state  # conv + recurrence states of the linear-attention layers, when attention runs


class Engine:
    """src/python_bindings.rs:104-311.  All six ``Qwen35MoEFusedExp*`` modes map to the one B200 engine."""

    def __init__(self, model: Model, pipeline_mode: str = "Qwen35MoEFusedExp2", num_active_experts: int = 0, *,
                 expert_cache_count: int = 0, device: int = 0):
        m = model.inner
        arch = m.architecture
        if pipeline_mode not in _MODES or arch not in ARCHS:
            # reference src/engine.rs:233-235
            raise ValueError(f"Config error: Unknown engine: engine_type={pipeline_mode!r}, arch={arch!r}")
        per_tok = m.get_usize("num_experts_per_tok", 8)
        k = num_active_experts or per_tok
        if k > per_tok or k > 8:
            raise ValueError(f"Config error: num_active_experts ({k}) exceeds num_experts_per_tok ({per_tok}) or MAX_K (8)")
        self.model = model
        self.pos = 0
        self._telemetry = {}
        self._last_h = np.zeros(m.get_usize("hidden_size"), np.float32)
        layers = m.get_usize("num_hidden_layers")
        mtp = m.get_usize("mtp_num_hidden_layers", 0)
        router_probe = m.tensor("model.layers.0.mlp.gate.weight")
        scheme = L.SCHEME_BQ4 if (router_probe is not None and router_probe.dtype == np.uint16) else L.SCHEME_INT4
        self.dims = Dims(hidden=m.get_usize("hidden_size"), inter=m.get_usize("moe_intermediate_size", 512),
                         shared_inter=m.get_usize("shared_expert_intermediate_size", 512),
                         num_experts=m.get_usize("num_experts", 256), top_k=k, num_layers=layers,
                         num_mtp_layers=mtp, vocab=m.get_usize("vocab_size"), scheme=scheme)
        self.native = NativeEngine(self.dims, device=device)  # ValueError for unsupported dimensions
        try:
            for l in range(layers + mtp):
                self._load_layer(l, f"model.layers.{l}" if l < layers else f"mtp.layers.{l - layers}")
            self._missing_head = self._load_head()
            self._missing_mtp = self._load_mtp() if mtp else ["an MTP layer (mtp_num_hidden_layers == 0)"]
            self._missing_attn = self._load_attn()
        except Exception:
            self.native.close()
            raise

    def _load_head(self):
        """Embedding table, final norm and lm_head, when the directory has them; returns the names that are missing."""
        m, eng = self.model.inner, self.native
        missing = []
        emb = m.q4("model.embed_tokens")
        if emb is not None:
            eng.load_embed(emb)
        else:
            missing.append("model.embed_tokens")
        norm = m.tensor("model.norm.weight")
        if norm is not None:
            eng.load_final_norm(norm)
        else:
            missing.append("model.norm.weight")
        w = m.tensor("lm_head.weight")
        if w is not None and w.dtype == np.uint8:       # INT8 rows + f32 scale per row (BQ4 scheme)
            eng.load_lm_head_int8(w, m.tensor("lm_head.scales"))
        elif w is not None and m.q4("lm_head") is not None:  # 4-bit triple (INT4 scheme)
            eng.load_lm_head_q4(m.q4("lm_head"))
        else:
            missing.append("lm_head")
        return missing

    def _load_attn(self):
        """The attention halves of the main layers, when the directory has the tensors of every layer
        (src/engine/qwen35_moe/cpu.rs:87-347 names them); returns what is missing, and then attention is passed through."""
        m, eng = self.model.inner, self.native
        need = ("num_attention_heads", "num_key_value_heads", "head_dim")
        if any(not m.get(k) for k in need):
            return [" / ".join(need) + " in config.json"]
        rope = m.get("rope_parameters") or {}
        heads, kv_heads, head_dim = (int(m.get(k)) for k in need)
        ad = dict(num_heads=heads, num_kv_heads=kv_heads, head_dim=head_dim,
                  rotary_dim=int(head_dim * float(m.get("partial_rotary_factor", rope.get("partial_rotary_factor", 0.25)))),
                  rope_theta=float(m.get("rope_theta", rope.get("rope_theta", 10_000_000.0))),
                  lin_num_k_heads=int(m.get("linear_num_key_heads", 16)), lin_num_v_heads=int(m.get("linear_num_value_heads", 32)),
                  lin_key_dim=int(m.get("linear_key_head_dim", 128)), lin_value_dim=int(m.get("linear_value_head_dim", 128)),
                  conv_kernel=int(m.get("linear_conv_kernel_dim", 4)), full_attn_interval=int(m.get("full_attention_interval", 4)))
        H = self.dims.hidden
        q_dim, kv_dim = heads * head_dim, kv_heads * head_dim
        total_key, total_value = ad["lin_num_k_heads"] * ad["lin_key_dim"], ad["lin_num_v_heads"] * ad["lin_value_dim"]
        conv_dim = 2 * total_key + total_value
        full_vecs = {L.A_Q_NORM: "self_attn.q_norm.weight", L.A_K_NORM: "self_attn.k_norm.weight"}
        full_projs = {L.A_Q_PROJ: ("self_attn.q_proj", 2 * q_dim, H), L.A_K_PROJ: ("self_attn.k_proj", kv_dim, H),
                      L.A_V_PROJ: ("self_attn.v_proj", kv_dim, H), L.A_O_PROJ: ("self_attn.o_proj", H, q_dim)}
        lin_vecs = {L.A_CONV1D: "linear_attn.conv1d.weight", L.A_A_LOG: "linear_attn.A_log", L.A_DT_BIAS: "linear_attn.dt_bias",
                    L.A_LIN_NORM: "linear_attn.norm.weight"}
        lin_projs = {L.A_IN_PROJ_QKV: ("linear_attn.in_proj_qkv", conv_dim, H), L.A_IN_PROJ_Z: ("linear_attn.in_proj_z", total_value, H),
                     L.A_IN_PROJ_B: ("linear_attn.in_proj_b", ad["lin_num_v_heads"], H),
                     L.A_IN_PROJ_A: ("linear_attn.in_proj_a", ad["lin_num_v_heads"], H), L.A_OUT_PROJ: ("linear_attn.out_proj", H, total_value)}
        plan, missing = [], []
        for l in range(self.dims.num_layers):
            pre = f"model.layers.{l}."
            full = (l + 1) % ad["full_attn_interval"] == 0
            vecs = {L.A_INPUT_NORM: "input_layernorm.weight", **(full_vecs if full else lin_vecs)}
            for which, name in vecs.items():
                t = m.tensor(pre + name)
                if t is None:
                    missing.append(pre + name)
                plan.append((l, which, t, None))
            for which, (base, rows, cols) in (full_projs if full else lin_projs).items():
                w = m.tensor(pre + base + ".weight")
                t = w.reshape(rows, cols) if (w is not None and w.dtype == np.uint16) else m.q4(pre + base)
                if t is None:
                    missing.append(pre + base)
                plan.append((l, which, t, "proj"))
        if missing:
            return missing
        eng.attn_configure(**ad)
        for l, which, t, kind in plan:
            (eng.attn_load_proj if kind else eng.attn_load_vec)(l, which, t)
        return []

    def _load_mtp(self):
        """The attention half of the MTP block, when the directory has its tensors (src/engine/qwen35_moe/mtp.rs:85-216
        names them); returns the names that are missing.  mtp.norm is optional: the model's final norm stands in."""
        m, eng = self.model.inner, self.native
        heads, kv_heads, head_dim = m.get("num_attention_heads"), m.get("num_key_value_heads"), m.get("head_dim")
        if not heads or not kv_heads or not head_dim:
            return ["num_attention_heads / num_key_value_heads / head_dim in config.json"]
        rope = m.get("rope_parameters") or {}
        factor = m.get("partial_rotary_factor", rope.get("partial_rotary_factor", 0.25))
        theta = m.get("rope_theta", rope.get("rope_theta", 10_000_000.0))
        norms = {L.M_PRE_FC_NORM_HIDDEN: "mtp.pre_fc_norm_hidden.weight", L.M_PRE_FC_NORM_EMBEDDING: "mtp.pre_fc_norm_embedding.weight",
                 L.M_INPUT_NORM: "mtp.layers.0.input_layernorm.weight", L.M_Q_NORM: "mtp.layers.0.self_attn.q_norm.weight",
                 L.M_K_NORM: "mtp.layers.0.self_attn.k_norm.weight"}
        q_dim, kv_dim, H = int(heads) * int(head_dim), int(kv_heads) * int(head_dim), self.dims.hidden
        projs = {L.M_FC: ("mtp.fc", H, 2 * H), L.M_Q_PROJ: ("mtp.layers.0.self_attn.q_proj", 2 * q_dim, H),
                 L.M_K_PROJ: ("mtp.layers.0.self_attn.k_proj", kv_dim, H), L.M_V_PROJ: ("mtp.layers.0.self_attn.v_proj", kv_dim, H),
                 L.M_O_PROJ: ("mtp.layers.0.self_attn.o_proj", H, q_dim)}
        found_n = {k: m.tensor(n) for k, n in norms.items()}
        found_p = {}
        for k, (base, rows, cols) in projs.items():
            w = m.tensor(base + ".weight")
            if w is not None and w.dtype == np.uint16:            # bf16, stored flat (src/dtype.rs:456-460)
                found_p[k] = w.reshape(rows, cols)
            else:
                found_p[k] = m.q4(base)
        missing = [norms[k] for k, v in found_n.items() if v is None] + [projs[k][0] for k, v in found_p.items() if v is None]
        if missing:
            return missing
        eng.mtp_configure(int(heads), int(kv_heads), int(head_dim), int(int(head_dim) * float(factor)), float(theta))
        for k, v in found_n.items():
            eng.mtp_load_norm(k, v)
        out_norm = m.tensor("mtp.norm.weight")
        if out_norm is not None:
            eng.mtp_load_norm(L.M_OUT_NORM, out_norm)
        for k, v in found_p.items():
            eng.mtp_load_proj(k, v)
        return []

    def _load_layer(self, layer: int, prefix: str) -> None:
        m, d, eng = self.model.inner, self.dims, self.native
        path = m.expert_file(layer)
        want = d.num_experts * eng.layout["expert_size"]
        if not os.path.exists(path) or os.path.getsize(path) != want:
            raise RuntimeError(f"I/O error: {path}: expected {want} bytes of packed experts")
        eng.load_layer(layer, np.memmap(path, dtype=np.uint8, mode="r"))
        norm = m.tensor(prefix + ".post_attention_layernorm.weight")
        if norm is None:
            raise RuntimeError(f"Config error: tensor {prefix}.post_attention_layernorm.weight missing")
        eng.load_bf16(layer, L.T_POST_NORM, norm)
        router = m.tensor(prefix + ".mlp.gate.weight")
        if router is not None and router.dtype == np.uint16:
            eng.load_bf16(layer, L.T_ROUTER, router.reshape(d.num_experts, d.hidden))
        else:
            eng.load_q4(layer, L.T_ROUTER, self._need_q4(prefix + ".mlp.gate"))
        eng.load_q4(layer, L.T_SHARED_GATE, self._need_q4(prefix + ".mlp.shared_expert.gate_proj"))
        eng.load_q4(layer, L.T_SHARED_UP, self._need_q4(prefix + ".mlp.shared_expert.up_proj"))
        eng.load_q4(layer, L.T_SHARED_DOWN, self._need_q4(prefix + ".mlp.shared_expert.down_proj"))
        eng.load_q4(layer, L.T_SHARED_SGATE, self._need_q4(prefix + ".mlp.shared_expert_gate"))

    def _need_q4(self, base: str):
        t = self.model.inner.q4(base)
        if t is None:
            raise RuntimeError(f"Config error: tensor {base}.weight/.scales/.biases missing")
        return t

    # ── reference surface ────────────────────────────────────────────────
    def _need_head(self, *names: str) -> None:
        miss = [n for n in names if n in self._missing_head]
        if miss:
            raise RuntimeError(f"Config error: tensor(s) {', '.join(miss)} missing from the model directory")

    def embed_lookup(self, input_ids: np.ndarray) -> np.ndarray:
        self._need_head("model.embed_tokens")
        try:
            return self.native.embed_lookup(np.ascontiguousarray(input_ids, np.int64).reshape(-1))
        except L.MoeError as e:
            raise RuntimeError(str(e)) from e

    def _sync_sequence(self, cache: Cache) -> None:
        """The attention state lives on the device.  A cache at position 0 starts a new sequence; any other position
        must be the one the device is at (the KV and recurrence states cannot be rebuilt from a position alone)."""
        dev = self.native.model_pos()
        if cache.pos == 0 and dev != 0:
            self.native.model_reset()
            self.pos = 0
        elif cache.pos != dev:
            raise RuntimeError(f"cache position {cache.pos} does not match the device state at position {dev}; "
                               "attention state can only continue or restart")

    def _after(self, n: int, cache: Cache) -> None:
        self.pos += n
        cache.pos = self.pos
        cache.gpu_dirty = True
        self._last_h = self.native.last_h_pre_norm()
        self._telemetry = self.native.telemetry()

    def forward_hidden_states(self, embeddings: np.ndarray, cache: Cache, *, batched: bool = False, mtp: bool = False) -> np.ndarray:
        """Not in the reference: the hidden states before the final norm, float32 [n, hidden]."""
        emb = np.ascontiguousarray(embeddings, np.float32).reshape(-1, self.dims.hidden)
        if cache.cpu_dirty:
            self.upload_cache(cache)
        try:
            if not self._missing_attn:
                # the whole decoder block per layer (token by token, or layer by layer for four tokens and more)
                self._sync_sequence(cache)
                out = self.native.model_forward_hidden(emb)
            else:
                out = self.native.forward_hidden(emb, batched=batched, mtp=mtp, check=_interrupt_pending)
        except L.MoeError as e:
            raise RuntimeError(str(e)) from e
        self._after(emb.shape[0], cache)
        return out

    def forward_hidden(self, embeddings: np.ndarray, cache: Cache, *, mtp: bool = False) -> np.ndarray:
        """src/python_bindings.rs:141-160: embeddings [n, hidden] -> logits [n, vocab]."""
        self._need_head("model.norm.weight", "lm_head")
        hidden = self.forward_hidden_states(embeddings, cache, mtp=mtp)
        try:
            return self.native.logits(hidden)
        except L.MoeError as e:
            raise RuntimeError(str(e)) from e

    def _forward_ids(self, tokens: np.ndarray, cache: Cache, batched: bool, mtp: bool) -> np.ndarray:
        toks = np.ascontiguousarray(tokens, np.int64).reshape(-1)
        if toks.size == 0:
            return np.zeros((0, self.dims.vocab), np.float32)
        self._need_head("model.embed_tokens", "model.norm.weight", "lm_head")
        if cache.cpu_dirty:
            self.upload_cache(cache)
        try:
            if not self._missing_attn:
                self._sync_sequence(cache)
                out = self.native.model_forward(toks)
            else:
                out = self.native.forward(toks, batched=batched, mtp=mtp, check=_interrupt_pending)
        except L.MoeError as e:
            raise RuntimeError(str(e)) from e
        self._after(toks.size, cache)
        return out

    def forward(self, tokens: np.ndarray, cache: Cache, *, mtp: bool = False) -> np.ndarray:
        """src/python_bindings.rs:172-202: token ids -> logits [n, vocab]; n = 0 gives [0, vocab]."""
        return self._forward_ids(tokens, cache, False, mtp)

    def forward_batched(self, tokens: np.ndarray, cache: Cache, *, mtp: bool = False) -> np.ndarray:
        """src/python_bindings.rs:208-244: same result, batched internals."""
        return self._forward_ids(tokens, cache, True, mtp)

    def upload_cache(self, cache: Cache) -> None:
        """src/engine.rs:64-71: the cache's state becomes the device's (a cache without states: a new sequence)."""
        if not self._missing_attn:
            eng = self.native
            try:
                if cache.states is None:
                    if cache.pos != 0:
                        raise RuntimeError(f"the cache is at position {cache.pos} but carries no state: attention state cannot "
                                           "be rebuilt from a position alone")
                    eng.model_reset()
                else:
                    if len(cache.states) != self.dims.num_layers:
                        raise RuntimeError(f"the cache holds {len(cache.states)} layers, the model {self.dims.num_layers}")
                    for l, st in enumerate(cache.states):
                        if "k_cache" in st:
                            if st["k_cache"].shape[0] < cache.pos:
                                raise RuntimeError(f"layer {l}: the cache holds {st['k_cache'].shape[0]} positions, pos is {cache.pos}")
                            eng.model_state_upload(l, L.ST_K_CACHE, st["k_cache"][:cache.pos])
                            eng.model_state_upload(l, L.ST_V_CACHE, st["v_cache"][:cache.pos])
                        else:
                            eng.model_state_upload(l, L.ST_CONV, _ring_from_shifted(st["conv_state"], cache.pos))
                            eng.model_state_upload(l, L.ST_SSM, st["ssm_state"])
                eng.model_set_pos(cache.pos)
            except L.MoeError as e:
                raise RuntimeError(str(e)) from e
        self.pos = cache.pos
        cache.cpu_dirty = False

    def download_cache(self, cache: Cache) -> None:
        """src/engine.rs:72-79: the device's state becomes the cache's."""
        if not self._missing_attn:
            eng, pos = self.native, self.native.model_pos()
            lay = Cache._layout_of(self.model.inner)
            probe = Cache.__new__(Cache)
            probe.layout = lay
            states = []
            try:
                for l in range(self.dims.num_layers):
                    if probe.is_full(l):
                        states.append({"k_cache": eng.model_state_download(l, L.ST_K_CACHE, pos * lay["kv_dim"]).reshape(pos, lay["kv_dim"]),
                                       "v_cache": eng.model_state_download(l, L.ST_V_CACHE, pos * lay["kv_dim"]).reshape(pos, lay["kv_dim"])})
                    else:
                        ring = eng.model_state_download(l, L.ST_CONV, lay["conv_kernel"] * lay["conv_dim"])
                        states.append({"conv_state": _shifted_from_ring(ring.reshape(lay["conv_kernel"], lay["conv_dim"]), pos),
                                       "ssm_state": eng.model_state_download(l, L.ST_SSM, lay["v_heads"] * lay["value_dim"] * lay["key_dim"])})
            except L.MoeError as e:
                raise RuntimeError(str(e)) from e
            cache.states, cache.layout = states, lay
            self.pos = pos
        cache.pos = self.pos
        cache.gpu_dirty = False

    def telemetry(self) -> dict:
        return dict(self._telemetry)

    def last_h_pre_norm(self) -> np.ndarray:
        return self._last_h.copy()

    def mtp_forward(self, token_id: int) -> np.ndarray:
        if self.dims.num_mtp_layers == 0:
            return np.zeros(0, np.float32)
        if not 0 <= int(token_id) < self.dims.vocab:
            raise ValueError(f"token id {token_id} outside [0, {self.dims.vocab})")
        if self._missing_mtp or self._missing_head:
            # without the block's attention tensors or the head only the MoE half can run: hidden state [hidden]
            return self.native.mtp_forward(self._last_h)
        # the reference's mtp_forward (src/python_bindings.rs:283-291): logits [vocab] of the next-next token
        return self.native.mtp_step(self._last_h, int(token_id))

    def mtp_reset(self) -> None:
        self.native.mtp_reset()

    def mtp_rollback(self, pos: int) -> None:
        self.native.mtp_rollback(pos)

    def snapshot_state(self) -> PyEngineSnapshot:
        dev = self.native.model_snapshot() if not self._missing_attn else None
        return PyEngineSnapshot(self.pos, self.native.mtp_pos(), self._last_h, dev)

    def restore_snapshot(self, snap: PyEngineSnapshot) -> None:
        if not self._missing_attn:
            if snap.device_state is None:
                raise RuntimeError("this snapshot carries no attention state")
            self.native.model_restore(snap.device_state)
        self.pos = snap.pos
        self._last_h = snap.last_h_pre_norm.copy()
        self.native.mtp_rollback(snap.mtp_pos)

    def __repr__(self) -> str:
        return f"Engine(loaded: {self.dims.num_layers} layers, hidden={self.dims.hidden})"


def _interrupt_pending() -> bool:
    """The reference polls ``py.check_signals()`` (src/python_bindings.rs:152); ctypes delivers
    KeyboardInterrupt after the call returns, so nothing is pending inside the callback."""
    return False


def qwen35_moe_quantize(model_path: str, output_dir: str, *, version: str, scheme: str = "bq4", device: int = 0) -> None:
    """src/python_bindings.rs:327-387: HF safetensors -> model_weights.{bin,json} + packed_experts/.

    Converts every tensor of the checkpoint the way the reference's pipeline does (manifest names,
    storage type per scheme, norm shift, conv1d axes, padding, config block); vision tensors are
    skipped.  Matrices are packed on the GPU.
    """
    if version not in ("3.5", "3.6"):
        raise ValueError(f"unknown Qwen version {version!r} (expected '3.5' or '3.6')")
    if scheme not in ("bq4", "int4"):
        raise ValueError(f"unknown scheme {scheme!r} (expected 'bq4' or 'int4')")
    from .quantize import quantize_moe_checkpoint
    quantize_moe_checkpoint(model_path, output_dir, version=version, scheme=scheme, device=device)


def _not_built(name: str):
    def f(*a, **k):
        raise NotImplementedError(f"{name} is outside the Qwen3.5/3.6 MoE path this library covers")
    f.__name__ = name
    return f


qwen35_dense_quantize = _not_built("qwen35_dense_quantize")
gemma4_moe_quantize = _not_built("gemma4_moe_quantize")
gemma4_dense_quantize = _not_built("gemma4_dense_quantize")


class PyHfRepo:
    def __init__(self, *a, **k):
        raise NotImplementedError("PyHfRepo (HF download) is outside the path this library covers; there is no network here")
