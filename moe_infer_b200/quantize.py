"""HF safetensors -> converted model directory, for the tensors of the MoE path and the model head.

Follows the reference's quantize pipeline (src/quantize.rs:71-365 and
src/quantize/qwen35_moe/{common,bq4,int4}.rs) for:
  * experts: `...mlp.experts.gate_up_proj` [E, 2I, H] and `...mlp.experts.down_proj` [E, H, I]
    -> packed_experts/layer_NN.bin (common.rs:300-345), packed on the GPU;
  * `mlp.gate` (bf16 in the BQ4 scheme, 4-bit in INT4: bq4.rs:25-32, int4.rs:24-35),
    `mlp.shared_expert.{gate,up,down}_proj`, `mlp.shared_expert_gate` (4-bit);
  * `post_attention_layernorm.weight` (bf16; +1 for Qwen3.6, bq4.rs:113-116);
  * the head: `embed_tokens` (4-bit in both schemes), the final `norm.weight` (bf16, +1 for Qwen3.6:
    common.rs is_final_zc_norm) and `lm_head` (INT8 with one f32 scale per row in BQ4, bq4.rs:29; 4-bit in INT4).
Tensor names in the manifest are the reference's (`language_model.model.layers.N...`, `language_model.lm_head`).
A 4-bit tensor whose inner dimension is not a multiple of 64 is zero-padded to one (src/quantize.rs:230-249).
The codecs and the bf16 rounding are the GPU packers' (bit-exact with src/dtype.rs:85-135, 164-179).
Attention and vision tensors are skipped.
"""
from __future__ import annotations

import json
import os
import re
import struct
from typing import Dict, Tuple

import numpy as np

from . import _lib as L
from .modeldir import ARCHS, ModelDirWriter
from .native import Dims, NativeEngine


def read_safetensors_index(model_path: str) -> Dict[str, Tuple[str, str, list, int, int]]:
    """name -> (file, dtype, shape, begin, end) over every *.safetensors shard (src/safetensors.rs:27-70)."""
    out = {}
    for fn in sorted(os.listdir(model_path)):
        if not fn.endswith(".safetensors"):
            continue
        full = os.path.join(model_path, fn)
        with open(full, "rb") as f:
            (hdr_len,) = struct.unpack("<Q", f.read(8))
            hdr = json.loads(f.read(hdr_len))
        base = 8 + hdr_len
        for name, meta in hdr.items():
            if name == "__metadata__":
                continue
            b, e = meta["data_offsets"]
            out[name] = (full, meta["dtype"], meta["shape"], base + b, base + e)
    return out


def _load(entry) -> np.ndarray:
    """Tensor as bf16 bit patterns (uint16) or float32, by source dtype."""
    full, dtype, shape, b, e = entry
    raw = np.memmap(full, dtype=np.uint8, mode="r")[b:e]
    if dtype == "BF16":
        return np.frombuffer(raw, np.uint16).reshape(shape)
    if dtype == "F32":
        return np.frombuffer(raw, np.float32).reshape(shape)
    if dtype == "F16":
        return np.frombuffer(raw, np.float16).astype(np.float32).reshape(shape)
    raise ValueError(f"unsupported safetensors dtype {dtype}")


def _f32(a: np.ndarray) -> np.ndarray:
    return (a.astype(np.uint32) << 16).view(np.float32) if a.dtype == np.uint16 else a.astype(np.float32)


def _ref_bf16(x: np.ndarray) -> np.ndarray:
    """The reference's f32 -> bf16 (src/dtype.rs:85-89): round_up = bit15 & (bit0 | bit16)."""
    u = np.ascontiguousarray(x, np.float32).view(np.uint32)
    up = ((u >> 15) & 1) & ((u & 1) | ((u >> 16) & 1))
    return ((u + (up << 16)) >> 16).astype(np.uint16)


def quantize_moe_checkpoint(model_path: str, output_dir: str, *, version: str, scheme: str, device: int = 0) -> None:
    with open(os.path.join(model_path, "config.json")) as f:
        config = json.load(f)
    tc = config.get("text_config", config)
    arch = (config.get("architectures") or [""])[0]
    if arch not in ARCHS:
        raise ValueError(f"architecture mismatch: found={arch!r}, expected one of {ARCHS}")
    g = lambda k, d=None: config.get(k, tc.get(k, d))
    H, I, SI, E = g("hidden_size"), g("moe_intermediate_size"), g("shared_expert_intermediate_size"), g("num_experts")
    n_layers, n_mtp = g("num_hidden_layers"), g("mtp_num_hidden_layers", 0)
    dims = Dims(hidden=H, inter=I, shared_inter=SI, num_experts=E, top_k=min(8, g("num_experts_per_tok", 8)),
                num_layers=n_layers, num_mtp_layers=n_mtp, vocab=g("vocab_size", 0),
                scheme=L.SCHEME_BQ4 if scheme == "bq4" else L.SCHEME_INT4)
    index = read_safetensors_index(model_path)
    eng = NativeEngine(dims, device=device)
    out = ModelDirWriter(output_dir, config, {"scheme": scheme, "version": version, "group_size": 64})

    def find(layer_prefix_pat: str, suffix: str):
        for name in index:
            if re.search(layer_prefix_pat + re.escape(suffix) + r"$", name):
                return index[name]
        return None

    def pack_q4(t: np.ndarray):
        """4-bit triple of a 2-D tensor; the inner dimension is zero-padded to a multiple of 64 first."""
        t = t if t.dtype == np.uint16 else _f32(t)
        rows, cols = t.shape
        if cols % 64:
            padded = np.zeros((rows, (cols + 63) // 64 * 64), t.dtype)
            padded[:, :cols] = t
            t = padded
        return eng.pack_int4(t)

    try:
        for l in range(n_layers + n_mtp):
            if l < n_layers:
                pat, dst = r"^(?!mtp\.).*" + rf"layers\.{l}\.", f"language_model.model.layers.{l}"
            else:
                pat, dst = rf"^mtp\.layers\.{l - n_layers}\.", f"mtp.layers.{l - n_layers}"
            gu, dn = find(pat, "mlp.experts.gate_up_proj"), find(pat, "mlp.experts.down_proj")
            if gu is None or dn is None:
                raise ValueError(f"layer {l}: expert tensors mlp.experts.gate_up_proj / down_proj not found")
            out.add_expert_layer(l, eng.pack_experts(_load(gu), _load(dn)))
            norm = find(pat, "post_attention_layernorm.weight")
            nv = _f32(_load(norm)).reshape(-1)
            if version == "3.6":
                nv = nv + np.float32(1.0)
            out.add_bf16(dst + ".post_attention_layernorm.weight", _ref_bf16(nv), flat=True)
            router = _load(find(pat, "mlp.gate.weight"))
            if scheme == "bq4":
                out.add_bf16(dst + ".mlp.gate.weight", _ref_bf16(_f32(router)), flat=True)
            else:
                out.add_q4(dst + ".mlp.gate", *pack_q4(router))
            for nm in ("shared_expert.gate_proj", "shared_expert.up_proj", "shared_expert.down_proj", "shared_expert_gate"):
                t = _load(find(pat, f"mlp.{nm}.weight"))
                t = t.reshape(t.shape[0], -1) if t.ndim == 2 else t.reshape(1, -1)
                out.add_q4(dst + ".mlp." + nm, *pack_q4(t))
        # the head (optional in stripped test checkpoints)
        emb = find(r"^(model\.language_model\.|model\.|language_model\.model\.)", "embed_tokens.weight")
        if emb is not None:
            out.add_q4("language_model.model.embed_tokens", *pack_q4(_load(emb)))
        fnorm = find(r"^(model\.language_model\.|model\.|language_model\.model\.)", "norm.weight")
        if fnorm is not None:
            nv = _f32(_load(fnorm)).reshape(-1)
            if version == "3.6":
                nv = nv + np.float32(1.0)
            out.add_bf16("language_model.model.norm.weight", _ref_bf16(nv), flat=True)
        head = find(r"^(language_model\.)?", "lm_head.weight")
        if head is not None:
            t = _load(head)
            if scheme == "bq4":
                q, sc = eng.pack_int8(t if t.dtype == np.uint16 else _f32(t))
                out.add_int8("language_model.lm_head", q, sc)
            else:
                out.add_q4("language_model.lm_head", *pack_q4(t))
    finally:
        out.close()
        eng.close()
