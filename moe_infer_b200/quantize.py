"""HF safetensors -> converted model directory, for the tensors of the MoE path.

Follows the reference's quantize pipeline (src/quantize.rs:71-365 and
src/quantize/qwen35_moe/{common,bq4,int4}.rs) for:
  * experts: `...mlp.experts.gate_up_proj` [E, 2I, H] and `...mlp.experts.down_proj` [E, H, I]
    -> packed_experts/layer_NN.bin (common.rs:300-345), packed on the GPU;
  * `mlp.gate` (bf16 in the BQ4 scheme, 4-bit in INT4: bq4.rs:25-32, int4.rs:24-35),
    `mlp.shared_expert.{gate,up,down}_proj`, `mlp.shared_expert_gate` (4-bit);
  * `post_attention_layernorm.weight` (bf16; +1 for Qwen3.6, bq4.rs:113-116).
The 4-bit codec and the bf16 rounding are the GPU packer's (bit-exact with
src/dtype.rs:85-135).  Attention, embedding, vision and lm_head tensors are skipped.
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

    try:
        for l in range(n_layers + n_mtp):
            if l < n_layers:
                pat, dst = r"^(?!mtp\.).*" + rf"layers\.{l}\.", f"model.layers.{l}"
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
            out.add_bf16(dst + ".post_attention_layernorm.weight", _ref_bf16(nv))
            router = _load(find(pat, "mlp.gate.weight"))
            if scheme == "bq4":
                out.add_bf16(dst + ".mlp.gate.weight", _ref_bf16(_f32(router)), flat=True)
            else:
                out.add_q4(dst + ".mlp.gate", *eng.pack_int4(router if router.dtype == np.uint16 else _f32(router)))
            for nm in ("shared_expert.gate_proj", "shared_expert.up_proj", "shared_expert.down_proj", "shared_expert_gate"):
                t = _load(find(pat, f"mlp.{nm}.weight"))
                t = t.reshape(t.shape[0], -1) if t.ndim == 2 else t.reshape(1, -1)
                out.add_q4(dst + ".mlp." + nm, *eng.pack_int4(t if t.dtype == np.uint16 else _f32(t)))
    finally:
        out.close()
        eng.close()
