"""HF safetensors checkpoint -> converted model directory (Qwen3.5 / Qwen3.6 MoE, BQ4 and INT4 schemes).

Follows the reference's quantize pipeline (src/quantize.rs:71-365 and
src/quantize/qwen35_moe/{common,bq4,int4}.rs):

  1. every tensor of every shard gets its manifest name (`manifest_name`: the reference's name table
     name_mapping.json, written here as rules) and a storage type by scheme (`storage_type`: bq4.rs:25-44,
     int4.rs:24-35); vision tensors are skipped (common.rs:183-185);
  2. values are sanitised (`sanitise`: +1 on zero-centred norms for Qwen3.6, common.rs:187-227; conv1d weights
     [C, K, S] -> [C, S, K], common.rs:229-242), 4-bit tensors get their inner dimension zero-padded to a multiple
     of 64 (src/quantize.rs:230-249), and the encoded tensor(s) go into model_weights.bin, 64-byte aligned, under
     `<name>` (bf16 / f32, shape [len]) or `<base>.weight/.scales/.biases` (4-bit) or `<base>.weight/.scales`
     (INT8) (src/quantize.rs:251-291, src/dtype.rs:443-475);
  3. the experts `...mlp.experts.gate_up_proj` [E, 2I, H] and `...mlp.experts.down_proj` [E, H, I] of every layer
     (MTP block = layer index num_hidden_layers) become packed_experts/layer_NN.bin (common.rs:243-358);
  4. the manifest carries the reference's `config` block (common.rs:362-411).

The 4-bit and INT8 codecs and the bf16 rounding are the GPU packers' (bit-exact with src/dtype.rs:85-135, 164-179);
tensors too small to matter (norms, biases, A_log) are encoded on the host with the same rounding.
"""
from __future__ import annotations

import json
import os
import struct
from typing import Dict, List, Optional, Tuple

import numpy as np

from . import _lib as L
from .modeldir import ARCHS, ModelDirWriter
from .native import Dims, NativeEngine

GROUP = 64


# ── safetensors ──────────────────────────────────────────────────────────────

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


# ── names, storage types, sanitisation ───────────────────────────────────────

def manifest_name(hf_name: str) -> str:
    """HF tensor name -> name in the manifest (what the reference's name table does, as rules).

    model.language_model.X -> language_model.model.X; lm_head.X -> language_model.lm_head.X;
    model.visual.X -> vision_tower.X; the fused expert tensors `mlp.experts.gate_up_proj` / `mlp.experts.down_proj`
    -> `mlp.switch_mlp.{gate_up,down}_proj.weight` (also under mtp.layers.N.); everything else keeps its name.
    """
    name = hf_name
    if name.startswith("model.language_model."):
        name = "language_model.model." + name[len("model.language_model."):]
    elif name.startswith("lm_head."):
        name = "language_model." + name
    elif name.startswith("model.visual."):
        name = "vision_tower." + name[len("model.visual."):]
    for hf_tail, tail in ((".mlp.experts.gate_up_proj", ".mlp.switch_mlp.gate_up_proj.weight"),
                          (".mlp.experts.down_proj", ".mlp.switch_mlp.down_proj.weight")):
        if name.endswith(hf_tail):
            name = name[:-len(hf_tail)] + tail
    return name


def is_expert_tensor(name: str) -> bool:
    return any(f".switch_mlp.{p}." in name for p in ("gate_proj", "gate_up_proj", "up_proj", "down_proj"))


def layer_of(name: str) -> Optional[int]:
    """First `layers.<digits>.` in the name (common.rs:154-176)."""
    pos = 0
    while True:
        pos = name.find("layers.", pos)
        if pos < 0:
            return None
        rest = name[pos + 7:]
        digits = len(rest) - len(rest.lstrip("0123456789"))
        if digits and len(rest) > digits and rest[digits] == ".":
            return int(rest[:digits])
        pos += 7


def _block_of(prefix: str) -> str:
    """The part of a tensor's prefix that names its block inside a layer (common.rs:130-150)."""
    for head, per_layer in (("language_model.model.layers.", True), ("language_model.", False),
                            ("vision_tower.blocks.", True), ("vision_tower.", False),
                            ("mtp.layers.", True), ("mtp.", False)):
        if prefix.startswith(head):
            rest = prefix[len(head):]
            if per_layer:
                dot = rest.find(".")
                return rest[dot + 1:] if dot >= 0 else rest
            return rest
    return prefix


_BQ4_BF16_BLOCKS = ("self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "self_attn.o_proj", "mlp.gate",
                    "attn.qkv", "attn.proj", "patch_embed.proj", "pos_embed")


def storage_type(name: str, shape, scheme: str) -> str:
    """'f32' | 'bf16' | 'int4' | 'int8' for a manifest name (bq4.rs:25-44, int4.rs:24-35)."""
    prefix, _, kind = name.rpartition(".")
    if kind == "A_log":
        return "f32"
    if kind != "weight" or len(shape) != 2:
        return "bf16"
    if scheme == "int4":
        return "int4"
    block = _block_of(prefix)
    if block in _BQ4_BF16_BLOCKS:
        return "bf16"
    return "int8" if block == "lm_head" else "int4"


_ZC_NORM_SUFFIXES = (".input_layernorm.weight", ".post_attention_layernorm.weight", ".q_norm.weight", ".k_norm.weight",
                     ".pre_fc_norm_hidden.weight", ".pre_fc_norm_embedding.weight")


def is_zero_centred_norm(name: str) -> bool:
    """Norms that the model applies as x * (1 + w) (common.rs:187-227); the gated norm of the linear-attention
    block is an ordinary RMS norm and is not one of them."""
    if name.endswith(".linear_attn.norm.weight"):
        return False
    if name.endswith(_ZC_NORM_SUFFIXES):
        return True
    return name.endswith("model.norm.weight") or name == "mtp.norm.weight"


def sanitise(name: str, vals: np.ndarray, version: str) -> np.ndarray:
    """+1 on zero-centred norms for Qwen3.6 (bq4.rs:113-116); conv1d [C, K, S] -> [C, S, K] (common.rs:229-242)."""
    if version == "3.6" and is_zero_centred_norm(name):
        vals = vals + np.float32(1.0)
    if "conv1d.weight" in name and vals.ndim == 3:
        vals = np.ascontiguousarray(np.moveaxis(vals, 2, 1))
    return vals


def manifest_config(tc: dict) -> dict:
    """The manifest's `config` block (common.rs:362-411), from the text config of config.json."""
    rope = tc.get("rope_parameters") or {}
    n_main, n_mtp = int(tc.get("num_hidden_layers", 0)), int(tc.get("mtp_num_hidden_layers", 0))
    interval = int(tc.get("full_attention_interval", 4))
    cfg = {
        "hidden_size": int(tc.get("hidden_size", 0)),
        "num_hidden_layers": n_main + n_mtp,
        "num_attention_heads": int(tc.get("num_attention_heads", 0)),
        "num_key_value_heads": int(tc.get("num_key_value_heads", 0)),
        "head_dim": int(tc.get("head_dim", 0)),
        "vocab_size": int(tc.get("vocab_size", 0)),
        "rms_norm_eps": float(tc.get("rms_norm_eps", 1e-6)),
        "num_experts": int(tc.get("num_experts", 0)),
        "num_experts_per_tok": int(tc.get("num_experts_per_tok", 0)),
        "moe_intermediate_size": int(tc.get("moe_intermediate_size", 0)),
        "shared_expert_intermediate_size": int(tc.get("shared_expert_intermediate_size", 0)),
        "full_attention_interval": interval,
        "linear_num_value_heads": int(tc.get("linear_num_value_heads", 32)),
        "linear_num_key_heads": int(tc.get("linear_num_key_heads", 16)),
        "linear_key_head_dim": int(tc.get("linear_key_head_dim", 128)),
        "linear_value_head_dim": int(tc.get("linear_value_head_dim", 128)),
        "linear_conv_kernel_dim": int(tc.get("linear_conv_kernel_dim", 4)),
        "partial_rotary_factor": float(tc.get("partial_rotary_factor", rope.get("partial_rotary_factor", 0.25))),
        "rope_theta": float(tc.get("rope_theta", rope.get("rope_theta", 10_000_000.0))),
        "mtp_num_hidden_layers": n_mtp,
    }
    # the MTP blocks count as full-attention layers
    cfg["layer_types"] = ["full_attention" if (i + 1) % interval == 0 else "linear_attention" for i in range(n_main)] \
        + ["full_attention"] * n_mtp
    return cfg


# ── the pipeline ─────────────────────────────────────────────────────────────

def quantize_moe_checkpoint(model_path: str, output_dir: str, *, version: str, scheme: str, device: int = 0) -> Dict[str, int]:
    """Converts a checkpoint directory; returns how many tensors were stored per storage type."""
    if scheme not in ("bq4", "int4"):
        raise ValueError(f"unknown scheme {scheme!r}")
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
    out = ModelDirWriter(output_dir, config, manifest_config(tc))
    summary: Dict[str, int] = {}
    experts: Dict[int, List[Optional[tuple]]] = {}

    def pack_q4(t: np.ndarray):
        """4-bit triple of a 2-D tensor; the inner dimension is zero-padded to a multiple of 64 first."""
        rows, cols = t.shape
        if cols % GROUP:
            padded = np.zeros((rows, (cols + GROUP - 1) // GROUP * GROUP), t.dtype)
            padded[:, :cols] = t
            t = padded
        return eng.pack_int4(t)

    try:
        # non-expert tensors, in name order (the reference walks a hash map: its order is unspecified)
        for hf_name in sorted(index):
            entry = index[hf_name]
            name = manifest_name(hf_name)
            if name.startswith("vision_tower."):
                continue
            if is_expert_tensor(name):
                layer = layer_of(hf_name)
                if layer is not None:
                    if hf_name.startswith("mtp."):
                        layer += n_layers
                    slot = experts.setdefault(layer, [None, None])
                    if "gate_up_proj" in name or "gate_proj" in name:
                        slot[0] = entry
                    elif "down_proj" in name:
                        slot[1] = entry
                    continue
            kind = storage_type(name, entry[2], scheme)
            summary[kind] = summary.get(kind, 0) + 1
            raw = _load(entry)
            touched = (version == "3.6" and is_zero_centred_norm(name)) or ("conv1d.weight" in name and raw.ndim == 3)
            if kind in ("int4", "int8"):
                base = name[:-len(".weight")] if name.endswith(".weight") else name
                # bf16 sources go to the GPU packer as they are (widening is exact); nothing sanitises a matrix
                t = raw if raw.dtype == np.uint16 else _f32(raw)
                if kind == "int4":
                    out.add_q4(base, *pack_q4(t))
                else:
                    out.add_int8(base, *eng.pack_int8(t))
            elif kind == "f32":
                out.add_f32(name, sanitise(name, _f32(raw), version).reshape(-1))
            else:
                bits = raw.reshape(-1) if (raw.dtype == np.uint16 and not touched) \
                    else _ref_bf16(sanitise(name, _f32(raw), version)).reshape(-1)
                out.add_bf16(name, bits, flat=True)
        # experts, one file per layer
        for l in range(n_layers + n_mtp):
            gu, dn = experts.get(l, [None, None])
            if gu is None or dn is None:
                raise ValueError(f"layer {l}: expert tensors mlp.experts.gate_up_proj / down_proj not found")
            out.add_expert_layer(l, eng.pack_experts(_load(gu), _load(dn)))
    finally:
        out.close()
        eng.close()
    return summary
