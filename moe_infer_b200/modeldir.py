"""Reader and writer of the reference's on-disk model directory.

Layout (reference src/model.rs:26-112, src/model/weights.rs:82-179,
src/quantize.rs:150-291, src/quantize/qwen35_moe/common.rs:314-348):

    config.json                      HF config; keys at top level or under "text_config"
    model_weights.json               {"tensors": {name: {offset, size, shape, dtype}}, "config": {...}}
    model_weights.bin                tensor bytes, 64-byte aligned
    packed_experts/layer_%02d.bin    num_experts packed experts back to back, one file per
                                     layer, MTP block = index num_hidden_layers

dtype strings follow src/dtype.rs:34-43: "f32", "bf16", "u32" (= 4-bit words), "u8".
The engine reads only the tensors of the MoE path and of the model head (embedding table, final norm, lm_head);
the converter writes every tensor of the checkpoint, attention included.
"""
from __future__ import annotations

import json
import os
from typing import Dict, Optional, Tuple

import numpy as np

ALIGN = 64
ARCHS = ("Qwen3_5MoeForConditionalGeneration", "Qwen3_5MoeForConditionalGeneration_Stripped")
_NP = {"f32": np.float32, "bf16": np.uint16, "u32": np.uint32, "u8": np.uint8}


class ModelDir:
    """mmap view of a converted model directory."""

    def __init__(self, path: str):
        self.path = path
        cfg_path = os.path.join(path, "config.json")
        if not os.path.exists(cfg_path):
            raise RuntimeError(f"Config error: cannot read {cfg_path}")
        with open(cfg_path) as f:
            self.config = json.load(f)
        man_path = os.path.join(path, "model_weights.json")
        bin_path = os.path.join(path, "model_weights.bin")
        if not os.path.exists(man_path) or not os.path.exists(bin_path):
            raise RuntimeError(f"I/O error: {man_path} / {bin_path} missing")
        with open(man_path) as f:
            manifest = json.load(f)
        if "tensors" not in manifest:
            raise RuntimeError("Config error: No 'tensors' key in manifest")
        self.tensors: Dict[str, dict] = manifest["tensors"]
        self.data = np.memmap(bin_path, dtype=np.uint8, mode="r")
        if os.path.isdir(os.path.join(path, "packed_experts_lz4")):
            raise RuntimeError("packed_experts_lz4 is not supported: experts stay resident in HBM, use packed_experts/")

    # reference src/model/config.rs:10-25: top level first, then text_config
    def get(self, key: str, default=None):
        if key in self.config:
            return self.config[key]
        return self.config.get("text_config", {}).get(key, default)

    def get_usize(self, key: str, default: Optional[int] = None) -> int:
        v = self.get(key, default)
        if v is None:
            raise KeyError(key)
        return int(v)

    @property
    def architecture(self) -> str:
        archs = self.get("architectures", []) or []
        return archs[0] if archs else ""

    def tensor(self, name: str) -> Optional[np.ndarray]:
        for prefix in ("", "language_model."):
            info = self.tensors.get(prefix + name)
            if info is not None:
                dt = _NP[info["dtype"]]
                raw = self.data[info["offset"]:info["offset"] + info["size"]]
                return np.frombuffer(raw, dtype=dt).reshape(info["shape"]) if info["shape"] else np.frombuffer(raw, dtype=dt)
        return None

    def q4(self, base: str) -> Optional[Tuple[np.ndarray, np.ndarray, np.ndarray]]:
        w, s, b = self.tensor(base + ".weight"), self.tensor(base + ".scales"), self.tensor(base + ".biases")
        if w is None or s is None or b is None:
            return None
        return w, s, b

    def expert_file(self, layer: int) -> str:
        return os.path.join(self.path, "packed_experts", f"layer_{layer:02d}.bin")


class ModelDirWriter:
    """Writes tensors in the reference's manifest format (64-byte aligned, same suffixes)."""

    def __init__(self, path: str, config: dict, manifest_config: Optional[dict] = None):
        self.path = path
        os.makedirs(os.path.join(path, "packed_experts"), exist_ok=True)
        with open(os.path.join(path, "config.json"), "w") as f:
            json.dump(config, f, indent=1)
        self.bin = open(os.path.join(path, "model_weights.bin"), "wb")
        self.offset = 0
        self.tensors: Dict[str, dict] = {}
        self.manifest_config = manifest_config or {}

    def _put(self, name: str, arr: np.ndarray, dtype: str, shape) -> None:
        if self.offset % ALIGN:
            pad = ALIGN - self.offset % ALIGN
            self.bin.write(b"\0" * pad)
            self.offset += pad
        raw = np.ascontiguousarray(arr).tobytes()
        self.bin.write(raw)
        self.tensors[name] = {"offset": self.offset, "size": len(raw), "shape": list(shape), "dtype": dtype}
        self.offset += len(raw)

    def add_bf16(self, name: str, bits: np.ndarray, flat: bool = False) -> None:
        # encode_bf16 writes matrices with shape [len] (reference src/dtype.rs:456-460)
        self._put(name, bits.astype(np.uint16), "bf16", [bits.size] if flat else bits.shape)

    def add_f32(self, name: str, vals: np.ndarray) -> None:
        # encode_fp32 (reference src/dtype.rs:462-465): shape [len]
        self._put(name, vals.astype(np.float32), "f32", [vals.size])

    def add_q4(self, base: str, w: np.ndarray, s: np.ndarray, b: np.ndarray) -> None:
        self._put(base + ".weight", w.astype(np.uint32), "u32", w.shape)
        self._put(base + ".scales", s.astype(np.uint16), "bf16", s.shape)
        self._put(base + ".biases", b.astype(np.uint16), "bf16", b.shape)

    def add_int8(self, base: str, q: np.ndarray, scales: np.ndarray) -> None:
        # encode_int8 (reference src/dtype.rs:466-475): ".weight" as "u8" [out, in], ".scales" as "f32" [out]
        self._put(base + ".weight", np.ascontiguousarray(q).view(np.uint8), "u8", q.shape)
        self._put(base + ".scales", scales.astype(np.float32), "f32", scales.shape)

    def add_expert_layer(self, layer: int, blob: np.ndarray) -> None:
        with open(os.path.join(self.path, "packed_experts", f"layer_{layer:02d}.bin"), "wb") as f:
            f.write(np.ascontiguousarray(blob).tobytes())

    def close(self) -> None:
        self.bin.close()
        with open(os.path.join(self.path, "model_weights.json"), "w") as f:
            json.dump({"model": self.path, "num_tensors": len(self.tensors), "config": self.manifest_config,
                       "tensors": self.tensors}, f)
