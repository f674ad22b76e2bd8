"""Seeded synthetic tensors with the shapes and value distributions of the
Qwen3.6-35B-A3B MoE blocks (no checkpoint or dataset is read).

Weights are N(0, 0.02^2); activations are N(0, 1) rounded to bf16 and widened
back to f32.  Packing is left to the caller (the GPU packer in the product, the
CPU oracle in tests), passed in as callables.
"""
from __future__ import annotations

import hashlib
from typing import Callable, Optional, Tuple

import numpy as np

ROLES = ("experts_gate_up", "experts_down", "router", "shared_gate", "shared_up", "shared_down",
         "shared_sgate", "post_norm", "hidden")


def tensor_seed(base_seed: int, config_id: int, layer: int, role: str, extra: int = 0) -> int:
    h = hashlib.sha256(f"{base_seed}:{config_id}:{layer}:{role}:{extra}".encode()).digest()
    return int.from_bytes(h[:8], "little")


def rng_for(base_seed: int, config_id: int, layer: int, role: str, extra: int = 0) -> np.random.Generator:
    return np.random.Generator(np.random.PCG64(tensor_seed(base_seed, config_id, layer, role, extra)))


def to_bf16_rne(x: np.ndarray) -> np.ndarray:
    """f32 -> bf16 bit patterns with IEEE round-to-nearest-even (input data only)."""
    u = np.ascontiguousarray(x, np.float32).view(np.uint32)
    r = ((u >> 16) & 1) + 0x7FFF
    return ((u + r) >> 16).astype(np.uint16)


def bf16_to_f32(u16: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(u16, np.uint16).astype(np.uint32) << 16).view(np.float32)


def normal_weights(rng: np.random.Generator, shape, sigma: float = 0.02, outlier_frac: float = 0.0,
                   outlier_sigmas: float = 20.0) -> np.ndarray:
    w = rng.standard_normal(shape, dtype=np.float32) * np.float32(sigma)
    if outlier_frac > 0.0:
        n = int(round(w.size * outlier_frac))
        if n:
            pos = rng.choice(w.size, size=n, replace=False)
            sign = rng.integers(0, 2, size=n) * 2 - 1
            w.reshape(-1)[pos] = (sign * outlier_sigmas * sigma).astype(np.float32)
    return w


def hidden_states(base_seed: int, config_id: int, n_tokens: int, hidden: int) -> np.ndarray:
    """N(0,1) rounded to bf16, returned as f32 [n, hidden]."""
    rng = rng_for(base_seed, config_id, 0, "hidden")
    return bf16_to_f32(to_bf16_rne(rng.standard_normal((n_tokens, hidden), dtype=np.float32)))


def layer_tensors(base_seed: int, config_id: int, layer: int, *, hidden: int, inter: int, shared_inter: int,
                  num_experts: int, bf16_source: bool = False, outlier_frac: float = 0.0) -> dict:
    """Raw (unpacked) f32 tensors of one MoE block in HF orientation.

    gate_up [E, 2I, H], down [E, H, I], router [E, H], shared_{gate,up} [SI, H],
    shared_down [H, SI], shared_sgate [1, H], post_norm [H] (all ones).
    With bf16_source the values are first rounded to bf16 (what an HF bf16
    checkpoint holds) and widened back, so f32 and bf16 packer inputs agree.
    """
    def gen(role, shape):
        w = normal_weights(rng_for(base_seed, config_id, layer, role), shape, outlier_frac=outlier_frac)
        return bf16_to_f32(to_bf16_rne(w)) if bf16_source else w

    return {
        "gate_up": gen("experts_gate_up", (num_experts, 2 * inter, hidden)),
        "down": gen("experts_down", (num_experts, hidden, inter)),
        "router": gen("router", (num_experts, hidden)),
        "shared_gate": gen("shared_gate", (shared_inter, hidden)),
        "shared_up": gen("shared_up", (shared_inter, hidden)),
        "shared_down": gen("shared_down", (hidden, shared_inter)),
        "shared_sgate": gen("shared_sgate", (1, hidden)),
        "post_norm": np.ones(hidden, np.float32),
    }


def zipf_logit_bias(base_seed: int, num_experts: int, alpha: float = 1.1, strength: float = 1.0) -> np.ndarray:
    """logit_bias[e] = strength * ln p_e with p_e ~ rank_e^-alpha over a seeded permutation."""
    rng = rng_for(base_seed, 3, 0, "router", 7)
    ranks = rng.permutation(num_experts) + 1
    p = ranks.astype(np.float64) ** (-alpha)
    p /= p.sum()
    return (strength * np.log(p)).astype(np.float32)
