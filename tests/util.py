"""Shared helpers of the test-suite: synthetic MoE blocks packed by the CPU oracle."""
from __future__ import annotations

import numpy as np

import oracle
from benchmarks import synth


def rel_l2(a: np.ndarray, b: np.ndarray) -> float:
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


def make_layer(seed: int, layer: int, *, hidden=2048, inter=512, shared_inter=512, num_experts=8,
               scheme="bq4", config_id=2) -> oracle.LayerWeights:
    t = synth.layer_tensors(seed, config_id, layer, hidden=hidden, inter=inter, shared_inter=shared_inter,
                            num_experts=num_experts)
    blob = oracle.pack_experts_layer(t["gate_up"], t["down"])
    router_bf16 = router_q4 = None
    if scheme == "bq4":
        router_bf16 = oracle.f32_to_bf16(t["router"])
    else:
        router_q4 = oracle.quant_int4(t["router"])
    return oracle.LayerWeights(
        hidden=hidden, inter=inter, shared_inter=shared_inter, num_experts=num_experts,
        post_norm_w=oracle.f32_to_bf16(t["post_norm"]), router_bf16=router_bf16, router_q4=router_q4,
        sh_gate=oracle.quant_int4(t["shared_gate"]), sh_up=oracle.quant_int4(t["shared_up"]),
        sh_down=oracle.quant_int4(t["shared_down"]), sgate=oracle.quant_int4(t["shared_sgate"]), experts=blob)


def upload_layer(eng, layer: int, lw: oracle.LayerWeights) -> None:
    from moe_infer_b200.native import load_layer_weights
    load_layer_weights(eng, layer, post_norm_w=lw.post_norm_w, router_bf16=lw.router_bf16,
                       router_q4=lw.router_q4, sh_gate=lw.sh_gate, sh_up=lw.sh_up, sh_down=lw.sh_down,
                       sgate=lw.sgate, experts=lw.experts)


def routing_maps(idx: np.ndarray, wts: np.ndarray):
    """[(sorted expert ids, weights in that order)] per token, for order-free comparison."""
    out = []
    for i, w in zip(np.atleast_2d(idx), np.atleast_2d(wts)):
        o = np.argsort(i, kind="stable")
        out.append((i[o], w[o]))
    return out
