"""Checks a full-size decode against the CPU oracle without copying the whole expert store to the host.

Test infrastructure: called only from ``tests/`` and from the ``cpu_baseline`` leg of ``bench.py``, as the checker
of what the GPU computed, never as the thing measured.

The oracle walks the stack layer by layer on the host copies of the non-expert tensors and on a sparse expert
blob: only the experts the GPU chose for the oracle's own hidden state are downloaded (8 x 1.77 MB per layer
instead of 453 MB).  The oracle still routes by itself; if it ever picked an expert that was not downloaded its
output would be computed from zeros and the comparison would fail, so a routing difference cannot hide.
"""
from __future__ import annotations

import numpy as np

from moe_infer_b200 import _lib as L
from moe_infer_b200.native import NativeEngine


def stack_against_oracle(eng: NativeEngine, host_tensors: dict, emb: np.ndarray, layers: int):
    """emb f32 [H]: one token.  Returns (oracle output [H], number of layers whose expert sets matched)."""
    import oracle
    oracle.build()
    d = eng.dims
    size = eng.layout["expert_size"]
    h = np.ascontiguousarray(emb, np.float32).reshape(1, d.hidden)
    matched = 0
    blob = np.zeros(d.num_experts * size, np.uint8)
    for l in range(layers):
        _, idx, _ = eng.layer_forward(l, h)  # the GPU's choice for this input: tells which experts to fetch
        base = eng.layer_dev(l)
        for e in idx[0]:
            e = int(e)
            L.check(eng.lib.moe_dev_download(eng.h, L.ptr(blob[e * size:(e + 1) * size]), base + e * size, size))
        t = host_tensors[l]
        lw = oracle.LayerWeights(hidden=d.hidden, inter=d.inter, shared_inter=d.shared_inter, num_experts=d.num_experts,
                                 post_norm_w=t["post_norm"], router_bf16=t["router_bf16"], router_q4=t["router_q4"],
                                 sh_gate=t["sh_gate"], sh_up=t["sh_up"], sh_down=t["sh_down"], sgate=t["sgate"], experts=blob)
        h, idx_ref, _ = oracle.moe_layer(lw, h, d.top_k)
        matched += int(set(idx_ref[0].tolist()) == set(idx[0].tolist()))
        for e in idx[0]:
            blob[int(e) * size:(int(e) + 1) * size] = 0
    return h[0], matched
