"""Kernel timeline of the whole-decoder decode: one token's kernels with their start, duration and the overlap with the
kernel after them, from CUPTI activity records (``torch.profiler``; no replay, no clock control).

    python -m benchmarks.timeline [--layers 40] [--head 30]
    python -m benchmarks.timeline --prompt 56        # one call of 56 tokens: per-kernel totals

Timed figures belong to ``bench.py``; this only shows where a token's time goes.  A negative "gap after" is an overlap:
the next kernel was resident (programmatic dependent launch) before this one ended.
"""
from __future__ import annotations

import argparse
import collections
import types

import numpy as np


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=40)
    ap.add_argument("--head", type=int, default=30, help="kernels of the token to list one by one")
    ap.add_argument("--prompt", type=int, default=0, help="trace one call of this many tokens instead of single tokens")
    a = ap.parse_args()
    import torch
    from torch.profiler import ProfilerActivity, profile

    from moe_infer_b200 import _lib as L
    from moe_infer_b200.native import Dims, NativeEngine

    from . import benchlib, workloads

    torch.cuda.init()
    eng = NativeEngine(Dims(num_layers=a.layers), device=0)
    benchlib.populate_synthetic(eng, base_seed=0)
    r = workloads.run_full_decode(types.SimpleNamespace(seed=0, warmup=3, steps=4), eng, 0)
    print(f"untraced: {r['ms_per_token']:.3f} ms per token, {r['gpu_launches'] // 4} kernels per token")
    H = eng.dims.hidden
    if a.prompt:
        n = a.prompt
        emb = np.random.default_rng(0).standard_normal((n, H)).astype(np.float32)
        out = np.empty((n, H), np.float32)
        for _ in range(2):  # the first call sizes the work areas
            eng.model_reset()
            L.check(eng.lib.moe_model_forward_hidden_host(eng.h, L.ptr(emb), n, L.ptr(out)))
        eng.model_reset()
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            L.check(eng.lib.moe_model_forward_hidden_host(eng.h, L.ptr(emb), n, L.ptr(out)))
        evs = sorted((e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA), key=lambda e: e.time_range.start)
        tot = collections.defaultdict(lambda: [0, 0.0])
        for e in evs:
            name = e.name.split("(")[0].replace("moe::", "").replace("void ", "")[:44]
            tot[name][0] += 1
            tot[name][1] += e.time_range.end - e.time_range.start
        span = evs[-1].time_range.end - evs[0].time_range.start
        print(f"one call of {n} tokens: {span / 1e3:.2f} ms under the tracer = {span / 1e3 / n:.3f} ms per token, {len(evs)} kernels and copies")
        print(f"{'kernel':<46}{'n':>6}{'total ms':>11}{'mean us':>10}")
        for k, v in sorted(tot.items(), key=lambda kv: -kv[1][1]):
            print(f"{k:<46}{v[0]:>6}{v[1] / 1e3:>11.2f}{v[1] / v[0]:>10.2f}")
        eng.close()
        return
    emb = np.random.default_rng(0).standard_normal((1, H)).astype(np.float32)
    out = np.empty((1, H), np.float32)
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(3):
            L.check(eng.lib.moe_model_forward_hidden_host(eng.h, L.ptr(emb), 1, L.ptr(out)))
    evs = sorted((e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA), key=lambda e: e.time_range.start)
    tok = evs[2 * (len(evs) // 3):]  # the last of the three tokens
    t0 = tok[0].time_range.start
    dur, gap = collections.defaultdict(list), collections.defaultdict(list)
    print(f"{'start us':>9} {'dur us':>8}  kernel")
    for i, e in enumerate(tok):
        name = e.name.split("(")[0].replace("moe::", "").replace("void ", "")[:44]
        d = e.time_range.end - e.time_range.start
        dur[name].append(d)
        if i + 1 < len(tok):
            gap[name].append(tok[i + 1].time_range.start - e.time_range.end)
        if i < a.head:
            print(f"{e.time_range.start - t0:9.2f} {d:8.2f}  {name}")
    print(f"token span under the tracer: {tok[-1].time_range.end - t0:.1f} us")
    print(f"{'kernel':<46}{'n':>4}{'mean dur us':>13}{'mean gap after us':>19}")
    for k, v in dur.items():
        print(f"{k:<46}{len(v):>4}{np.mean(v):>13.2f}{(np.mean(gap[k]) if gap[k] else 0.0):>19.2f}")
    eng.close()


if __name__ == "__main__":
    main()
