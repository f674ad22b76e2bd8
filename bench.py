#!/usr/bin/env python3
"""Benchmark of the 4-bit MoE hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Default workload `decode`: one token through a 40-layer Qwen3.6-35B-A3B-shaped MoE stack
(256 experts, top-8, hidden 2048, BQ4 scheme), synthetic seeded weights resident in HBM.
One step = one 40-layer decode of one token; metric = decode tokens/s.
With N > 1 (torchrun) every rank holds its own replica and decodes its own token stream
(batch-1 decode does not shard; no data-path collective): weak scaling.

Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

NCU_DRAM_BYTES_PER_LAYER = 17.24e6  # (68.00 MB read + 0.97 MB written) / 4 layers
N_ROTATE = 64  # distinct input tokens cycled through, so routing differs from step to step


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None,
                    help="timed steps (default 2000; 20 for --impl reference and the prefill workload)")
    ap.add_argument("--warmup", type=int, default=None,
                    help="untimed steps (default 20; 3 for --impl reference and the prefill workload)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="decode", choices=["decode", "layer", "pack", "matvec", "batched64", "prefill"])
    ap.add_argument("--layers", type=int, default=40)
    ap.add_argument("--tokens", type=int, default=0, help="tokens per step for the batched workloads")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    slow = args.impl == "reference" or args.workload == "prefill"
    if args.steps is None:
        args.steps = 20 if slow else 2000
    if args.warmup is None:
        args.warmup = 3 if slow else 20
    return args


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


class Dist:
    """Barrier and max-over-ranks; torch.distributed only when there is more than one rank."""

    def __init__(self, world: int, local: int):
        self.world = world
        self.t = None
        if world > 1:
            import torch
            import torch.distributed as dist
            torch.cuda.set_device(local)
            dist.init_process_group("nccl", device_id=torch.device("cuda", local))
            self.t, self.d = torch, dist

    def barrier(self):
        if self.t is not None:
            self.d.barrier()
            self.t.cuda.synchronize()

    def max(self, v: float) -> float:
        if self.t is None:
            return v
        x = self.t.tensor([v], dtype=self.t.float64, device="cuda")
        self.d.all_reduce(x, op=self.d.ReduceOp.MAX)
        return float(x.item())

    def sum(self, v: float) -> float:
        if self.t is None:
            return v
        x = self.t.tensor([v], dtype=self.t.float64, device="cuda")
        self.d.all_reduce(x, op=self.d.ReduceOp.SUM)
        return float(x.item())

    def close(self):
        if self.t is not None:
            self.d.destroy_process_group()


# ─── CPU arm: the oracle port timed on the host cores ─────────────────────────

def cpu_decode_sample(dims, n_layers_sample: int, threads: int, target_s: float = 12.0, seed: int = 0):
    """Times the CPU restatement of the reference's decode path on a bounded sample.

    `threads` independent token streams (one per thread, like `threads` copies of the
    reference's single-threaded CpuEngine) each walk `n_layers_sample` MoE blocks.
    Expert words are random nibbles with fixed plausible scale/bias: the CPU time of
    the scalar loop does not depend on the values.  Returns (tok/s scaled to the
    full stack, description).
    """
    import oracle
    from benchmarks import synth
    oracle.build()
    rng = np.random.default_rng(seed)
    H, I, E, K = dims.hidden, dims.inter, dims.num_experts, dims.top_k
    lay = oracle.expert_layout(H, I)
    s_bits = int(oracle.f32_to_bf16(np.array([0.0063], np.float32))[0])
    b_bits = int(oracle.f32_to_bf16(np.array([-0.047], np.float32))[0])

    def q4(rows, cols):
        w = rng.integers(0, 2**32, size=(rows, cols // 8), dtype=np.uint64).astype(np.uint32)
        return w, np.full((rows, cols // 64), s_bits, np.uint16), np.full((rows, cols // 64), b_bits, np.uint16)

    layers = []
    for _ in range(n_layers_sample):
        blob = np.empty(E * lay["expert_size"], np.uint8)
        one = np.empty(lay["expert_size"], np.uint8)
        for name, rows, cols in (("gate", I, H), ("up", I, H), ("down", H, I)):
            w, s, b = q4(rows, cols)
            o = lay[name + "_w"]
            one[o:o + w.nbytes] = w.view(np.uint8).ravel()
            one[lay[name + "_s"]:lay[name + "_s"] + s.nbytes] = s.view(np.uint8).ravel()
            one[lay[name + "_b"]:lay[name + "_b"] + b.nbytes] = b.view(np.uint8).ravel()
        blob.reshape(E, -1)[:] = one  # every expert the same bytes: timing only
        layers.append(oracle.LayerWeights(
            hidden=H, inter=I, shared_inter=dims.shared_inter, num_experts=E,
            post_norm_w=oracle.f32_to_bf16(np.ones(H, np.float32)),
            router_bf16=oracle.f32_to_bf16((rng.standard_normal((E, H)) * 0.02).astype(np.float32)),
            router_q4=None, sh_gate=q4(dims.shared_inter, H), sh_up=q4(dims.shared_inter, H),
            sh_down=q4(H, dims.shared_inter), sgate=q4(1, H), experts=blob))
    h = synth.hidden_states(seed, 2, threads, H)
    # warm-up + calibration
    t0 = time.perf_counter()
    oracle.moe_layer(layers[0], h, K, threads=threads)
    per_layer = time.perf_counter() - t0
    reps = max(1, int(target_s / max(per_layer * n_layers_sample, 1e-6)))
    t0 = time.perf_counter()
    for _ in range(reps):
        x = h
        for lw in layers:
            x, _, _ = oracle.moe_layer(lw, x, K, threads=threads)
    dt = time.perf_counter() - t0
    layer_tokens_per_s = reps * n_layers_sample * threads / dt
    tok_s = layer_tokens_per_s / dims.num_layers
    desc = (f"{threads} independent token streams (1 thread each) x {n_layers_sample} of {dims.num_layers} MoE blocks "
            f"x {reps} reps, {dt:.1f} s of CPU work, scaled to the full stack; random packed bytes of the config's shapes")
    return tok_s, desc


def run_reference(args, rank, world):
    if rank != 0:
        return
    from moe_infer_b200.native import Dims
    dims = Dims(num_layers=args.layers)
    threads = os.cpu_count() or 1
    # one step of this arm = one bounded sample; K steps + W warm-ups must end within minutes
    per = max(2.0, min(12.0, 120.0 / max(args.steps + args.warmup, 1)))
    vals = []
    desc = ""
    for i in range(args.warmup + args.steps):
        v, desc = cpu_decode_sample(dims, 2, threads, target_s=per, seed=args.seed + i)
        if i >= args.warmup:
            vals.append(v)
    value = float(np.mean(vals)) if vals else 0.0
    line = {
        "impl": "reference", "metric": "moe_decode_tokens_per_s", "value": value, "unit": "tok/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1000.0 / value if value else None,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"decode 1 token x {dims.num_layers} MoE layers, 256 experts top-8, hidden 2048, BQ4",
                   "note": "CPU restatement of the reference's CpuEngine MoE path (the Rust crate cannot be built here)"},
        "cpu_baseline": {"value": value, "unit": "tok/s", "cores": threads, "kind": "port", "sample": desc},
        "e2e": {"value": value, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ─── our arm ──────────────────────────────────────────────────────────────────

def run_decode(args, rank, world, local, dist):
    from moe_infer_b200 import _lib as L
    from benchmarks import benchlib, synth
    from moe_infer_b200.native import Dims, NativeEngine, PinnedArray

    dims = Dims(num_layers=args.layers)
    eng = NativeEngine(dims, device=local)
    t_build = benchlib.populate_synthetic(eng, base_seed=args.seed + 1000 * rank)
    H = dims.hidden
    emb_host = synth.hidden_states(args.seed + rank, 2, N_ROTATE, H)
    emb_dev = eng.alloc(emb_host.nbytes).upload(emb_host)
    out_dev = eng.alloc(N_ROTATE * H * 4)
    K, W = args.steps, args.warmup

    def step_dev(i):
        t = i % N_ROTATE
        eng.forward_hidden_dev(emb_dev.ptr + t * H * 4, 1, False, out_dev.ptr + t * H * 4)

    for i in range(W):
        step_dev(i)
    eng.sync()
    dist.barrier()
    n0 = eng.launch_count()
    with benchlib.ClockSampler(local) as clk:
        eng.timer_start()
        for i in range(K):
            step_dev(W + i)
        ms = eng.timer_stop()
        eng.sync()
    launches = eng.launch_count() - n0
    dist.barrier()
    ms_max = dist.max(ms)

    # end to end through the host-pointer C ABI: pinned host input, host output
    pin_in = PinnedArray((N_ROTATE, H), np.float32)
    pin_in.array[:] = emb_host
    pin_out = PinnedArray((1, H), np.float32)
    for i in range(min(W, 5)):
        eng.forward_hidden(pin_in.array[i % N_ROTATE], out=pin_out.array)
    dist.barrier()
    t0 = time.perf_counter()
    for i in range(K):
        eng.forward_hidden(pin_in.array[(W + i) % N_ROTATE], out=pin_out.array)
    e2e_s = time.perf_counter() - t0
    e2e_s = dist.max(e2e_s)
    finite = bool(np.isfinite(pin_out.array).all())

    tok_s = world * K / (ms_max / 1e3)
    e2e_tok_s = world * K / e2e_s
    peaks = benchlib.measured_peaks()
    bytes_per_launch = benchlib.layer_token_bytes(dims) * dims.num_layers
    achieved = bytes_per_launch / (ms / K / 1e3) / 1e9

    # DRAM bytes (read + write) per layer from the ncu capture of a 4-layer launch of this kernel; every layer's
    # weights are read once, so a launch's traffic is that figure times the layer count.
    default_shape = (dims.hidden, dims.inter, dims.num_experts, dims.top_k) == (2048, 512, 256, 8)
    traffic = NCU_DRAM_BYTES_PER_LAYER * dims.num_layers if default_shape else None
    traffic_src = "ncu dram__bytes_read+write of a 4-layer launch, per layer, x layers" if default_shape else None

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        v, desc = cpu_decode_sample(dims, 2, 1, target_s=10.0, seed=args.seed)
        cpu = {"value": v, "unit": "tok/s", "cores": 1, "kind": "port", "sample": desc}

    if rank == 0:
        line = {
            "metric": "moe_decode_tokens_per_s", "value": tok_s, "unit": "tok/s", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": ms_max / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "u4 weights x 24-bit fixed-point activations (three s8 digits), exact s32 dp4a sums, f32 scales", "data": "synthetic",
            "config": {"workload": f"decode 1 token x {dims.num_layers} MoE layers, 256 experts top-8, hidden 2048, "
                                   "inter 512, BQ4 (bf16 router), attention passed through",
                       "replicas": world, "resident_store_GB": round(eng.resident_bytes() / 1e9, 2),
                       "l2": f"each step streams {bytes_per_launch / 1e6:.0f} MB of weights (> 126 MB L2); inputs rotate over "
                             f"{N_ROTATE} tokens so routing changes every step",
                       "store_build_s": round(t_build, 1), "finite": finite},
            "clocks": clk.summary(),
            "e2e": {"value": e2e_tok_s, "unit": "tok/s", "h2d_bytes_per_step": H * 4, "d2h_bytes_per_step": H * 4},
            "gpu_launches": int(launches),
            "roofline": {"bound": "hbm", "kernel": "decode_fused_kernel", "achieved": achieved, "peak": peaks["hbm_gbs"],
                         "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"], "peak_source": peaks["source"],
                         "frac_of_nominal_8TBs": achieved / 8000.0, "bytes_per_launch": bytes_per_launch,
                         "traffic": traffic, "traffic_source": traffic_src},
        }
        if cpu:
            line["cpu_baseline"] = cpu
        print(json.dumps(line), flush=True)
    for b in (emb_dev, out_dev):
        b.free()
    pin_in.free()
    pin_out.free()
    eng.close()


def main():
    args = parse()
    rank, world, local = dist_env()
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    dist = Dist(world, local)
    try:
        if args.workload == "decode":
            run_decode(args, rank, world, local, dist)
        else:
            from benchmarks import workloads as bench_extra
            bench_extra.run(args, rank, world, local, dist)
    finally:
        dist.close()


if __name__ == "__main__":
    main()
