#!/usr/bin/env python3
"""Benchmark of the 4-bit MoE hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Headline (default workload `decode`): one token through a 40-layer Qwen3.6-35B-A3B-shaped MoE stack (256 experts,
top-8, hidden 2048, BQ4 scheme), synthetic seeded weights resident in HBM.  One step = one 40-layer decode of one
token; metric = decode tokens/s.  With N > 1 (torchrun) every rank holds its own replica and decodes its own token
stream (batch-1 decode does not shard; no data-path collective): weak scaling.

The same JSON line carries a `secondary` object, filled in the same process after the headline: the 4,096-token
prefill (one GPU: grouped tensor-core path; N > 1: experts sharded over the ranks, dispatch/combine over NVLink),
the packer (N > 1: layers split over the ranks) and, on one GPU, the 64-token batched decode, the single-block decode
and the dequant-matvec at 512 x 2048 and at an HBM-sized shape.  Every timed figure is the median over repeats of its
timed region (CUDA events, barrier + synchronize on both sides, max over ranks).

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

NCU_DRAM_BYTES_PER_LAYER = 17.44e6  # (68.05 MB read + 1.70 MB written) / 4 layers: profiles/decode_slots_kernel_4layers.md
N_ROTATE = 64  # distinct input tokens cycled through, so routing differs from step to step
DECODE_DTYPE = "u4 weights x 24-bit fixed-point activations (three s8 digits), exact s32 dp4a sums, f32 scales"


def decode_workload(layers: int) -> str:
    """The headline workload's name: printed identically by both arms."""
    return (f"decode 1 token x {layers} MoE layers, 256 experts top-8, hidden 2048, inter 512, BQ4 (bf16 router), "
            "attention passed through")


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None,
                    help="timed steps per region (default 200; 20 for --impl reference)")
    ap.add_argument("--warmup", type=int, default=None, help="untimed steps (default 20; 3 for --impl reference)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="decode",
                    choices=["decode", "layer", "pack", "matvec", "matvec_hbm", "lm_head", "full_decode", "batched64", "prefill"])
    ap.add_argument("--layers", type=int, default=40)
    ap.add_argument("--tokens", type=int, default=0, help="tokens per step for the batched workloads")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-secondary", action="store_true", help="headline only")
    args = ap.parse_args()
    slow = args.impl == "reference"
    if args.steps is None:
        args.steps = 20 if slow else 200
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

    def close(self):
        if self.t is not None:
            self.d.destroy_process_group()


# ─── CPU arm: the oracle port timed on the host cores ─────────────────────────

def cpu_decode_sample(dims, n_layers_sample: int, threads: int, target_s: float = 12.0, seed: int = 0):
    """Times the CPU restatement of the reference's decode path on a bounded sample.

    `threads` independent token streams (one per thread, like `threads` copies of the reference's single-threaded
    CpuEngine) each walk `n_layers_sample` MoE blocks.  Expert words are random nibbles with fixed plausible
    scale/bias: the CPU time of the scalar loop does not depend on the values.  Returns (tok/s scaled to the full
    stack, description).
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
        "config": {"workload": decode_workload(dims.num_layers),
                   "note": "CPU restatement of the reference's CpuEngine MoE path (the Rust crate cannot be built here). "
                           "The figure is a throughput over one independent batch-1 token stream per host thread, which "
                           "favours this arm against the GPU arm's single-stream latency; every sampled block reads the "
                           "same expert bytes, which favours it again (cache-resident weights)."},
        "cpu_baseline": {"value": value, "unit": "tok/s", "cores": threads, "kind": "port", "sample": desc},
        "e2e": {"value": value, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ─── our arm ──────────────────────────────────────────────────────────────────

def run_decode(args, rank, world, local, dist):
    from benchmarks import benchlib, synth, workloads
    from moe_infer_b200.native import Dims, NativeEngine, PinnedArray

    dims = Dims(num_layers=args.layers)
    eng = NativeEngine(dims, device=local)
    host_tensors = {} if (rank == 0 and world == 1 and not args.no_cpu_baseline) else None
    t_build = benchlib.populate_synthetic(eng, base_seed=args.seed + 1000 * rank, keep_host=host_tensors)
    H = dims.hidden
    emb_host = synth.hidden_states(args.seed + rank, 2, N_ROTATE, H)
    emb_dev = eng.alloc(emb_host.nbytes).upload(emb_host)
    out_dev = eng.alloc(N_ROTATE * H * 4)
    K, W = args.steps, args.warmup

    def step_dev(i):
        t = i % N_ROTATE
        eng.forward_hidden_dev(emb_dev.ptr + t * H * 4, 1, False, out_dev.ptr + t * H * 4)

    # device-resident: regions of exactly K steps, repeated for about 1.5 s so that the clock sampler sees the load
    with benchlib.ClockSampler(local) as clk:
        t = workloads.timed_repeats(eng, step_dev, W, K, dist, min_repeats=7, fill_s=1.5)
    ms_region = t["ms"]

    # end to end through the host-pointer C ABI: pinned host input, host output, copies inside the timed region
    pin_in = PinnedArray((N_ROTATE, H), np.float32)
    pin_in.array[:] = emb_host
    pin_out = PinnedArray((1, H), np.float32)
    for i in range(min(W, 5)):
        eng.forward_hidden(pin_in.array[i % N_ROTATE], out=pin_out.array)
    e2e_regions = []
    for r in range(7):
        dist.barrier()
        t0 = time.perf_counter()
        for i in range(K):
            eng.forward_hidden(pin_in.array[(W + r * K + i) % N_ROTATE], out=pin_out.array)
        e2e_regions.append(dist.max(time.perf_counter() - t0))
    e2e_s = float(np.median(e2e_regions))
    finite = bool(np.isfinite(pin_out.array).all())

    tok_s = world * K / (ms_region / 1e3)
    e2e_tok_s = world * K / e2e_s
    bytes_per_launch = benchlib.layer_token_bytes(dims) * dims.num_layers
    default_shape = (dims.hidden, dims.inter, dims.num_experts, dims.top_k) == (2048, 512, 256, 8)
    traffic = NCU_DRAM_BYTES_PER_LAYER * dims.num_layers if default_shape else None
    roof = workloads.hbm_roofline("decode_slots_kernel", bytes_per_launch, ms_region / K, traffic=traffic,
                                  traffic_source="ncu dram__bytes_read+write of a 4-layer launch, per layer, x layers"
                                  if default_shape else None)
    roof["bytes_per_launch"] = bytes_per_launch

    parity = {}
    cpu = None
    if host_tensors is not None:
        # the checker: the CPU oracle walks the same 40 layers on the same weights for one token
        from benchmarks import oracle_check
        got = eng.forward_hidden(emb_host[0])
        ref, matched = oracle_check.stack_against_oracle(eng, host_tensors, emb_host[0], dims.num_layers)
        parity["decode"] = {"rel_l2_vs_oracle": workloads.rel_l2(got[0], ref),
                            "rel_l2_of_update_vs_oracle": workloads.rel_l2(got[0] - emb_host[0], ref - emb_host[0]),
                            "layers_with_identical_expert_sets": f"{matched}/{dims.num_layers}"}
        v, desc = cpu_decode_sample(dims, 2, 1, target_s=10.0, seed=args.seed)
        cpu = {"value": v, "unit": "tok/s", "cores": 1, "kind": "port", "sample": desc}

    secondary = {}
    if not args.no_secondary and default_shape and args.layers >= 8:
        if world == 1:
            secondary["layer_decode"] = workloads.run_layer(args, eng, local)
            secondary["batched64"] = workloads.run_batched64(args, eng, local)
            parity["batched64"] = {"rel_l2_vs_decode_path": secondary["batched64"]["parity_rel_l2_vs_decode_path"]}
            secondary["matvec_512x2048"] = workloads.run_matvec(args, eng, local)
            secondary["matvec_hbm"] = workloads.run_matvec(args, eng, local, rows=248320, cols=2048, copies=2)
            secondary["full_decode"] = workloads.run_full_decode(args, eng, local)
    resident_gb = eng.resident_bytes() / 1e9
    for b in (emb_dev, out_dev):
        b.free()
    pin_in.free()
    pin_out.free()
    eng.close()
    if not args.no_secondary and default_shape and args.layers >= 8:
        secondary["prefill_4096x40"] = workloads.run_prefill(args, rank, world, local, dist, 4096, args.layers)
        parity["prefill_4096x40"] = {"rel_l2_vs_decode_path": secondary["prefill_4096x40"]["parity_rel_l2_vs_decode_path"],
                                     "rel_l2_vs_single_gpu": secondary["prefill_4096x40"]["parity_rel_l2_vs_single_gpu"]}
        secondary["pack"] = workloads.run_pack(args, rank, world, local, dist)
        if world == 1:
            secondary["lm_head_int8"] = workloads.run_lm_head(args, local, "int8")

    if rank == 0:
        line = {
            "metric": "moe_decode_tokens_per_s", "value": tok_s, "unit": "tok/s", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": ms_region / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": DECODE_DTYPE, "data": "synthetic",
            "config": {"workload": decode_workload(dims.num_layers), "replicas": world,
                       "resident_store_GB": round(resident_gb, 2),
                       "l2": f"each step streams {bytes_per_launch / 1e6:.0f} MB of weights (> 126 MB L2); inputs rotate over "
                             f"{N_ROTATE} tokens so routing changes every step",
                       "timing": f"median of {t['repeats']} regions of {K} steps (min {t['min_ms'] / K:.4f}, max "
                                 f"{t['max_ms'] / K:.4f} ms per step)",
                       "store_build_s": round(t_build, 1), "finite": finite, "parity_rel_l2": parity},
            "clocks": clk.summary(),
            "e2e": {"value": e2e_tok_s, "unit": "tok/s", "h2d_bytes_per_step": H * 4, "d2h_bytes_per_step": H * 4},
            "gpu_launches": int(t["launches"]),
            "roofline": roof,
        }
        if cpu:
            line["cpu_baseline"] = cpu
        if secondary:
            line["secondary"] = secondary
        print(json.dumps(line), flush=True)


def run_single(args, rank, world, local, dist):
    """One secondary workload by itself (`--workload NAME`): the same dict, printed as the line's `config`."""
    from benchmarks import benchlib, workloads
    from moe_infer_b200.native import Dims, NativeEngine
    name = args.workload
    if name == "prefill":
        r = workloads.run_prefill(args, rank, world, local, dist, args.tokens or 4096, args.layers)
        metric, unit, value, ms = "moe_prefill_tokens_per_s", "tok/s", r["tok_per_s"], r["ms_per_step"]
    elif name == "pack":
        r = workloads.run_pack(args, rank, world, local, dist)
        metric, unit, value, ms = "quantize_GB_per_s", "GB/s", r["GB_per_s"], r["ms_per_checkpoint"]
    elif name == "lm_head":
        r = workloads.run_lm_head(args, local, "int8")
        metric, unit, value, ms = "lm_head_GB_per_s", "GB/s", r["roofline"]["achieved"], r["us_per_call"] / 1e3
    else:
        small = name in ("matvec", "matvec_hbm")
        dims = Dims(num_layers=1, num_experts=4, top_k=4) if small else Dims(num_layers=args.layers if name == "full_decode" else min(args.layers, 12))
        eng = NativeEngine(dims, device=local)
        if not small:
            benchlib.populate_synthetic(eng, base_seed=args.seed)
        if name == "full_decode":
            r = workloads.run_full_decode(args, eng, local)
            metric, unit, value, ms = "decoder_decode_tokens_per_s", "tok/s", r["tok_per_s"], r["ms_per_token"]
        elif name == "layer":
            r = workloads.run_layer(args, eng, local)
            metric, unit, value, ms = "moe_layer_decode_us", "us", r["us_per_layer"], r["us_per_layer"] / 1e3
        elif name == "batched64":
            r = workloads.run_batched64(args, eng, local, args.tokens or 64)
            metric, unit, value, ms = "moe_batched_decode_tokens_per_s", "tok/s", r["tok_per_s"], r["ms_per_step"]
        elif name == "matvec":
            r = workloads.run_matvec(args, eng, local)
            metric, unit, value, ms = "matvec_GB_per_s", "GB/s", r["roofline"]["achieved"], r["us_per_call"] / 1e3
        else:
            r = workloads.run_matvec(args, eng, local, rows=248320, cols=2048, copies=2)
            metric, unit, value, ms = "matvec_GB_per_s", "GB/s", r["roofline"]["achieved"], r["us_per_call"] / 1e3
        eng.close()
    if rank == 0:
        roof = r.pop("roofline")
        print(json.dumps({"metric": metric, "value": value, "unit": unit, "n_gpus": world, "steps": args.steps,
                          "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": name != "layer",
                          "scaling": r.get("scaling", "weak"), "vs_baseline": None, "data": "synthetic", "config": r,
                          "gpu_launches": r.get("gpu_launches"), "roofline": roof}), flush=True)


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
            run_single(args, rank, world, local, dist)
    finally:
        dist.close()


if __name__ == "__main__":
    main()
