"""Secondary benchmark workloads (selected with ``bench.py --workload``).

layer      config 2: one MoE block, batch-1 decode, rotating over distinct layer copies
batched64  config 3: 64 tokens through one block, Zipf(1.1)-skewed routing
prefill    config 4: T tokens through the 40-block stack (INT4 scheme), grouped tensor-core path
pack       config 5: GPU quantisation of expert tensors into the packed blob layout
matvec     config 1 on the GPU: one 512x2048 dequant-matvec

Each prints one JSON line with the same keys as the default workload.
"""
from __future__ import annotations

import json
import time

import numpy as np

from moe_infer_b200 import _lib as L
from moe_infer_b200.native import Dims, NativeEngine, PinnedArray

from . import benchlib, synth


# Router logits of random weights have a spread of about +-2.5; the Zipf(1.1) popularity prior ln p_e spans 6.1.
# Scaling the prior by this factor gives the hottest expert about 40 of 64 tokens, as config 3 asks.
ZIPF_STRENGTH = 0.5


def _line(args, world, metric, unit, value, ms_per_step, workload, roofline, e2e, launches, clocks, extra=None,
          dtype="bf16 x 4-bit -> f32"):
    line = {"metric": metric, "value": value, "unit": unit, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": dtype, "data": "synthetic", "config": {"workload": workload},
            "clocks": clocks, "e2e": e2e, "gpu_launches": int(launches), "roofline": roofline}
    if extra:
        line["config"].update(extra)
    return line


def _time_loop(eng, fn, warmup, steps, local):
    for i in range(warmup):
        fn(i)
    eng.sync()
    n0 = eng.launch_count()
    with benchlib.ClockSampler(local) as clk:
        eng.timer_start()
        for i in range(steps):
            fn(warmup + i)
        ms = eng.timer_stop()
        eng.sync()
    return ms, eng.launch_count() - n0, clk.summary()


def run_layer(args, rank, world, local, dist):
    n_copies = 12  # 12 x 453 MB of experts: the weights a step touches were evicted from L2 long ago
    dims = Dims(num_layers=n_copies)
    eng = NativeEngine(dims, device=local)
    benchlib.populate_synthetic(eng, base_seed=args.seed)
    H = dims.hidden
    emb = synth.hidden_states(args.seed, 2, 64, H)
    d_in = eng.alloc(emb.nbytes).upload(emb)
    d_out = eng.alloc(emb.nbytes)

    def step(i):
        eng.layer_forward_dev(i % n_copies, d_in.ptr + (i % 64) * H * 4, 1, d_out.ptr + (i % 64) * H * 4)

    ms, launches, clocks = _time_loop(eng, step, args.warmup, args.steps, local)
    pin = PinnedArray((1, H), np.float32)
    pin.array[:] = emb[:1]
    t0 = time.perf_counter()
    for i in range(args.steps):
        eng.layer_forward(i % n_copies, pin.array)
    e2e_s = time.perf_counter() - t0
    peaks = benchlib.measured_peaks()
    b = benchlib.layer_token_bytes(dims)
    ach = b / (ms / args.steps / 1e3) / 1e9
    roof = {"bound": "hbm", "kernel": "decode_fused_kernel (1 layer)", "achieved": ach, "peak": peaks["hbm_gbs"],
            "unit": "GB/s", "frac": ach / peaks["hbm_gbs"], "peak_source": peaks["source"],
            "frac_of_nominal_8TBs": ach / 8000.0, "bytes_per_launch": b, "traffic": None}
    if rank == 0:
        print(json.dumps(_line(args, world, "moe_layer_decode_tokens_per_s", "layer-tok/s", args.steps / (ms / 1e3),
                               ms / args.steps, "config 2: one MoE layer, batch-1 decode, 256 experts top-8, BQ4; "
                               f"rotating over {n_copies} layer copies (L2 cannot hold them)", roof,
                               {"value": args.steps / e2e_s, "unit": "layer-tok/s", "h2d_bytes_per_step": H * 4,
                                "d2h_bytes_per_step": H * 4 + 64}, launches, clocks,
                               dtype="u4 weights x 24-bit fixed-point activations (three s8 digits), exact s32 dp4a sums, f32 scales")),
              flush=True)
    eng.close()


def run_batched(args, rank, world, local, dist, n_tokens, n_layers, scheme, zipf, workload, metric):
    dims = Dims(num_layers=n_layers, scheme=scheme)
    eng = NativeEngine(dims, device=local)
    benchlib.populate_synthetic(eng, base_seed=args.seed, config_id=4 if scheme == L.SCHEME_INT4 else 3)
    H, E, K, I = dims.hidden, dims.num_experts, dims.top_k, dims.inter
    emb = synth.hidden_states(args.seed, 3, n_tokens, H)
    d_in = eng.alloc(emb.nbytes).upload(emb)
    d_out = eng.alloc(emb.nbytes)
    d_idx = eng.alloc(n_tokens * K * 4)
    d_w = eng.alloc(n_tokens * K * 4)
    d_bias = None
    if zipf:
        bias = synth.zipf_logit_bias(args.seed, E, alpha=1.1, strength=ZIPF_STRENGTH)
        d_bias = eng.alloc(bias.nbytes).upload(bias)
    single = n_layers if zipf else 0  # zipf workload: one block per step, rotating over the copies

    def step(i):
        if single:
            eng.layer_forward_dev(i % n_layers, d_in.ptr, n_tokens, d_out.ptr, out_idx=d_idx.ptr, out_w=d_w.ptr,
                                  logit_bias=d_bias.ptr if d_bias else 0)
        else:
            eng.forward_hidden_dev(d_in.ptr, n_tokens, True, d_out.ptr)

    ms, launches, clocks = _time_loop(eng, step, args.warmup, args.steps, local)
    ms_step = ms / args.steps
    # end to end through the host-pointer entry point
    pin_in = PinnedArray((n_tokens, H), np.float32)
    pin_in.array[:] = emb
    pin_out = PinnedArray((n_tokens, H), np.float32)
    reps = max(1, min(args.steps, 20))
    if single:
        eng.layer_forward(0, pin_in.array, logit_bias=None if not zipf else bias)
        t0 = time.perf_counter()
        for i in range(reps):
            eng.layer_forward(i % n_layers, pin_in.array, logit_bias=None if not zipf else bias)
    else:
        eng.forward_hidden(pin_in.array, batched=True, out=pin_out.array)
        t0 = time.perf_counter()
        for i in range(reps):
            eng.forward_hidden(pin_in.array, batched=True, out=pin_out.array)
    e2e_s = (time.perf_counter() - t0) / reps
    peaks = benchlib.measured_peaks()
    lay = eng.layout["expert_size"]
    layers_per_step = 1 if single else n_layers
    flops_layer = n_tokens * K * 6 * H * I + n_tokens * 6 * H * I + n_tokens * 2 * E * H + n_tokens * 2 * H
    extra = {"tokens_per_step": n_tokens, "layers_per_step": layers_per_step}
    if zipf:
        idx = d_idx.download(np.int32, (n_tokens, K))
        counts = np.bincount(idx.ravel(), minlength=E)
        U = int((counts > 0).sum())
        router_b = E * H * 2 if scheme == L.SCHEME_BQ4 else E * H // 2 + 2 * E * (H // 64) * 2
        b = U * lay + lay + 1152 + router_b + n_tokens * H * (2 + 4)
        ach = b / (ms_step / 1e3) / 1e9
        roof = {"bound": "hbm", "kernel": "grouped_gemm_kernel<1>+<2>", "achieved": ach, "peak": peaks["hbm_gbs"],
                "unit": "GB/s", "frac": ach / peaks["hbm_gbs"], "peak_source": peaks["source"],
                "bytes_per_step": b, "tflops": flops_layer / (ms_step / 1e3) / 1e12, "traffic": None}
        extra.update({"distinct_experts_hit": U, "max_tokens_per_expert": int(counts.max()),
                      "l2": f"rotating over {n_layers} layer copies"})
    else:
        tf = flops_layer * layers_per_step / (ms_step / 1e3) / 1e12
        roof = {"bound": "tensor", "kernel": "grouped_gemm_kernel<1>+<2>", "achieved": tf,
                "peak": peaks["bf16_tflops_sustained"], "unit": "TFLOP/s", "frac": tf / peaks["bf16_tflops_sustained"],
                "peak_source": peaks["source"] + " (sustained cuBLAS bf16)", "flops_per_step": flops_layer * layers_per_step,
                "traffic": None}
        extra.update({"l2": "each layer reads 455 MB of unique weights (> 126 MB L2)"})
    tok_s = n_tokens / (ms_step / 1e3)
    if rank == 0:
        print(json.dumps(_line(args, world, metric, "tok/s", tok_s, ms_step, workload, roof,
                               {"value": n_tokens / e2e_s, "unit": "tok/s", "h2d_bytes_per_step": n_tokens * H * 4,
                                "d2h_bytes_per_step": n_tokens * H * 4}, launches, clocks, extra)), flush=True)
    eng.close()


def run_prefill_ep(args, rank, world, local, dist):
    """Config 4 across `world` GPUs: experts sharded 256/P, tokens T/P per rank, dispatch/combine over peer memory."""
    from moe_infer_b200 import ep as ephost
    T = args.tokens or 4096
    n_local = T // world
    dims = Dims(num_layers=args.layers, scheme=L.SCHEME_INT4)
    eng = NativeEngine(dims, device=local)
    benchlib.populate_synthetic(eng, base_seed=args.seed, config_id=4)  # same seed on every rank: replicated tensors agree
    H, E, K, I = dims.hidden, dims.num_experts, dims.top_k, dims.inter
    emb = synth.hidden_states(args.seed, 3, T, H)[rank * n_local:(rank + 1) * n_local]
    d_in = eng.alloc(emb.nbytes).upload(emb)
    d_out = eng.alloc(emb.nbytes)
    eng.ep_init(ephost.exchange_handles(eng.ep_export(rank, world, n_local)))
    dist.barrier()

    def step(i):
        eng.ep_forward_hidden_dev(d_in.ptr, n_local, d_out.ptr)

    for i in range(args.warmup):
        step(i)
    eng.sync()
    dist.barrier()
    n0 = eng.launch_count()
    with benchlib.ClockSampler(local) as clk:
        eng.timer_start()
        for i in range(args.steps):
            step(i)
        ms = eng.timer_stop()
        eng.sync()
    launches = eng.launch_count() - n0
    dist.barrier()
    ms = dist.max(ms)
    out = d_out.download(np.float32, (n_local, H))
    finite = bool(np.isfinite(out).all())
    ms_step = ms / args.steps
    flops_layer = T * K * 6 * H * I + T * 6 * H * I + T * 2 * E * H + T * 2 * H
    tf = flops_layer * args.layers / (ms_step / 1e3) / 1e12
    peaks = benchlib.measured_peaks()
    roof = {"bound": "tensor", "kernel": "grouped_gemm_kernel<1>+<2> (per GPU)", "achieved": tf / world,
            "peak": peaks["bf16_tflops_sustained"], "unit": "TFLOP/s per GPU",
            "frac": tf / world / peaks["bf16_tflops_sustained"], "peak_source": peaks["source"] + " (sustained cuBLAS bf16)",
            "aggregate_tflops": tf, "traffic": None}
    dist.barrier()
    if rank == 0:
        line = _line(args, world, "moe_prefill_tokens_per_s", "tok/s", T / (ms_step / 1e3), ms_step,
                     f"config 4: {T}-token prefill through {args.layers} MoE layers, INT4 scheme, experts sharded "
                     f"{E}/{world} per GPU, token dispatch/combine over NVLink peer memory", roof,
                     {"value": None, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, launches,
                     clk.summary(), {"tokens_per_step": T, "tokens_per_rank": n_local, "finite": finite,
                                     "parallelism": f"ep{world}"})
        line["scaling"] = "strong"
        print(json.dumps(line), flush=True)
    dist.barrier()
    eng.close()


def run_pack(args, rank, world, local, dist):
    dims = Dims(num_layers=1)
    eng = NativeEngine(dims, device=local)
    H, I, E = dims.hidden, dims.inter, dims.num_experts
    n_src = 3  # three distinct 1.6 GB source sets, rotated: 4.8 GB >> L2
    gus, dns = [], []
    for s in range(n_src):
        gu = eng.alloc(E * 2 * I * H * 2)
        dn = eng.alloc(E * H * I * 2)
        eng.synth_normal(gu.ptr, L.DT_BF16, E * 2 * I * H, 100 + s, 0.02, 0.001, 0.4)
        eng.synth_normal(dn.ptr, L.DT_BF16, E * H * I, 200 + s, 0.02, 0.001, 0.4)
        gus.append(gu)
        dns.append(dn)
    blob = eng.layer_dev(0)

    def step(i):
        eng.pack_experts_dev(gus[i % n_src].ptr, dns[i % n_src].ptr, L.DT_BF16, E, blob)

    ms, launches, clocks = _time_loop(eng, step, args.warmup, args.steps, local)
    elems = E * 3 * I * H
    b = elems * 2 + elems * 0.5625
    peaks = benchlib.measured_peaks()
    ach = b / (ms / args.steps / 1e3) / 1e9
    roof = {"bound": "hbm", "kernel": "pack_int4_kernel<bf16>", "achieved": ach, "peak": peaks["hbm_gbs"],
            "unit": "GB/s", "frac": ach / peaks["hbm_gbs"], "peak_source": peaks["source"], "bytes_per_step": b,
            "traffic": None}
    # end to end: 8 experts from pinned host memory and back
    n_e = 8
    gu_h = PinnedArray((n_e, 2 * I, H), np.uint16)
    dn_h = PinnedArray((n_e, H, I), np.uint16)
    gu_h.array[:] = 0x3C00
    dn_h.array[:] = 0x3C00
    eng.pack_experts(gu_h.array, dn_h.array)
    t0 = time.perf_counter()
    for _ in range(3):
        eng.pack_experts(gu_h.array, dn_h.array)
    e2e_s = (time.perf_counter() - t0) / 3
    if rank == 0:
        print(json.dumps(_line(args, world, "quantize_GB_per_s", "GB/s", ach, ms / args.steps,
                               "config 5: one layer's experts (256 x 3 matrices of 1,048,576 bf16, 0.1% outliers) -> packed blob",
                               roof, {"value": n_e * 3 * I * H * 2.5625 / e2e_s / 1e9, "unit": "GB/s",
                                      "h2d_bytes_per_step": n_e * 3 * I * H * 2,
                                      "d2h_bytes_per_step": n_e * eng.layout["expert_size"]},
                               launches, clocks, {"full_checkpoint_ms_extrapolated": ms / args.steps * 40.1},
                               dtype="f32 (exactly rounded), u8 nibbles")), flush=True)
    eng.close()


def run_matvec(args, rank, world, local, dist):
    dims = Dims(num_experts=4, top_k=4, num_layers=1)
    eng = NativeEngine(dims, device=local)
    rows, cols = 512, 2048
    n_copies = 512  # 512 x 0.59 MB = 302 MB of distinct matrices, rotated
    wb, sb = rows * cols // 2, rows * (cols // 64) * 2
    w = eng.alloc(n_copies * wb)
    s = eng.alloc(n_copies * sb)
    b = eng.alloc(n_copies * sb)
    src = eng.alloc(n_copies * rows * cols * 2)
    eng.synth_normal(src.ptr, L.DT_BF16, n_copies * rows * cols, 7, 0.02)
    eng.pack_int4_dev(src.ptr, L.DT_BF16, n_copies * rows, cols, w.ptr, s.ptr, b.ptr)
    x = synth.hidden_states(0, 1, 1, cols)
    dx = eng.alloc(x.nbytes).upload(x)
    dy = eng.alloc(rows * 4)

    def step(i):
        c = i % n_copies
        eng.matvec_int4_dev(w.ptr + c * wb, s.ptr + c * sb, b.ptr + c * sb, dx.ptr, dy.ptr, rows, cols)

    ms, launches, clocks = _time_loop(eng, step, args.warmup, args.steps, local)
    by = 595968
    peaks = benchlib.measured_peaks()
    ach = by / (ms / args.steps / 1e3) / 1e9
    roof = {"bound": "hbm (launch-latency dominated at this size)", "kernel": "matvec_int4_kernel", "achieved": ach,
            "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": ach / peaks["hbm_gbs"], "peak_source": peaks["source"],
            "bytes_per_launch": by, "traffic": None}
    if rank == 0:
        print(json.dumps(_line(args, world, "matvec_GB_per_s", "GB/s", ach, ms / args.steps,
                               "config 1 on the GPU: one 512x2048 4-bit dequant-matvec per launch", roof,
                               {"value": None, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                               launches, clocks, dtype="f32 accumulate over 4-bit weights")), flush=True)
    eng.close()


def run(args, rank, world, local, dist):
    if args.workload == "layer":
        run_layer(args, rank, world, local, dist)
    elif args.workload == "batched64":
        run_batched(args, rank, world, local, dist, args.tokens or 64, 8, L.SCHEME_BQ4, True,
                    "config 3: 64 tokens through one MoE layer, top-8 of 256, Zipf(1.1) routing, BQ4",
                    "moe_batched_decode_tokens_per_s")
    elif args.workload == "prefill" and world > 1:
        run_prefill_ep(args, rank, world, local, dist)
    elif args.workload == "prefill":
        run_batched(args, rank, world, local, dist, args.tokens or 4096, args.layers, L.SCHEME_INT4, False,
                    f"config 4: {args.tokens or 4096}-token prefill through {args.layers} MoE layers, INT4 scheme, "
                    "attention passed through, 1 GPU", "moe_prefill_tokens_per_s")
    elif args.workload == "pack":
        run_pack(args, rank, world, local, dist)
    elif args.workload == "matvec":
        run_matvec(args, rank, world, local, dist)
    else:
        raise SystemExit(f"unknown workload {args.workload}")
