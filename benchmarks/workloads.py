"""Timed workloads behind ``bench.py``.

decode     config 2 x 40 layers: one token through the MoE stack (the headline, in ``bench.py``)
layer      config 2: one MoE block, batch-1 decode, rotating over distinct layer copies
batched64  config 3: 64 tokens through one block, Zipf(1.1)-skewed routing
prefill    config 4: T tokens through the 40-block stack (INT4 scheme); one GPU = grouped tensor-core path,
           several GPUs = experts sharded over the ranks, token dispatch/combine over NVLink peer memory
pack       config 5: GPU quantisation of expert tensors into the packed blob layout; several GPUs = layers
           split over the ranks, no communication
matvec     config 1 on the GPU (512 x 2048, launch-bound) and an HBM-sized matrix of the lm_head shape

Every function returns a dict (one JSON line's worth).  A timed figure is the median over several repeats of its
timed region (CUDA events on the engine's stream, max over ranks per repeat), so that short regions give steady numbers.
"""
from __future__ import annotations

import time
from typing import Callable, List, Optional

import numpy as np

from moe_infer_b200 import _lib as L
from moe_infer_b200.native import Dims, NativeEngine, PinnedArray

from . import benchlib, synth

# Router logits of random weights have a spread of about +-2.5; the Zipf(1.1) popularity prior ln p_e spans 6.1.
# Scaling the prior by this factor gives the hottest expert about 40 of 64 tokens, as config 3 asks.
ZIPF_STRENGTH = 0.5
MIN_REPEATS = 5


def timed_repeats(eng: NativeEngine, fn: Callable[[int], None], warmup: int, steps: int, dist=None,
                  min_repeats: int = MIN_REPEATS, fill_s: float = 0.0, max_repeats: int = 400) -> dict:
    """Runs `warmup` untimed steps, then repeats a region of exactly `steps` steps at least `min_repeats` times (and
    until `fill_s` seconds of device time have passed); every region is bracketed by a barrier + synchronize and timed
    with CUDA events, max over ranks.  Returns the median region and the launch count of one region."""
    for i in range(warmup):
        fn(i)
    eng.sync()
    regions: List[float] = []
    launches = 0
    i0 = warmup
    while len(regions) < min_repeats or (sum(regions) / 1e3 < fill_s and len(regions) < max_repeats):
        if dist is not None:
            dist.barrier()
        n0 = benchlib.launch_count(eng)
        benchlib.timer_start(eng)
        for i in range(steps):
            fn(i0 + i)
        ms = benchlib.timer_stop(eng)
        eng.sync()
        launches = benchlib.launch_count(eng) - n0
        if dist is not None:
            dist.barrier()
            ms = dist.max(ms)
        regions.append(ms)
        i0 += steps
    med = float(np.median(regions))
    return {"ms": med, "ms_per_step": med / steps, "repeats": len(regions), "min_ms": float(min(regions)),
            "max_ms": float(max(regions)), "launches": int(launches)}


def hbm_roofline(kernel: str, bytes_per_step: float, ms_per_step: float, traffic=None, **extra) -> dict:
    peaks = benchlib.measured_peaks()
    ach = bytes_per_step / (ms_per_step / 1e3) / 1e9
    r = {"bound": "hbm", "kernel": kernel, "achieved": ach, "peak": peaks["hbm_gbs"], "unit": "GB/s",
         "frac": ach / peaks["hbm_gbs"], "peak_source": peaks["source"], "frac_of_nominal_8TBs": ach / 8000.0,
         "bytes_per_step": bytes_per_step, "traffic": traffic}
    r.update(extra)
    return r


def tensor_roofline(kernel: str, flops_per_step: float, ms_per_step: float, n_gpus: int = 1, **extra) -> dict:
    peaks = benchlib.measured_peaks()
    tf = flops_per_step / (ms_per_step / 1e3) / 1e12
    r = {"bound": "tensor", "kernel": kernel, "achieved": tf / n_gpus, "peak": peaks["bf16_tflops_sustained"],
         "unit": "TFLOP/s per GPU", "frac": tf / n_gpus / peaks["bf16_tflops_sustained"],
         "peak_source": peaks["source"] + " (sustained cuBLAS bf16)", "flops_per_step": flops_per_step,
         "aggregate_tflops": tf, "traffic": None}
    r.update(extra)
    return r


def layer_flops(d: Dims, n_tokens: int) -> float:
    """Useful flops of one MoE block over n tokens: routed experts, shared expert, router, gate score."""
    H, I, E, K = d.hidden, d.inter, d.num_experts, d.top_k
    return float(n_tokens) * (K * 6 * H * I + 6 * H * d.shared_inter + 2 * E * H + 2 * H)


def rel_l2(a, b) -> float:
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


# ─── config 2: one block, one token ───────────────────────────────────────────

def run_layer(args, eng: NativeEngine, local: int) -> dict:
    dims = eng.dims
    n_copies = dims.num_layers  # distinct layer copies: the weights a step touches were evicted from L2 long ago
    H = dims.hidden
    emb = synth.hidden_states(args.seed, 2, 64, H)
    d_in = eng.alloc(emb.nbytes).upload(emb)
    d_out = eng.alloc(emb.nbytes)

    def step(i):
        eng.layer_forward_dev(i % n_copies, d_in.ptr + (i % 64) * H * 4, 1, d_out.ptr + (i % 64) * H * 4)

    t = timed_repeats(eng, step, args.warmup, args.steps)
    b = benchlib.layer_token_bytes(dims)
    out = {"workload": f"config 2: one MoE layer, batch-1 decode, {dims.num_experts} experts top-{dims.top_k}, BQ4; "
                       f"rotating over {n_copies} layer copies (L2 cannot hold them)",
           "us_per_layer": t["ms_per_step"] * 1e3, "repeats": t["repeats"], "gpu_launches": t["launches"],
           "roofline": hbm_roofline("decode_slots_kernel (1 layer)", b, t["ms_per_step"])}
    d_in.free()
    d_out.free()
    return out


# ─── config 3: 64 tokens, Zipf routing ────────────────────────────────────────

def run_batched64(args, eng: NativeEngine, local: int, n_tokens: int = 64) -> dict:
    dims = eng.dims
    H, E, K = dims.hidden, dims.num_experts, dims.top_k
    n_layers = dims.num_layers
    emb = synth.hidden_states(args.seed, 3, n_tokens, H)
    d_in = eng.alloc(emb.nbytes).upload(emb)
    d_out = eng.alloc(emb.nbytes)
    d_idx = eng.alloc(n_tokens * K * 4)
    d_w = eng.alloc(n_tokens * K * 4)
    bias = synth.zipf_logit_bias(args.seed, E, alpha=1.1, strength=ZIPF_STRENGTH)
    d_bias = eng.alloc(bias.nbytes).upload(bias)

    def step(i):
        eng.layer_forward_dev(i % n_layers, d_in.ptr, n_tokens, d_out.ptr, out_idx=d_idx.ptr, out_w=d_w.ptr,
                              logit_bias=d_bias.ptr)

    t = timed_repeats(eng, step, args.warmup, args.steps)
    idx = d_idx.download(np.int32, (n_tokens, K))
    counts = np.bincount(idx.ravel(), minlength=E)
    U = int((counts > 0).sum())
    lay = eng.layout["expert_size"]
    router_b = E * H * 2 if dims.scheme == L.SCHEME_BQ4 else E * H // 2 + 2 * E * (H // 64) * 2
    b = U * lay + lay + 1152 + router_b + n_tokens * H * (2 + 4)
    # parity of the grouped path (bf16 operands) against the decode path (f32-class) on the same tokens and layer
    last = (args.warmup + t["repeats"] * args.steps - 1) % n_layers
    got = d_out.download(np.float32, (n_tokens, H))
    errs = []
    for tok in range(min(8, n_tokens)):
        ref, _, _ = eng.layer_forward(last, emb[tok], logit_bias=bias)
        errs.append(rel_l2(got[tok] - emb[tok], ref[0] - emb[tok]))
    out = {"workload": f"config 3: {n_tokens} tokens through one MoE layer, top-{K} of {E}, Zipf(1.1) routing, BQ4; "
                       f"rotating over {n_layers} layer copies",
           "ms_per_step": t["ms_per_step"], "tok_per_s": n_tokens / (t["ms_per_step"] / 1e3), "repeats": t["repeats"],
           "gpu_launches": t["launches"], "distinct_experts_hit": U, "max_tokens_per_expert": int(counts.max()),
           "parity_rel_l2_vs_decode_path": float(max(errs)),
           "roofline": hbm_roofline("grouped_gemm_kernel<1>+<2>", b, t["ms_per_step"],
                                    tflops=layer_flops(dims, n_tokens) / (t["ms_per_step"] / 1e3) / 1e12)}
    for buf in (d_in, d_out, d_idx, d_w, d_bias):
        buf.free()
    return out


# ─── config 4: prefill ────────────────────────────────────────────────────────

def run_prefill(args, rank: int, world: int, local: int, dist, n_tokens: int = 4096, layers: Optional[int] = None) -> dict:
    """T tokens through the INT4-scheme stack.  world == 1: the grouped path on one GPU.  world > 1: experts sharded
    E / world per rank, tokens T / world per rank, dispatch and combine over peer memory (strong scaling)."""
    layers = layers or args.layers
    dims = Dims(num_layers=layers, scheme=L.SCHEME_INT4)
    eng = NativeEngine(dims, device=local)
    benchlib.populate_synthetic(eng, base_seed=args.seed, config_id=4)  # same seed on every rank: replicated tensors agree
    H, E, K = dims.hidden, dims.num_experts, dims.top_k
    n_local = n_tokens // world
    emb_all = synth.hidden_states(args.seed, 3, n_tokens, H)
    emb = emb_all[rank * n_local:(rank + 1) * n_local]
    d_in = eng.alloc(emb.nbytes).upload(emb)
    d_out = eng.alloc(emb.nbytes)
    steps = max(1, min(args.steps, 5))
    warm = max(3, min(args.warmup, 5))
    if world > 1:
        from moe_infer_b200 import ep as ephost
        eng.ep_init(ephost.exchange_handles(eng.ep_export(rank, world, n_local)))
        dist.barrier()

        def step(i):
            eng.ep_forward_hidden_dev(d_in.ptr, n_local, d_out.ptr)
    else:
        def step(i):
            eng.forward_hidden_dev(d_in.ptr, n_local, True, d_out.ptr)

    t = timed_repeats(eng, step, warm, steps, dist if world > 1 else None)
    finite = bool(np.isfinite(d_out.download(np.float32, (n_local, H))).all())
    # parity, outside the timed region: layer 0 over this rank's tokens as the timed path computes it, against the
    # single-GPU entry point on the first 64 of them (every rank holds all experts of this synthetic store), and
    # against the decode path (f32-class arithmetic) on the first 8
    n_chk = min(64, n_local)
    if world > 1:
        eng.ep_layer_forward_dev(0, d_in.ptr, n_local, d_out.ptr)
    else:
        eng.layer_forward_dev(0, d_in.ptr, n_local, d_out.ptr)
    eng.sync()
    got = d_out.download(np.float32, (n_local, H))[:n_chk]
    parity_single = None
    if world > 1:
        if rank == 0:
            single, _, _ = eng.layer_forward(0, emb[:n_chk])
            parity_single = rel_l2(got - emb[:n_chk], single - emb[:n_chk])
        dist.barrier()
    errs = []
    if rank == 0:
        for tok in range(min(8, n_chk)):
            ref, _, _ = eng.layer_forward(0, emb[tok])
            errs.append(rel_l2(got[tok] - emb[tok], ref[0] - emb[tok]))
    fl = layer_flops(dims, n_tokens) * layers
    ms_step = t["ms_per_step"]
    out = {"workload": f"config 4: {n_tokens}-token prefill through {layers} MoE layers, INT4 scheme, attention passed through; "
                       + (f"experts sharded {E}/{world} per GPU, tokens {n_local} per GPU, dispatch/combine over NVLink peer memory"
                          if world > 1 else "1 GPU"),
           "n_gpus": world, "parallelism": f"ep{world}" if world > 1 else "single", "scaling": "strong",
           "ms_per_step": ms_step, "tok_per_s": n_tokens / (ms_step / 1e3), "tflops": fl / (ms_step / 1e3) / 1e12,
           "repeats": t["repeats"], "steps_per_repeat": steps, "gpu_launches": t["launches"], "finite": finite,
           "parity_rel_l2_vs_decode_path": float(max(errs)) if errs else None,
           "parity_rel_l2_vs_single_gpu": parity_single,
           "l2": "each layer reads 455 MB of unique weights (> 126 MB L2)",
           "roofline": tensor_roofline("grouped_gemm_kernel<1>+<2>", fl, ms_step, world)}
    d_in.free()
    d_out.free()
    if world > 1:
        dist.barrier()
    eng.close()
    return out


# ─── config 5: packer ─────────────────────────────────────────────────────────

def run_pack(args, rank: int, world: int, local: int, dist) -> dict:
    """One step = this rank's share of a 40-layer checkpoint's expert tensors (40 / world layers) packed into the blob
    layout; ranks work on disjoint layers with no communication, the figure is the aggregate."""
    dims = Dims(num_layers=1)
    eng = NativeEngine(dims, device=local)
    H, I, E = dims.hidden, dims.inter, dims.num_experts
    total_layers = 40
    my_layers = len(range(rank, total_layers, world))
    n_src = 3  # three distinct 1.6 GB source sets, rotated: 4.8 GB >> L2
    gus, dns = [], []
    for s in range(n_src):
        gu = eng.alloc(E * 2 * I * H * 2)
        dn = eng.alloc(E * H * I * 2)
        benchlib.synth_normal(eng, gu.ptr, L.DT_BF16, E * 2 * I * H, 100 + s + 10 * rank, 0.02, 0.001, 0.4)
        benchlib.synth_normal(eng, dn.ptr, L.DT_BF16, E * H * I, 200 + s + 10 * rank, 0.02, 0.001, 0.4)
        gus.append(gu)
        dns.append(dn)
    blob = eng.layer_dev(0)

    def step(i):
        for l in range(my_layers):
            k = (i * my_layers + l) % n_src
            eng.pack_experts_dev(gus[k].ptr, dns[k].ptr, L.DT_BF16, E, blob)

    steps = max(1, min(args.steps, 3))
    t = timed_repeats(eng, step, 3, steps, dist if world > 1 else None)
    elems = float(E * 3 * I * H) * total_layers
    b = elems * 2 + elems * 0.5625
    ms_step = t["ms_per_step"]
    per_gpu_b = (float(E * 3 * I * H) * my_layers) * 2.5625
    out = {"workload": f"config 5: the experts of a 40-layer checkpoint (40 x 256 x 3 matrices of 1,048,576 bf16, 0.1% outliers) "
                       f"-> packed blobs; layers split over {world} GPU(s), no communication",
           "n_gpus": world, "ms_per_checkpoint": ms_step, "GB_per_s": b / (ms_step / 1e3) / 1e9, "repeats": t["repeats"],
           "gpu_launches": t["launches"], "layers_per_gpu": my_layers,
           "roofline": hbm_roofline("pack_int4_kernel<bf16> (per GPU)", per_gpu_b, ms_step)}
    for buf in gus + dns:
        buf.free()
    eng.close()
    return out


# ─── lm_head: the largest single read of a decode step ────────────────────────

def run_lm_head(args, local: int, kind: str = "int8", vocab: int = 248320) -> dict:
    """final norm + lm_head for one token: vocab x 2048 INT8 rows (BQ4 scheme) or 4-bit rows (INT4 scheme)."""
    import ctypes as C
    dims = Dims(num_layers=1, num_experts=4, top_k=4, vocab=vocab)
    eng = NativeEngine(dims, device=local)
    H = dims.hidden
    rng = np.random.default_rng(args.seed)
    eng.load_final_norm(synth.to_bf16_rne(np.ones(H, np.float32)))
    if kind == "int8":
        q = rng.integers(-127, 128, size=(vocab, H), dtype=np.int8)
        eng.load_lm_head_int8(q, np.full(vocab, 2e-4, np.float32))
        by = vocab * H + vocab * 4
    else:
        w = rng.integers(0, 2**32, size=(vocab, H // 8), dtype=np.uint64).astype(np.uint32)
        sb = np.full((vocab, H // 64), 0x3C00, np.uint16)
        eng.load_lm_head_q4((w, sb, sb))
        by = vocab * H // 2 + 2 * vocab * (H // 64) * 2
    h = synth.hidden_states(args.seed, 2, 4, H)
    d_h = eng.alloc(h.nbytes).upload(h)
    d_l = eng.alloc(vocab * 4)

    def step(i):
        L.check(eng.lib.moe_logits_dev(eng.h, C.c_void_p(d_h.ptr + (i % 4) * H * 4), 1, C.c_void_p(d_l.ptr)))

    t = timed_repeats(eng, step, max(3, min(args.warmup, 10)), max(1, min(args.steps, 20)))
    out = {"workload": f"final norm + lm_head, 1 token: {vocab} x {H} {'INT8 rows, one f32 scale per row' if kind == 'int8' else '4-bit rows'} "
                       f"({by / 1e6:.0f} MB per call, larger than L2)",
           "us_per_call": t["ms_per_step"] * 1e3, "repeats": t["repeats"], "gpu_launches": t["launches"],
           "roofline": hbm_roofline("matvec_int8_stream_kernel" if kind == "int8" else "matvec_int4_stream_kernel", by + vocab * 4,
                                    t["ms_per_step"])}
    d_h.free()
    d_l.free()
    eng.close()
    return out


# ─── the whole decoder: attention half + MoE half of every layer, one token ──

QWEN36_ATTN = dict(num_heads=16, num_kv_heads=2, head_dim=256, rotary_dim=64, rope_theta=1.0e7, lin_num_k_heads=16,
                   lin_num_v_heads=32, lin_key_dim=128, lin_value_dim=128, conv_kernel=4, full_attn_interval=4)


def run_full_decode(args, eng: NativeEngine, local: int) -> dict:
    """One token through attention + MoE of every layer of `eng` (whose MoE store is populated): the model's own
    attention shapes (10 gated full-attention layers with bf16 projections, 30 Gated DeltaNet layers with 4-bit
    projections, as the BQ4 scheme stores them).  The same random projection values are uploaded to every layer of a
    kind (each layer has its own device copy, so the traffic is real); context length stays below 64 positions."""
    a = QWEN36_ATTN
    H, n_layers = eng.dims.hidden, eng.dims.num_layers
    rng = np.random.default_rng(args.seed + 77)
    q_dim, kv_dim = a["num_heads"] * a["head_dim"], a["num_kv_heads"] * a["head_dim"]
    total_key, total_value = a["lin_num_k_heads"] * a["lin_key_dim"], a["lin_num_v_heads"] * a["lin_value_dim"]
    conv_dim = 2 * total_key + total_value
    eng.attn_configure(max_seq=64, **a)
    bfm = lambda r, c: synth.to_bf16_rne((rng.standard_normal((r, c)) * 0.02).astype(np.float32))
    q4m = lambda r, c: (rng.integers(0, 2**32, size=(r, c // 8), dtype=np.uint64).astype(np.uint32),
                        np.full((r, c // 64), 0x3B00, np.uint16), np.full((r, c // 64), 0xBC80, np.uint16))  # scale 2^-9, bias -2^-6
    ones = lambda n: synth.to_bf16_rne(np.ones(n, np.float32))
    full = {L.A_Q_PROJ: bfm(2 * q_dim, H), L.A_K_PROJ: bfm(kv_dim, H), L.A_V_PROJ: bfm(kv_dim, H), L.A_O_PROJ: bfm(H, q_dim)}
    lin = {L.A_IN_PROJ_QKV: q4m(conv_dim, H), L.A_IN_PROJ_Z: q4m(total_value, H), L.A_IN_PROJ_B: q4m(a["lin_num_v_heads"], H),
           L.A_IN_PROJ_A: q4m(a["lin_num_v_heads"], H), L.A_OUT_PROJ: q4m(H, total_value)}
    conv = synth.to_bf16_rne((rng.standard_normal((conv_dim, a["conv_kernel"])) * 0.5).astype(np.float32))
    attn_bytes = 0
    for l in range(n_layers):
        eng.attn_load_vec(l, L.A_INPUT_NORM, ones(H))
        if (l + 1) % a["full_attn_interval"] == 0:
            eng.attn_load_vec(l, L.A_Q_NORM, ones(a["head_dim"]))
            eng.attn_load_vec(l, L.A_K_NORM, ones(a["head_dim"]))
            for which, t in full.items():
                eng.attn_load_proj(l, which, t)
                attn_bytes += t.nbytes
        else:
            eng.attn_load_vec(l, L.A_CONV1D, conv)
            eng.attn_load_vec(l, L.A_A_LOG, np.zeros(a["lin_num_v_heads"], np.float32))
            eng.attn_load_vec(l, L.A_DT_BIAS, synth.to_bf16_rne(np.zeros(a["lin_num_v_heads"], np.float32)))
            eng.attn_load_vec(l, L.A_LIN_NORM, ones(a["lin_value_dim"]))
            for which, t in lin.items():
                eng.attn_load_proj(l, which, t)
                attn_bytes += sum(x.nbytes for x in t)
            attn_bytes += 2 * total_value * a["lin_key_dim"] * 4  # the recurrence state is read and written
    emb = synth.hidden_states(args.seed, 2, 8, H)
    out = np.empty((1, H), np.float32)

    def step(i):
        if eng.model_pos() >= 60:
            eng.model_reset()
        L.check(eng.lib.moe_model_forward_hidden_host(eng.h, L.ptr(emb[i % 8:i % 8 + 1]), 1, L.ptr(out)))

    t = timed_repeats(eng, step, max(3, min(args.warmup, 5)), max(1, min(args.steps, 10)))
    # where the host's time goes, from the engine's own telemetry over a few more tokens (outside the timed region)
    eng.lib.moe_set_record_telemetry(1)
    t0 = eng.telemetry()
    for i in range(8):
        step(i)
    t1 = eng.telemetry()
    eng.lib.moe_set_record_telemetry(0)
    host = {k: (t1.get(k, 0.0) - t0.get(k, 0.0)) / 8 for k in ("phase.op2_encode_ms", "phase.hidden_wait_ms")}
    # a prompt through the same path: 56 tokens in one call (layer by layer: projections, attention, DeltaNet recurrence and
    # MoE halves each over all the tokens of the call)
    n_prompt = 56
    pe = synth.hidden_states(args.seed, 4, n_prompt, H)
    po = np.empty((n_prompt, H), np.float32)

    def prompt_step(i):
        eng.model_reset()
        L.check(eng.lib.moe_model_forward_hidden_host(eng.h, L.ptr(pe), n_prompt, L.ptr(po)))

    tp = timed_repeats(eng, prompt_step, 1, 1, min_repeats=3)
    eng.model_reset()
    moe_bytes = benchlib.layer_token_bytes(eng.dims) * n_layers
    res = {"workload": f"whole decoder, 1 token x {n_layers} layers: attention half (10 full-attention layers with bf16 projections, "
                       "30 Gated DeltaNet layers with 4-bit projections; Qwen3.6-35B-A3B head counts) + MoE half, host buffers, "
                       "context below 64 positions",
           "ms_per_token": t["ms_per_step"], "tok_per_s": 1e3 / t["ms_per_step"], "repeats": t["repeats"],
           "gpu_launches": t["launches"], "finite": bool(np.isfinite(out).all()),
           "host_enqueue_ms_per_token": host["phase.op2_encode_ms"], "host_wait_ms_per_token": host["phase.hidden_wait_ms"],
           "prompt": {"tokens": n_prompt, "ms": tp["ms_per_step"], "ms_per_token": tp["ms_per_step"] / n_prompt,
                      "tok_per_s": n_prompt / (tp["ms_per_step"] / 1e3), "finite": bool(np.isfinite(po).all()),
                      "gpu_launches": tp["launches"]},
           "attention_MB_per_token": attn_bytes / 1e6, "moe_MB_per_token": moe_bytes / 1e6,
           "roofline": hbm_roofline("attention kernels + decode_slots_kernel per layer", attn_bytes + moe_bytes, t["ms_per_step"])}
    return res


# ─── config 1 on the GPU, and the matvec at HBM size ──────────────────────────

def run_matvec(args, eng: NativeEngine, local: int, rows: int = 512, cols: int = 2048, copies: int = 512) -> dict:
    wb, sb = rows * cols // 2, rows * (cols // 64) * 2
    w = eng.alloc(copies * wb)
    s = eng.alloc(copies * sb)
    b = eng.alloc(copies * sb)
    chunk_rows = min(copies * rows, 65536)
    src = eng.alloc(chunk_rows * cols * 2)
    done = 0
    while done < copies * rows:  # pack in chunks so the bf16 source stays small
        n = min(chunk_rows, copies * rows - done)
        benchlib.synth_normal(eng, src.ptr, L.DT_BF16, n * cols, 7 + done, 0.02)
        eng.pack_int4_dev(src.ptr, L.DT_BF16, n, cols, w.ptr + done * (cols // 2), s.ptr + done * (cols // 64) * 2,
                          b.ptr + done * (cols // 64) * 2)
        done += n
    x = synth.hidden_states(0, 1, 1, cols)
    dx = eng.alloc(x.nbytes).upload(x)
    dy = eng.alloc(rows * 4)

    def step(i):
        c = i % copies
        eng.matvec_int4_dev(w.ptr + c * wb, s.ptr + c * sb, b.ptr + c * sb, dx.ptr, dy.ptr, rows, cols)

    steps = args.steps if rows <= 4096 else max(1, min(args.steps, 20))
    t = timed_repeats(eng, step, max(3, min(args.warmup, 10)), steps)
    by = wb + 2 * sb + cols * 4 + rows * 4
    out = {"workload": f"{rows} x {cols} 4-bit dequant-matvec per launch, rotating over {copies} distinct matrices "
                       f"({copies * (wb + 2 * sb) / 1e6:.0f} MB)",
           "us_per_call": t["ms_per_step"] * 1e3, "repeats": t["repeats"], "gpu_launches": t["launches"],
           "roofline": hbm_roofline("matvec_int4_stream_kernel" if (cols == 2048 and rows >= 4096) else "matvec_int4_kernel", by,
                                    t["ms_per_step"])}
    for buf in (w, s, b, src, dx, dy):
        buf.free()
    return out
