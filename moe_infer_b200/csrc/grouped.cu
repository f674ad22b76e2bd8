// Batched (n > 1 tokens) path of one MoE block: tokens are sorted by expert on the
// device and each expert's tokens run through a grouped 4-bit GEMM on the
// 5th-generation tensor cores.
//
// Replaces forward_hidden_batched's per-layer MoE half (reference
// src/engine/qwen35_moe/fused_exp3.rs:216-276 and batched.rs:334-447), which
// routes every token on the CPU and then issues 3 matvec dispatches per (token,
// expert), re-reading the expert weights for each token.  Here every expert's
// weights are read and dequantised once per tile of up to 256 of its tokens.
//
//   prep     per token: x = rmsnorm(h) as three bf16 terms (hi for the GEMMs, all three for the router),
//            sigmoid(shared_expert_gate . x)
//   router   logits = x . Wr^T on the tensor cores with three-way bf16 splits (f32 accuracy)
//   route    per token softmax / top-k / renormalise (one warp), expert histogram
//   plan     exclusive scan of the histogram, list of (expert, token tile) work items
//   scatter  token -> expert-sorted slot
//   gemm1    per (tile, 128-row block): D_gate, D_up [128 rows x N tokens] in TMEM =
//            dequant(W_gate/up rows) . X_tile^T ; epilogue silu(g) * u -> act (bf16)
//   gemm2    per (tile, 128-row block): D [128 rows x N tokens] = dequant(W_down rows)
//            . act_tile^T ; epilogue -> O (bf16, one row per slot)
//   combine  per token: h_out = h_in + sum_k w_k O[slot(t,k)] + sigmoid(sg) O[shared slot]
//
// GEMM operand staging: weights are dequantised by the 512 producer threads of the CTA
// (128-bit nibble loads, bf16x2 arithmetic) straight into shared memory in the
// K-major 128-byte-swizzled layout tcgen05.mma reads; one K step = one 64-column
// quantisation group = one 128-byte swizzle row.  A 4-bit word holds columns
// c..c+7; masking pairs (n, n+4) without shifting them into order yields the
// column order [0,4,1,5,2,6,3,7] inside every 8-column block, so the activations
// are stored with the same interleave (the dot product does not care about the
// order of its terms).  A dedicated warp issues the MMAs (hand-off through "full"
// mbarriers); their completion frees the stage through tcgen05.commit on an mbarrier.  Weights (A) take the M = 128
// side, tokens (B) the N side, so ragged per-expert token counts only change N.
#include "umma.cuh"
#include <cuda.h>
#include <vector>
#include <utility>
#include <cstdlib>
#include <cstdio>

namespace moe {

constexpr int kBH = 2048;  // hidden
constexpr int kBI = 512;   // moe_intermediate_size == shared_expert_intermediate_size
constexpr int kNT = 256;   // tokens per tile (MMA N, padded to a multiple of 16)
constexpr int kProdWarps = 16;                  // operand producers / epilogue
constexpr int kProdThreads = kProdWarps * 32;
constexpr int kGemmThreads = kProdThreads + 32;  // + one MMA-issuing warp
constexpr int kAStages = 2;   // dequantised weight tiles (produced locally: shallow ring)
constexpr int kBStages = 4;   // activation tiles (copied from L2: deep ring, kBStages - 1 K steps of lookahead)
constexpr int kFullRing = 4;  // "operands in place" barriers (producers run at most kAStages steps ahead of the MMAs)
constexpr int kMaxEPerLane = 16;
constexpr int kSlotPathMaxTokens = 256;  // the slot-wise expert FFN's work area is sized for this many tokens
constexpr int kSlotPathDefault = 48;     // batches up to this size take it: 76 against 128 us at 8 tokens, 147 against 191 us
                                         // at 32, level at 64 (L2-to-SM traffic grows with the slots), behind from there

// position of logical column j (0..7) inside a K-interleaved 8-block
__host__ __device__ __forceinline__ int ipos(int j) { return ((j & 3) << 1) | (j >> 2); }

// ─── prep: norm, bf16/f32 activations, shared gate ──────────────────────────
__global__ void __launch_bounds__(256) batch_prep_kernel(const float* __restrict__ h_in, int n, LayerDev ly,
                                                         __nv_bfloat16* __restrict__ x_bf,
                                                         __nv_bfloat16* __restrict__ x_mid,
                                                         __nv_bfloat16* __restrict__ x_lo, float* __restrict__ sgate,
                                                         int32_t* __restrict__ counts, int n_counts) {
    const int t = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    __shared__ float red[8];
    // the expert histogram of this layer starts from zero (it is filled two kernels later)
    if (t == 0)
        for (int i = tid; i < n_counts; i += 256) counts[i] = 0;
    const float4* hp = reinterpret_cast<const float4*>(h_in + (size_t)t * kBH) + tid * 2;
    const float4 a = hp[0], b = hp[1];
    float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) ss += v[i] * v[i];
    ss = warp_sum(ss);
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    float tot = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) tot += red[i];
    // rms_norm_bf16 (reference src/math_util.rs:282-288)
    const float inv_rms = 1.0f / sqrtf(tot / (float)kBH + 1e-6f);
    const uint4 nw = reinterpret_cast<const uint4*>(ly.post_norm)[tid];
    const uint32_t nwr[4] = {nw.x, nw.y, nw.z, nw.w};
    float x[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        x[2 * i] = v[2 * i] * inv_rms * __uint_as_float(nwr[i] << 16);
        x[2 * i + 1] = v[2 * i + 1] * inv_rms * __uint_as_float(nwr[i] & 0xFFFF0000u);
    }
    // bf16, K-interleaved: stored order [0,4,1,5,2,6,3,7]; x = hi + mid + lo to 24 significant bits
    // (hi feeds the expert GEMMs, all three the f32-accurate router)
    uint16_t ph[8], pm[8], pl[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int q = ((i & 3) << 1) | (i >> 2);
        const __nv_bfloat16 hb = __float2bfloat16_rn(x[i]);
        const float r1 = x[i] - __bfloat162float(hb);
        const __nv_bfloat16 mb = __float2bfloat16_rn(r1);
        const __nv_bfloat16 lb = __float2bfloat16_rn(r1 - __bfloat162float(mb));
        ph[q] = __bfloat16_as_ushort(hb); pm[q] = __bfloat16_as_ushort(mb); pl[q] = __bfloat16_as_ushort(lb);
    }
    auto pack8 = [](const uint16_t (&v)[8]) {
        return make_uint4(v[0] | ((uint32_t)v[1] << 16), v[2] | ((uint32_t)v[3] << 16), v[4] | ((uint32_t)v[5] << 16),
                          v[6] | ((uint32_t)v[7] << 16));
    };
    reinterpret_cast<uint4*>(x_bf + (size_t)t * kBH)[tid] = pack8(ph);
    reinterpret_cast<uint4*>(x_mid + (size_t)t * kBH)[tid] = pack8(pm);
    reinterpret_cast<uint4*>(x_lo + (size_t)t * kBH)[tid] = pack8(pl);
    // shared_expert_gate . x : thread tid owns word tid of the single 4-bit row
    const uint32_t w = ly.sgate.w[tid];
    const float s = bf16_bits_to_f32(ly.sgate.s[tid >> 3]);
    const float bb = bf16_bits_to_f32(ly.sgate.b[tid >> 3]);
    float acc = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) acc += ((float)((w >> (4 * i)) & 0xFu) * s + bb) * x[i];
    acc = warp_sum(acc);
    __syncthreads();
    if (lane == 0) red[warp] = acc;
    __syncthreads();
    if (tid == 0) {
        float sc = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) sc += red[i];
        sgate[t] = 1.0f / (1.0f + expf(-sc));  // sigmoid (reference src/math_util.rs:67-69)
    }
}

// 16-byte asynchronous copy global -> shared; src_bytes == 0 writes zeros.
__device__ __forceinline__ void cp16_zfill(uint32_t dst_smem, const void* src, uint32_t src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst_smem), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_commit_group() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_wait_group() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// ─── router logits on the tensor cores, to f32 accuracy ─────────────────────
// logits[n, E] = X[n, H] . Wr[E, H]^T.  The expert choice must match an f32
// evaluation, so neither operand may simply be rounded to bf16: every f32 value
// v is split into three bf16 terms hi + mid + lo (24 significant bits) and the
// products of total order <= 2 are accumulated in f32 by tcgen05.mma:
//   bf16 router (BQ4):  W . (x_hi + x_mid + x_lo)                         3 MMAs per K block
//   4-bit router (INT4): W_hi.x_hi + W_hi.x_mid + W_mid.x_hi + W_hi.x_lo + W_lo.x_hi + W_mid.x_mid   6 MMAs
// The weight planes are built once per layer (router_planes_kernel), the
// activation planes by the prep kernel, both K-interleaved; the GEMM kernel only
// copies tiles (16-byte asynchronous copies, three stages) and issues MMAs.
// One CTA = 128 experts x 64 tokens.
constexpr int kRtTok = 64;
constexpr int kRtMaxStages = 5;
constexpr int kRtATile = 128 * 128;   // 128 rows x 64 bf16
constexpr int kRtBTile = kRtTok * 128;
constexpr int kRtRing = 216 * 1024;   // bytes of operand stages: 3 for a bf16 router (256 rows per CTA), 3 for a 4-bit one (128 rows)
constexpr int kRtMaxSplit = 8;        // the contraction may be split over up to this many CTAs; batch_route_kernel adds the partial sums
// how many ways to split so that a small token count still fills the machine
static int router_split(int n, int E, int nplanes) {
    const int ctas = ((n + kRtTok - 1) / kRtTok) * (nplanes == 1 ? (E + 255) / 256 : (E + 127) / 128);
    int s = 1;
    while (s < kRtMaxSplit && ctas * s < 100) s *= 2;
    return s;
}
constexpr int kRtSmem = kRtRing + 1024;
constexpr int kRtAccCols = 256;       // TMEM columns per accumulator (3 x 64 used)
constexpr int kRtTmemCols = 512;

__device__ __forceinline__ void split3(float v, uint16_t& hi, uint16_t& mid, uint16_t& lo) {
    const __nv_bfloat16 h = __float2bfloat16_rn(v);
    const float r1 = v - __bfloat162float(h);
    const __nv_bfloat16 m = __float2bfloat16_rn(r1);
    const float r2 = r1 - __bfloat162float(m);
    const __nv_bfloat16 l = __float2bfloat16_rn(r2);
    hi = __bfloat16_as_ushort(h); mid = __bfloat16_as_ushort(m); lo = __bfloat16_as_ushort(l);
}

// planes[p][row][H] (bf16, K-interleaved, rows padded to a multiple of 128 with zeros);
// one thread per 8-column block.  4-bit weights are dequantised as the reference does,
// (nibble as f32) * scale + bias (src/math_util.rs:47), before the split.
__global__ void __launch_bounds__(256) router_planes_kernel(LayerDev ly, int E, int rows_padded, uint16_t* planes) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    const int per_row = kBH / 8;
    if (i >= rows_padded * per_row) return;
    const int row = i / per_row, blk = i - row * per_row;
    const bool q4 = ly.router_bf16 == nullptr;
    float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (row < E) {
        if (!q4) {
            const uint4 q = *reinterpret_cast<const uint4*>(ly.router_bf16 + (size_t)row * kBH + blk * 8);
            const uint32_t r[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) { v[2 * k] = __uint_as_float(r[k] << 16); v[2 * k + 1] = __uint_as_float(r[k] & 0xFFFF0000u); }
        } else {
            const uint32_t w = ly.router_q4.w[(size_t)row * per_row + blk];
            const float s = bf16_bits_to_f32(ly.router_q4.s[(size_t)row * (kBH / kGroup) + (blk >> 3)]);
            const float b = bf16_bits_to_f32(ly.router_q4.b[(size_t)row * (kBH / kGroup) + (blk >> 3)]);
#pragma unroll
            for (int k = 0; k < 8; ++k) v[k] = (float)((w >> (4 * k)) & 0xFu) * s + b;
        }
    }
    const int np = q4 ? 3 : 1;
    uint16_t pl[3][8];
#pragma unroll
    for (int k = 0; k < 8; ++k) split3(v[k], pl[0][ipos(k)], pl[1][ipos(k)], pl[2][ipos(k)]);
    for (int p = 0; p < np; ++p) {
        uint4 o;
        o.x = pl[p][0] | ((uint32_t)pl[p][1] << 16); o.y = pl[p][2] | ((uint32_t)pl[p][3] << 16);
        o.z = pl[p][4] | ((uint32_t)pl[p][5] << 16); o.w = pl[p][6] | ((uint32_t)pl[p][7] << 16);
        *reinterpret_cast<uint4*>(planes + ((size_t)p * rows_padded + row) * kBH + blk * 8) = o;
    }
}

// Operands arrive by tiled TMA loads (one instruction per 128 x 64 or 64 x 64 bf16 box, 128-byte
// swizzle applied by the copy engine): a thread-issued cp.async costs its warp about 130 cycles
// per instruction, which made this short, latency-bound kernel several times slower.
// Warp 0 lane 0 requests tiles, warp 1 lane 0 issues the MMAs, all 8 warps run the epilogue.
__device__ __forceinline__ void tma_load_2d(uint32_t dst_smem, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst_smem),
        "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
        : "memory");
}
__device__ __forceinline__ bool wait_or_abort(uint64_t* bar, uint32_t parity, volatile int* s_abort);

// map_w: the layer's router planes as one [nplanes * rows_padded][H] bf16 tensor;
// map_x: the activation planes hi/mid/lo as one [3 * x_rows][H] bf16 tensor.
__global__ void __launch_bounds__(256, 1) router_gemm_kernel(const __grid_constant__ CUtensorMap map_w,
                                                             const __grid_constant__ CUtensorMap map_x, int n, int E,
                                                             int nplanes, int rows_padded, int x_rows,
                                                             float* __restrict__ logits, unsigned int* err) {
    // A CTA computes logits for 64 tokens x (256 experts when the router is bf16, 128 when it is three
    // planes of a 4-bit one) over one kRtSplit-th of the contraction, into its own partial-sum slab.
    const int nacc = (nplanes == 1) ? 2 : 1;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* stages = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ uint64_t bar_full[kRtMaxStages];
    __shared__ uint64_t bar_empty[kRtMaxStages];
    __shared__ uint64_t bar_acc;
    __shared__ uint32_t tmem_slot;
    __shared__ int s_abort_mem;
    volatile int* s_abort = &s_abort_mem;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int t0 = blockIdx.x * kRtTok, e0 = blockIdx.y * 128 * nacc;
    logits += (size_t)blockIdx.z * n * E;
    // a stage holds nacc * nplanes weight tiles and the three activation tiles
    const int na = nacc * nplanes;
    const uint32_t stage_bytes = (uint32_t)na * kRtATile + 3u * kRtBTile;
    const int S = min(kRtMaxStages, (int)(kRtRing / stage_bytes));
    if (tid == 0) {
        for (int i = 0; i < kRtMaxStages; ++i) { mbar_init(&bar_full[i], 1); mbar_init(&bar_empty[i], 1); }
        mbar_init(&bar_acc, 1);
        s_abort_mem = 0;
        mbar_fence_init();
    }
    if (warp == 0) umma::tmem_alloc(&tmem_slot, kRtTmemCols);
    umma::fence_before_sync();
    __syncthreads();
    umma::fence_after_sync();
    const uint32_t tmem = tmem_slot;
    const uint32_t stages_addr = smem_u32(stages);
    const int kSteps = kBH / 64 / (int)gridDim.z;
    const int kc0 = blockIdx.z * kSteps;  // first K step of this CTA's share

    if (tid == 0) {
        // ─── tile requests ────────────────────────────────────────────────────
        for (int kc = 0; kc < kSteps; ++kc) {
            const int st = kc % S, use = kc / S;
            if (use > 0 && !wait_or_abort(&bar_empty[st], (uint32_t)(use - 1) & 1u, s_abort)) break;
            const uint32_t base = stages_addr + (uint32_t)st * stage_bytes;
            mbar_expect_tx(&bar_full[st], stage_bytes);
            // weight tile i = a * nplanes + p: plane p of expert rows e0 + 128 a ..
            for (int i = 0; i < na; ++i) {
                const int a = i / nplanes, p = i - a * nplanes;
                tma_load_2d(base + i * kRtATile, &map_w, (kc0 + kc) * 64, p * rows_padded + e0 + 128 * a, &bar_full[st]);
            }
            for (int p = 0; p < 3; ++p)
                tma_load_2d(base + na * kRtATile + p * kRtBTile, &map_x, (kc0 + kc) * 64, p * x_rows + t0, &bar_full[st]);
        }
    } else if (tid == 32) {
        // ─── MMA issue ────────────────────────────────────────────────────────
        // The three activation tiles (hi, mid, lo; 64 token rows each) are stacked in shared memory, so one MMA
        // with N = 192 multiplies a weight tile with all three (N = 128, 64 for the smaller weight terms); the
        // three column groups of the accumulator are added in the epilogue.
        const uint32_t idesc3 = umma::make_idesc_bf16(128, 3 * kRtTok), idesc2 = umma::make_idesc_bf16(128, 2 * kRtTok),
                       idesc1 = umma::make_idesc_bf16(128, kRtTok);
        for (int kc = 0; kc < kSteps; ++kc) {
            const int st = kc % S, use = kc / S;
            if (!wait_or_abort(&bar_full[st], (uint32_t)use & 1u, s_abort)) break;
            umma::fence_after_sync();
            const uint32_t a0 = stages_addr + (uint32_t)st * stage_bytes, b0 = a0 + na * kRtATile;
#pragma unroll
            for (int k16 = 0; k16 < 4; ++k16) {
                const uint32_t o = k16 * 32;
                const uint64_t bx = umma::make_desc_sw128_kmajor(b0 + o);
                const uint32_t first = (kc > 0 || k16 > 0) ? 1u : 0u;
                for (int a = 0; a < nacc; ++a) {
                    const uint32_t d = tmem + a * kRtAccCols, aa = a0 + a * nplanes * kRtATile + o;
                    umma::mma_bf16(d, umma::make_desc_sw128_kmajor(aa), bx, idesc3, first);  // W_hi . {x_hi, x_mid, x_lo}
                    if (nplanes == 3) {
                        umma::mma_bf16(d, umma::make_desc_sw128_kmajor(aa + kRtATile), bx, idesc2, 1u);      // W_mid . {x_hi, x_mid}
                        umma::mma_bf16(d, umma::make_desc_sw128_kmajor(aa + 2 * kRtATile), bx, idesc1, 1u);  // W_lo . x_hi
                    }
                }
            }
            umma::commit(&bar_empty[st]);
            if (kc == kSteps - 1) umma::commit(&bar_acc);
        }
    }
    __syncwarp();
    const bool acc_ok = wait_or_abort(&bar_acc, 0, s_abort);
    const bool alive = __syncthreads_and(acc_ok ? 1 : 0) != 0;
    if (alive) {
        umma::fence_after_sync();
        {
            const int quad = warp & 3, cb = warp >> 2;  // 8 warps: 4 lane quadrants x 2 column blocks of 32 tokens
            for (int a = 0; a < nacc; ++a) {
                const int e = e0 + 128 * a + quad * 32 + lane;
                float g[32], gm[32], gl[32];
                const uint32_t ta = tmem + ((uint32_t)(quad * 32) << 16) + (uint32_t)(a * kRtAccCols + cb * 32);
                umma::ld_32x32(ta, g);
                umma::ld_32x32(ta + kRtTok, gm);
                umma::ld_32x32(ta + 2 * kRtTok, gl);
#pragma unroll
                for (int c = 0; c < 32; ++c) {
                    const int t = t0 + cb * 32 + c;
                    if (t < n && e < E) logits[(size_t)t * E + e] = (g[c] + gm[c]) + gl[c];
                }
            }
        }
    } else if (tid == 0) {
        atomicExch(err, 8u);
    }
    umma::fence_before_sync();
    __syncthreads();
    if (warp == 0) umma::tmem_dealloc(tmem, kRtTmemCols);
}

// every rank's exported buffer as mapped into this process (expert parallelism)
struct EpPeers {
    uint8_t* base[kEpMaxWorld];
};
// what the route kernel needs to send the histogram to the peers (world = 0: single GPU, nothing is sent)
struct EpPush {
    EpPeers peers;
    size_t counts_off, flags_off;
    int me, world;
    unsigned int epoch;
    unsigned int* done;
};

// ─── route: one warp per token ──────────────────────────────────────────────
// route_experts (reference src/engine/qwen35_moe/cpu.rs:78-85; softmax, top-k and
// renormalise of src/math_util.rs:77-126).  Ties go to the lower index.  Results in
// descending order.  Also counts tokens per expert.
template <int NPER>  // experts per lane: 8 covers 256 experts, 16 covers 512
__global__ void __launch_bounds__(256) batch_route_kernel(const float* __restrict__ logits, int n, int E, int K,
                                                          const float* __restrict__ bias,
                                                          const int32_t* __restrict__ forced,
                                                          int32_t* __restrict__ topk_idx, float* __restrict__ topk_w,
                                                          int32_t* __restrict__ counts, int nsplit, EpPush ep,
                                                          unsigned int* err) {
    const int t = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (t < n) {
    const float* lg = logits + (size_t)t * E;
    const size_t slab = (size_t)n * E;  // the router GEMM leaves kRtSplit partial sums, added here in a fixed order
    float p[NPER];
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < NPER; ++i) {
        const int e = lane + 32 * i;
        float v = -INFINITY;
        if (e < E) {
            // all partial sums are requested before the first is used; they are added in slab order
            float part[kRtMaxSplit];
#pragma unroll
            for (int z = 0; z < kRtMaxSplit; ++z) part[z] = (z < nsplit) ? __ldg(lg + e + z * slab) : 0.0f;
            v = part[0];
#pragma unroll
            for (int z = 1; z < kRtMaxSplit; ++z)
                if (z < nsplit) v += part[z];
            if (bias) v += bias[e];
        }
        p[i] = v;
        mx = fmaxf(mx, v);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float sum = 0.0f;
#pragma unroll
    for (int i = 0; i < NPER; ++i) {
        p[i] = (lane + 32 * i < E) ? expf(p[i] - mx) : 0.0f;
        sum += p[i];
    }
    sum = warp_sum(sum);
    const float inv = 1.0f / sum;
#pragma unroll
    for (int i = 0; i < NPER; ++i) p[i] = (lane + 32 * i < E) ? p[i] * inv : -1.0f;
    float myw = 0.0f;
    int myi = 0;
    if (forced) {
        for (int k = 0; k < K; ++k) {
            int e = forced[(size_t)t * K + k];
            if ((unsigned)e >= (unsigned)E) {  // a caller's index outside [0, E): reported, never dereferenced
                if (lane == 0) atomicExch(err, 10u);
                e = 0;
            }
            float v = 0.0f;
#pragma unroll
            for (int i = 0; i < NPER; ++i)
                if (lane + 32 * i == e) v = p[i];
            v = __shfl_sync(0xffffffffu, v, e & 31);
            if (lane == k) { myw = v; myi = e; }
        }
    } else {
        uint32_t taken = 0;  // bit i: this lane's i-th expert has been chosen
        for (int k = 0; k < K; ++k) {
            float bv = -1.0f;  // chosen experts and lanes beyond E hold -1: never greater than this
            int be = 0x7fffffff;
#pragma unroll
            for (int i = 0; i < NPER; ++i)
                if (p[i] > bv) { bv = p[i]; be = lane + 32 * i; }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
                const int oe = __shfl_xor_sync(0xffffffffu, be, o);
                if (ov > bv || (ov == bv && oe < be)) { bv = ov; be = oe; }
            }
            if (be >= E) {
                // Nothing compared greater: the remaining probabilities are NaN.  Take the lowest expert not
                // chosen yet (all-NaN logits give experts 0..K-1, as the reference's heap does,
                // src/math_util.rs:89-99); an index outside [0, E) must never reach the histogram.
                int lo = 0x7fffffff;
#pragma unroll
                for (int i = NPER - 1; i >= 0; --i)
                    if (lane + 32 * i < E && !((taken >> i) & 1u)) lo = lane + 32 * i;
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) lo = min(lo, __shfl_xor_sync(0xffffffffu, lo, o));
                be = lo;  // K <= E, so one exists
                bv = NAN;
            }
            if (lane == k) { myw = bv; myi = be; }
#pragma unroll
            for (int i = 0; i < NPER; ++i)
                if (lane + 32 * i == be) { p[i] = -1.0f; taken |= 1u << i; }
        }
    }
    const float ws = warp_sum(lane < K ? myw : 0.0f);
    if (ws > 0.0f) myw *= (1.0f / ws);
    if (lane < K) {
        topk_idx[(size_t)t * K + lane] = myi;
        topk_w[(size_t)t * K + lane] = myw;
        atomicAdd(&counts[myi], 1);
    }
    }
    // expert parallelism: the last block to finish sends this rank's histogram to every peer and
    // publishes the epoch (the plan kernel of every rank waits for it)
    if (ep.world > 0) {
        __shared__ int s_last;
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) {
            const unsigned int prev = atomicAdd(ep.done, 1u);
            s_last = (prev == gridDim.x - 1) ? 1 : 0;
            if (s_last) *ep.done = 0u;
        }
        __syncthreads();
        if (s_last) {
            __threadfence();
            for (int i = threadIdx.x; i < ep.world * E; i += blockDim.x) {
                const int d = i / E, e = i - d * E;
                reinterpret_cast<int32_t*>(ep.peers.base[d] + ep.counts_off)[(size_t)ep.me * E + e] = __ldcg(counts + e);
            }
            __threadfence_system();
            __syncthreads();
            if (threadIdx.x < 32 && (int)threadIdx.x < ep.world) {
                unsigned int* f = reinterpret_cast<unsigned int*>(ep.peers.base[threadIdx.x] + ep.flags_off) + ep.me * 16;
                asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(f), "r"(ep.epoch) : "memory");
            }
        }
    }
}

// ─── plan: scan of the histogram and the tile list; one block ───────────────
__global__ void __launch_bounds__(1024) batch_plan_kernel(int32_t* counts, int32_t* offsets, int32_t* cursor, int E,
                                                          int n, int32_t* tile_list, int32_t* n_tiles, int max_tiles) {
    __shared__ int s_off[1024 + 1];
    __shared__ int s_tile[1024 + 1];
    const int tid = threadIdx.x;
    if (tid == 0) counts[E] = n;  // the shared expert sees every token
    __syncthreads();
    const int c = (tid <= E) ? counts[tid] : 0;
    const int nt = (c + kNT - 1) / kNT;
    s_off[tid] = c;
    s_tile[tid] = nt;
    __syncthreads();
    if (tid == 0) {  // E + 1 <= 513 entries: a serial scan is a few microseconds
        int a = 0, b = 0;
        for (int i = 0; i <= E; ++i) {
            const int ca = s_off[i], cb = s_tile[i];
            s_off[i] = a; s_tile[i] = b;
            a += ca; b += cb;
        }
        s_off[E + 1] = a;
        s_tile[E + 1] = b;
        *n_tiles = b < max_tiles ? b : max_tiles;
    }
    __syncthreads();
    if (tid <= E + 1) offsets[tid] = s_off[tid];
    if (tid <= E) {
        cursor[tid] = 0;
        for (int i = 0; i < nt; ++i) {
            const int k = s_tile[tid] + i;
            if (k < max_tiles) {
                tile_list[3 * k] = tid;
                tile_list[3 * k + 1] = s_off[tid] + i * kNT;
                tile_list[3 * k + 2] = min(kNT, c - i * kNT);
            }
        }
    }
}

// ─── scatter: (token, k) -> expert-sorted slot ──────────────────────────────
__global__ void __launch_bounds__(256) batch_scatter_kernel(const int32_t* __restrict__ topk_idx, int n, int K, int E,
                                                            const int32_t* __restrict__ offsets, int32_t* cursor,
                                                            int32_t* __restrict__ slot_token,
                                                            int32_t* __restrict__ slot_of,
                                                            int32_t* __restrict__ slot_expert) {  // nullable
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n * K) {
        const int t = i / K;
        const int e = topk_idx[i];
        const int slot = offsets[e] + atomicAdd(&cursor[e], 1);
        slot_token[slot] = t;
        slot_of[i] = slot;
        if (slot_expert) slot_expert[slot] = e;
    }
    if (i < n) {
        slot_token[offsets[E] + i] = i;
        if (slot_expert) slot_expert[offsets[E] + i] = E;
    }
}

// ─── grouped GEMM ───────────────────────────────────────────────────────────
struct GemmParams {
    const uint8_t* experts;       // E packed experts of this layer
    const uint8_t* shared;        // shared expert, same layout
    moe_expert_layout_t lay;
    int E;
    const __nv_bfloat16* x;       // [n, H] bf16 K-interleaved           (gemm1 B operand)
    __nv_bfloat16* act;           // [slots, I] bf16 K-interleaved         (gemm1 out, gemm2 B operand)
    __nv_bfloat16* o;             // [slots, H] bf16                       (gemm2 out)
    const int32_t* tile_list;
    const int32_t* n_tiles;
    const int32_t* slot_token;
    unsigned int* err;
    // expert-parallel use: before touching x, wait until every peer has published `ep_epoch` (ep_world = 0: no wait)
    const uint8_t* ep_local;
    size_t ep_flags;
    int ep_world;
    unsigned int ep_epoch;
};

// Hand-offs between the GPUs of an expert-parallel group are epoch numbers in a flag word per
// (receiver, sender).  Lanes 0..P-1 of the calling warp wait until every sender has published
// `epoch` to this rank; bounded (an error word is raised and the caller goes on).
__device__ __forceinline__ void ep_wait_warp(const uint8_t* local, size_t flags_off, int P, unsigned int epoch,
                                             unsigned int* err, int lane) {
    if (lane < P) {
        const unsigned int* f = reinterpret_cast<const unsigned int*>(local + flags_off) + lane * 16;
        const long long t0 = clock64();
        for (;;) {
            unsigned int v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
            if ((int)(v - epoch) >= 0) break;
            if (clock64() - t0 > kWaitCycles) { atomicExch(err, 9u); break; }
        }
    }
    __threadfence_system();
    __syncwarp();
}

// 8 nibbles of one word -> 8 bf16 (n * s + b) in the order [0,4,1,5,2,6,3,7]
__device__ __forceinline__ uint4 dequant_word(uint32_t w, __nv_bfloat162 s2, __nv_bfloat162 b2) {
    const uint32_t kMask = 0x000F000Fu, kMagic = 0x43004300u;  // bf16 128.0 in both halves
    const __nv_bfloat162 c128 = __floats2bfloat162_rn(128.0f, 128.0f);
    uint32_t t[4];
    t[0] = (w & kMask) | kMagic;
    t[1] = ((w >> 4) & kMask) | kMagic;
    t[2] = ((w >> 8) & kMask) | kMagic;
    t[3] = ((w >> 12) & kMask) | kMagic;
    uint32_t r[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        // (128 + n) - 128 = n exactly; n * s + b rounded once to bf16
        const __nv_bfloat162 nn = __hsub2(*reinterpret_cast<__nv_bfloat162*>(&t[i]), c128);
        const __nv_bfloat162 v = __hfma2(nn, s2, b2);
        r[i] = *reinterpret_cast<const uint32_t*>(&v);
    }
    return make_uint4(r[0], r[1], r[2], r[3]);
}

// Bounded, abort-aware mbarrier wait: gives up after about a second of SM clocks or as
// soon as another warp of the CTA has given up (s_abort), so that a broken pipeline
// drains instead of hanging.
__device__ __forceinline__ bool wait_or_abort(uint64_t* bar, uint32_t parity, volatile int* s_abort) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (uint32_t i = 1;; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 63u) == 0u && (*s_abort || clock64() - t0 > kWaitCycles)) {
            *s_abort = 1;
            return false;
        }
    }
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}


// Warp roles: warps 0..15 produce the operand tiles (dequantised weights, copied
// activations) and run the epilogue; warp 16 only issues the MMAs, because a
// tcgen05.mma issue blocks its thread for about as long as the MMA runs.
template <int MODE>  // 1: gate/up + SwiGLU -> act ; 2: down -> o
__global__ void __launch_bounds__(kGemmThreads, 1) grouped_gemm_kernel(GemmParams p) {
    constexpr int kIn = (MODE == 1) ? kBH : kBI;            // contraction length
    constexpr int kKC = kIn / 64;                           // K steps (one quantisation group each)
    // work item = (token tile, row block): 128 gate rows + the same 128 up rows, or 256 down rows;
    // either way two M = 128 accumulators share one activation tile
    constexpr int kRB = (MODE == 1) ? kBI / 128 : kBH / 256;
    constexpr int kARows = 256;
    constexpr int kABytes = kARows * 128;
    constexpr int kBBytes = kNT * 128;
    constexpr int kLook = kBStages - 1;  // K steps between requesting an activation tile and using it
    constexpr uint32_t kTmemCols = 512;
    static_assert(kKC > kLook, "the prologue requests the first kLook activation tiles");
    static_assert(kARows * 2 == kProdThreads, "one (row, half-group) dequant task per producer thread");
    constexpr int kWRing = 4;  // K steps of weight words in flight in registers
    static_assert(kKC % kWRing == 0, "the weight prefetch ring cycles through kWRing register sets");

    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* stages = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ uint64_t bar_full[kFullRing];    // producers -> MMA warp: operands of a K step are in place
    __shared__ uint64_t bar_empty_a[kAStages];  // MMA completion -> producers: weight stage may be overwritten
    __shared__ uint64_t bar_empty_b[kBStages];  // MMA completion -> producers: activation stage may be overwritten
    __shared__ uint64_t bar_acc;             // MMA completion -> epilogue: accumulators are final
    __shared__ uint64_t bar_tfree;           // epilogue -> MMA warp: accumulators have been read
    __shared__ uint32_t tmem_slot;
    __shared__ int s_abort_mem;
    volatile int* s_abort = &s_abort_mem;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) {
        for (int i = 0; i < kFullRing; ++i) mbar_init(&bar_full[i], kProdWarps);
        for (int i = 0; i < kAStages; ++i) mbar_init(&bar_empty_a[i], 1);
        for (int i = 0; i < kBStages; ++i) mbar_init(&bar_empty_b[i], 1);
        mbar_init(&bar_acc, 1);
        mbar_init(&bar_tfree, kProdWarps);
        s_abort_mem = 0;
        mbar_fence_init();
    }
    if (warp == 0) umma::tmem_alloc(&tmem_slot, kTmemCols);
    if (warp == 1 && p.ep_world > 0) ep_wait_warp(p.ep_local, p.ep_flags, p.ep_world, p.ep_epoch, p.err, lane);
    umma::fence_before_sync();
    __syncthreads();
    umma::fence_after_sync();
    const uint32_t tmem = tmem_slot;
    const uint32_t stages_addr = smem_u32(stages);
    const uint32_t b_ring_addr = stages_addr + kAStages * kABytes;  // activation stages follow the weight stages

    const int n_items = *p.n_tiles * kRB;
    uint32_t it = 0;       // K steps so far (drives the stage ring and the mbarrier parities)
    uint32_t n_done = 0;   // items finished by this CTA
    bool alive = true;

    if (warp == kProdWarps) {
        // ─── MMA issuer ───────────────────────────────────────────────────────
        for (int item = blockIdx.x; item < n_items && alive; item += gridDim.x) {
            const int tile = item / kRB;
            const int nt = p.tile_list[3 * tile + 2];
            const uint32_t idesc = umma::make_idesc_bf16(128, (uint32_t)((nt + 15) & ~15));
            for (int kc = 0; kc < kKC && alive; ++kc, ++it) {
                const uint32_t sa = it % kAStages, sb = it % kBStages, sf = it % kFullRing;
                bool ok = wait_or_abort(&bar_full[sf], (it / kFullRing) & 1, s_abort);
                // the previous item's accumulators must have been read before they are overwritten
                if (kc == 0 && n_done > 0) ok = wait_or_abort(&bar_tfree, (n_done - 1) & 1, s_abort) && ok;
                alive = __all_sync(0xffffffffu, ok);
                if (!alive) break;
                if (lane == 0) {
                    umma::fence_after_sync();
                    const uint32_t a_addr = stages_addr + sa * kABytes, b_addr = b_ring_addr + sb * kBBytes;
#pragma unroll
                    for (int k16 = 0; k16 < 4; ++k16) {
                        const uint64_t db = umma::make_desc_sw128_kmajor(b_addr + k16 * 32);
                        const uint32_t acc = (kc > 0 || k16 > 0) ? 1u : 0u;
                        umma::mma_bf16(tmem, umma::make_desc_sw128_kmajor(a_addr + k16 * 32), db, idesc, acc);
                        umma::mma_bf16(tmem + kNT, umma::make_desc_sw128_kmajor(a_addr + 128 * 128 + k16 * 32), db, idesc, acc);
                    }
                    umma::commit(&bar_empty_a[sa]);
                    umma::commit(&bar_empty_b[sb]);
                    if (kc == kKC - 1) umma::commit(&bar_acc);
                }
                __syncwarp();
            }
            ++n_done;
        }
    } else {
        // ─── producers + epilogue ─────────────────────────────────────────────
        for (int item = blockIdx.x; item < n_items && alive; item += gridDim.x) {
            const int tile = item / kRB, rb = item - tile * kRB;
            const int e = p.tile_list[3 * tile], s0 = p.tile_list[3 * tile + 1], nt = p.tile_list[3 * tile + 2];
            const int N = (nt + 15) & ~15;
            const uint8_t* ex = (e < p.E) ? p.experts + (size_t)e * p.lay.expert_size : p.shared;

            // this thread's dequant task: (row of the A tile, half of the 64-column group)
            const int r = tid >> 1, half = tid & 1;
            const uint32_t* wp;
            const uint16_t* sp;
            const uint16_t* bp;
            if (MODE == 1) {
                const int up = r >> 7, row = rb * 128 + (r & 127);
                wp = reinterpret_cast<const uint32_t*>(ex + (up ? p.lay.up_w : p.lay.gate_w)) + (size_t)row * (kBH / 8) + half * 4;
                sp = reinterpret_cast<const uint16_t*>(ex + (up ? p.lay.up_s : p.lay.gate_s)) + (size_t)row * (kBH / kGroup);
                bp = reinterpret_cast<const uint16_t*>(ex + (up ? p.lay.up_b : p.lay.gate_b)) + (size_t)row * (kBH / kGroup);
            } else {
                const int row = rb * 256 + r;
                wp = reinterpret_cast<const uint32_t*>(ex + p.lay.down_w) + (size_t)row * (kBI / 8) + half * 4;
                sp = reinterpret_cast<const uint16_t*>(ex + p.lay.down_s) + (size_t)row * (kBI / kGroup);
                bp = reinterpret_cast<const uint16_t*>(ex + p.lay.down_b) + (size_t)row * (kBI / kGroup);
            }
            uint32_t aoff[4];  // swizzled byte offsets of the task's four 16-byte outputs inside a stage
            {
                const uint32_t sub = (r >= 128) ? 128u * 128u : 0u;
#pragma unroll
                for (int wi = 0; wi < 4; ++wi) aoff[wi] = sub + umma::sw128_offset((uint32_t)(r & 127), (uint32_t)(half * 4 + wi));
            }
            // this thread's pieces of the activation tile: piece q = tid + 512 * i -> (token row q >> 3, chunk q & 7)
            constexpr int kBPieces = kNT * 8 / kProdThreads;  // 4
            const __nv_bfloat16* bsrc[kBPieces];
            uint32_t boff[kBPieces];
#pragma unroll
            for (int i = 0; i < kBPieces; ++i) {
                const int q = tid + i * kProdThreads;
                const int j = q >> 3, c = q & 7;
                const int jj = j < nt ? j : 0;
                // (the map may have been written by a peer GPU after this kernel started: read it through L2)
                bsrc[i] = ((MODE == 1) ? p.x + (size_t)__ldcg(p.slot_token + s0 + jj) * kBH : p.act + (size_t)(s0 + jj) * kBI) + c * 8;
                boff[i] = umma::sw128_offset((uint32_t)j, (uint32_t)c);
            }
            // asynchronous copy of the activation tile of K step kc into activation stage st (rows >= nt zero-filled)
            auto issue_b = [&](int kc, uint32_t st) {
                const uint32_t base = b_ring_addr + st * kBBytes;
#pragma unroll
                for (int i = 0; i < kBPieces; ++i) {
                    const int j = (tid + i * kProdThreads) >> 3;
                    if (j < N) cp16_zfill(base + boff[i], bsrc[i] + kc * 64, j < nt ? 16u : 0u);
                }
            };
            // weight words, scales and biases of kWRing K steps in flight in registers
            uint4 wq[kWRing];
            uint16_t sq[kWRing], bq[kWRing];
            auto load_a = [&](int kc, uint4& w, uint16_t& sc, uint16_t& bi) {
                w = ld_stream_u4(wp + kc * 8);
                sc = __ldg(sp + kc);
                bi = __ldg(bp + kc);
            };

            bool ok = true;
            {   // prologue: weights of the first kWRing K steps, activations of the first kLook K steps
#pragma unroll
                for (int i = 0; i < kWRing; ++i) load_a(i, wq[i], sq[i], bq[i]);
#pragma unroll
                for (int j = 0; j < kLook; ++j) {
                    const uint32_t g = it + j, sb = g % kBStages, use = g / kBStages;
                    if (use > 0) ok = wait_or_abort(&bar_empty_b[sb], (use - 1) & 1, s_abort) && ok;
                    issue_b(j, sb);
                    cp_commit_group();
                }
            }
            auto k_step = [&](int kc, uint4& w, uint16_t& sc, uint16_t& bi) {
                const uint32_t sa = it % kAStages;
                // dequantise this K step's 64 columns of this thread's row half, once the MMAs that read
                // this weight stage kAStages K steps ago are done
                {
                    const uint32_t use = it / kAStages;
                    if (use > 0) ok = wait_or_abort(&bar_empty_a[sa], (use - 1) & 1, s_abort) && ok;
                }
                unsigned char* a_tile = stages + sa * kABytes;
                const uint32_t s32 = (uint32_t)sc | ((uint32_t)sc << 16);
                const uint32_t b32 = (uint32_t)bi | ((uint32_t)bi << 16);
                const __nv_bfloat162 s2 = *reinterpret_cast<const __nv_bfloat162*>(&s32);
                const __nv_bfloat162 b2 = *reinterpret_cast<const __nv_bfloat162*>(&b32);
                const uint32_t words[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
                for (int wi = 0; wi < 4; ++wi)
                    *reinterpret_cast<uint4*>(a_tile + aoff[wi]) = dequant_word(words[wi], s2, b2);
                if (kc + kWRing < kKC) load_a(kc + kWRing, w, sc, bi);  // refill this register set
                cp_wait_group<kLook - 1>();  // this K step's activation pieces have landed (later ones may be in flight)
                umma::fence_smem_to_async();
                __syncwarp();
                if (lane == 0) mbar_arrive(&bar_full[it % kFullRing]);
                // The activations of K step kc + kLook go into the stage that K step kc - 1 used: its MMAs
                // were issued a whole dequantisation ago, so this wait is short, and it sits after this
                // step's hand-off so that it never delays the tensor pipe.
                if (kc + kLook < kKC) {
                    const uint32_t g = it + kLook, sb = g % kBStages, use = g / kBStages;
                    if (use > 0) ok = wait_or_abort(&bar_empty_b[sb], (use - 1) & 1, s_abort) && ok;
                    issue_b(kc + kLook, sb);
                }
                cp_commit_group();
                ++it;
            };
            for (int kc = 0; kc < kKC; kc += kWRing) {
#pragma unroll
                for (int i = 0; i < kWRing; ++i) k_step(kc + i, wq[i], sq[i], bq[i]);
                if (!__all_sync(0xffffffffu, ok)) { alive = false; break; }
            }
            if (!alive) break;

            // ---- epilogue: TMEM -> registers -> global ----
            alive = __all_sync(0xffffffffu, wait_or_abort(&bar_acc, n_done & 1, s_abort));
            if (!alive) break;
            umma::fence_after_sync();
            {
                const int quad = warp & 3;                 // TMEM lanes 32*quad .. +31 belong to this warp
                constexpr int kColGroups = kProdWarps / 4;  // warps sharing a lane quadrant split the columns
                for (int cb = (warp >> 2); cb * 32 < N; cb += kColGroups) {
                    const uint32_t taddr = tmem + ((uint32_t)(quad * 32) << 16) + (uint32_t)(cb * 32);
                    float g[32], u[32];
                    umma::ld_32x32(taddr, g);
                    umma::ld_32x32(taddr + kNT, u);
                    if (MODE == 1) {
                        const int row = rb * 128 + quad * 32 + lane;  // gate/up row inside the expert matrix
                        const int pos = (row & ~7) | ipos(row & 7);
#pragma unroll
                        for (int c = 0; c < 32; ++c) {
                            const int col = cb * 32 + c;
                            if (col < nt) {
                                // swiglu_fused (reference src/math_util.rs:254-259)
                                const float a = __fdividef(g[c], 1.0f + __expf(-g[c])) * u[c];
                                p.act[(size_t)(s0 + col) * kBI + pos] = __float2bfloat16_rn(a);
                            }
                        }
                    } else {
                        const int row = rb * 256 + quad * 32 + lane;  // first accumulator: rows +0, second: rows +128
#pragma unroll
                        for (int c = 0; c < 32; ++c) {
                            const int col = cb * 32 + c;
                            if (col < nt) {
                                p.o[(size_t)(s0 + col) * kBH + row] = __float2bfloat16_rn(g[c]);
                                p.o[(size_t)(s0 + col) * kBH + row + 128] = __float2bfloat16_rn(u[c]);
                            }
                        }
                    }
                }
            }
            ++n_done;
            umma::fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bar_tfree);  // this warp has read its part of the accumulators
        }
        cp_wait_group<0>();
    }

    if (!alive && lane == 0) atomicExch(p.err, 7u);
    umma::fence_before_sync();
    __syncthreads();  // the only CTA-wide barrier after set-up: every role has left its loop
    if (warp == 0) umma::tmem_dealloc(tmem, kTmemCols);
}

// ─── combine ────────────────────────────────────────────────────────────────
// moe_combine_residual (reference src/math_util.rs:599-612) per token, reading the
// expert outputs through the token's slots.
__global__ void __launch_bounds__(256) batch_combine_kernel(const float* __restrict__ h_in, float* __restrict__ h_out,
                                                            int n, int K, int E, const __nv_bfloat16* __restrict__ o,
                                                            const int32_t* __restrict__ slot_of,
                                                            const float* __restrict__ topk_w,
                                                            const float* __restrict__ sgate,
                                                            const int32_t* __restrict__ offsets) {
    const int t = blockIdx.x, tid = threadIdx.x;
    const float4* hp = reinterpret_cast<const float4*>(h_in + (size_t)t * kBH) + tid * 2;
    const float4 a = hp[0], b = hp[1];
    float moe[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    auto add = [&](int slot, float w, float (&dst)[8]) {
        const uint4 q = __ldg(reinterpret_cast<const uint4*>(o + (size_t)slot * kBH) + tid);
        const uint32_t r[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            dst[2 * i] += w * __uint_as_float(r[i] << 16);
            dst[2 * i + 1] += w * __uint_as_float(r[i] & 0xFFFF0000u);
        }
    };
    for (int k = 0; k < K; ++k) add(slot_of[(size_t)t * K + k], topk_w[(size_t)t * K + k], moe);
    float sh[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    add(offsets[E] + t, sgate[t], sh);
    const float hin[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    float out[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) out[i] = hin[i] + moe[i] + sh[i];
    float4* op = reinterpret_cast<float4*>(h_out + (size_t)t * kBH) + tid * 2;
    op[0] = make_float4(out[0], out[1], out[2], out[3]);
    op[1] = make_float4(out[4], out[5], out[6], out[7]);
}

// ─── expert parallelism: dispatch / combine over peer memory ────────────────
// No counterpart in the reference (one device).  Rank r owns experts
// [r*E/P, (r+1)*E/P) of every layer; router, shared expert and norms are
// replicated; each rank brings its own tokens.  Per layer:
//   counts   every rank writes its expert histogram into every peer's table
//   plan     from the full table each rank derives (a) where its rows go inside the
//            owner's receive buffer and (b) the tile list over the rows it receives
//   scatter  each (token, k) row of bf16 activations is written straight into the
//            owner's buffer with 16-byte peer stores, with a return address
//   gemm     the owner runs the grouped GEMMs over what it received (+ the shared
//            expert over its own tokens)
//   return   the owner writes each output row back into the sender's buffer
//   combine  the sender adds residual, weighted expert rows and the shared expert
// Ranks meet through per-source epoch flags in the mapped buffers; every wait
// is bounded and raises the engine's error word instead of hanging.
// Lanes 0..P-1 of the calling warp publish this rank's epoch to every peer, after a system-scope
// fence: whatever this thread has observed as written is visible before the flag.
__device__ __forceinline__ void ep_signal_warp(const EpPeers& peers, const EpSym& sym, int me, int P, unsigned int epoch, int lane) {
    __threadfence_system();
    if (lane < P) {
        unsigned int* f = reinterpret_cast<unsigned int*>(peers.base[lane] + sym.flags) + me * 16;
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(f), "r"(epoch) : "memory");
    }
}

// True in exactly one block of the grid: the last one whose threads have all finished their stores
// (each thread fences at system scope before its block is counted).  That block resets the counter.
__device__ __forceinline__ bool ep_last_block(unsigned int* counter) {
    __shared__ int s_last;
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned int prev = atomicAdd(counter, 1u);
        s_last = (prev == gridDim.x - 1) ? 1 : 0;
        if (s_last) *counter = 0u;
    }
    __syncthreads();
    return s_last != 0;
}

// plan: one block.  counts_all[s][e] = rows rank s sends to expert e.
__global__ void __launch_bounds__(1024) ep_plan_kernel(const int32_t* counts_all, int me, int P, int E, int n_local,
                                                       int32_t* base_send, int32_t* cursor, int32_t* tile_list,
                                                       int32_t* n_tiles, int max_tiles, int32_t* total_recv,
                                                       const uint8_t* local, size_t flags_off, unsigned int epoch,
                                                       unsigned int* err) {
    // every peer's histogram must have arrived
    if (threadIdx.x < 32) ep_wait_warp(local, flags_off, P, epoch, err, threadIdx.x);
    __syncthreads();
    __shared__ int tot[1024];      // rows expert e receives from everybody
    __shared__ int before[1024];   // ... from ranks below me
    __shared__ int estart[1024];   // first slot of expert e inside its owner's buffer
    __shared__ int tstart[1024];   // first tile of my local expert
    __shared__ int s_total, s_tiles;
    const int tid = threadIdx.x, Eloc = E / P;
    if (tid < E) {
        int t = 0, b = 0;
        for (int s = 0; s < P; ++s) {
            const int c = counts_all[(size_t)s * E + tid];
            if (s < me) b += c;
            t += c;
        }
        tot[tid] = t;
        before[tid] = b;
    }
    __syncthreads();
    if (tid < P) {  // exclusive scan of each owner's experts
        int a = 0;
        for (int i = 0; i < Eloc; ++i) { estart[tid * Eloc + i] = a; a += tot[tid * Eloc + i]; }
        if (tid == me) s_total = a;
    }
    __syncthreads();
    if (tid < E) {
        base_send[tid] = estart[tid] + before[tid];
        cursor[tid] = 0;
    }
    if (tid == 0) {
        int b = 0;
        for (int i = 0; i < Eloc; ++i) { tstart[i] = b; b += (tot[me * Eloc + i] + kNT - 1) / kNT; }
        tstart[Eloc] = b;
        const int sh = (n_local + kNT - 1) / kNT;
        s_tiles = b + sh;
        *n_tiles = s_tiles < max_tiles ? s_tiles : max_tiles;
        *total_recv = s_total;
    }
    __syncthreads();
    if (tid < Eloc) {
        const int e = me * Eloc + tid, c = tot[e];
        for (int i = 0; i * kNT < c; ++i) {
            const int k = tstart[tid] + i;
            if (k < max_tiles) {
                tile_list[3 * k] = e;
                tile_list[3 * k + 1] = estart[e] + i * kNT;
                tile_list[3 * k + 2] = min(kNT, c - i * kNT);
            }
        }
    }
    if (tid == 0) {  // shared expert over this rank's own tokens, stored after the received rows
        for (int i = 0; i * kNT < n_local; ++i) {
            const int k = tstart[Eloc] + i;
            if (k < max_tiles) {
                tile_list[3 * k] = E;
                tile_list[3 * k + 1] = s_total + i * kNT;
                tile_list[3 * k + 2] = min(kNT, n_local - i * kNT);
            }
        }
    }
}

// scatter: one warp per token.  A token's activations go once to every GPU that owns at least one of its
// experts (into the slot of the first such expert, the "leader"); the other experts' slots on that GPU are
// mapped to the same row.  The leader slot also receives the list of its members and their routing weights,
// so that the owner can add up the token's expert outputs and send back one row.
__global__ void __launch_bounds__(256) ep_scatter_kernel(EpPeers peers, EpSym sym, int me, int P, int E, int K, int n,
                                                         const __nv_bfloat16* __restrict__ x,
                                                         const int32_t* __restrict__ topk_idx,
                                                         const float* __restrict__ topk_w,
                                                         const int32_t* __restrict__ base_send, int32_t* cursor,
                                                         const int32_t* __restrict__ total_recv, uint8_t* lead_mask,
                                                         unsigned int* done, unsigned int epoch) {
    const int t = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    const int Eloc = E / P;
    if (t < n) {
        int d = -1 - lane, slot = 0;  // lanes beyond K: destinations that match nobody
        float w = 0.0f;
        if (lane < K) {
            const int e = topk_idx[(size_t)t * K + lane];
            d = e / Eloc;
            slot = base_send[e] + atomicAdd(&cursor[e], 1);
            w = topk_w[(size_t)t * K + lane];
        }
        // leader = lowest k with the same destination; rank = position among that destination's experts
        int leader = lane, rank = 0, cnt = 0;
        for (int k2 = 0; k2 < K; ++k2) {
            const int d2 = __shfl_sync(0xffffffffu, d, k2);
            if (d2 == d) {
                if (k2 < leader) leader = k2;
                if (k2 < lane) ++rank;
                ++cnt;
            }
        }
        const int lslot = __shfl_sync(0xffffffffu, slot, leader);
        const bool is_leader = lane < K && leader == lane;
        if (lane < K) {
            uint8_t* pb = peers.base[d];
            reinterpret_cast<int32_t*>(pb + sym.xmap)[slot] = lslot;
            // return address: rank and (token * K + leader's k); member count for leaders, 0 otherwise
            reinterpret_cast<int4*>(pb + sym.meta)[slot] = make_int4(me, t * K + leader, is_leader ? cnt : 0, 0);
            reinterpret_cast<int32_t*>(pb + sym.memb)[(size_t)lslot * kMaxK + rank] = slot;
            reinterpret_cast<float*>(pb + sym.mwt)[(size_t)lslot * kMaxK + rank] = w;
        }
        const unsigned lmask = __ballot_sync(0xffffffffu, is_leader);
        if (lane == 0) lead_mask[t] = (uint8_t)lmask;
        // the row: read once, stored once per destination and once locally for the shared expert
        uint4 r[kBH * 2 / 16 / 32];
        const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)t * kBH);
#pragma unroll
        for (int i = 0; i < kBH * 2 / 16 / 32; ++i) r[i] = src[lane + 32 * i];
        for (unsigned m = lmask; m; m &= m - 1) {
            const int k = __ffs(m) - 1;
            const int dk = __shfl_sync(0xffffffffu, d, k), sk = __shfl_sync(0xffffffffu, slot, k);
            uint4* dst = reinterpret_cast<uint4*>(peers.base[dk] + sym.xrecv + (size_t)sk * kBH * 2);
#pragma unroll
            for (int i = 0; i < kBH * 2 / 16 / 32; ++i) dst[lane + 32 * i] = r[i];
        }
        const int ls = *total_recv + t;
        uint4* dst = reinterpret_cast<uint4*>(peers.base[me] + sym.xrecv + (size_t)ls * kBH * 2);
#pragma unroll
        for (int i = 0; i < kBH * 2 / 16 / 32; ++i) dst[lane + 32 * i] = r[i];
        if (lane == 0) reinterpret_cast<int32_t*>(peers.base[me] + sym.xmap)[ls] = ls;
    }
    // the last block to finish tells every peer that this rank's rows are in place
    if (ep_last_block(done) && threadIdx.x < 32) ep_signal_warp(peers, sym, me, P, epoch, threadIdx.x);
}

// return: one warp per received row; a leader row adds up the weighted outputs of its members (in the order
// of the sender's expert list) and sends the sum to the rank the token came from.
__global__ void __launch_bounds__(256) ep_return_kernel(EpPeers peers, EpSym sym, int me, int P,
                                                        const __nv_bfloat16* __restrict__ o,
                                                        const int32_t* __restrict__ total_recv, unsigned int* done,
                                                        unsigned int epoch) {
    const int lane = threadIdx.x & 31;
    const int total = *total_recv;
    const int4* meta = reinterpret_cast<const int4*>(peers.base[me] + sym.meta);
    const int32_t* memb = reinterpret_cast<const int32_t*>(peers.base[me] + sym.memb);
    const float* mwt = reinterpret_cast<const float*>(peers.base[me] + sym.mwt);
    constexpr int kPer = kBH * 2 / 16 / 32;  // 16-byte pieces of a row per lane
    for (int s = blockIdx.x * 8 + (threadIdx.x >> 5); s < total; s += gridDim.x * 8) {
        const int4 m = __ldcg(meta + s);
        if (m.z <= 0) continue;  // not a leader: its output travels inside its leader's sum
        float acc[kPer * 8];
#pragma unroll
        for (int i = 0; i < kPer * 8; ++i) acc[i] = 0.0f;
        for (int j = 0; j < m.z; ++j) {
            const int sj = __ldcg(memb + (size_t)s * kMaxK + j);
            const float wj = __ldcg(mwt + (size_t)s * kMaxK + j);
            const uint4* src = reinterpret_cast<const uint4*>(o + (size_t)sj * kBH);
#pragma unroll
            for (int i = 0; i < kPer; ++i) {
                const uint4 q = src[lane + 32 * i];
                const uint32_t rr[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    acc[i * 8 + 2 * c] = fmaf(wj, __uint_as_float(rr[c] << 16), acc[i * 8 + 2 * c]);
                    acc[i * 8 + 2 * c + 1] = fmaf(wj, __uint_as_float(rr[c] & 0xFFFF0000u), acc[i * 8 + 2 * c + 1]);
                }
            }
        }
        uint4* dst = reinterpret_cast<uint4*>(peers.base[m.x] + sym.oback + (size_t)m.y * kBH * 2);
#pragma unroll
        for (int i = 0; i < kPer; ++i) {
            uint32_t pk[4];
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const __nv_bfloat162 v = __floats2bfloat162_rn(acc[i * 8 + 2 * c], acc[i * 8 + 2 * c + 1]);
                pk[c] = *reinterpret_cast<const uint32_t*>(&v);
            }
            dst[lane + 32 * i] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
        }
    }
    if (ep_last_block(done) && threadIdx.x < 32) ep_signal_warp(peers, sym, me, P, epoch, threadIdx.x);
}

// combine: moe_combine_residual (reference src/math_util.rs:599-612); the routed experts' outputs arrive already
// weighted and summed per owning GPU (one row per leader, see the scatter kernel); routed rows come from the
// returned buffer in (token, k) order, the shared expert's row from this rank's own output.
__global__ void __launch_bounds__(256) ep_combine_kernel(const float* __restrict__ h_in, float* __restrict__ h_out,
                                                         int n, int K, const __nv_bfloat16* __restrict__ oback,
                                                         const __nv_bfloat16* __restrict__ o_local,
                                                         const int32_t* __restrict__ total_recv,
                                                         const uint8_t* __restrict__ lead_mask,
                                                         const float* __restrict__ sgate, const uint8_t* local,
                                                         size_t flags_off, int P, unsigned int epoch, unsigned int* err) {
    const int t = blockIdx.x, tid = threadIdx.x;
    // every peer's output rows must have arrived
    if (tid < 32) ep_wait_warp(local, flags_off, P, epoch, err, tid);
    __syncthreads();
    const float4* hp = reinterpret_cast<const float4*>(h_in + (size_t)t * kBH) + tid * 2;
    const float4 a = hp[0], b = hp[1];
    float moe[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, sh[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    auto add = [&](const __nv_bfloat16* row, float w, float (&dst)[8]) {
        const uint4 q = *(reinterpret_cast<const uint4*>(row) + tid);  // plain load: written by peers during this launch sequence
        const uint32_t r[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            dst[2 * i] += w * __uint_as_float(r[i] << 16);
            dst[2 * i + 1] += w * __uint_as_float(r[i] & 0xFFFF0000u);
        }
    };
    const unsigned lm = lead_mask[t];
    for (int k = 0; k < K; ++k)
        if (lm >> k & 1u) add(oback + ((size_t)t * K + k) * kBH, 1.0f, moe);
    add(o_local + (size_t)(*total_recv + t) * kBH, sgate[t], sh);
    const float hin[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    float4* op = reinterpret_cast<float4*>(h_out + (size_t)t * kBH) + tid * 2;
    op[0] = make_float4(hin[0] + moe[0] + sh[0], hin[1] + moe[1] + sh[1], hin[2] + moe[2] + sh[2], hin[3] + moe[3] + sh[3]);
    op[1] = make_float4(hin[4] + moe[4] + sh[4], hin[5] + moe[5] + sh[5], hin[6] + moe[6] + sh[6], hin[7] + moe[7] + sh[7]);
}

// ─── host side ──────────────────────────────────────────────────────────────

static size_t al256(size_t v) { return (v + 255) / 256 * 256; }

template <int MODE>
static constexpr size_t gemm_smem_bytes() {
    return (size_t)kAStages * (256 * 128) + (size_t)kBStages * (kNT * 128) + 1024;
}

// Tensor map of a row-major [rows][H] bf16 tensor read in boxes of box_rows x 64 columns with the
// 128-byte swizzle the MMA descriptors expect.  The encoder lives in the driver library; its entry
// point is looked up through the runtime so that nothing links against the driver directly.
typedef CUresult (*tmap_encode_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static int encode_rows_map(void* out128, const void* base, uint64_t rows, uint32_t box_rows) {
    static tmap_encode_fn fn = nullptr;
    if (!fn) {
        void* pfn = nullptr;
        cudaDriverEntryPointQueryResult q;
        MOE_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &pfn, cudaEnableDefault, &q));
        MOE_REQUIRE(pfn && q == cudaDriverEntryPointSuccess, "the driver does not provide cuTensorMapEncodeTiled");
        fn = reinterpret_cast<tmap_encode_fn>(pfn);
    }
    static_assert(sizeof(CUtensorMap) == 128, "tensor maps are stored in 128-byte fields");
    const cuuint64_t gdim[2] = {(cuuint64_t)kBH, (cuuint64_t)rows};
    const cuuint64_t gstride[1] = {(cuuint64_t)kBH * 2};
    const cuuint32_t box[2] = {64u, box_rows};
    const cuuint32_t estr[2] = {1u, 1u};
    const CUresult r = fn(reinterpret_cast<CUtensorMap*>(out128), CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), gdim,
                          gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    MOE_REQUIRE(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed with driver status %d", (int)r);
    return MOE_OK;
}

// Builds the router's bf16 planes of a layer on first batched use (and after the router is reloaded).
static int ensure_router_planes(moe_engine* e, int layer) {
    LayerHost& lh = e->layers[layer];
    if (lh.planes_valid) return MOE_OK;
    const int E = e->dims.num_experts, rows = (E + 127) / 128 * 128;
    if (!lh.planes) {
        MOE_CUDA(cudaMalloc(&lh.planes, (size_t)3 * rows * kBH * 2));
        int rcm = encode_rows_map(lh.planes_map, lh.planes, (uint64_t)3 * rows, 128);
        if (rcm) return rcm;
        e->resident += (size_t)3 * rows * kBH * 2;
    }
    int rc = refresh_layer_table(e);
    if (rc) return rc;
    router_planes_kernel<<<(rows * (kBH / 8) + 255) / 256, 256, 0, e->stream>>>(lh.dev, E, rows, (uint16_t*)lh.planes);
    MOE_CUDA(cudaGetLastError());
    e->launches++;
    lh.planes_valid = true;
    e->table_dirty = true;
    return refresh_layer_table(e);
}

int batch_reserve(moe_engine* e, int32_t n_tokens) {
    BatchWork& bw = e->bw;
    if (n_tokens <= bw.capacity) return MOE_OK;
    MOE_CUDA(cudaStreamSynchronize(e->stream));
    batch_destroy(e);
    const moe_dims_t& d = e->dims;
    const size_t n = (size_t)n_tokens, H = d.hidden, I = d.inter, E = d.num_experts, K = d.top_k;
    const size_t slots = n * K + n;
    const int max_tiles = (int)(slots / kNT + E + 2);
    size_t off = 0;
    auto take = [&](size_t bytes) { size_t o = off; off += al256(bytes); return o; };
    const size_t o_ha = take(n * H * 4), o_hb = take(n * H * 4), o_x = take(n * H * 2), o_xm = take(n * H * 2), o_xl = take(n * H * 2);
    // the router GEMM leaves router_split(n') slabs of n' x E partial sums for any n' up to the capacity
    size_t lg_rows = n;
    for (int np = 1; np <= n_tokens; ++np) {
        const int s = router_split(np, (int)E, 1) > router_split(np, (int)E, 3) ? router_split(np, (int)E, 1) : router_split(np, (int)E, 3);
        if ((size_t)s * np > lg_rows) lg_rows = (size_t)s * np;
        if (s == 1) break;  // the split only shrinks as the token count grows
    }
    const size_t o_lg = take(lg_rows * E * 4);
    const size_t o_ti = take(n * K * 4), o_tw = take(n * K * 4), o_sg = take(n * 4);
    const size_t o_cnt = take((E + 1) * 4), o_off = take((E + 2) * 4), o_cur = take((E + 1) * 4);
    const size_t o_st = take(slots * 4), o_so = take(n * K * 4), o_act = take(slots * I * 2), o_o = take(slots * H * 2);
    const size_t o_tl = take((size_t)max_tiles * 3 * 4), o_nt = take(4);
    // the slot-wise expert FFN of small batches: the expert of every slot, f32 SwiGLU outputs of up to kSlotPathMaxTokens tokens
    const size_t small_n = n < (size_t)kSlotPathMaxTokens ? n : (size_t)kSlotPathMaxTokens;
    const size_t o_se = take(slots * 4), o_a32 = take((small_n * K + small_n) * I * 4);
    MOE_CUDA(cudaMalloc(&bw.base, off));
    uint8_t* b = bw.base;
    bw.h_a = (float*)(b + o_ha); bw.h_b = (float*)(b + o_hb);
    bw.x = (__nv_bfloat16*)(b + o_x); bw.x_mid = (__nv_bfloat16*)(b + o_xm); bw.x_lo = (__nv_bfloat16*)(b + o_xl);
    bw.logits = (float*)(b + o_lg); bw.topk_idx = (int32_t*)(b + o_ti); bw.topk_w = (float*)(b + o_tw);
    bw.sgate = (float*)(b + o_sg);
    bw.counts = (int32_t*)(b + o_cnt); bw.offsets = (int32_t*)(b + o_off); bw.cursor = (int32_t*)(b + o_cur);
    bw.slot_token = (int32_t*)(b + o_st); bw.slot_of = (int32_t*)(b + o_so);
    bw.act = (__nv_bfloat16*)(b + o_act); bw.o = (__nv_bfloat16*)(b + o_o);
    bw.tile_list = (int32_t*)(b + o_tl); bw.n_tiles = (int32_t*)(b + o_nt);
    bw.slot_expert = (int32_t*)(b + o_se); bw.act32 = (float*)(b + o_a32);
    bw.max_tiles = max_tiles;
    bw.capacity = n_tokens;
    bw.logit_rows = (int64_t)lg_rows;
    {
        int rcm = encode_rows_map(bw.x_map, bw.x, (uint64_t)3 * n, kRtTok);
        if (rcm) return rcm;
    }
    MOE_CUDA(cudaFuncSetAttribute(grouped_gemm_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)gemm_smem_bytes<1>()));
    MOE_CUDA(cudaFuncSetAttribute(grouped_gemm_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)gemm_smem_bytes<2>()));
    MOE_CUDA(cudaFuncSetAttribute(router_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kRtSmem));
    return MOE_OK;
}

void batch_destroy(moe_engine* e) {
    BatchWork& bw = e->bw;
    if (bw.base) cudaFree(bw.base);
    bw = BatchWork{};
}

int launch_batched_layer(moe_engine* e, int layer, const float* h_in, int32_t n, float* h_out,
                         const float* logit_bias, const int32_t* forced_idx, int32_t* out_idx, float* out_w) {
    const moe_dims_t& d = e->dims;
    MOE_REQUIRE(d.hidden == kBH && d.inter == kBI && d.shared_inter == kBI,
                "batched path is built for hidden=%d, inter=shared_inter=%d (got %d/%d/%d)", kBH, kBI, d.hidden,
                d.inter, d.shared_inter);
    MOE_REQUIRE(d.num_experts <= 32 * kMaxEPerLane, "batched path supports at most %d experts", 32 * kMaxEPerLane);
    MOE_REQUIRE((((uintptr_t)h_in) & 15) == 0 && (((uintptr_t)h_out) & 15) == 0, "batched: h must be 16-byte aligned");
    int rc = check_layer_ready(e, layer);
    if (rc) return rc;
    rc = refresh_layer_table(e);
    if (rc) return rc;
    rc = batch_reserve(e, n);
    if (rc) return rc;
    rc = ensure_router_planes(e, layer);
    if (rc) return rc;
    BatchWork& bw = e->bw;
    const LayerDev ly = e->layers[layer].dev;
    const int E = d.num_experts, K = d.top_k;
    cudaStream_t st = e->stream;
    int32_t* idx = out_idx ? out_idx : bw.topk_idx;
    float* wts = out_w ? out_w : bw.topk_w;

    batch_prep_kernel<<<n, 256, 0, st>>>(h_in, n, ly, bw.x, bw.x_mid, bw.x_lo, bw.sgate, bw.counts, E + 1);
    const int rsplit = router_split(n, E, ly.router_nplanes);
    MOE_REQUIRE((int64_t)rsplit * n <= bw.logit_rows, "router partial sums (%d x %d rows) exceed the logits work area (%lld rows)",
                rsplit, n, (long long)bw.logit_rows);
    router_gemm_kernel<<<dim3((n + kRtTok - 1) / kRtTok, ly.router_nplanes == 1 ? (E + 255) / 256 : (E + 127) / 128, rsplit), 256, kRtSmem, st>>>(
        *reinterpret_cast<const CUtensorMap*>(e->layers[layer].planes_map), *reinterpret_cast<const CUtensorMap*>(bw.x_map), n, E,
        ly.router_nplanes, (E + 127) / 128 * 128, bw.capacity, bw.logits, e->dec_sync + 2);
    if (E <= 256) batch_route_kernel<8><<<(n + 7) / 8, 256, 0, st>>>(bw.logits, n, E, K, logit_bias, forced_idx, idx, wts, bw.counts, rsplit, EpPush{}, e->dec_sync + 2);
    else batch_route_kernel<16><<<(n + 7) / 8, 256, 0, st>>>(bw.logits, n, E, K, logit_bias, forced_idx, idx, wts, bw.counts, rsplit, EpPush{}, e->dec_sync + 2);
    batch_plan_kernel<<<1, 1024, 0, st>>>(bw.counts, bw.offsets, bw.cursor, E, n, bw.tile_list, bw.n_tiles, bw.max_tiles);
    // Few tokens per expert: the slot-wise matvec form of the expert FFN (slots_ffn.cu); otherwise the grouped GEMMs.
    static const int slot_max = [] { const char* v = getenv("MOE_B200_SLOT_FFN_MAX"); return v ? atoi(v) : kSlotPathDefault; }();
    const bool by_slot = n <= slot_max && n <= kSlotPathMaxTokens;
    batch_scatter_kernel<<<(n * K + 255) / 256, 256, 0, st>>>(idx, n, K, E, bw.offsets, bw.cursor, bw.slot_token, bw.slot_of,
                                                               by_slot ? bw.slot_expert : nullptr);
    if (by_slot) {
        rc = launch_slot_ffn(e, ly, h_in, n * K + n, bw.slot_token, bw.slot_expert, bw.act32, bw.o);
        if (rc) return rc;
        e->launches -= 2;  // counted with the layer's eight below
    } else {
    GemmParams gp{};
    gp.experts = ly.experts; gp.shared = ly.shared; gp.lay = e->lay; gp.E = E;
    gp.x = bw.x; gp.act = bw.act; gp.o = bw.o;
    gp.tile_list = bw.tile_list; gp.n_tiles = bw.n_tiles; gp.slot_token = bw.slot_token;
    gp.err = e->dec_sync + 2;
    grouped_gemm_kernel<1><<<e->sm_count, kGemmThreads, gemm_smem_bytes<1>(), st>>>(gp);
    grouped_gemm_kernel<2><<<e->sm_count, kGemmThreads, gemm_smem_bytes<2>(), st>>>(gp);
    }
    batch_combine_kernel<<<n, 256, 0, st>>>(h_in, h_out, n, K, E, bw.o, bw.slot_of, wts, bw.sgate, bw.offsets);
    e->launches += 8;
    MOE_CUDA(cudaGetLastError());
    return MOE_OK;
}


// Private work areas of the expert-parallel path (sized at moe_ep_export time).
int ep_alloc_work(moe_engine* e) {
    EpState& ep = e->ep;
    const moe_dims_t& d = e->dims;
    const size_t rows = (size_t)ep.slots_cap + ep.cap;
    ep.max_tiles = (int)(rows / kNT + d.num_experts + 2);
    size_t off = 0;
    auto take = [&](size_t bytes) { size_t o = off; off += al256(bytes); return o; };
    const size_t o_act = take(rows * d.inter * 2), o_o = take(rows * d.hidden * 2), o_tl = take((size_t)ep.max_tiles * 12);
    const size_t o_nt = take(4), o_bs = take((size_t)d.num_experts * 4), o_cu = take((size_t)d.num_experts * 4);
    const size_t o_tr = take(4), o_dn = take(4), o_lm = take((size_t)ep.cap);
    MOE_CUDA(cudaMalloc(&ep.work, off));
    ep.done = (unsigned int*)(ep.work + o_dn);
    ep.lead_mask = ep.work + o_lm;
    MOE_CUDA(cudaMemsetAsync(ep.done, 0, 4, e->stream));
    ep.act = (__nv_bfloat16*)(ep.work + o_act); ep.o = (__nv_bfloat16*)(ep.work + o_o);
    ep.tile_list = (int32_t*)(ep.work + o_tl); ep.n_tiles = (int32_t*)(ep.work + o_nt);
    ep.base_send = (int32_t*)(ep.work + o_bs); ep.cursor = (int32_t*)(ep.work + o_cu);
    ep.total_recv = (int32_t*)(ep.work + o_tr);
    return batch_reserve(e, ep.cap);
}

// One MoE block, expert-parallel; every rank of the group must call it for the same layer.
int ep_layer(moe_engine* e, int layer, const float* h_in, int32_t n, float* h_out) {
    EpState& ep = e->ep;
    const moe_dims_t& d = e->dims;
    MOE_REQUIRE(ep.ready, "expert parallelism is not initialised (moe_ep_export + moe_ep_init)");
    MOE_REQUIRE(n >= 1 && n <= ep.cap, "token count %d outside 1..%d (max_tokens_per_rank)", n, ep.cap);
    MOE_REQUIRE((((uintptr_t)h_in) & 15) == 0 && (((uintptr_t)h_out) & 15) == 0, "h must be 16-byte aligned");
    int rc = check_layer_ready(e, layer);
    if (rc) return rc;
    rc = refresh_layer_table(e);
    if (rc) return rc;
    rc = ensure_router_planes(e, layer);
    if (rc) return rc;
    BatchWork& bw = e->bw;
    const LayerDev ly = e->layers[layer].dev;
    const int E = d.num_experts, K = d.top_k, P = ep.world, me = ep.rank;
    cudaStream_t st = e->stream;
    unsigned int* err = e->dec_sync + 2;
    EpPeers peers{};
    for (int i = 0; i < P; ++i) peers.base[i] = ep.peer[i];
    const int32_t* counts_all = reinterpret_cast<const int32_t*>(ep.local + ep.sym.counts);

    batch_prep_kernel<<<n, 256, 0, st>>>(h_in, n, ly, bw.x, bw.x_mid, bw.x_lo, bw.sgate, bw.counts, E + 1);
    const int rsplit = router_split(n, E, ly.router_nplanes);
    MOE_REQUIRE((int64_t)rsplit * n <= bw.logit_rows, "router partial sums (%d x %d rows) exceed the logits work area (%lld rows)",
                rsplit, n, (long long)bw.logit_rows);
    router_gemm_kernel<<<dim3((n + kRtTok - 1) / kRtTok, ly.router_nplanes == 1 ? (E + 255) / 256 : (E + 127) / 128, rsplit), 256, kRtSmem, st>>>(
        *reinterpret_cast<const CUtensorMap*>(e->layers[layer].planes_map), *reinterpret_cast<const CUtensorMap*>(bw.x_map), n, E,
        ly.router_nplanes, (E + 127) / 128 * 128, bw.capacity, bw.logits, err);
    // 1. histogram exchange: the last block of the route kernel pushes it and publishes the epoch; the plan waits for everybody's
    EpPush push{};
    push.peers = peers; push.counts_off = ep.sym.counts; push.flags_off = ep.sym.flags;
    push.me = me; push.world = P; push.epoch = ++ep.epoch; push.done = ep.done;
    if (E <= 256) batch_route_kernel<8><<<(n + 7) / 8, 256, 0, st>>>(bw.logits, n, E, K, nullptr, nullptr, bw.topk_idx, bw.topk_w, bw.counts, rsplit, push, err);
    else batch_route_kernel<16><<<(n + 7) / 8, 256, 0, st>>>(bw.logits, n, E, K, nullptr, nullptr, bw.topk_idx, bw.topk_w, bw.counts, rsplit, push, err);
    ep_plan_kernel<<<1, 1024, 0, st>>>(counts_all, me, P, E, n, ep.base_send, ep.cursor, ep.tile_list, ep.n_tiles,
                                       ep.max_tiles, ep.total_recv, ep.local, ep.sym.flags, ep.epoch, err);
    // 2. dispatch (the last block of the scatter publishes the epoch)
    ep_scatter_kernel<<<(n + 7) / 8, 256, 0, st>>>(peers, ep.sym, me, P, E, K, n, bw.x, bw.topk_idx, bw.topk_w, ep.base_send,
                                                  ep.cursor, ep.total_recv, ep.lead_mask, ep.done, ++ep.epoch);
    // 3. grouped GEMMs over the received rows (+ shared expert over the local ones); the first one waits for the rows
    GemmParams gp{};
    gp.experts = ly.experts; gp.shared = ly.shared; gp.lay = e->lay; gp.E = E;
    gp.x = reinterpret_cast<const __nv_bfloat16*>(ep.local + ep.sym.xrecv);
    gp.act = ep.act; gp.o = ep.o;
    gp.tile_list = ep.tile_list; gp.n_tiles = ep.n_tiles; gp.slot_token = reinterpret_cast<const int32_t*>(ep.local + ep.sym.xmap);
    gp.err = err;
    gp.ep_local = ep.local; gp.ep_flags = ep.sym.flags; gp.ep_world = P; gp.ep_epoch = ep.epoch;
    grouped_gemm_kernel<1><<<e->sm_count, kGemmThreads, gemm_smem_bytes<1>(), st>>>(gp);
    gp.ep_world = 0;
    grouped_gemm_kernel<2><<<e->sm_count, kGemmThreads, gemm_smem_bytes<2>(), st>>>(gp);
    // 4. return (the last block publishes the epoch), 5. combine (waits for everybody's rows)
    ep_return_kernel<<<e->sm_count * 2, 256, 0, st>>>(peers, ep.sym, me, P, ep.o, ep.total_recv, ep.done, ++ep.epoch);
    ep_combine_kernel<<<n, 256, 0, st>>>(h_in, h_out, n, K, reinterpret_cast<const __nv_bfloat16*>(ep.local + ep.sym.oback),
                                         ep.o, ep.total_recv, ep.lead_mask, bw.sgate, ep.local, ep.sym.flags, P, ep.epoch, err);
    e->launches += 9;
    MOE_CUDA(cudaGetLastError());
    return MOE_OK;
}

}  // namespace moe
