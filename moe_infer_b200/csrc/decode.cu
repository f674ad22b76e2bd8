// Batch-1 decode of the MoE stack: one persistent cooperative kernel walks the
// layers; every CTA owns a fixed, contiguous slice of each weight matrix and
// pulls it from the resident HBM store into shared memory with bulk (TMA)
// copies issued as early as the data dependencies allow; nibbles are
// dequantised in registers and reduced with warp shuffles.
//
// Replaces, per layer, the tail of op1 (post-attention norm, router matvec,
// shared-expert gate/up, shared_expert_gate), the CPU route_experts round trip and
// op2 (8 x gate/up/SwiGLU/down, shared down, moe_combine_residual) of the
// reference's decode engines (src/engine/qwen35_moe/fused_exp1.rs:149-365,
// 734-856; CPU statement src/engine/qwen35_moe/cpu.rs:187-205, 78-85, 398-483).
// Where the reference commits 41 command buffers per token with a blocking
// GPU->CPU wait each, this is one launch for the whole stack; top-k runs on
// the device.
//
// Two kernels live here.  decode_stack_kernel is the three-phase form (serves the
// allocation-free single-block entry point):
//
//   phase A  x = rmsnorm(h) (every CTA, redundantly); router logits, shared
//            expert gate/up + SwiGLU, shared gate score            [~2.2 MB]
//   phase B  softmax + top-k (every CTA, redundantly); gate/up/SwiGLU of the K
//            chosen experts                                         [~9.4 MB]
//   phase C  down projections of the K experts and the shared expert, combine
//            with the residual: one warp owns one output element    [~5.3 MB]
//
// with a counting grid barrier after each phase.  decode_fused_kernel (further down,
// used by the engine) folds phase A into the neighbouring phases and needs two
// grid-wide exchanges per layer, one of them without a barrier.
//
// HBM-bound: 16,974,976 weight bytes per layer-token at the reference sizes.
// Every wait (grid barrier, mbarrier, tag poll) is bounded and a timeout raises an
// error word instead of hanging.
#include "decode_common.cuh"
#include <mutex>

namespace moe {

constexpr int kProfPoints = 12;

// Per-CTA slice capacities; the host checks that the grid is large enough.
constexpr int kMaxRouterRows = 4;   // ceil(E / grid)
constexpr int kMaxSharedRows = 4;   // ceil(I / grid) gate/up row pairs of the shared expert
constexpr int kMaxBItems = 28;      // ceil(K * I / grid) gate/up row pairs of routed experts
constexpr int kMaxCRows = 14;       // ceil(H / grid) output elements

#define PROF(idx)                                                                                  \
    do {                                                                                           \
        if (p.prof && cta == 0 && tid == 0) p.prof[(l - p.l0) * kProfPoints + (idx)] = clock64();  \
    } while (0)

struct DecodeParams {
    const LayerDev* layers;  // table in device memory, or nullptr: then `one` is the only layer
    LayerDev one;
    int l0, l1;
    const float* h_in;
    float* h_out;
    float* h_buf0;
    float* h_buf1;
    float* logits;      // [E]
    float* act;         // [(K + 1) * I]
    float* misc;        // [0] shared gate score
    const float* logit_bias;
    const int32_t* forced_idx;
    int32_t* out_idx;
    float* out_w;
    unsigned int* sync; // [0] arrivals, [1] exits, [2] error word
    long long* prof;    // nullable: [layer][kProfPoints] SM-clock stamps taken by CTA 0
    int E, K;
    moe_expert_layout_t lay;
};

struct __align__(128) DecodeSmem {
    // prefetched weight slices (destinations of bulk copies: 16-byte aligned offsets)
    uint4 a_router[kMaxRouterRows * (kH * 2 / 16)];      // bf16 rows (4096 B each) or 4-bit rows (1024 B each)
    uint4 a_shw[2][kMaxSharedRows][kChH];                // shared expert gate / up rows
    uint4 a_sgw[kChH];                                   // shared_expert_gate row
    uint4 b_w[2][kMaxBItems][kChH];                      // routed gate / up rows
    uint4 c_w[kMaxK + 1][kMaxCRows][kChI];               // down rows of the K experts + shared expert
    uint16_t a_router_s[kMaxRouterRows][kH / kGroup];
    uint16_t a_router_b[kMaxRouterRows][kH / kGroup];
    uint16_t a_shs[2][kMaxSharedRows][kH / kGroup];
    uint16_t a_shb[2][kMaxSharedRows][kH / kGroup];
    uint16_t a_sgs[kH / kGroup];
    uint16_t a_sgb[kH / kGroup];
    uint16_t b_s[2][kMaxBItems][kH / kGroup];
    uint16_t b_b[2][kMaxBItems][kH / kGroup];
    uint16_t c_s[kMaxK + 1][kMaxCRows][kI / kGroup];
    uint16_t c_b[kMaxK + 1][kMaxCRows][kI / kGroup];
    // activations
    float raw[kH];              // bulk-copy landing zone for h
    float xn[kH];               // normalised x, plain order (bf16 router rows)
    float4 xs[8 * kChH];        // normalised x, chunk-transposed
    float sumx[kChH];
    float4 acts[(kMaxK + 1) * 8 * kChI];  // SwiGLU outputs, chunk-transposed per expert
    float suma[(kMaxK + 1) * kChI];
    float prob[kMaxE];
    float red[kDecWarps];
    float red2[kDecWarps];
    float inv_rms;
    float cand_p[kMaxE];
    int cand_i[kMaxE];
    int ncand;
    float topw[kMaxK + 1];      // combine weights; [K] = sigmoid(shared gate)
    float topp[kMaxK];
    int topi[kMaxK];
    int flag;
    uint64_t bar_h;
};
static_assert(sizeof(DecodeSmem) <= 227 * 1024, "decode staging exceeds shared memory");
static_assert((sizeof(uint16_t) * (kMaxK + 1) * kMaxCRows * (kI / kGroup)) % 16 == 0, "bulk-copy destinations stay aligned");

__device__ __forceinline__ int slice_lo(int c, int n, int G) { return (int)(((long long)c * n) / G); }

// ─── grid barrier with a bounded wait ───────────────────────────────────────
// Arrivals are counted on one monotonically increasing word; `target` is the
// count that completes this barrier.  Returns false (for the whole CTA) when
// the wait gave up or another CTA already raised the error word.
template <class SM>
__device__ __forceinline__ bool grid_barrier(unsigned int* sync, unsigned int target, SM* sm) {
    // h is written with generic stores and read back by bulk (async-proxy) copies
    asm volatile("fence.proxy.async;" ::: "memory");
    __syncthreads();
    if (threadIdx.x == 0) {
        // release: publishes this CTA's writes (ordered before it by the bar.sync above)
        asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(sync), "r"(1u) : "memory");
        int ok = 0;
        const long long t0 = clock64();
        for (uint32_t i = 0;; ++i) {
            unsigned int v;
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(sync) : "memory");
            if (v >= target) { ok = 1; break; }
            if ((i & 63u) == 63u) {
                unsigned int err;
                asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(err) : "l"(sync + 2) : "memory");
                if (err || clock64() - t0 > kWaitCycles) break;
            }
        }
        if (!ok) atomicExch(&sync[2], 2u);
        sm->flag = ok;
        asm volatile("fence.proxy.async;" ::: "memory");
    }
    __syncthreads();
    return sm->flag != 0;
}

// phase A slice: router rows [e0, e0+ne), shared gate/up pairs [p0, p0+np), shared gate (last CTA)
__device__ __forceinline__ void prefetch_A(DecodeSmem* sm, const LayerDev& ly, const moe_expert_layout_t& S,
                                           int cta, int G, int E, int tid) {
    const int e0 = slice_lo(cta, E, G), ne = slice_lo(cta + 1, E, G) - e0;
    const int p0 = slice_lo(cta, kI, G), np = slice_lo(cta + 1, kI, G) - p0;
    constexpr int kRowW = kH / 2, kRowS = (kH / kGroup) * 2;  // bytes of one 4-bit row / of its scales
    if (ly.router_bf16) {
        copy_flat(sm->a_router, ly.router_bf16 + (size_t)e0 * kH, ne * (kH * 2 / 16), tid);
    } else {
        copy_flat(sm->a_router, ly.router_q4.w + (size_t)e0 * (kH / 8), ne * (kRowW / 16), tid);
        copy_flat(sm->a_router_s, ly.router_q4.s + (size_t)e0 * (kH / kGroup), ne * (kRowS / 16), tid);
        copy_flat(sm->a_router_b, ly.router_q4.b + (size_t)e0 * (kH / kGroup), ne * (kRowS / 16), tid);
    }
    const uint8_t* sh = ly.shared;
    copy_flat(sm->a_shw[0], sh + S.gate_w + (size_t)p0 * kRowW, np * (kRowW / 16), tid);
    copy_flat(sm->a_shw[1], sh + S.up_w + (size_t)p0 * kRowW, np * (kRowW / 16), tid);
    // the four small arrays: one piece per thread at most
    {
        const int per = np * (kRowS / 16);
        if (tid < 4 * per) {
            const int a = tid / per, q = tid - a * per;
            const int64_t off = a == 0 ? S.gate_s : a == 1 ? S.up_s : a == 2 ? S.gate_b : S.up_b;
            uint16_t* d = a == 0 ? sm->a_shs[0][0] : a == 1 ? sm->a_shs[1][0] : a == 2 ? sm->a_shb[0][0] : sm->a_shb[1][0];
            cp16(reinterpret_cast<uint8_t*>(d) + q * 16, sh + off + (size_t)p0 * kRowS + q * 16);
        }
    }
    if (cta == G - 1) {
        copy_flat(sm->a_sgw, ly.sgate.w, kRowW / 16, tid);
        if (tid < kRowS / 16) cp16(reinterpret_cast<uint8_t*>(sm->a_sgs) + tid * 16, reinterpret_cast<const uint8_t*>(ly.sgate.s) + tid * 16);
        else if (tid < 2 * (kRowS / 16))
            cp16(reinterpret_cast<uint8_t*>(sm->a_sgb) + (tid - kRowS / 16) * 16,
                 reinterpret_cast<const uint8_t*>(ly.sgate.b) + (tid - kRowS / 16) * 16);
    }
    cp_commit();
}

// phase B: a warp copies the items it will compute itself, j = warp and warp + 16
// of this CTA's [i0, i0 + nb) (item = slot k * I + row r: gate row r and up row r of
// the k-th chosen expert).  Warp-private, so only a __syncwarp is needed before use
// and warps start computing as soon as their own bytes land.
template <class SM>
__device__ __forceinline__ void prefetch_B_warp(SM* sm, const LayerDev& ly, const moe_expert_layout_t& L,
                                                int i0, int nb, int warp, int lane) {
    constexpr int kPW = kH / 2 / 16;  // 64 pieces per weight row; scales/biases: 4 pieces per row
#pragma unroll
    for (int t = 0; t < 2; ++t) {
        const int j = warp + t * kDecWarps;
        if (j < nb) {
            const int i = i0 + j, k = i / kI, r = i - k * kI;
            const uint8_t* ex = ly.experts + (size_t)sm->topi[k] * L.expert_size;
            const uint8_t* gw = ex + L.gate_w + (size_t)r * (kH / 2);
            const uint8_t* uw = ex + L.up_w + (size_t)r * (kH / 2);
            cp16(&sm->b_w[0][j][lane], gw + lane * 16);
            cp16(&sm->b_w[0][j][lane + 32], gw + (lane + 32) * 16);
            cp16(&sm->b_w[1][j][lane], uw + lane * 16);
            cp16(&sm->b_w[1][j][lane + 32], uw + (lane + 32) * 16);
            if (lane < 16) {
                const int a = lane >> 2, c = lane & 3;
                const int64_t off = a == 0 ? L.gate_s : a == 1 ? L.up_s : a == 2 ? L.gate_b : L.up_b;
                uint16_t* d = a == 0 ? sm->b_s[0][j] : a == 1 ? sm->b_s[1][j] : a == 2 ? sm->b_b[0][j] : sm->b_b[1][j];
                cp16(reinterpret_cast<uint8_t*>(d) + c * 16, ex + off + (size_t)r * (kH / kGroup) * 2 + c * 16);
            }
        }
    }
    static_assert(kPW == 64, "two pieces per lane per row");
    cp_commit();
}

// phase C: a warp copies the down rows of the output element it owns (row r0 + warp)
// for the K chosen experts and the shared expert.
template <class SM>
__device__ __forceinline__ void prefetch_C_warp(SM* sm, const LayerDev& ly, const moe_expert_layout_t& L,
                                                int r0, int nc, int K, int warp, int lane) {
    for (int j = warp; j < nc; j += kDecWarps) {
        const int pw = (K + 1) * kChI;  // 16 pieces per row
        for (int q = lane; q < pw; q += 32) {
            const int m = q / kChI, c = q - m * kChI;
            const uint8_t* ex = (m < K) ? ly.experts + (size_t)sm->topi[m] * L.expert_size : ly.shared;
            cp16(&sm->c_w[m][j][c], ex + L.down_w + (size_t)(r0 + j) * (kI / 2) + c * 16);
        }
        if (lane < 2 * (K + 1)) {
            const int m = lane >> 1, a = lane & 1;
            const uint8_t* ex = (m < K) ? ly.experts + (size_t)sm->topi[m] * L.expert_size : ly.shared;
            cp16(a ? sm->c_b[m][j] : sm->c_s[m][j], ex + (a ? L.down_b : L.down_s) + (size_t)(r0 + j) * (kI / kGroup) * 2);
        }
    }
    cp_commit();
}

// ─── x = rmsnorm(h) * w, staged three ways (plain, chunk-transposed, chunk sums) ──
// rms_norm_bf16 (reference src/math_util.rs:282-288), eps 1e-6.
template <class SM>
__device__ __forceinline__ bool stage_norm(SM* sm, const float* h, const uint16_t* norm_w,
                                           uint32_t parity) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) {
        mbar_expect_tx(&sm->bar_h, kH * 4u);
        bulk_g2s(sm->raw, h, kH * 4u, &sm->bar_h);
    }
    const uint2 wb = __ldg(reinterpret_cast<const uint2*>(norm_w) + tid);  // 4 bf16, in flight during the wait
    if (!__syncthreads_and(mbar_wait(&sm->bar_h, parity) ? 1 : 0)) return false;
    static_assert(kH == kDecThreads * 4, "one float4 per thread");
    const float4 v = reinterpret_cast<const float4*>(sm->raw)[tid];
    float ss = warp_sum(v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w);
    if (lane == 0) sm->red[warp] = ss;
    __syncthreads();
    float tot = 0.0f;
#pragma unroll
    for (int i = 0; i < kDecWarps; ++i) tot += sm->red[i];
    const float inv_rms = 1.0f / sqrtf(tot / (float)kH + 1e-6f);
    if (tid == 0) sm->inv_rms = inv_rms;
    float4 o;
    o.x = v.x * inv_rms * __uint_as_float(wb.x << 16);
    o.y = v.y * inv_rms * __uint_as_float(wb.x & 0xFFFF0000u);
    o.z = v.z * inv_rms * __uint_as_float(wb.y << 16);
    o.w = v.w * inv_rms * __uint_as_float(wb.y & 0xFFFF0000u);
    reinterpret_cast<float4*>(sm->xn)[tid] = o;
    const int c = tid >> 3, j = tid & 7;   // float4 j of chunk c
    sm->xs[j * kChH + c] = o;
    float s = (o.x + o.y) + (o.z + o.w);
    s += __shfl_xor_sync(0xffffffffu, s, 1);
    s += __shfl_xor_sync(0xffffffffu, s, 2);
    s += __shfl_xor_sync(0xffffffffu, s, 4);
    if (j == 0) sm->sumx[c] = s;
    __syncthreads();
    return true;
}

// Dot products of NR 4-bit rows of length kH (staged in shared memory) with the staged x.
template <int NR, class SM>
__device__ __forceinline__ void rows_dot_h(const SM* sm, const uint4* const (&w)[NR],
                                           const uint16_t* const (&s)[NR], const uint16_t* const (&b)[NR],
                                           float (&out)[NR], int lane) {
#pragma unroll
    for (int r = 0; r < NR; ++r) out[r] = 0.0f;
#pragma unroll
    for (int it = 0; it < 2; ++it) {
        const int c = lane + 32 * it;
        float4 xv[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) xv[j] = sm->xs[j * kChH + c];
        const float sx = sm->sumx[c];
#pragma unroll
        for (int r = 0; r < NR; ++r) out[r] += chunk_term(w[r][c], xv, sx, s[r][c >> 1], b[r][c >> 1]);
    }
#pragma unroll
    for (int r = 0; r < NR; ++r) out[r] = warp_sum(out[r]);
}

// One bf16 row of length kH (BQ4-scheme router; reference matvec_bf16,
// src/engine/shaders.metal:2392), the row staged in shared memory.
__device__ __forceinline__ float row_dot_bf16(const DecodeSmem* sm, const uint4* wrow, int lane) {
    float acc = 0.0f;
#pragma unroll
    for (int it = 0; it < kH / 256; ++it) {
        const uint4 q = wrow[lane + 32 * it];
        const int base = (lane + 32 * it) * 8;
        const float4 x0 = *reinterpret_cast<const float4*>(sm->xn + base);
        const float4 x1 = *reinterpret_cast<const float4*>(sm->xn + base + 4);
        acc = fmaf(__uint_as_float(q.x << 16), x0.x, acc);
        acc = fmaf(__uint_as_float(q.x & 0xFFFF0000u), x0.y, acc);
        acc = fmaf(__uint_as_float(q.y << 16), x0.z, acc);
        acc = fmaf(__uint_as_float(q.y & 0xFFFF0000u), x0.w, acc);
        acc = fmaf(__uint_as_float(q.z << 16), x1.x, acc);
        acc = fmaf(__uint_as_float(q.z & 0xFFFF0000u), x1.y, acc);
        acc = fmaf(__uint_as_float(q.w << 16), x1.z, acc);
        acc = fmaf(__uint_as_float(q.w & 0xFFFF0000u), x1.w, acc);
    }
    return warp_sum(acc);
}

// ─── softmax + top-k + renormalise, whole CTA ───────────────────────────────
// route_experts (reference src/engine/qwen35_moe/cpu.rs:78-85): softmax over all
// E logits (src/math_util.rs:77-88), the K largest probabilities (ties: lower
// index first, matching the strict `>` of src/math_util.rs:101), divided by their
// sum (:120-126).  Thread t owns expert t.  The K-th largest of the 16 per-warp
// maxima is a lower bound of the K-th largest probability, so only experts at
// or above it are candidates; each candidate finds its rank by counting the
// candidates that beat it.  Results come out in descending order.
template <class SM>
__device__ __forceinline__ void route_cta(SM* sm, float v, const int32_t* forced, int E, int K, unsigned int* err) {
    // v: this thread's router logit (thread t owns expert t; -INFINITY for t >= E)
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    float mx = v;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if (lane == 0) sm->red[warp] = mx;
    if (tid == 0) sm->ncand = 0;
    __syncthreads();
    const float wmx = mx;  // this warp's max logit
    mx = sm->red[0];
#pragma unroll
    for (int i = 1; i < kDecWarps; ++i) mx = fmaxf(mx, sm->red[i]);
    const float ex = (tid < E) ? expf(v - mx) : 0.0f;
    const float ws = warp_sum(ex);
    __syncthreads();
    if (lane == 0) { sm->red[warp] = ws; sm->red2[warp] = (warp * 32 < E) ? expf(wmx - mx) : -1.0f; }
    __syncthreads();
    float sum = 0.0f;
#pragma unroll
    for (int i = 0; i < kDecWarps; ++i) sum += sm->red[i];
    const float inv = 1.0f / sum;
    const float pr = ex * inv;
    static_assert(kMaxE == kDecThreads, "one thread per expert slot");
    sm->prob[tid] = (tid < E) ? pr : -1.0f;
    // default choice (experts 0..K-1): stands only when NaN logits leave fewer than K candidates, as the
    // reference's heap keeps its first K entries then (src/math_util.rs:89-99); never an undefined index
    if (tid < K) { sm->topi[tid] = tid; sm->topp[tid] = pr; }
    if (forced) {
        __syncthreads();
        if (tid < K) {
            int fe = forced[tid];
            if ((unsigned)fe >= (unsigned)E) { atomicExch(err, 10u); fe = 0; }  // reported, never dereferenced
            sm->topi[tid] = fe;
            sm->topp[tid] = sm->prob[fe];
        }
    } else {
        // threshold = K-th largest warp maximum (as a probability); -1 when fewer than K warps hold experts
        float tau;
        {
            const int me = lane & (kDecWarps - 1);
            const float mine = sm->red2[me] * inv;  // bit-identical to the owning thread's pr; negative for empty warps
            int cnt = 0;
#pragma unroll
            for (int j = 0; j < kDecWarps; ++j) {
                const float o = __shfl_sync(0xffffffffu, mine, j);
                cnt += (o > mine) || (o == mine && j < me);
            }
            // exactly one of lanes 0..15 has K-1 warp maxima ahead of it
            const unsigned hit = __ballot_sync(0xffffffffu, cnt == K - 1 && lane < kDecWarps);
            tau = __shfl_sync(0xffffffffu, mine, __ffs(hit) - 1);
            if (tau < 0.0f) tau = -1.0f;  // fewer than K warps hold experts: everything is a candidate
        }
        if (tid < E && pr >= tau) {
            const int slot = atomicAdd(&sm->ncand, 1);
            sm->cand_p[slot] = pr;
            sm->cand_i[slot] = tid;
        }
        __syncthreads();
        const int nc = sm->ncand;
        if (tid < nc) {
            const float cp = sm->cand_p[tid];
            const int ci = sm->cand_i[tid];
            int rank = 0;
            for (int j = 0; j < nc; ++j) {
                const float q = sm->cand_p[j];
                rank += (q > cp) || (q == cp && sm->cand_i[j] < ci);
            }
            if (rank < K) { sm->topi[rank] = ci; sm->topp[rank] = cp; }
        }
    }
    __syncthreads();
    if (tid == 0) {
        // normalize_weights: divide by the sum of the K selected probabilities
        float s = 0.0f;
        for (int k = 0; k < K; ++k) s += sm->topp[k];
        const float invs = s > 0.0f ? 1.0f / s : 1.0f;
        for (int k = 0; k < K; ++k) sm->topw[k] = sm->topp[k] * invs;
    }
    __syncthreads();
}

// ─── the persistent kernel ──────────────────────────────────────────────────
__global__ void __launch_bounds__(kDecThreads, 1) decode_stack_kernel(DecodeParams p) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    DecodeSmem* sm = reinterpret_cast<DecodeSmem*>(smem_raw);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int G = gridDim.x;
    const int cta = blockIdx.x;
    const int E = p.E, K = p.K;
    const moe_expert_layout_t L = p.lay;

    if (tid == 0) {
        mbar_init(&sm->bar_h, 1);
        mbar_fence_init();
    }
    __syncthreads();

    // this CTA's slices
    const int e0 = slice_lo(cta, E, G), ne = slice_lo(cta + 1, E, G) - e0;
    const int p0 = slice_lo(cta, kI, G), np = slice_lo(cta + 1, kI, G) - p0;
    const int i0 = slice_lo(cta, K * kI, G), nb = slice_lo(cta + 1, K * kI, G) - i0;
    const int r0 = slice_lo(cta, kH, G), nc = slice_lo(cta + 1, kH, G) - r0;

    unsigned int bar_target = 0;
    uint32_t parity = 0;
    bool alive = true;

    prefetch_A(sm, p.layers ? p.layers[p.l0] : p.one, L, cta, G, E, tid);

    for (int l = p.l0; l < p.l1 && alive; ++l) {
        const LayerDev ly = p.layers ? p.layers[l] : p.one;
        const float* h_cur = (l == p.l0) ? p.h_in : (((l - p.l0) & 1) ? p.h_buf0 : p.h_buf1);
        float* h_nxt = (l == p.l1 - 1) ? p.h_out : (((l - p.l0) & 1) ? p.h_buf1 : p.h_buf0);

        // ── phase A ────────────────────────────────────────────────────────
        PROF(0);
        if (!stage_norm(sm, h_cur, ly.post_norm, parity)) {
            if (tid == 0) atomicExch(&p.sync[2], 3u);
            alive = false;
            break;
        }
        cp_wait<0>();  // this layer's phase-A slice (requested one layer ago)
        __syncthreads();
        PROF(1);
        {
            // warps [0, ne): router rows; [4, 4 + np): shared gate/up pairs; 8: shared gate score
            if (warp < ne) {
                float v;
                if (ly.router_bf16) {
                    v = row_dot_bf16(sm, sm->a_router + warp * (kH * 2 / 16), lane);
                } else {
                    const uint4* const w[1] = {sm->a_router + warp * kChH};
                    const uint16_t* const s[1] = {sm->a_router_s[warp]};
                    const uint16_t* const b[1] = {sm->a_router_b[warp]};
                    float o[1];
                    rows_dot_h<1>(sm, w, s, b, o, lane);
                    v = o[0];
                }
                if (lane == 0) p.logits[e0 + warp] = v;
            } else if (warp >= 4 && warp < 4 + np) {
                const int j = warp - 4;
                const uint4* const w[2] = {sm->a_shw[0][j], sm->a_shw[1][j]};
                const uint16_t* const s[2] = {sm->a_shs[0][j], sm->a_shs[1][j]};
                const uint16_t* const b[2] = {sm->a_shb[0][j], sm->a_shb[1][j]};
                float o[2];
                rows_dot_h<2>(sm, w, s, b, o, lane);
                if (lane == 0) p.act[K * kI + p0 + j] = swiglu(o[0], o[1]);
            } else if (warp == 8 && cta == G - 1) {
                const uint4* const w[1] = {sm->a_sgw};
                const uint16_t* const s[1] = {sm->a_sgs};
                const uint16_t* const b[1] = {sm->a_sgb};
                float o[1];
                rows_dot_h<1>(sm, w, s, b, o, lane);
                if (lane == 0) p.misc[0] = o[0];
            }
        }
        PROF(2);
        bar_target += G;
        if (!grid_barrier(p.sync, bar_target, sm)) { alive = false; break; }
        PROF(3);
        PROF(4);

        // ── phase B ────────────────────────────────────────────────────────
        {
            float v = -INFINITY;
            if (tid < E) {
                v = __ldcg(p.logits + tid);  // written by other CTAs: read through L2
                if (p.logit_bias) v += p.logit_bias[tid];
            }
            route_cta(sm, v, p.forced_idx, E, K, p.sync + 2);
        }
        PROF(5);
        // request this warp's gate/up rows now; its down rows and the next layer's
        // phase-A slice are requested after the gate/up arithmetic, so that their
        // issue (which stalls while the load queues are full) overlaps barrier 2
        prefetch_B_warp(sm, ly, L, i0, nb, warp, lane);
        if (warp == 0) {
            if (lane == 0) {
                // sigmoid (reference src/math_util.rs:67-69) of the shared gate score
                sm->topw[K] = 1.0f / (1.0f + expf(-__ldcg(p.misc)));
            }
            if (cta == 0 && lane < K) {
                if (p.out_idx) p.out_idx[lane] = sm->topi[lane];
                if (p.out_w) p.out_w[lane] = sm->topw[lane];
            }
        }
        PROF(6);
        cp_wait<0>();  // this warp's gate/up rows landed
        __syncwarp();
        PROF(7);
        {
            // item j of this CTA = (gate row, up row) pair; two items per warp pass
            for (int j = warp; j < nb; j += 2 * kDecWarps) {
                const int j2 = j + kDecWarps;
                const bool two = j2 < nb;
                const int jb = two ? j2 : j;
                const uint4* const w[4] = {sm->b_w[0][j], sm->b_w[1][j], sm->b_w[0][jb], sm->b_w[1][jb]};
                const uint16_t* const s[4] = {sm->b_s[0][j], sm->b_s[1][j], sm->b_s[0][jb], sm->b_s[1][jb]};
                const uint16_t* const b[4] = {sm->b_b[0][j], sm->b_b[1][j], sm->b_b[0][jb], sm->b_b[1][jb]};
                float o[4];
                rows_dot_h<4>(sm, w, s, b, o, lane);
                if (lane == 0) {
                    p.act[i0 + j] = swiglu(o[0], o[1]);
                    if (two) p.act[i0 + j2] = swiglu(o[2], o[3]);
                }
            }
        }
        prefetch_C_warp(sm, ly, L, r0, nc, K, warp, lane);
        if (l + 1 < p.l1) prefetch_A(sm, p.layers ? p.layers[l + 1] : p.one, L, cta, G, E, tid);
        else cp_commit();  // keep the group count per layer fixed
        PROF(8);
        bar_target += G;
        if (!grid_barrier(p.sync, bar_target, sm)) { alive = false; break; }
        PROF(9);

        // ── phase C ────────────────────────────────────────────────────────
        {
            // stage the (K + 1) x I SwiGLU outputs chunk-transposed, with chunk sums
            const int n_f4 = (K + 1) * (kI / 4);
            for (int i = tid; i < n_f4; i += kDecThreads) {
                const float4 v = __ldcg(reinterpret_cast<const float4*>(p.act) + i);
                const int m = i / (kI / 4), f = i - m * (kI / 4);
                const int c = f >> 3, j = f & 7;
                sm->acts[(m * 8 + j) * kChI + c] = v;
                float sv = (v.x + v.y) + (v.z + v.w);
                sv += __shfl_xor_sync(0xffffffffu, sv, 1);
                sv += __shfl_xor_sync(0xffffffffu, sv, 2);
                sv += __shfl_xor_sync(0xffffffffu, sv, 4);
                if (j == 0) sm->suma[m * kChI + c] = sv;
            }
            cp_wait<1>();  // this warp's down rows landed
            __syncthreads();  // the staged activations above are shared by all warps
            PROF(10);
            // one warp per output element: half-warp `sub` takes matrices sub, sub+2, ...
            const int sub = lane >> 4, c = lane & 15;
            constexpr int kMats = (kMaxK + 2) / 2;  // 5 matrix slots per half-warp
            for (int j = warp; j < nc; j += kDecWarps) {
                float acc = 0.0f;
#pragma unroll
                for (int jm = 0; jm < kMats; ++jm) {
                    const int m = sub + 2 * jm;
                    if (m <= K) {
                        float4 xv[8];
#pragma unroll
                        for (int q = 0; q < 8; ++q) xv[q] = sm->acts[(m * 8 + q) * kChI + c];
                        acc = fmaf(sm->topw[m],
                                   chunk_term(sm->c_w[m][j][c], xv, sm->suma[m * kChI + c], sm->c_s[m][j][c >> 1],
                                              sm->c_b[m][j][c >> 1]),
                                   acc);
                    }
                }
                acc = warp_sum(acc);
                // moe_combine_residual (reference src/math_util.rs:599-612)
                if (lane == 0) h_nxt[r0 + j] = sm->raw[r0 + j] + acc;
            }
        }
        PROF(11);
        parity ^= 1u;
        if (l + 1 < p.l1) {
            bar_target += G;
            if (!grid_barrier(p.sync, bar_target, sm)) { alive = false; break; }
        }
    }

    // Last CTA out rewinds the barrier words for the next launch.
    __syncthreads();
    if (tid == 0) {
        __threadfence();
        const unsigned int done = atomicAdd(&p.sync[1], 1u) + 1u;
        if (done == (unsigned int)G) {
            p.sync[0] = 0u;
            p.sync[1] = 0u;
            __threadfence();
        }
    }
}

// ════════════════════════════════════════════════════════════════════════════
// Fused variant: the next layer's router is folded into the down phase.
//
// logits_{l+1}[e] = inv_rms * sum_i Wr[e][i] * nw[i] * h_{l+1}[i] is linear in h, and after
// the down phase every CTA owns ~14 finished elements of h_{l+1}: it multiplies them
// with its slice of the transposed router (built once per layer) and adds the 256 partial
// sums into a global accumulator.  Partial sums are added as 64-bit fixed point (2^-32
// units, scaled by the current 1/rms so magnitudes stay near a finished logit): integer
// addition is associative, so the total does not depend on the order of arrival and
// repeated runs give identical bits.  The sum of squares the next norm needs travels the
// same way, so routing starts from 2 KB of accumulators.  The shared expert's gate/up rows
// ride along with the routed experts' as a ninth "slot".
//
// Nothing that crosses CTAs waits for a fence:
//  * SwiGLU outputs and the hidden state travel as 8-byte words (tag, value), tag = the
//    producing layer's epoch.  8-byte accesses are single-copy atomic: a reader that sees
//    the current tag sees the value, and re-reads a word whose tag is stale.
//  * Accumulator words carry a contribution count in their low 8 bits (value in the upper
//    56); they are never cleared, a reader subtracts what it read two layers earlier and
//    knows the sum is complete when the count has advanced by the number of CTAs.
//  * "This CTA is done" is a relaxed increment of a counter that readers watch before they
//    read at all: a hint that keeps 148 CTAs from hammering lines that are still being
//    written (polling the data itself was 2-3x slower), never a proof of visibility.
// Every wait is bounded (about a second of SM clocks) and ends in an error word.
// ════════════════════════════════════════════════════════════════════════════
constexpr size_t kActLLWords = (size_t)(kMaxK + 1) * kI + 8;
constexpr int kMaxB3Items = 32;   // ceil((K + 1) * I / grid) gate/up row pairs incl. the shared expert
constexpr float kFix = 4294967296.0f;  // 2^32
constexpr int kMaxDecLayers = 64;  // layer table rows staged in shared memory per launch
constexpr int kAccPitch = 1;  // distance between accumulators in words (spreading them over sectors measured no faster)
constexpr int kAccStride = (kMaxE + 8) * kAccPitch;
constexpr int kLLGroups = ((kMaxK + 1) * (kI / 4) + kDecThreads - 1) / kDecThreads;  // 4-value groups per thread

struct Decode3Params {
    const LayerDev* layers;
    int l0, l1;
    const float* h_in;
    float* h_out;
    long long* acc;     // [2][kAccStride] fixed-point accumulators (router logits; [kMaxE] = sum of squares), zero at launch
    unsigned long long* act_ll;  // [(K + 1) * I + 1] (tag << 32 | float bits): SwiGLU outputs, then the shared gate score
    unsigned int epoch_base;     // tags in act_ll are <= epoch_base when the kernel starts
    unsigned long long* hint;    // counts CTAs that have written their SwiGLU outputs (a hint: the tags decide)
    unsigned long long* hint2;   // counts CTAs that have finished a layer (h stored, partial logits added); same base
    unsigned long long hint_base;
    unsigned long long* h_ll;    // [H] (tag << 32 | float bits): the hidden state between layers
    const float* logit_bias;
    const int32_t* forced_idx;
    int32_t* out_idx;
    float* out_w;
    unsigned int* err;
    long long* prof;
    int E, K;
    moe_expert_layout_t lay;
};

struct __align__(128) DecodeSmem3 {
    uint4 b_w[2][kMaxB3Items][kChH];
    uint4 c_w[kMaxK + 1][kMaxCRows][kChI];
    float wt[kMaxCRows * kMaxE];          // slice of the next layer's transposed router (bf16 or f32 rows of E)
    uint4 sg_w[kChH];                     // shared_expert_gate row (CTA 0 only)
    uint16_t sg_s[kH / kGroup];
    uint16_t sg_b[kH / kGroup];
    uint16_t b_s[2][kMaxB3Items][kH / kGroup];
    uint16_t b_b[2][kMaxB3Items][kH / kGroup];
    uint16_t c_s[kMaxK + 1][kMaxCRows][kI / kGroup];
    uint16_t c_b[kMaxK + 1][kMaxCRows][kI / kGroup];
    float raw[kH];
    float xn[kH];
    float4 xs[8 * kChH];
    float sumx[kChH];
    float4 acts[(kMaxK + 1) * 8 * kChI];
    float suma[(kMaxK + 1) * kChI];
    float prob[kMaxE];
    float red[kDecWarps];
    float red2[kDecWarps];
    float inv_rms;
    float cand_p[kMaxE];
    int cand_i[kMaxE];
    int ncand;
    float topw[kMaxK + 1];
    float topp[kMaxK];
    int topi[kMaxK];
    uint4 xq[6 * kChH];                   // x as three signed-byte digit planes, [plane * 2 + odd][chunk] (see stage_digits)
    float xdl[kChH];                      // value of one unit of a chunk's digits
    uint4 aq[(kMaxK + 1) * 6 * kChI];     // SwiGLU outputs as digit planes, per matrix [plane * 2 + odd][chunk]
    float adl[(kMaxK + 1) * kChI];
    float hn[kMaxCRows + 2];              // this CTA's finished elements of the next h, times the next norm weight
    float hraw[kMaxCRows + 2];            // the same elements as they are
    float hmax[32];                       // routing: maxima of 16-expert groups
    float tau;                            // routing: candidate threshold
    int flag;
    uint64_t bar_h;
    uint64_t bar_b;   // gate/up slices landed
    LayerDev tab[kMaxDecLayers];  // this launch's rows of the layer table
};
static_assert(sizeof(DecodeSmem3) <= 227 * 1024, "decode staging exceeds shared memory");

// gate/up rows of item j (slot m = item / I: the m-th chosen expert, or the shared expert for m == K)
__device__ __forceinline__ void prefetch_B3_warp(DecodeSmem3* sm, const LayerDev& ly, const moe_expert_layout_t& L,
                                                 int i0, int nb, int K, bool with_sgate, int warp, int lane) {
    if (with_sgate) {
        cp16(&sm->sg_w[lane], reinterpret_cast<const uint8_t*>(ly.sgate.w) + lane * 16);
        cp16(&sm->sg_w[lane + 32], reinterpret_cast<const uint8_t*>(ly.sgate.w) + (lane + 32) * 16);
        if (lane < 4) cp16(reinterpret_cast<uint8_t*>(sm->sg_s) + lane * 16, reinterpret_cast<const uint8_t*>(ly.sgate.s) + lane * 16);
        else if (lane < 8) cp16(reinterpret_cast<uint8_t*>(sm->sg_b) + (lane - 4) * 16, reinterpret_cast<const uint8_t*>(ly.sgate.b) + (lane - 4) * 16);
    }
#pragma unroll
    for (int t = 0; t < 2; ++t) {
        const int j = warp + t * kDecWarps;
        if (j < nb) {
            const int i = i0 + j, m = i / kI, r = i - m * kI;
            const uint8_t* ex = (m < K) ? ly.experts + (size_t)sm->topi[m] * L.expert_size : ly.shared;
            const uint8_t* gw = ex + L.gate_w + (size_t)r * (kH / 2);
            const uint8_t* uw = ex + L.up_w + (size_t)r * (kH / 2);
            cp16(&sm->b_w[0][j][lane], gw + lane * 16);
            cp16(&sm->b_w[0][j][lane + 32], gw + (lane + 32) * 16);
            cp16(&sm->b_w[1][j][lane], uw + lane * 16);
            cp16(&sm->b_w[1][j][lane + 32], uw + (lane + 32) * 16);
            if (lane < 16) {
                const int a = lane >> 2, c = lane & 3;
                const int64_t off = a == 0 ? L.gate_s : a == 1 ? L.up_s : a == 2 ? L.gate_b : L.up_b;
                uint16_t* d = a == 0 ? sm->b_s[0][j] : a == 1 ? sm->b_s[1][j] : a == 2 ? sm->b_b[0][j] : sm->b_b[1][j];
                cp16(reinterpret_cast<uint8_t*>(d) + c * 16, ex + off + (size_t)r * (kH / kGroup) * 2 + c * 16);
            }
        }
    }
    cp_commit();
}

__device__ __forceinline__ int router_t_stride(int E) { return (E + 7) & ~7; }  // elements per row: 16-byte multiples

// ─── weight slices by bulk copy ─────────────────────────────────────────────
// A CTA's gate/up items are consecutive (slot, row) pairs, so each of the six arrays it needs
// (gate/up weights, scales, biases) is at most two contiguous byte ranges (one per slot
// touched): twelve bulk copies, issued by twelve different threads, each announcing its own
// bytes on the mbarrier (which counts kBCopies arrivals per phase).
constexpr int kBCopies = 12;

__device__ __forceinline__ void bulk_B_copy(DecodeSmem3* sm, const LayerDev& ly, const moe_expert_layout_t& L,
                                            int i0, int nb, int K, int q) {
    const int a = q >> 1, sg = q & 1;
    const int m0 = i0 / kI, ra = i0 - m0 * kI;
    const int n0 = min(nb, kI - ra), n1 = nb - n0;
    const int m = m0 + sg, row = sg ? 0 : ra, n = sg ? n1 : n0, j0 = sg ? n0 : 0;
    uint32_t bytes = 0;
    if (n > 0) {
        const uint8_t* ex = (m < K) ? ly.experts + (size_t)sm->topi[m] * L.expert_size : ly.shared;
        const bool is_w = a < 2;
        const int64_t off = a == 0 ? L.gate_w : a == 1 ? L.up_w : a == 2 ? L.gate_s : a == 3 ? L.up_s : a == 4 ? L.gate_b : L.up_b;
        const uint32_t row_bytes = is_w ? kH / 2 : (kH / kGroup) * 2;
        void* dst = a == 0 ? (void*)sm->b_w[0][j0] : a == 1 ? (void*)sm->b_w[1][j0] : a == 2 ? (void*)sm->b_s[0][j0]
                  : a == 3 ? (void*)sm->b_s[1][j0] : a == 4 ? (void*)sm->b_b[0][j0] : (void*)sm->b_b[1][j0];
        bytes = (uint32_t)n * row_bytes;
        mbar_expect_tx(&sm->bar_b, bytes);
        bulk_g2s(dst, ex + off + (size_t)row * row_bytes, bytes, &sm->bar_b);
    } else {
        mbar_expect_tx(&sm->bar_b, 0u);
    }
}

// rows [r0, r0 + nc) of a layer's transposed router (contiguous: nc * E elements), all threads
__device__ __forceinline__ void prefetch_wt(DecodeSmem3* sm, const void* router_t, bool bf16, int r0, int nc, int E, int tid) {
    const size_t row_bytes = (size_t)router_t_stride(E) * (bf16 ? 2 : 4);
    copy_flat(sm->wt, reinterpret_cast<const uint8_t*>(router_t) + (size_t)r0 * row_bytes, (int)(nc * row_bytes / 16), tid);
    cp_commit();
}

// This CTA's contribution to the router logits of a layer: sum over its rows j of
// Wr[e][r0 + j] * (h[r0 + j] * norm_w[r0 + j]), times `scale` (the caller's estimate of
// 1 / rms(h), which keeps the fixed-point value near the size of a finished logit).
__device__ __forceinline__ void push_partial_logits(const DecodeSmem3* sm, bool bf16, long long* acc, int nc, int E,
                                                    float scale, int tid) {
    if (tid < E) {
        const int Ep = router_t_stride(E);
        float part = 0.0f;
        if (bf16) {
            const uint16_t* w = reinterpret_cast<const uint16_t*>(sm->wt);
            for (int j = 0; j < nc; ++j) part = fmaf(__uint_as_float((uint32_t)w[j * Ep + tid] << 16), sm->hn[j], part);
        } else {
            for (int j = 0; j < nc; ++j) part = fmaf(sm->wt[j * Ep + tid], sm->hn[j], part);
        }
        // value in the upper 56 bits, a contribution count in the low 8: a reader knows the sum is complete
        // when the count has advanced by the number of CTAs (fewer than 256)
        const long long fx = __float2ll_rn(part * scale * kFix);
        atomicAdd(reinterpret_cast<unsigned long long*>(acc) + tid * kAccPitch, ((unsigned long long)fx << 8) + 1ull);
    }
    if (tid == kDecThreads - 1) {
        // this CTA's share of sum((h * scale)^2)
        float q = 0.0f;
        for (int j = 0; j < nc; ++j) {
            const float t = sm->hraw[j] * scale;
            q = fmaf(t, t, q);
        }
        atomicAdd(reinterpret_cast<unsigned long long*>(acc) + kMaxE * kAccPitch,
                  ((unsigned long long)__float2ll_rn(q * kFix) << 8) + 1ull);
    }
}

__device__ __forceinline__ void st_ll(unsigned long long* ptr, unsigned int tag, float v) {
    const unsigned long long w = ((unsigned long long)tag << 32) | (unsigned long long)__float_as_uint(v);
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(ptr), "l"(w) : "memory");
}
__device__ __forceinline__ void ld_ll2(const unsigned long long* ptr, unsigned long long& a, unsigned long long& b) {
    asm volatile("ld.relaxed.gpu.global.v2.u64 {%0, %1}, [%2];" : "=l"(a), "=l"(b) : "l"(ptr) : "memory");
}

// Reads an accumulator until the contributions of all G CTAs are in: the word is never reset, the reader
// subtracts what it read two layers ago (`prev`, updated).  Returns the sum (2^-32 units); bounded.
__device__ __forceinline__ long long read_counted(const long long* word, unsigned long long& prev, int G, int* ok) {
    const long long t0 = clock64();
    for (uint32_t it = 0;; ++it) {
        unsigned long long raw;
        asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(raw) : "l"(word) : "memory");
        const unsigned long long d = raw - prev;
        if ((int)(d & 0xFFull) == G) {
            prev = raw;
            return (long long)d >> 8;
        }
        if ((it & 15u) == 15u && clock64() - t0 > kWaitCycles) { *ok = 0; return 0; }
    }
}

// x = rmsnorm(h) * w staged as digit planes, h given as this thread's float4 (elements 4 tid ..)
__device__ __forceinline__ void stage_from_regs(DecodeSmem3* sm, const uint16_t* norm_w, const float4 v) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint2 wb = __ldg(reinterpret_cast<const uint2*>(norm_w) + tid);
    reinterpret_cast<float4*>(sm->raw)[tid] = v;  // the down phase adds the residual from here
    float ss = warp_sum(v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w);
    if (lane == 0) sm->red[warp] = ss;
    __syncthreads();
    float tot = 0.0f;
#pragma unroll
    for (int i = 0; i < kDecWarps; ++i) tot += sm->red[i];
    const float inv_rms = 1.0f / sqrtf(tot / (float)kH + 1e-6f);
    if (tid == 0) sm->inv_rms = inv_rms;
    float4 o;
    o.x = v.x * inv_rms * __uint_as_float(wb.x << 16);
    o.y = v.y * inv_rms * __uint_as_float(wb.x & 0xFFFF0000u);
    o.z = v.z * inv_rms * __uint_as_float(wb.y << 16);
    o.w = v.w * inv_rms * __uint_as_float(wb.y & 0xFFFF0000u);
    const int c = tid >> 3, j = tid & 7;
    stage_digits(sm->xq, sm->xdl, kChH, c, j, o);
    float s = (o.x + o.y) + (o.z + o.w);
    s += __shfl_xor_sync(0xffffffffu, s, 1);
    s += __shfl_xor_sync(0xffffffffu, s, 2);
    s += __shfl_xor_sync(0xffffffffu, s, 4);
    if (j == 0) sm->sumx[c] = s;
    __syncthreads();
}

#define PROF3(idx)                                                                                 \
    do {                                                                                           \
        if (p.prof && cta == 0 && tid == 0) p.prof[(l - p.l0) * kProfPoints + (idx)] = clock64();  \
    } while (0)

static_assert(kMaxCRows <= kDecWarps, "one finished element of h per warp");

__global__ void __launch_bounds__(kDecThreads, 1) decode_fused_kernel(Decode3Params p) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    DecodeSmem3* sm = reinterpret_cast<DecodeSmem3*>(smem_raw);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int G = gridDim.x;
    const int cta = blockIdx.x;
    const int E = p.E, K = p.K;
    const moe_expert_layout_t L = p.lay;

    if (tid == 0) {
        mbar_init(&sm->bar_h, 1);
        mbar_init(&sm->bar_b, kBCopies);
        mbar_fence_init();
    }
    {
        // pointer loads from shared memory instead of dependent global loads on the critical path
        static_assert(sizeof(LayerDev) % 4 == 0, "table rows are copied as words");
        const uint32_t* src = reinterpret_cast<const uint32_t*>(p.layers + p.l0);
        uint32_t* dst = reinterpret_cast<uint32_t*>(sm->tab);
        const int words = (p.l1 - p.l0) * (int)(sizeof(LayerDev) / 4);
        for (int i = tid; i < words; i += kDecThreads) dst[i] = __ldg(src + i);
    }
    __syncthreads();

    const int n_items = (K + 1) * kI;
    const int i0 = slice_lo(cta, n_items, G), nb = slice_lo(cta + 1, n_items, G) - i0;
    const int r0 = slice_lo(cta, kH, G), nc = slice_lo(cta + 1, kH, G) - r0;
    // the shared expert's gate score is one more row: CTA 0's last warp takes it
    const bool sg_here = (cta == 0 && warp == kDecWarps - 1);

    uint32_t parity = 0, wpar = 0;
    bool alive = true;
    float pscale = 1.0f;  // scale the pending accumulators were pushed with
    // what this thread read from its accumulator words the last time each of the two sets was used
    unsigned long long pa_cur = 0, pa_oth = 0, pq_cur = 0, pq_oth = 0;
    // "this CTA has finished": a relaxed count, no fence; the data it announces validates itself
    auto announce = [&]() {
        __syncthreads();
        if (tid == 0) asm volatile("red.relaxed.gpu.global.add.u64 [%0], %1;" ::"l"(p.hint2), "l"(1ull) : "memory");
    };

    // ── prologue: router logits and sum of squares of the first layer from h_in ──
    {
        const LayerDev& ly = sm->tab[0];
        prefetch_wt(sm, ly.router_t, ly.router_bf16 != nullptr, r0, nc, E, tid);
        if (!stage_norm(sm, p.h_in, ly.post_norm, parity)) {
            if (tid == 0) atomicExch(p.err, 3u);
            alive = false;
        }
        parity ^= 1u;
        if (alive) {
            pscale = sm->inv_rms;
            if (tid < nc) {
                const float hv = sm->raw[r0 + tid];
                sm->hraw[tid] = hv;
                sm->hn[tid] = hv * __uint_as_float((uint32_t)ly.post_norm[r0 + tid] << 16);
            }
            cp_wait<0>();
            __syncthreads();
            push_partial_logits(sm, ly.router_bf16 != nullptr, p.acc, nc, E, pscale, tid);
            announce();
        }
    }

    for (int l = p.l0; l < p.l1 && alive; ++l) {
        const LayerDev& ly = sm->tab[l - p.l0];
        const int rel = l - p.l0;
        const bool has_next = l + 1 < p.l1;
        long long* acc_cur = p.acc + (rel & 1) * kAccStride;
        long long* acc_nxt = p.acc + ((rel + 1) & 1) * kAccStride;
        const unsigned int epoch = p.epoch_base + (unsigned int)rel + 1u;

        // ── route (from the accumulators) while h is being staged ──────────
        PROF3(0);
        float vlogit = -INFINITY;  // this thread's router logit (thread t owns expert t)
        {
            // every CTA has announced the end of the previous phase (a hint: the words below validate themselves)
            if (tid == 0) {
                const unsigned long long want_n = p.hint_base + (unsigned long long)G * (unsigned long long)(rel + 1);
                const long long t0 = clock64();
                int okh = 1;
                for (uint32_t it = 0;; ++it) {
                    unsigned long long nn;
                    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(nn) : "l"(p.hint2) : "memory");
                    if (nn >= want_n) break;
                    if ((it & 63u) == 63u && clock64() - t0 > kWaitCycles) { okh = 0; break; }
                }
                sm->flag = okh;
            }
            __syncthreads();
            int okr = sm->flag;
            float v = -INFINITY;
            const long long aq = read_counted(acc_cur + kMaxE * kAccPitch, pq_cur, G, &okr);
            long long a = 0;
            if (tid < E) a = read_counted(acc_cur + tid * kAccPitch, pa_cur, G, &okr);
            { unsigned long long t = pa_cur; pa_cur = pa_oth; pa_oth = t; t = pq_cur; pq_cur = pq_oth; pq_oth = t; }
            if (!__syncthreads_and(okr)) {
                if (tid == 0) atomicExch(p.err, 5u);
                alive = false;
                break;
            }
            // mean of (h * pscale)^2 -> 1 / rms(h); the logits were accumulated times pscale
            const float r = 1.0f / pscale;
            const float msq = __ll2float_rn(aq) * (1.0f / kFix) * (1.0f / (float)kH);
            const float inv_rms_acc = 1.0f / sqrtf(msq * r * r + 1e-6f);
            if (tid < E) {
                v = __ll2float_rn(a) * (1.0f / kFix) * r * inv_rms_acc;
                if (p.logit_bias) v += p.logit_bias[tid];
            }
            route_select(sm, v, p.forced_idx, E, K, p.err);
            vlogit = v;
        }
        PROF3(1);
        // one bulk copy per thread: gate/up slices first, then everything the down phase needs
        if (lane == 0 && warp < kBCopies) bulk_B_copy(sm, ly, L, i0, nb, K, warp);
        if (sg_here) prefetch_B3_warp(sm, ly, L, i0, 0, K, true, warp, lane);  // the gate-score row only
        else cp_commit();
        // the copies are on their way: now the softmax weights of the chosen experts
        route_weights(sm, vlogit, E, K);
        if (cta == 0 && warp == 0 && lane < K) {
            if (p.out_idx) p.out_idx[lane] = sm->topi[lane];
            if (p.out_w) p.out_w[lane] = sm->topw[lane];
        }
        // next layer's norm weight of the element of h this warp will finish
        float nwn = 0.0f;
        if (has_next && warp < nc && lane == 0)
            nwn = __uint_as_float((uint32_t)__ldg(sm->tab[rel + 1].post_norm + r0 + warp) << 16);
        PROF3(2);
        {
            // this thread's four elements of h: plain floats for the first layer, tagged words afterwards
            float4 hv4;
            int okh = 1;
            if (rel == 0) {
                hv4 = __ldg(reinterpret_cast<const float4*>(p.h_in) + tid);
            } else {
                const unsigned int want_tag = p.epoch_base + (unsigned int)rel;  // the producing layer's epoch
                const unsigned long long* src = p.h_ll + 4 * tid;
                unsigned long long q0, q1, q2, q3;
                const long long t0 = clock64();
                for (uint32_t it = 0;; ++it) {
                    ld_ll2(src, q0, q1);
                    ld_ll2(src + 2, q2, q3);
                    if ((unsigned int)(q0 >> 32) == want_tag && (unsigned int)(q1 >> 32) == want_tag &&
                        (unsigned int)(q2 >> 32) == want_tag && (unsigned int)(q3 >> 32) == want_tag)
                        break;
                    if ((it & 15u) == 15u && clock64() - t0 > kWaitCycles) { okh = 0; break; }
                }
                hv4 = make_float4(__uint_as_float((unsigned int)q0), __uint_as_float((unsigned int)q1),
                                  __uint_as_float((unsigned int)q2), __uint_as_float((unsigned int)q3));
            }
            if (!__syncthreads_and(okh)) {
                if (tid == 0) atomicExch(p.err, 3u);
                alive = false;
                break;
            }
            stage_from_regs(sm, ly.post_norm, hv4);
        }
        const float inv_rms = sm->inv_rms;
        PROF3(3);
        int landed = 1;
        cp_wait<0>();  // this warp's gate/up rows (and the gate-score row) landed
        landed = mbar_wait(&sm->bar_b, wpar) ? 1 : 0;
        __syncwarp();
        PROF3(4);
        {
            bool sg_done = !sg_here;
            for (int j = warp; j < nb; j += 2 * kDecWarps) {
                const int j2 = j + kDecWarps;
                const bool two = j2 < nb;
                const bool sg_now = !two && !sg_done;  // the spare half of the pass takes the gate-score row
                const int jb = two ? j2 : j;
                const uint4* const w[4] = {sm->b_w[0][j], sm->b_w[1][j], sg_now ? sm->sg_w : sm->b_w[0][jb], sm->b_w[1][jb]};
                const uint16_t* const s[4] = {sm->b_s[0][j], sm->b_s[1][j], sg_now ? sm->sg_s : sm->b_s[0][jb], sm->b_s[1][jb]};
                const uint16_t* const b[4] = {sm->b_b[0][j], sm->b_b[1][j], sg_now ? sm->sg_b : sm->b_b[0][jb], sm->b_b[1][jb]};
                float o[4];
                rows_dot_q<4>(sm, w, s, b, o, lane);
                if (lane == 0) {
                    st_ll(p.act_ll + i0 + j, epoch, swiglu(o[0], o[1]));
                    if (two) st_ll(p.act_ll + i0 + j2, epoch, swiglu(o[2], o[3]));
                    if (sg_now) st_ll(p.act_ll + n_items, epoch, o[2]);
                }
                sg_done |= sg_now;
            }
            if (!sg_done) {
                const uint4* const w[1] = {sm->sg_w};
                const uint16_t* const s[1] = {sm->sg_s};
                const uint16_t* const b[1] = {sm->sg_b};
                float o[1];
                rows_dot_q<1>(sm, w, s, b, o, lane);
                if (lane == 0) st_ll(p.act_ll + n_items, epoch, o[0]);
            }
        }
        // Tell the others that this CTA's outputs are on their way.  Not ordered against the
        // stores above (no fence): readers use it only to decide when to start reading.
        __syncthreads();
        if (tid == 0) asm volatile("red.relaxed.gpu.global.add.u64 [%0], %1;" ::"l"(p.hint), "l"(1ull) : "memory");
        // down rows and the next router's slice: requested after the gate/up arithmetic, so that their
        // issue (which stalls while the load queues are full) does not delay it
        prefetch_C_warp(sm, ly, L, r0, nc, K, warp, lane);
        if (has_next) {
            const LayerDev& nx = sm->tab[rel + 1];
            prefetch_wt(sm, nx.router_t, nx.router_bf16 != nullptr, r0, nc, E, tid);
        } else {
            cp_commit();  // keep the group count per layer fixed
        }
        PROF3(5);

        // ── gather every CTA's SwiGLU outputs: re-read until all tags are current ──
        {
            const int n_g = (K + 1) * (kI / 4);  // groups of 4 values
            unsigned long long q[kLLGroups][4];
            unsigned long long qs = 0;
            unsigned int pending = 0;
#pragma unroll
            for (int t = 0; t < kLLGroups; ++t)
                if (tid + t * kDecThreads < n_g) pending |= 1u << t;
            const bool sg_reader = (tid == kDecThreads - 1);
            if (sg_reader) pending |= 1u << kLLGroups;
            const long long t0 = clock64();
            int ok = landed;
            if (tid == 0) {
                const unsigned long long want_n = p.hint_base + (unsigned long long)G * (unsigned long long)(rel + 1);
                for (uint32_t it = 0;; ++it) {
                    unsigned long long n;
                    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(n) : "l"(p.hint) : "memory");
                    if (n >= want_n) break;
                    if ((it & 63u) == 63u && clock64() - t0 > kWaitCycles) { ok = 0; break; }
                }
            }
            __syncthreads();
            // the groups are taken in an order rotated by the CTA index, so that the CTAs do not
            // all ask for the same lines at the same moment
            const int n_wg = n_g / 32;
            int gidx[kLLGroups];
#pragma unroll
            for (int t = 0; t < kLLGroups; ++t) {
                const int wg = warp + t * kDecWarps;
                gidx[t] = ((wg + cta) % n_wg) * 32 + lane;
            }
            for (uint32_t it = 0; pending; ++it) {
#pragma unroll
                for (int t = 0; t < kLLGroups; ++t)
                    if (pending >> t & 1u) {
                        const unsigned long long* src = p.act_ll + 4 * (size_t)gidx[t];
                        ld_ll2(src, q[t][0], q[t][1]);
                        ld_ll2(src + 2, q[t][2], q[t][3]);
                    }
                if (pending >> kLLGroups & 1u)
                    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(qs) : "l"(p.act_ll + n_items) : "memory");
#pragma unroll
                for (int t = 0; t < kLLGroups; ++t)
                    if (pending >> t & 1u) {
                        const bool cur = (unsigned int)(q[t][0] >> 32) == epoch && (unsigned int)(q[t][1] >> 32) == epoch &&
                                         (unsigned int)(q[t][2] >> 32) == epoch && (unsigned int)(q[t][3] >> 32) == epoch;
                        if (cur) pending &= ~(1u << t);
                    }
                if ((pending >> kLLGroups & 1u) && (unsigned int)(qs >> 32) == epoch) pending &= ~(1u << kLLGroups);
                if (pending && (it & 15u) == 15u) {
                    unsigned int e;
                    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(e) : "l"(p.err) : "memory");
                    if (e != 0u || clock64() - t0 > kWaitCycles) { ok = 0; break; }
                }
            }
            __syncwarp();
#pragma unroll
            for (int t = 0; t < kLLGroups; ++t) {
                const int i = gidx[t];
                if (tid + t * kDecThreads < n_g) {  // uniform per warp: n_g and the stride are multiples of 32
                    float4 v;
                    v.x = __uint_as_float((unsigned int)q[t][0]);
                    v.y = __uint_as_float((unsigned int)q[t][1]);
                    v.z = __uint_as_float((unsigned int)q[t][2]);
                    v.w = __uint_as_float((unsigned int)q[t][3]);
                    const int m = i / (kI / 4), f = i - m * (kI / 4);
                    const int c = f >> 3, j = f & 7;
                    stage_digits(sm->aq + m * 6 * kChI, sm->adl + m * kChI, kChI, c, j, v);
                    float sv = (v.x + v.y) + (v.z + v.w);
                    sv += __shfl_xor_sync(0xffffffffu, sv, 1);
                    sv += __shfl_xor_sync(0xffffffffu, sv, 2);
                    sv += __shfl_xor_sync(0xffffffffu, sv, 4);
                    if (j == 0) sm->suma[m * kChI + c] = sv;
                }
            }
            // sigmoid (reference src/math_util.rs:67-69) of the shared gate score
            if (sg_reader) sm->topw[K] = 1.0f / (1.0f + expf(-__uint_as_float((unsigned int)qs)));
            PROF3(6);
            cp_wait<1>();  // this warp's down rows landed (the next router's slice may still be in flight)
            wpar ^= 1u;
            if (!__syncthreads_and(ok)) {
                if (tid == 0) atomicExch(p.err, 4u);
                alive = false;
                break;
            }
        }
        PROF3(7);
        {
            const int sub = lane >> 4, c = lane & 15;
            constexpr int kMats = (kMaxK + 2) / 2;
            if (warp < nc) {
                const int j = warp;
                float acc = 0.0f;
#pragma unroll
                for (int jm = 0; jm < kMats; ++jm) {
                    const int m = sub + 2 * jm;
                    if (m <= K) {
                        uint4 xe[3], xo[3];
#pragma unroll
                        for (int q = 0; q < 3; ++q) {
                            xe[q] = sm->aq[(m * 6 + q * 2 + 0) * kChI + c];
                            xo[q] = sm->aq[(m * 6 + q * 2 + 1) * kChI + c];
                        }
                        const float sc = bf16_bits_to_f32(sm->c_s[m][j][c >> 1]), bi = bf16_bits_to_f32(sm->c_b[m][j][c >> 1]);
                        const float term = fmaf(sc * sm->adl[m * kChI + c], dot32_int(sm->c_w[m][j][c], xe, xo),
                                                bi * sm->suma[m * kChI + c]);
                        acc = fmaf(sm->topw[m], term, acc);
                    }
                }
                acc = warp_sum(acc);
                // moe_combine_residual (reference src/math_util.rs:599-612)
                if (lane == 0) {
                    const float hv = sm->raw[r0 + j] + acc;
                    if (has_next) st_ll(p.h_ll + r0 + j, epoch, hv);
                    else p.h_out[r0 + j] = hv;
                    sm->hraw[j] = hv;
                    sm->hn[j] = hv * nwn;
                }
            }
            PROF3(8);
            if (has_next) {
                cp_wait<0>();  // the next router's slice landed
                __syncthreads();
                push_partial_logits(sm, sm->tab[rel + 1].router_bf16 != nullptr, acc_nxt, nc, E, inv_rms, tid);
                pscale = inv_rms;
                PROF3(9);
                announce();
                PROF3(10);
            }
        }
    }
}

// Transposed router of a layer for the fused decode kernel: out[i][e] = Wr[e][i], as bf16
// bit patterns when the router is bf16 and as dequantised f32 when it is 4-bit; rows are
// padded with zeros to router_t_stride(E) elements.
__global__ void __launch_bounds__(256) router_transpose_kernel(LayerDev ly, int E, void* out) {
    const int Ep = router_t_stride(E);
    __shared__ float tile[32][33];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
    const int i_blk = blockIdx.x * 32, e_blk = blockIdx.y * 32;
    for (int r = ty; r < 32; r += 8) {
        const int e = e_blk + r, i = i_blk + tx;
        float v = 0.0f;
        if (e < E) {
            if (ly.router_bf16) {
                v = __uint_as_float((uint32_t)ly.router_bf16[(size_t)e * kH + i] << 16);
            } else {
                const uint32_t word = ly.router_q4.w[(size_t)e * (kH / 8) + (i >> 3)];
                const float q = (float)((word >> (4 * (i & 7))) & 15u);
                const size_t g = (size_t)e * (kH / kGroup) + i / kGroup;
                v = fmaf(q, __uint_as_float((uint32_t)ly.router_q4.s[g] << 16), __uint_as_float((uint32_t)ly.router_q4.b[g] << 16));
            }
        }
        tile[r][tx] = v;
    }
    __syncthreads();
    for (int r = ty; r < 32; r += 8) {
        const int i = i_blk + r, e = e_blk + tx;
        if (e < Ep) {
            const float v = tile[tx][r];  // zero beyond E
            if (ly.router_bf16) reinterpret_cast<uint16_t*>(out)[(size_t)i * Ep + e] = (uint16_t)(__float_as_uint(v) >> 16);
            else reinterpret_cast<float*>(out)[(size_t)i * Ep + e] = v;
        }
    }
}

// ─── host side ──────────────────────────────────────────────────────────────

int decode_init(moe_engine* e) {
    const moe_dims_t& d = e->dims;
    MOE_CUDA(cudaMalloc(&e->dec_sync, 16 * sizeof(unsigned int)));
    MOE_CUDA(cudaMemset(e->dec_sync, 0, 16 * sizeof(unsigned int)));
    e->dec_prof = nullptr;
    MOE_CUDA(cudaMallocHost(&e->stage_host, ((size_t)2 * d.hidden + 16) * sizeof(float)));  // + the error word's landing place
    MOE_CUDA(cudaMalloc(&e->dec_act_ll, kActLLWords * sizeof(unsigned long long)));
    MOE_CUDA(cudaMemset(e->dec_act_ll, 0, kActLLWords * sizeof(unsigned long long)));
    MOE_CUDA(cudaMalloc(&e->dec_hint, 256));  // two counters, a cache line apart
    MOE_CUDA(cudaMemset(e->dec_hint, 0, 256));
    e->dec_hint_base = 0;
    MOE_CUDA(cudaMalloc(&e->dec_h_ll, kH * sizeof(unsigned long long)));
    MOE_CUDA(cudaMemset(e->dec_h_ll, 0, kH * sizeof(unsigned long long)));
    MOE_CUDA(cudaMalloc(&e->dec_acc, 2 * kAccStride * sizeof(long long)));
    MOE_CUDA(cudaMemset(e->dec_acc, 0, 2 * kAccStride * sizeof(long long)));
    e->dec_epoch = 0;
    MOE_CUDA(cudaFuncSetAttribute(decode_stack_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  (int)sizeof(DecodeSmem)));
    MOE_CUDA(cudaFuncSetAttribute(decode_fused_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  (int)sizeof(DecodeSmem3)));
    int per_sm = 0;
    MOE_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_fused_kernel, kDecThreads,
                                                           sizeof(DecodeSmem3)));
    MOE_REQUIRE(per_sm >= 1, "fused decode kernel does not fit on an SM");
    MOE_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_stack_kernel, kDecThreads,
                                                           sizeof(DecodeSmem)));
    MOE_REQUIRE(per_sm >= 1, "decode kernel does not fit on an SM");
    e->dec_grid = e->sm_count;  // one CTA per SM, all co-resident (cooperative launch)
    return slots_decode_init(e);
}

// Turns the per-phase clock stamps on or off (a device buffer of
// layers x kProfPoints stamps, written by CTA 0 of the decode kernel).
int decode_profile_enable(moe_engine* e, bool on) {
    if (on && !e->dec_prof) {
        MOE_CUDA(cudaMalloc(&e->dec_prof, e->layers.size() * kProfPoints * sizeof(long long)));
        MOE_CUDA(cudaMemset(e->dec_prof, 0, e->layers.size() * kProfPoints * sizeof(long long)));
    } else if (!on && e->dec_prof) {
        MOE_CUDA(cudaStreamSynchronize(e->stream));
        cudaFree(e->dec_prof);
        e->dec_prof = nullptr;
    }
    return MOE_OK;
}

int decode_profile_read(moe_engine* e, long long* out, int max_layers, int* points) {
    *points = kProfPoints;
    if (!e->dec_prof) { set_error("decode profiling is off"); return MOE_ERR_STATE; }
    int n = (int)e->layers.size() < max_layers ? (int)e->layers.size() : max_layers;
    MOE_CUDA(cudaMemcpyAsync(out, e->dec_prof, (size_t)n * kProfPoints * sizeof(long long), cudaMemcpyDeviceToHost, e->stream));
    MOE_CUDA(cudaStreamSynchronize(e->stream));
    return MOE_OK;
}

void decode_destroy(moe_engine* e) {
    slots_decode_destroy(e);
    if (e->dec_prof) cudaFree(e->dec_prof);
    cudaFree(e->dec_sync);
    cudaFree(e->dec_act_ll); cudaFree(e->dec_acc); cudaFree(e->dec_hint); cudaFree(e->dec_h_ll);
    if (e->stage_host) cudaFreeHost(e->stage_host);
}

// After a failed device-side wait (and before the epoch counter would wrap) the tagged
// exchange buffer and the router accumulators are in an unknown state: put them back to the state a launch expects.
int decode_reset_after_error(moe_engine* e) {
    MOE_CUDA(cudaMemsetAsync(e->dec_act_ll, 0, kActLLWords * sizeof(unsigned long long), e->stream));
    MOE_CUDA(cudaMemsetAsync(e->dec_acc, 0, 2 * kAccStride * sizeof(long long), e->stream));
    MOE_CUDA(cudaMemsetAsync(e->dec_hint, 0, 256, e->stream));
    MOE_CUDA(cudaMemsetAsync(e->dec_h_ll, 0, kH * sizeof(unsigned long long), e->stream));
    e->dec_hint_base = 0;
    int rc = slots_decode_reset(e);
    if (rc != MOE_OK) return rc;
    MOE_CUDA(cudaStreamSynchronize(e->stream));
    e->dec_epoch = 0;
    return MOE_OK;
}

// Builds the transposed router of a layer: when the router tensor is loaded, and again on first
// decode use if it is missing.
int ensure_router_t(moe_engine* e, int layer) {
    LayerHost& lh = e->layers[layer];
    if (lh.router_t_valid || e->dims.hidden != kH) return MOE_OK;  // other widths never reach the decode kernel
    const int E = e->dims.num_experts;
    const int Ep = (E + 7) & ~7;
    if (!lh.router_t) MOE_CUDA(cudaMalloc(&lh.router_t, (size_t)kH * Ep * sizeof(float)));
    int rc = refresh_layer_table(e);  // lh.dev must point at the current router
    if (rc != MOE_OK) return rc;
    router_transpose_kernel<<<dim3(kH / 32, (Ep + 31) / 32), 256, 0, e->stream>>>(lh.dev, E, lh.router_t);
    MOE_CUDA(cudaGetLastError());
    e->launches++;
    lh.router_t_valid = true;
    e->table_dirty = true;
    return MOE_OK;
}

static int launch_decode_chunk(moe_engine* e, int l0, int l1, const float* h_in, float* h_out,
                               const float* logit_bias, const int32_t* forced_idx, int32_t* out_idx, float* out_w);

// Layers [l0, l1) for one token.  Long stacks run as several launches of at most kMaxDecLayers
// layers; a later launch reads its input from h_out (a CTA writes its part of the output
// only after every CTA has staged the input, so the two may be the same buffer).
int launch_decode(moe_engine* e, int l0, int l1, const float* h_in, float* h_out,
                  const float* logit_bias, const int32_t* forced_idx, int32_t* out_idx, float* out_w, bool pdl) {
    MOE_REQUIRE(l0 >= 0 && l1 > l0 && l1 <= (int)e->layers.size(), "decode: bad layer range [%d, %d)", l0, l1);
    for (int a = l0; a < l1; a += kMaxDecLayers) {
        const int b = a + kMaxDecLayers < l1 ? a + kMaxDecLayers : l1;
        // the slot-grouped kernel where the device and the model shape allow it, the grid-wide kernel otherwise
        int rc = slots_decode_usable(e, a, b)
                     ? launch_decode_slots(e, a, b, a == l0 ? h_in : h_out, h_out, logit_bias, forced_idx, out_idx, out_w, pdl && a == l0)
                     : launch_decode_chunk(e, a, b, a == l0 ? h_in : h_out, h_out, logit_bias, forced_idx, out_idx, out_w);
        if (rc != MOE_OK) return rc;
    }
    return MOE_OK;
}

static int launch_decode_chunk(moe_engine* e, int l0, int l1, const float* h_in, float* h_out,
                               const float* logit_bias, const int32_t* forced_idx, int32_t* out_idx, float* out_w) {
    const moe_dims_t& d = e->dims;
    MOE_REQUIRE(d.hidden == kH && d.inter == kI && d.shared_inter == kI,
                "decode path is built for hidden=%d, inter=shared_inter=%d (got %d/%d/%d)", kH, kI,
                d.hidden, d.inter, d.shared_inter);
    MOE_REQUIRE(d.num_experts <= kMaxE, "decode path supports at most %d experts", kMaxE);
    const int G = e->dec_grid;
    auto cdiv = [](int a, int b) { return (a + b - 1) / b; };
    // every CTA's weight slice must fit its shared-memory staging area
    MOE_REQUIRE(cdiv((d.top_k + 1) * kI, G) <= kMaxB3Items && cdiv(kH, G) <= kMaxCRows,
                "decode kernel needs at least 147 SMs for these dimensions (device has %d)", G);
    MOE_REQUIRE(l0 >= 0 && l1 > l0 && l1 <= (int)e->layers.size(), "decode: bad layer range [%d, %d)", l0, l1);
    MOE_REQUIRE(l1 - l0 <= kMaxDecLayers, "decode: at most %d layers per launch", kMaxDecLayers);
    MOE_REQUIRE(G < 256, "decode kernel counts CTAs in 8 bits (grid of %d)", G);
    MOE_REQUIRE((((uintptr_t)h_in) & 15) == 0 && (((uintptr_t)h_out) & 15) == 0, "decode: h must be 16-byte aligned");
    for (int l = l0; l < l1; ++l) {
        int rc = check_layer_ready(e, l);
        if (rc != MOE_OK) return rc;
        rc = ensure_router_t(e, l);
        if (rc != MOE_OK) return rc;
    }
    int rc = refresh_layer_table(e);
    if (rc != MOE_OK) return rc;
    Decode3Params p{};
    p.layers = e->layers_dev;
    p.l0 = l0; p.l1 = l1;
    p.h_in = h_in; p.h_out = h_out;
    if (e->dec_epoch > 0xFFFF0000u - (unsigned int)(l1 - l0)) {
        rc = decode_reset_after_error(e);  // tags must never repeat: start the epochs over on a cleared buffer
        if (rc != MOE_OK) return rc;
    }
    p.acc = e->dec_acc; p.act_ll = e->dec_act_ll;
    p.epoch_base = e->dec_epoch;
    e->dec_epoch += (unsigned int)(l1 - l0);
    p.hint = e->dec_hint;
    p.hint2 = e->dec_hint + 16;  // 128 bytes further
    p.h_ll = e->dec_h_ll;
    p.hint_base = e->dec_hint_base;
    // the accumulators are never cleared by the kernel (readers subtract what they saw before): start from zero
    MOE_CUDA(cudaMemsetAsync(e->dec_acc, 0, 2 * kAccStride * sizeof(long long), e->stream));
    e->dec_hint_base += (unsigned long long)G * (unsigned long long)(l1 - l0);
    p.logit_bias = logit_bias; p.forced_idx = forced_idx;
    p.out_idx = out_idx; p.out_w = out_w;
    p.err = e->dec_sync + 2;
    p.prof = e->dec_prof;
    p.E = d.num_experts; p.K = d.top_k;
    p.lay = e->lay;
    void* args[] = {&p};
    MOE_CUDA(cudaLaunchCooperativeKernel((const void*)decode_fused_kernel, dim3(e->dec_grid), dim3(kDecThreads),
                                         args, sizeof(DecodeSmem3), e->stream));
    e->launches++;
    return MOE_OK;
}

// ─── decode of one block for callers that must not allocate ─────────────────
//
// Some hosts cannot let a library call cudaMalloc: a serving process whose device
// memory is carved up once at start-up and owned by its own pool, a plug-in
// running inside such a process, or a latency-critical loop in which cudaMalloc /
// cudaFree (which synchronise the device and can fail when memory is fragmented)
// are banned after initialisation.  For them the decode kernel's work areas (the
// router logits, the SwiGLU outputs, the grid-barrier words) live in the
// fixed array below instead of in engine-owned
// allocations.  The array is part of the library image: every GPU that loads
// the library holds these 40 KiB until the process exits.
constexpr size_t kNaSync = 0;        // 16 barrier / error words
constexpr size_t kNaLayer = 256;     // one LayerDev
constexpr size_t kNaMisc = 512;      // float[16]
constexpr size_t kNaLogits = 1024;   // float[kMaxE + 4]
constexpr size_t kNaAct = 3328;      // float[(kMaxK + 1) * kI]
constexpr size_t kNaH0 = kNaAct + sizeof(float) * (kMaxK + 1) * kI;
constexpr size_t kNaH1 = kNaH0 + sizeof(float) * kH;
constexpr size_t kNoAllocScratchBytes = 40960;
static_assert(kNaH1 + sizeof(float) * kH <= kNoAllocScratchBytes, "scratch layout exceeds the array");
static_assert(kNaLogits + sizeof(float) * (kMaxE + 4) <= kNaAct && sizeof(LayerDev) <= kNaMisc - kNaLayer, "scratch layout overlaps");
static_assert(kNaAct % 256 == 0 && kNaH0 % 256 == 0 && kNaH1 % 256 == 0, "scratch parts stay 256-byte aligned");

static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];

constexpr int kNaMaxDevices = 64;
// In host code `g_noalloc_scratch` is only a handle for the runtime, not an address a
// kernel can use; the device address is looked up once per device and kept here.
static unsigned char* g_noalloc_dev_ptr[kNaMaxDevices] = {};
static int g_noalloc_grid[kNaMaxDevices] = {};
static std::mutex g_noalloc_mutex;  // two host threads may make a device's first call at the same time

}  // namespace moe

using namespace moe;

extern "C" int moe_layer_decode_noalloc(const moe_dims_t* dims, int device, const moe_layer_ptrs_t* lp,
                                        const float* h_in_dev, float* h_out_dev, int32_t* out_idx_dev,
                                        float* out_w_dev, void* cuda_stream, int wait) {
    MOE_REQUIRE(dims && lp && h_in_dev && h_out_dev, "null argument");
    const moe_dims_t& d = *dims;
    MOE_REQUIRE(d.hidden == kH && d.inter == kI && d.shared_inter == kI && d.group == kGroup,
                "no-alloc decode is built for hidden=%d, inter=shared_inter=%d, group=%d", kH, kI, kGroup);
    MOE_REQUIRE(d.top_k >= 1 && d.top_k <= kMaxK && d.top_k <= d.num_experts, "num_active_experts (%d) must be in 1..%d",
                d.top_k, kMaxK);
    // the fixed scratch array holds the logits of at most kMaxE experts
    MOE_REQUIRE(d.num_experts >= 1 && d.num_experts <= kMaxE,
                "num_experts (%d) exceeds the static scratch of the no-alloc entry point (at most %d experts)",
                d.num_experts, kMaxE);
    MOE_REQUIRE(lp->experts && lp->post_norm && lp->shared && lp->sgate_w && lp->sgate_s && lp->sgate_b &&
                    (lp->router_bf16 || (lp->router_w && lp->router_s && lp->router_b)),
                "no-alloc decode: a tensor pointer is missing");
    MOE_REQUIRE(device >= 0 && device < kNaMaxDevices, "device %d out of range", device);
    MOE_REQUIRE((((uintptr_t)h_in_dev) & 15) == 0 && (((uintptr_t)h_out_dev) & 15) == 0, "h must be 16-byte aligned");
    int prev = 0;
    MOE_CUDA(cudaGetDevice(&prev));
    MOE_CUDA(cudaSetDevice(device));
    int rc = MOE_OK;
    cudaStream_t st = (cudaStream_t)cuda_stream;
    do {
        unsigned char* base = nullptr;
        int G = 0;
        {
            std::lock_guard<std::mutex> lock(g_noalloc_mutex);  // held for the set-up only
            if (!g_noalloc_dev_ptr[device]) {
                // one-time set-up on this device (with the device current): device address of the array
                unsigned char* ptr = nullptr;
                cudaError_t ce = cudaGetSymbolAddress((void**)&ptr, g_noalloc_scratch);
                if (ce != cudaSuccess || !ptr) { rc = cuda_fail(ce, "cudaGetSymbolAddress(g_noalloc_scratch)", __FILE__, __LINE__); break; }
                ce = cudaFuncSetAttribute(decode_stack_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(DecodeSmem));
                int sms = 0;
                if (ce == cudaSuccess) ce = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
                if (ce != cudaSuccess) { rc = cuda_fail(ce, "no-alloc decode set-up", __FILE__, __LINE__); break; }
                g_noalloc_grid[device] = sms;
                g_noalloc_dev_ptr[device] = ptr;
            }
            base = g_noalloc_dev_ptr[device];
            G = g_noalloc_grid[device];
        }
        auto cdiv = [](int a, int b) { return (a + b - 1) / b; };
        if (!(cdiv(d.num_experts, G) <= kMaxRouterRows && cdiv(kI, G) <= kMaxSharedRows &&
              cdiv(d.top_k * kI, G) <= kMaxBItems && cdiv(kH, G) <= kMaxCRows)) {
            set_error("decode kernel needs at least 147 SMs for these dimensions (device has %d)", G);
            rc = MOE_ERR_INVALID;
            break;
        }
        DecodeParams p{};
        p.layers = nullptr;  // the layer travels inside the kernel parameters: no host copy is queued on the stream
        LayerDev& ld = p.one;
        ld.experts = (const uint8_t*)lp->experts;
        ld.post_norm = (const uint16_t*)lp->post_norm;
        ld.router_bf16 = (const uint16_t*)lp->router_bf16;
        ld.router_q4.w = (const uint32_t*)lp->router_w;
        ld.router_q4.s = (const uint16_t*)lp->router_s;
        ld.router_q4.b = (const uint16_t*)lp->router_b;
        ld.shared = (const uint8_t*)lp->shared;
        ld.sgate.w = (const uint32_t*)lp->sgate_w;
        ld.sgate.s = (const uint16_t*)lp->sgate_s;
        ld.sgate.b = (const uint16_t*)lp->sgate_b;
        // the array keeps whatever the previous call left: the barrier and error words must start at zero
        cudaError_t ce = cudaMemsetAsync(base + kNaSync, 0, 64, st);
        if (ce != cudaSuccess) { rc = cuda_fail(ce, "no-alloc decode: scratch set-up", __FILE__, __LINE__); break; }
        p.l0 = 0; p.l1 = 1;
        p.h_in = h_in_dev; p.h_out = h_out_dev;
        p.h_buf0 = reinterpret_cast<float*>(base + kNaH0);
        p.h_buf1 = reinterpret_cast<float*>(base + kNaH1);
        p.logits = reinterpret_cast<float*>(base + kNaLogits);
        p.act = reinterpret_cast<float*>(base + kNaAct);
        p.misc = reinterpret_cast<float*>(base + kNaMisc);
        p.logit_bias = nullptr; p.forced_idx = nullptr;
        p.out_idx = out_idx_dev; p.out_w = out_w_dev;
        p.sync = reinterpret_cast<unsigned int*>(base + kNaSync);
        p.prof = nullptr;
        p.E = d.num_experts; p.K = d.top_k;
        if (moe_expert_layout(d.hidden, d.inter, d.group, &p.lay) != MOE_OK) { rc = MOE_ERR_INVALID; break; }
        void* args[] = {&p};
        ce = cudaLaunchCooperativeKernel((const void*)decode_stack_kernel, dim3(G), dim3(kDecThreads), args,
                                         sizeof(DecodeSmem), st);
        if (ce != cudaSuccess) { rc = cuda_fail(ce, "no-alloc decode launch", __FILE__, __LINE__); break; }
        if (wait) {
            unsigned int flag = 0;
            ce = cudaMemcpyAsync(&flag, base + kNaSync + 8, sizeof(flag), cudaMemcpyDeviceToHost, st);
            if (ce == cudaSuccess) ce = cudaStreamSynchronize(st);
            if (ce != cudaSuccess) { rc = cuda_fail(ce, "no-alloc decode wait", __FILE__, __LINE__); break; }
            if (flag) {
                set_error("a bounded device-side wait gave up (code %u); the result of this call is invalid", flag);
                rc = MOE_ERR_DEVICE_WAIT;
            }
        }
    } while (0);
    cudaSetDevice(prev);
    return rc;
}

extern "C" int moe_layer_decode_noalloc_status(int device, void* cuda_stream, unsigned int* code) {
    MOE_REQUIRE(code, "null argument");
    MOE_REQUIRE(device >= 0 && device < kNaMaxDevices, "device %d out of range", device);
    *code = 0;
    unsigned char* base = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_noalloc_mutex);
        base = g_noalloc_dev_ptr[device];
    }
    if (!base) return MOE_OK;  // no call has run on this device yet
    int prev = 0;
    MOE_CUDA(cudaGetDevice(&prev));
    MOE_CUDA(cudaSetDevice(device));
    cudaStream_t st = (cudaStream_t)cuda_stream;
    unsigned int flag = 0;
    cudaError_t ce = cudaMemcpyAsync(&flag, base + kNaSync + 8, sizeof(flag), cudaMemcpyDeviceToHost, st);
    if (ce == cudaSuccess) ce = cudaStreamSynchronize(st);
    cudaSetDevice(prev);
    if (ce != cudaSuccess) return cuda_fail(ce, "no-alloc decode status", __FILE__, __LINE__);
    *code = flag;
    if (flag) {
        set_error("a bounded device-side wait gave up (code %u); the result of the last no-alloc call is invalid", flag);
        return MOE_ERR_DEVICE_WAIT;
    }
    return MOE_OK;
}
