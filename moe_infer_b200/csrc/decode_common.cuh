// Device helpers shared by the decode kernels (decode.cu, decode_slots.cu): model
// constants, 16-byte asynchronous copies, the integer dot product of staged 4-bit rows,
// and the on-device routing (softmax / top-k / renormalise of the reference's
// route_experts, src/engine/qwen35_moe/cpu.rs:78-85).
#pragma once
#include "q4dot.cuh"
#include "stage.cuh"

namespace moe {

constexpr int kH = 2048;        // hidden (both reference models)
constexpr int kI = 512;         // moe_intermediate_size == shared_expert_intermediate_size
constexpr int kDecWarps = 16;
constexpr int kDecThreads = kDecWarps * 32;
constexpr int kChH = kH / 32;   // 64 chunks (128-bit loads) per hidden row
constexpr int kChI = kI / 32;   // 16 chunks per intermediate row
constexpr int kMaxE = 512;      // routing supports up to 512 experts

// ─── weight prefetch with per-thread 16-byte asynchronous copies ─────────────
// Every thread of the CTA copies pieces p = tid, tid + 512, ... of a slice;
// completion is tracked with cp.async groups (one group per slice), then a CTA
// barrier makes the bytes visible to every warp.
__device__ __forceinline__ void cp16(void* dst_smem, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst_smem)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void copy_flat(void* dst, const void* src, int pieces, int tid) {
    for (int q = tid; q < pieces; q += kDecThreads)
        cp16(reinterpret_cast<uint8_t*>(dst) + (size_t)q * 16, reinterpret_cast<const uint8_t*>(src) + (size_t)q * 16);
}

// swiglu_fused (reference src/math_util.rs:254-259): silu(gate) * up.
__device__ __forceinline__ float swiglu(float g, float u) { return g / (1.0f + expf(-g)) * u; }

// Dot products of NR 4-bit rows of length kH with the staged x (integer path).
template <int NR, class SM>
__device__ __forceinline__ void rows_dot_q(const SM* sm, const uint4* const (&w)[NR],
                                           const uint16_t* const (&s)[NR], const uint16_t* const (&b)[NR],
                                           float (&out)[NR], int lane) {
#pragma unroll
    for (int r = 0; r < NR; ++r) out[r] = 0.0f;
#pragma unroll
    for (int it = 0; it < 2; ++it) {
        const int c = lane + 32 * it;
        uint4 xe[3], xo[3];
#pragma unroll
        for (int p = 0; p < 3; ++p) {
            xe[p] = sm->xq[(p * 2 + 0) * kChH + c];
            xo[p] = sm->xq[(p * 2 + 1) * kChH + c];
        }
        const float sx = sm->sumx[c], dl = sm->xdl[c];
#pragma unroll
        for (int r = 0; r < NR; ++r) {
            const float sc = bf16_bits_to_f32(s[r][c >> 1]), bi = bf16_bits_to_f32(b[r][c >> 1]);
            out[r] += fmaf(sc * dl, dot32_int(w[r][c], xe, xo), bi * sx);
        }
    }
#pragma unroll
    for (int r = 0; r < NR; ++r) out[r] = warp_sum(out[r]);
}

// route_cta rearranged for latency, in two halves.  route_select picks the K experts from the raw logits
// (softmax is monotonic, so the K largest logits are the K largest probabilities) and is all that the
// weight copies wait for; route_weights forms the probabilities of the chosen experts afterwards, while the
// copies are in flight.  Ranks are found with warp votes instead of per-thread loops: the rank of a value
// among 32 is the population count of one ballot.  The candidate threshold comes from the maxima of
// 16-expert groups (32 of them, one per lane): warp w ranks group maxima 2w and 2w+1, and whichever has K-1
// maxima ahead of it is the threshold.  Values: p = exp(v - max) * (1 / sum), weights p_k * (1 / sum_k p_k),
// as route_cta; ties between equal logits go to the lower index.  (Two different logits whose probabilities
// round to the same float are ordered by logit here and by index in the reference: a difference below the
// rounding of the logits themselves.)
template <class SM>
__device__ __forceinline__ void route_select(SM* sm, float v, const int32_t* forced, int E, int K, unsigned int* err) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    float m = v;
    m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
    m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
    m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 4));
    m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 8));
    if ((lane & 15) == 0) sm->hmax[tid >> 4] = m;
    m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 16));
    if (lane == 0) sm->red[warp] = m;  // per-warp maxima: kept for route_weights
    if (tid == 0) { sm->ncand = 0; sm->tau = -INFINITY; }
    // Default choice: experts 0..K-1.  It stands only where the ranking below writes nothing, i.e. when logits are
    // NaN (comparisons with NaN are false, so fewer than K candidates exist): the reference's heap keeps its first
    // K entries in that case (src/math_util.rs:89-99), and an expert index must never be left undefined.
    if (tid < K) { sm->topi[tid] = tid; sm->topp[tid] = v; }
    if (forced) sm->prob[tid] = v;
    __syncthreads();
    if (forced) {
        if (tid < K) {
            int fe = forced[tid];
            if ((unsigned)fe >= (unsigned)E) { atomicExch(err, 10u); fe = 0; }  // reported, never dereferenced
            sm->topi[tid] = fe;
            sm->topp[tid] = sm->prob[fe];
        }
        __syncthreads();
        return;
    }
    {
        // group maxima; -inf for groups beyond E (then everything is a candidate)
        const float mine = (lane * 16 < E) ? sm->hmax[lane] : -INFINITY;
#pragma unroll
        for (int t = 0; t < 2; ++t) {
            const int iu = 2 * warp + t;
            const float u = __shfl_sync(0xffffffffu, mine, iu);
            const int ahead = __popc(__ballot_sync(0xffffffffu, (mine > u) || (mine == u && lane < iu)));
            // exactly one group has K-1 ahead of it; lowered by a hair (harmless: it only adds candidates)
            if (ahead == K - 1 && lane == 0) sm->tau = u - 1e-6f * fmaxf(1.0f, fabsf(u));
        }
    }
    __syncthreads();
    {
        const bool is_c = tid < E && v >= sm->tau;
        const unsigned bal = __ballot_sync(0xffffffffu, is_c);
        int base = 0;
        if (lane == 0 && bal) base = atomicAdd(&sm->ncand, __popc(bal));
        base = __shfl_sync(0xffffffffu, base, 0);
        if (is_c) {
            const int slot = base + __popc(bal & ((1u << lane) - 1u));
            sm->cand_p[slot] = v;
            sm->cand_i[slot] = tid;
        }
    }
    __syncthreads();
    {
        // warp w ranks candidates w, w + 16, ...: every lane compares one other candidate per vote
        const int nc = sm->ncand;
        for (int c = warp; c < nc; c += kDecWarps) {
            const float cp = sm->cand_p[c];
            const int ci = sm->cand_i[c];
            int rank = 0;
            for (int j0 = 0; j0 < nc; j0 += 32) {
                const int j = j0 + lane;
                bool beats = false;
                if (j < nc) {
                    const float q = sm->cand_p[j];
                    beats = (q > cp) || (q == cp && sm->cand_i[j] < ci);
                }
                rank += __popc(__ballot_sync(0xffffffffu, beats));
            }
            if (rank < K && lane == 0) { sm->topi[rank] = ci; sm->topp[rank] = cp; }  // topp: the logit, for now
        }
    }
    __syncthreads();
}

// Probabilities and renormalised weights of the experts route_select chose (their logits are in topp).
template <class SM>
__device__ __forceinline__ void route_weights(SM* sm, float v, int E, int K) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    float mx = sm->red[0];
#pragma unroll
    for (int i = 1; i < kDecWarps; ++i) mx = fmaxf(mx, sm->red[i]);
    const float ex = (tid < E) ? expf(v - mx) : 0.0f;
    const float ws = warp_sum(ex);
    if (lane == 0) sm->red2[warp] = ws;
    __syncthreads();
    if (warp == 0) {
        float sum = 0.0f;
#pragma unroll
        for (int i = 0; i < kDecWarps; ++i) sum += sm->red2[i];
        const float inv = 1.0f / sum;
        // same expression as the owning thread's exp(v - max) * inv
        const float pk = (lane < K) ? expf(sm->topp[lane] - mx) * inv : 0.0f;
        // normalize_weights: divide by the sum of the K selected probabilities, added in order
        float s = 0.0f;
        for (int k = 0; k < K; ++k) s += __shfl_sync(0xffffffffu, pk, k);
        const float invs = s > 0.0f ? 1.0f / s : 1.0f;
        if (lane < K) sm->topw[lane] = pk * invs;
    }
    __syncthreads();
}


// Entry points of the slot-grouped decode kernel (decode_slots.cu).
int slots_decode_init(moe_engine* e);
void slots_decode_destroy(moe_engine* e);
bool slots_decode_usable(const moe_engine* e, int l0, int l1);
int slots_decode_reset(moe_engine* e);
int slots_decode_prefetch_stats(moe_engine* e, double* checks, double* hits);
int launch_decode_slots(moe_engine* e, int l0, int l1, const float* h_in, float* h_out, const float* logit_bias,
                        const int32_t* forced_idx, int32_t* out_idx, float* out_w, bool pdl = false);

}  // namespace moe
