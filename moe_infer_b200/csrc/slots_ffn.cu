// Expert FFN of a small batch, one (token, expert) slot at a time.
//
// The grouped GEMM (grouped.cu) spends the same time on an expert's weight tiles whether 1 or 256 of the batch's tokens
// chose that expert: its producers dequantise every tile to bf16 for the tensor cores.  With a few tokens per expert
// (batched decode: 64 tokens over 256 experts) that work is wasted, and the matvec formulation of the decode path is
// the cheaper one: integer dot products on the packed nibbles, weights read once from HBM per expert and again from L2
// for the expert's other tokens (the slots are sorted by expert, so they run back to back).
//
// Replaces, for n <= kSlotPathMaxTokens tokens, the two grouped GEMMs of forward_hidden_batched's MoE half (reference
// src/engine/qwen35_moe/batched.rs:334-447: per (token, expert) gate / up matvecs, SwiGLU, down matvec) between the
// shared routing front end (prep, router, route, plan, scatter) and the combine kernel:
//   slot_gateup_kernel   act[slot][r] = silu(Wg[r] . x) * (Wu[r] . x), x = rmsnorm(h[token]) * post_norm, f32
//   slot_down_kernel     o[slot][r]   = Wd[r] . act[slot], written as bf16 rows for batch_combine_kernel
// Arithmetic as in the decode kernel (q4dot.cuh): activations as three signed-byte digit planes per 32-element chunk,
// dp4a sums that are exact integers.
#include "q4dot.cuh"
#include "stage.cuh"
#include <cuda_bf16.h>

namespace moe {

constexpr int kSfH = 2048, kSfI = 512;
constexpr int kSfWarps = 8, kSfThreads = kSfWarps * 32;
constexpr int kSfGuCtas = 4;                       // CTAs per slot, gate/up: 128 row pairs each
constexpr int kSfGuRows = kSfI / kSfGuCtas;        // row pairs per CTA
constexpr int kSfDnCtas = 4;                       // CTAs per slot, down: 512 rows each
constexpr int kSfDnRows = kSfH / kSfDnCtas;
static_assert(kSfGuRows % (kSfWarps * 2) == 0 && kSfDnRows % (kSfWarps * 4 * 2) == 0, "work split below assumes these shapes");

struct SlotFfnParams {
    const uint8_t* experts;       // E packed experts of this layer
    const uint8_t* shared;        // shared expert, same layout
    moe_expert_layout_t lay;
    int E;
    const float* h_in;            // [n, H]
    const uint16_t* post_norm;    // bf16 [H]
    const int32_t* slot_token;    // token of every slot
    const int32_t* slot_expert;   // expert of every slot (E: the shared expert)
    float* act;                   // [slots, I]
    __nv_bfloat16* o;             // [slots, H]
    unsigned int* err;
};

__device__ __forceinline__ const uint8_t* slot_weights(const SlotFfnParams& p, int e) {
    return e >= p.E ? p.shared : p.experts + (size_t)e * p.lay.expert_size;
}

// ─── gate / up + SwiGLU ─────────────────────────────────────────────────────
// grid (kSfGuCtas, slots).  The CTA stages its token's h (bulk copy), norms it, writes the digit planes; every lane
// keeps the planes of its own 64-column group in registers; a warp then takes two row pairs (gate row r and up row r)
// at a time: eight 128-bit loads per lane in flight.
__global__ void __launch_bounds__(kSfThreads, 2) slot_gateup_kernel(SlotFfnParams p) {
    constexpr int nch = kSfH / 32;
    __shared__ __align__(128) float raw[kSfH];
    __shared__ __align__(16) uint4 xq[6 * nch];
    __shared__ float xdl[nch];
    __shared__ float sumx[nch];
    __shared__ float red[kSfWarps];
    __shared__ uint64_t bar;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int slot = blockIdx.y;
    const int token = p.slot_token[slot], expert = p.slot_expert[slot];
    if (tid == 0) {
        mbar_init(&bar, 1);
        mbar_fence_init();
    }
    __syncthreads();
    if (tid == 0) {
        mbar_expect_tx(&bar, kSfH * 4u);
        bulk_g2s(raw, p.h_in + (size_t)token * kSfH, kSfH * 4u, &bar);
    }
    // this warp's first two row pairs do not depend on x: requested before it is waited for
    const uint8_t* ex = slot_weights(p, expert);
    const uint4* gw = reinterpret_cast<const uint4*>(ex + p.lay.gate_w);
    const uint4* uw = reinterpret_cast<const uint4*>(ex + p.lay.up_w);
    const uint16_t* gs = reinterpret_cast<const uint16_t*>(ex + p.lay.gate_s);
    const uint16_t* gb = reinterpret_cast<const uint16_t*>(ex + p.lay.gate_b);
    const uint16_t* us = reinterpret_cast<const uint16_t*>(ex + p.lay.up_s);
    const uint16_t* ub = reinterpret_cast<const uint16_t*>(ex + p.lay.up_b);
    constexpr int kU = 2;  // row pairs per batch
    const int row_first = blockIdx.x * kSfGuRows + warp * kU;
    uint4 qg[kU][2], qu[kU][2];
    uint16_t sg[kU], bg[kU], su[kU], bu[kU];
    auto load_batch = [&](int r0) {
#pragma unroll
        for (int u = 0; u < kU; ++u) {
            const size_t r = (size_t)(r0 + u);
            qg[u][0] = ld_stream_u4(gw + r * (kSfH / 32) + 2 * lane);
            qg[u][1] = ld_stream_u4(gw + r * (kSfH / 32) + 2 * lane + 1);
            qu[u][0] = ld_stream_u4(uw + r * (kSfH / 32) + 2 * lane);
            qu[u][1] = ld_stream_u4(uw + r * (kSfH / 32) + 2 * lane + 1);
            sg[u] = __ldg(gs + r * (kSfH / kGroup) + lane);
            bg[u] = __ldg(gb + r * (kSfH / kGroup) + lane);
            su[u] = __ldg(us + r * (kSfH / kGroup) + lane);
            bu[u] = __ldg(ub + r * (kSfH / kGroup) + lane);
        }
    };
    load_batch(row_first);
    const int ok = __syncthreads_and(mbar_wait(&bar, 0) ? 1 : 0);
    if (!ok) {
        if (tid == 0) atomicExch(p.err, 1u);
        return;
    }
    // x = rmsnorm(h) * post_norm (rms_norm_bf16, reference src/math_util.rs:282-288)
    float ss = 0.0f;
#pragma unroll
    for (int it = 0; it < kSfH / 4 / kSfThreads; ++it) {
        const float4 v = reinterpret_cast<const float4*>(raw)[tid + it * kSfThreads];
        ss = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, ss))));
    }
    ss = warp_sum(ss);
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    float tot = 0.0f;
#pragma unroll
    for (int i = 0; i < kSfWarps; ++i) tot += red[i];
    const float inv_rms = 1.0f / sqrtf(tot / (float)kSfH + 1e-6f);
#pragma unroll
    for (int it = 0; it < kSfH / 4 / kSfThreads; ++it) {
        const int f = tid + it * kSfThreads;  // float4 index: chunk f >> 3, part f & 7
        float4 v = reinterpret_cast<const float4*>(raw)[f];
        const uint2 wb = __ldg(reinterpret_cast<const uint2*>(p.post_norm) + f);
        v.x = v.x * inv_rms * __uint_as_float(wb.x << 16);
        v.y = v.y * inv_rms * __uint_as_float(wb.x & 0xFFFF0000u);
        v.z = v.z * inv_rms * __uint_as_float(wb.y << 16);
        v.w = v.w * inv_rms * __uint_as_float(wb.y & 0xFFFF0000u);
        stage_digits(xq, xdl, nch, f >> 3, f & 7, v);
        float sv = (v.x + v.y) + (v.z + v.w);
        sv += __shfl_xor_sync(0xffffffffu, sv, 1);
        sv += __shfl_xor_sync(0xffffffffu, sv, 2);
        sv += __shfl_xor_sync(0xffffffffu, sv, 4);
        if ((f & 7) == 0) sumx[f >> 3] = sv;
    }
    __syncthreads();
    uint4 xe[2][3], xo[2][3];
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int pl = 0; pl < 3; ++pl) {
            xe[h][pl] = xq[(pl * 2 + 0) * nch + 2 * lane + h];
            xo[h][pl] = xq[(pl * 2 + 1) * nch + 2 * lane + h];
        }
    const float dl0 = xdl[2 * lane], dl1 = xdl[2 * lane + 1];
    const float sx = sumx[2 * lane] + sumx[2 * lane + 1];

    const int row_end = (blockIdx.x + 1) * kSfGuRows;
    for (int r0 = row_first; r0 < row_end;) {
        float ag[kU], au[kU];
#pragma unroll
        for (int u = 0; u < kU; ++u) {
            const float dg = fmaf(dl0, dot32_regs(qg[u][0], xe[0], xo[0]), dl1 * dot32_regs(qg[u][1], xe[1], xo[1]));
            const float du = fmaf(dl0, dot32_regs(qu[u][0], xe[0], xo[0]), dl1 * dot32_regs(qu[u][1], xe[1], xo[1]));
            ag[u] = fmaf(bf16_bits_to_f32(sg[u]), dg, bf16_bits_to_f32(bg[u]) * sx);
            au[u] = fmaf(bf16_bits_to_f32(su[u]), du, bf16_bits_to_f32(bu[u]) * sx);
        }
        const int done = r0;
        r0 += kSfWarps * kU;
        if (r0 < row_end) load_batch(r0);  // the next batch is on its way while this one is reduced
#pragma unroll
        for (int u = 0; u < kU; ++u) {
            const float g = warp_sum(ag[u]), up = warp_sum(au[u]);
            if (lane == 0) p.act[(size_t)slot * kSfI + done + u] = g / (1.0f + expf(-g)) * up;  // swiglu_fused (math_util.rs:254-259)
        }
    }
}

// ─── down ───────────────────────────────────────────────────────────────────
// grid (kSfDnCtas, slots).  A down row has 512 columns = 8 groups: eight lanes cover a row, a warp four rows at a time,
// two such sets in flight.  The slot's 512 SwiGLU outputs are staged as digit planes like x above.
__global__ void __launch_bounds__(kSfThreads, 2) slot_down_kernel(SlotFfnParams p) {
    constexpr int nch = kSfI / 32;
    __shared__ __align__(16) uint4 aq[6 * nch];
    __shared__ float adl[nch];
    __shared__ float suma[nch];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int slot = blockIdx.y;
    const int expert = p.slot_expert[slot];
    const uint8_t* ex = slot_weights(p, expert);
    const uint4* dw = reinterpret_cast<const uint4*>(ex + p.lay.down_w);
    const uint16_t* ds = reinterpret_cast<const uint16_t*>(ex + p.lay.down_s);
    const uint16_t* db = reinterpret_cast<const uint16_t*>(ex + p.lay.down_b);
    const int sub = lane >> 3, grp = lane & 7;  // row of the warp's four, 64-column group of the row
    constexpr int kU = 2;
    const int row_first = blockIdx.x * kSfDnRows + warp * 4 * kU;
    uint4 q[kU][2];
    uint16_t sc[kU], bi[kU];
    auto load_batch = [&](int r0) {
#pragma unroll
        for (int u = 0; u < kU; ++u) {
            const size_t r = (size_t)(r0 + u * 4 + sub);
            q[u][0] = ld_stream_u4(dw + r * (kSfI / 32) + 2 * grp);
            q[u][1] = ld_stream_u4(dw + r * (kSfI / 32) + 2 * grp + 1);
            sc[u] = __ldg(ds + r * (kSfI / kGroup) + grp);
            bi[u] = __ldg(db + r * (kSfI / kGroup) + grp);
        }
    };
    load_batch(row_first);  // weights: independent of the activations staged below
    if (tid < kSfI / 4) {   // 128 threads: one float4 each, eight consecutive lanes per chunk
        const float4 v = *reinterpret_cast<const float4*>(p.act + (size_t)slot * kSfI + tid * 4);
        stage_digits(aq, adl, nch, tid >> 3, tid & 7, v);
        float sv = (v.x + v.y) + (v.z + v.w);
        sv += __shfl_xor_sync(0xffffffffu, sv, 1);
        sv += __shfl_xor_sync(0xffffffffu, sv, 2);
        sv += __shfl_xor_sync(0xffffffffu, sv, 4);
        if ((tid & 7) == 0) suma[tid >> 3] = sv;
    }
    __syncthreads();
    uint4 xe[2][3], xo[2][3];
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int pl = 0; pl < 3; ++pl) {
            xe[h][pl] = aq[(pl * 2 + 0) * nch + 2 * grp + h];
            xo[h][pl] = aq[(pl * 2 + 1) * nch + 2 * grp + h];
        }
    const float dl0 = adl[2 * grp], dl1 = adl[2 * grp + 1];
    const float sx = suma[2 * grp] + suma[2 * grp + 1];

    const int row_end = (blockIdx.x + 1) * kSfDnRows;
    for (int r0 = row_first; r0 < row_end;) {
        float acc[kU];
#pragma unroll
        for (int u = 0; u < kU; ++u) {
            const float d = fmaf(dl0, dot32_regs(q[u][0], xe[0], xo[0]), dl1 * dot32_regs(q[u][1], xe[1], xo[1]));
            acc[u] = fmaf(bf16_bits_to_f32(sc[u]), d, bf16_bits_to_f32(bi[u]) * sx);
        }
        const int done = r0;
        r0 += kSfWarps * 4 * kU;
        if (r0 < row_end) load_batch(r0);
#pragma unroll
        for (int u = 0; u < kU; ++u) {
            float a = acc[u];  // the eight lanes of a row
            a += __shfl_xor_sync(0xffffffffu, a, 1);
            a += __shfl_xor_sync(0xffffffffu, a, 2);
            a += __shfl_xor_sync(0xffffffffu, a, 4);
            if (grp == 0) p.o[(size_t)slot * kSfH + done + u * 4 + sub] = __float2bfloat16_rn(a);
        }
    }
}

// Both kernels over `slots` slots (every token's K routed slots and its shared-expert slot).
int launch_slot_ffn(moe_engine* e, const LayerDev& ly, const float* h_in, int slots, const int32_t* slot_token,
                    const int32_t* slot_expert, float* act, void* o) {
    MOE_REQUIRE(e->dims.hidden == kSfH && e->dims.inter == kSfI && e->dims.shared_inter == kSfI,
                "the slot-wise expert FFN is built for hidden=%d, inter=shared_inter=%d", kSfH, kSfI);
    MOE_REQUIRE(slots > 0 && slots <= 65535, "slot count %d outside 1..65535", slots);
    SlotFfnParams p{};
    p.experts = ly.experts; p.shared = ly.shared; p.lay = e->lay; p.E = e->dims.num_experts;
    p.h_in = h_in; p.post_norm = reinterpret_cast<const uint16_t*>(ly.post_norm);
    p.slot_token = slot_token; p.slot_expert = slot_expert;
    p.act = act; p.o = reinterpret_cast<__nv_bfloat16*>(o);
    p.err = e->dec_sync + 2;
    slot_gateup_kernel<<<dim3(kSfGuCtas, slots), kSfThreads, 0, e->stream>>>(p);
    slot_down_kernel<<<dim3(kSfDnCtas, slots), kSfThreads, 0, e->stream>>>(p);
    e->launches += 2;
    MOE_CUDA(cudaGetLastError());
    return MOE_OK;
}

}  // namespace moe
