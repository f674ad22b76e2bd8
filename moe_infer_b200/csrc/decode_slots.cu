// Batch-1 decode of the MoE stack, one persistent cooperative launch of 9 x 16 CTAs.
//
// Same arithmetic and reference as decode.cu (op1 tail, route_experts, op2 of the
// reference's decode engines: src/engine/qwen35_moe/fused_exp1.rs:149-365, 734-856;
// CPU statement src/engine/qwen35_moe/cpu.rs:187-205, 78-85, 398-483), a different
// division of the work.  Each of the nine "slots" of a layer (the eight chosen experts
// and the shared expert) belongs to a group of sixteen CTAs.  CTA j of a group computes
// gate/up/SwiGLU for rows 32 j .. 32 j + 31 of its slot's expert and, after the group has
// exchanged those 512 outputs, the down projection of output rows 128 j .. 128 j + 127:
// every weight slice is one contiguous range of the expert blob (bulk copies only), and
// the SwiGLU outputs cross sixteen CTAs instead of the whole grid.  The down projection
// is linear in its input, so the nine slots' weighted outputs simply add up:
//
//   * every CTA adds its 128 outputs into fixed-point accumulators in global memory
//     (integer addition is associative: the result does not depend on arrival order,
//     repeated runs give identical bits) and its share of the NEXT layer's router logits
//     (logits are linear in h: rows 128 j .. of the transposed router times the CTA's
//     outputs; the first group adds the layer's input rows).  An accumulator word carries
//     its contribution count in the low 16 bits and is never cleared: a reader subtracts
//     what it read two layers earlier and knows the sum is complete when the count has
//     advanced by the number of contributors.  At the top of the next layer every CTA
//     reads the 2,048 sums and 256 logits and routes.
//   * inside a group the SwiGLU outputs travel as 8-byte words (tag, value), tag = the
//     layer's epoch: 8-byte accesses are single-copy atomic, so a reader that sees the
//     current tag sees the value; a relaxed per-group counter tells readers when to look.
//
// Every wait is bounded (about a second of SM clocks) and ends in an error word.
// The host uses this kernel for top-k = 8, a bf16 router and at most 256 experts on a
// device with at least 144 SMs, and the grid-wide kernel of decode.cu otherwise.
#include "decode_common.cuh"
#include <stdlib.h>
#include <string.h>

namespace moe {

constexpr int kGrpCtas = 16;                       // CTAs per slot group
constexpr int kNSlots = kMaxK + 1;                 // 8 chosen experts + the shared expert
constexpr int kSG = kGrpCtas * kNSlots;            // grid: 144 CTAs
constexpr int kItems = kI / kGrpCtas;              // 32 gate/up row pairs per CTA
constexpr int kBatch = kItems / 2;                 // they arrive in two batches of one row pair per warp
constexpr int kDnRows = kH / kGrpCtas;             // 128 output rows per CTA
constexpr int kRtRows = kDnRows / 4;               // rows of the transposed router per thread (two experts each)
constexpr int kSlMaxLayers = 64;
constexpr int kSlProfPoints = 12;
constexpr float kHFix = 268435456.0f;              // 2^28: unit of the hidden-state accumulators
constexpr float kLFix = 4294967296.0f;             // 2^32: unit of the logit accumulators
constexpr unsigned long long kCntMask = 0xFFFFull;
constexpr int kHintStride = 16;                    // u64 words between the per-group counters (128 bytes)
static_assert(kBatch == kDecWarps && kDnRows == 8 * kDecWarps && kChI == 16, "work split below assumes these shapes");

struct SlotParams {
    const LayerDev* layers;
    int l0, l1;
    const float* h_in;
    float* h_out;
    unsigned long long* hacc;     // [2][kH] accumulators: (sum of weighted slot outputs in 2^-28 units) << 16 | count
    unsigned long long* lacc;     // [2][kMaxE] accumulators of the router logits, same format in 2^-32 units
    unsigned long long* hint;     // counts CTAs that have finished a layer (a hint: the accumulators validate themselves)
    unsigned long long hint_base;
    unsigned long long* act_ll;   // [kNSlots][kI] (tag << 32 | float bits): SwiGLU outputs of a slot
    unsigned int epoch_base;      // tags in act_ll are <= epoch_base when the kernel starts
    const float* logit_bias;
    const int32_t* forced_idx;
    int32_t* out_idx;
    float* out_w;
    unsigned int* err;
    long long* prof;              // nullable: [layer][kSlProfPoints] SM-clock stamps taken by CTA 0
    int E;
    moe_expert_layout_t lay;
    int prefetch_same;            // 1: request the next layer's copy of this layer's experts into L2 (the reference's predictor)
    unsigned long long* pf_stats; // [2]: predictions checked, predictions that were among the next layer's experts
};

struct __align__(128) SlotSmem {
    uint4 gu_w[2][kItems][kChH];             // gate / up rows of this CTA's items
    uint4 dn_w[kDnRows][kChI];               // this CTA's down rows
    uint4 sg_w[kChH];                        // shared_expert_gate row (shared-expert group only)
    uint4 xq[6 * kChH];                      // x as three signed-byte digit planes (see stage_digits)
    uint4 aq[6 * kChI];                      // the slot's SwiGLU outputs as digit planes
    uint16_t gu_s[2][kItems][kH / kGroup];
    uint16_t gu_b[2][kItems][kH / kGroup];
    uint16_t dn_s[kDnRows][kI / kGroup];
    uint16_t dn_b[kDnRows][kI / kGroup];
    uint16_t sg_s[kH / kGroup];
    uint16_t sg_b[kH / kGroup];
    float lpart[4][kMaxE];                   // partial router logits of the four row quarters
    float hn[kDnRows];                       // this CTA's finished rows times the next norm weight
    float hrow[kDnRows];                     // this CTA's rows of the layer's input (first group; zeros elsewhere)
    float nwn[kDnRows];                      // next layer's norm weight of this CTA's rows
    float xdl[kChH];
    float sumx[kChH];
    float adl[kChI];
    float suma[kChI];
    float myact[kItems];                     // this CTA's SwiGLU outputs
    float prob[kMaxE];
    float cand_p[kMaxE];
    int cand_i[kMaxE];
    float red[kDecWarps];
    float red2[kDecWarps];
    float red3[kDecWarps];
    float hmax[32];
    float tau;
    float inv_rms;
    int ncand;
    float topw[kMaxK + 1];                   // combine weights; [K] = sigmoid(shared gate score)
    float topp[kMaxK];
    int topi[kMaxK];
    int pred_prev;                           // the expert this CTA requested ahead for the layer now running (-1: none)
    int flag;
    uint64_t bar_g[2];                       // gate/up batches landed
    uint64_t bar_d;                          // down rows landed
    LayerDev tab[kSlMaxLayers];              // this launch's rows of the layer table
};
static_assert(sizeof(SlotSmem) <= 227 * 1024, "decode staging exceeds shared memory");

// Bounded wait on one of this CTA's mbarriers; gives up early when any CTA has raised the error word.
__device__ __forceinline__ bool wait_bar(uint64_t* bar, uint32_t parity, const unsigned int* err) {
    long long t0 = 0;
    for (uint32_t it = 0;; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((it & 127u) == 127u) {
            unsigned int e;
            asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(e) : "l"(err) : "memory");
            if (e != 0u) return false;
            if (t0 == 0) t0 = clock64();
            else if (clock64() - t0 > kWaitCycles) return false;
        }
    }
}
// Bounded wait until a relaxed counter has reached `want` (one thread).
__device__ __forceinline__ int wait_count(const unsigned long long* ctr, unsigned long long want, const unsigned int* err) {
    long long t0 = 0;
    for (uint32_t it = 0;; ++it) {
        unsigned long long n;
        asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(n) : "l"(ctr) : "memory");
        if (n >= want) return 1;
        if ((it & 63u) == 63u) {
            unsigned int e;
            asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(e) : "l"(err) : "memory");
            if (t0 == 0) t0 = clock64();
            if (e != 0u || clock64() - t0 > kWaitCycles) return 0;
        }
    }
}

// x = rmsnorm(h) * w (rms_norm_bf16, reference src/math_util.rs:282-288, eps 1e-6) staged as digit planes;
// h given as this thread's float4 (elements 4 tid ..), its four norm weights as bf16 pairs, 1 / rms(h) already known.
__device__ __forceinline__ void stage_x(SlotSmem* sm, const uint2 wb, const float4 v, float inv_rms) {
    const int tid = threadIdx.x;
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
}

// 1 / rms(h) from every thread's four elements (one CTA barrier)
__device__ __forceinline__ float block_inv_rms(SlotSmem* sm, const float4 v) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float ss = warp_sum(v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w);
    if (lane == 0) sm->red3[warp] = ss;  // an array of its own: the routing code reuses red / red2 right away
    __syncthreads();
    float tot = 0.0f;
#pragma unroll
    for (int i = 0; i < kDecWarps; ++i) tot += sm->red3[i];
    return 1.0f / sqrtf(tot / (float)kH + 1e-6f);
}

// This thread's part of a layer's transposed router ([H][Ep] bf16): experts 2 e2 and 2 e2 + 1 of rows
// row0 .. row0 + 31, one 32-bit load per row, consecutive lanes on consecutive words.
__device__ __forceinline__ void load_router_slice(uint32_t (&rt)[kRtRows], const void* router_t, int Ep, int row0, int e2) {
    if (2 * e2 >= Ep) return;
    const uint32_t* src = reinterpret_cast<const uint32_t*>(router_t) + (size_t)row0 * (Ep / 2) + e2;
#pragma unroll
    for (int i = 0; i < kRtRows; ++i) rt[i] = __ldg(src + (size_t)i * (Ep / 2));
}

// Adds this CTA's share of the next layer's router logits to the accumulators: logits are linear in h, so the
// product of this CTA's 128 output rows (sm->hn, already times the next norm weight) with its rows of the
// transposed router is a partial sum that the other CTAs' shares complete.  Fixed point, times `scale`.
__device__ __forceinline__ void push_partial_logits(SlotSmem* sm, const uint32_t (&rt)[kRtRows], unsigned long long* lacc,
                                                    int E, int Ep, float scale) {
    const int tid = threadIdx.x, e2 = tid & 127, qt = tid >> 7;
    float a0 = 0.0f, a1 = 0.0f;
    if (2 * e2 < Ep) {
#pragma unroll
        for (int i = 0; i < kRtRows; ++i) {
            const float hn = sm->hn[qt * kRtRows + i];
            a0 = fmaf(__uint_as_float(rt[i] << 16), hn, a0);
            a1 = fmaf(__uint_as_float(rt[i] & 0xFFFF0000u), hn, a1);
        }
    }
    sm->lpart[qt][2 * e2] = a0;
    sm->lpart[qt][2 * e2 + 1] = a1;
    __syncthreads();
    if (tid < E) {
        const float part = (sm->lpart[0][tid] + sm->lpart[1][tid]) + (sm->lpart[2][tid] + sm->lpart[3][tid]);
        const long long fx = __float2ll_rn(part * scale * kLFix);
        asm volatile("red.relaxed.gpu.global.add.u64 [%0], %1;" ::"l"(lacc + tid), "l"(((unsigned long long)fx << 16) + 1ull) : "memory");
    }
}


#define SPROF(idx)                                                                                   \
    do {                                                                                             \
        if (p.prof && blockIdx.x == 0 && tid == 0) p.prof[rel * kSlProfPoints + (idx)] = clock64();  \
    } while (0)

__global__ void __launch_bounds__(kDecThreads, 1) decode_slots_kernel(SlotParams p) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    SlotSmem* sm = reinterpret_cast<SlotSmem*>(smem_raw);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int slot = blockIdx.x / kGrpCtas, grank = blockIdx.x % kGrpCtas;
    const int E = p.E, Ep = (E + 7) & ~7;
    constexpr int K = kMaxK;
    const moe_expert_layout_t L = p.lay;
    const int n_layers = p.l1 - p.l0;
    const bool shared_slot = slot == K;

    pdl_trigger();
    if (tid == 0) {
        mbar_init(&sm->bar_g[0], 6);
        mbar_init(&sm->bar_g[1], 6 + (shared_slot ? 3 : 0));
        mbar_init(&sm->bar_d, 3);
        mbar_fence_init();
    }
    // Launched as a programmatic dependent (the whole-decoder path), the kernel may be resident while the one that
    // produces h_in still runs: until the wait below it reads only the layer table and the first layer's router slice,
    // which no kernel of the chain writes (the host launches the ordinary way when it has just refreshed them).
    {
        static_assert(sizeof(LayerDev) % 4 == 0, "table rows are copied as words");
        const uint32_t* src = reinterpret_cast<const uint32_t*>(p.layers + p.l0);
        uint32_t* dst = reinterpret_cast<uint32_t*>(sm->tab);
        const int words = n_layers * (int)(sizeof(LayerDev) / 4);
        for (int i = tid; i < words; i += kDecThreads) dst[i] = __ldg(src + i);
    }
    __syncthreads();

    const int r0 = kDnRows * grank;       // this CTA's output rows
    const int item0 = kItems * grank;     // this CTA's gate/up rows inside its slot's expert
    const int rt_e2 = tid & 127, rt_row0 = r0 + (tid >> 7) * kRtRows;  // this thread's part of the router slice

    uint32_t rt[kRtRows];
    load_router_slice(rt, sm->tab[0].router_t, Ep, rt_row0, rt_e2);
    pdl_wait();
    float4 hv = ld_dep_f4(reinterpret_cast<const float4*>(p.h_in) + tid);  // this thread's four elements of h
    // what this thread last read from its accumulator words: of the set about to be read / of the other set
    unsigned long long hprev_cur[4] = {0ull, 0ull, 0ull, 0ull}, hprev_oth[4] = {0ull, 0ull, 0ull, 0ull};
    unsigned long long lprev_cur = 0ull, lprev_oth = 0ull;
    bool alive = true;
    float pscale = 1.0f;  // scale the pending logit accumulators were pushed with

    // Waits until `n_done` pushes of every CTA are announced, then reads this thread's accumulator words until
    // they are complete: the hidden-state sums of the layer just finished (added to hv) when with_h, the router
    // logits of the layer about to run (returned through `logit`, in 2^-32 units times pscale) when with_l.
    unsigned long long l_expect = (unsigned long long)kSG;  // contributions a finished logit sum carries
    auto read_acc = [&](int n_done, bool with_h, int hset, bool with_l, int lset, long long& logit) -> bool {
        if (tid == 0) sm->flag = wait_count(p.hint, p.hint_base + (unsigned long long)kSG * (unsigned long long)n_done, p.err);
        __syncthreads();
        int ok = sm->flag;
        const unsigned long long* hsrc = p.hacc + (size_t)hset * kH + 4 * tid;
        const unsigned long long* lsrc = p.lacc + (size_t)lset * kMaxE + tid;
        const bool my_l = with_l && tid < E;
        unsigned long long q[4] = {0ull, 0ull, 0ull, 0ull}, ql = 0ull;
        long long t0 = 0;
        for (uint32_t it = 0; ok; ++it) {
            bool done = true;
            if (with_h) {
                asm volatile("ld.relaxed.gpu.global.v2.u64 {%0, %1}, [%2];" : "=l"(q[0]), "=l"(q[1]) : "l"(hsrc) : "memory");
                asm volatile("ld.relaxed.gpu.global.v2.u64 {%0, %1}, [%2];" : "=l"(q[2]), "=l"(q[3]) : "l"(hsrc + 2) : "memory");
            }
            if (my_l) asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(ql) : "l"(lsrc) : "memory");
            if (with_h) {
#pragma unroll
                for (int i = 0; i < 4; ++i) done = done && (((q[i] - hprev_cur[i]) & kCntMask) == (unsigned long long)kNSlots);
            }
            if (my_l) done = done && (((ql - lprev_cur) & kCntMask) == l_expect);
            if (done) break;
            if ((it & 15u) == 15u) {
                if (t0 == 0) t0 = clock64();
                else if (clock64() - t0 > kWaitCycles) ok = 0;
            }
        }
        if (ok && with_h) {
            float d[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                d[i] = __ll2float_rn((long long)(q[i] - hprev_cur[i]) >> 16) * (1.0f / kHFix);
                hprev_cur[i] = hprev_oth[i];  // the sets alternate from layer to layer
                hprev_oth[i] = q[i];
            }
            // moe_combine_residual (reference src/math_util.rs:599-612): h + sum of the weighted expert outputs
            hv.x += d[0]; hv.y += d[1]; hv.z += d[2]; hv.w += d[3];
        }
        if (ok && with_l) {
            logit = (long long)(ql - lprev_cur) >> 16;
            lprev_cur = lprev_oth;
            lprev_oth = ql;
        }
        return __syncthreads_and(ok) != 0;
    };

    // Requests this CTA's weight slices of a layer: every slice is one contiguous range of the slot's expert.  One copy
    // per warp (lane 0): copies issued by several lanes of one warp would go out one after the other.
    auto request_weights = [&](const LayerDev& ly) {
        const uint8_t* ex = shared_slot ? ly.shared : ly.experts + (size_t)sm->topi[slot] * L.expert_size;
        if (lane == 0 && warp < 12) {
            const int b = warp / 6, a = warp - b * 6;  // batch, array
            const bool is_w = a < 2;
            const int64_t off = a == 0 ? L.gate_w : a == 1 ? L.up_w : a == 2 ? L.gate_s : a == 3 ? L.up_s : a == 4 ? L.gate_b : L.up_b;
            const uint32_t row_bytes = is_w ? kH / 2 : (kH / kGroup) * 2;
            const int j0 = b * kBatch;
            void* dst = a == 0 ? (void*)sm->gu_w[0][j0] : a == 1 ? (void*)sm->gu_w[1][j0] : a == 2 ? (void*)sm->gu_s[0][j0]
                      : a == 3 ? (void*)sm->gu_s[1][j0] : a == 4 ? (void*)sm->gu_b[0][j0] : (void*)sm->gu_b[1][j0];
            const uint32_t bytes = kBatch * row_bytes;
            mbar_expect_tx(&sm->bar_g[b], bytes);
            bulk_g2s_stream(dst, ex + off + (size_t)(item0 + j0) * row_bytes, bytes, &sm->bar_g[b]);
        } else if (lane == 0 && warp < 15) {
            const int q = warp - 12;
            const int64_t off = q == 0 ? L.down_w : q == 1 ? L.down_s : L.down_b;
            const uint32_t row_bytes = q == 0 ? kI / 2 : (kI / kGroup) * 2;
            void* dst = q == 0 ? (void*)sm->dn_w : q == 1 ? (void*)sm->dn_s : (void*)sm->dn_b;
            const uint32_t bytes = kDnRows * row_bytes;
            mbar_expect_tx(&sm->bar_d, bytes);
            bulk_g2s_stream(dst, ex + off + (size_t)r0 * row_bytes, bytes, &sm->bar_d);
        }
        if (shared_slot && lane == 1 && warp < 3) {
            const void* src = warp == 0 ? (const void*)ly.sgate.w : warp == 1 ? (const void*)ly.sgate.s : (const void*)ly.sgate.b;
            void* dst = warp == 0 ? (void*)sm->sg_w : warp == 1 ? (void*)sm->sg_s : (void*)sm->sg_b;
            const uint32_t bytes = warp == 0 ? kH / 2 : (kH / kGroup) * 2;
            mbar_expect_tx(&sm->bar_g[1], bytes);
            bulk_g2s(dst, src, bytes, &sm->bar_g[1]);
        }
    };

    // The reference hides expert fetches by assuming that layer L + 1 picks the experts layer L picked
    // (src/engine/qwen35_moe/fused_exp6.rs:4-8, expert_prefetch.rs:95-135) and reading them ahead.  Here: once layer L is
    // routed, a routed CTA asks for its own slices of the same expert in layer L + 1 to be brought into L2 (nine ranges, one
    // per warp), and the first CTA of each group counts how often the expert it asked for was indeed chosen.  Off by default:
    // with routers that are independent from layer to layer (the synthetic store) the guess is right 8 times in 256.
    if (tid == 0) sm->pred_prev = -1;
    auto prefetch_same_experts = [&](int rel) {
        if (!p.prefetch_same || shared_slot) return;
        if (tid == 0) {
            if (sm->pred_prev >= 0 && grank == 0) {
                bool hit = false;
                for (int k = 0; k < K; ++k) hit = hit || sm->topi[k] == sm->pred_prev;
                atomicAdd(p.pf_stats, 1ull);
                if (hit) atomicAdd(p.pf_stats + 1, 1ull);
            }
            sm->pred_prev = (rel + 1 < n_layers) ? sm->topi[slot] : -1;
        }
        if (rel + 1 < n_layers && lane == 0 && warp < 9) {
            const uint8_t* ex = sm->tab[rel + 1].experts + (size_t)sm->topi[slot] * L.expert_size;
            const int a = warp;
            const bool gu = a < 6;
            const int64_t off = a == 0 ? L.gate_w : a == 1 ? L.up_w : a == 2 ? L.gate_s : a == 3 ? L.up_s : a == 4 ? L.gate_b : a == 5 ? L.up_b
                              : a == 6 ? L.down_w : a == 7 ? L.down_s : L.down_b;
            const uint32_t row_bytes = a < 2 ? kH / 2 : gu ? (kH / kGroup) * 2 : a == 6 ? kI / 2 : (kI / kGroup) * 2;
            const int row = gu ? item0 : r0, rows = gu ? kItems : kDnRows;
            prefetch_l2(ex + off + (size_t)row * row_bytes, (uint32_t)rows * row_bytes);
        }
    };

    // ── prologue: router logits of the first layer from h_in (the first group's rows cover all of h) ──
    {
        pscale = block_inv_rms(sm, hv);
        if (warp == grank) {
            const uint2 nw = __ldg(reinterpret_cast<const uint2*>(sm->tab[0].post_norm) + tid);
            float4 o = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (slot == 0) {
                o.x = hv.x * __uint_as_float(nw.x << 16);
                o.y = hv.y * __uint_as_float(nw.x & 0xFFFF0000u);
                o.z = hv.z * __uint_as_float(nw.y << 16);
                o.w = hv.w * __uint_as_float(nw.y & 0xFFFF0000u);
            }
            reinterpret_cast<float4*>(sm->hn)[lane] = o;
        }
        __syncthreads();
        // only the first group holds rows of h here: the other groups' shares would be zeros
        if (slot == 0) {
            push_partial_logits(sm, rt, p.lacc, E, Ep, pscale);
            __syncthreads();
        }
        if (tid == 0) asm volatile("red.relaxed.gpu.global.add.u64 [%0], %1;" ::"l"(p.hint), "l"(1ull) : "memory");
    }

    for (int rel = 0; rel < n_layers; ++rel) {
        const LayerDev& ly = sm->tab[rel];
        const uint32_t ph = (uint32_t)rel & 1u;
        const bool has_next = rel + 1 < n_layers;
        const unsigned int epoch = p.epoch_base + (unsigned int)rel + 1u;
        SPROF(0);
        // the shared expert's slices depend on nothing but the layer: requested before the layer's input is known
        if (shared_slot) request_weights(ly);
        // norm weights of this thread's elements (this layer) and of this CTA's output rows (next layer): requested now,
        // used after the layer's input has arrived
        const uint2 norm_wb = __ldg(reinterpret_cast<const uint2*>(ly.post_norm) + tid);
        uint16_t nwn_bits = 0;
        if (has_next && tid < kDnRows) nwn_bits = __ldg(sm->tab[rel + 1].post_norm + r0 + tid);
        // ── this layer's input: h (sums of the layer before) and the router logits ──
        long long lq = 0;
        l_expect = (unsigned long long)(rel == 0 ? kGrpCtas : kSG);  // the first layer's sums come from the first group alone
        if (!read_acc(rel + 1, rel > 0, (rel + 1) & 1, true, rel & 1, lq)) {
            if (tid == 0) atomicExch(p.err, 3u);
            alive = false;
            break;
        }
        SPROF(1);
        float inv_rms, v = -INFINITY;
        if (p.logit_bias == nullptr) {
            // The logits are the accumulated sums times a positive factor (1 / rms of this layer's input over the
            // factor they were pushed with): the selection needs only their order, so it runs on the raw sums and
            // the weight requests go out before the norm's reduction; the factor is applied afterwards.
            const float u = (tid < E) ? __ll2float_rn(lq) : -INFINITY;
            route_select(sm, u, p.forced_idx, E, K, p.err);
            SPROF(2);
            if (!shared_slot) request_weights(ly);
            SPROF(3);
            prefetch_same_experts(rel);
            inv_rms = block_inv_rms(sm, hv);
            const float f1 = 1.0f / kLFix, f2 = inv_rms / pscale;
            if (tid < E) v = u * f1 * f2;
            // what route_weights reads later (behind the barrier that follows the staging): chosen logits, warp maxima
            if (tid < K) sm->topp[tid] = sm->topp[tid] * f1 * f2;
            if (tid >= 32 && tid < 32 + kDecWarps) sm->red[tid - 32] = sm->red[tid - 32] * f1 * f2;
        } else {
            inv_rms = block_inv_rms(sm, hv);
            if (tid < E) v = __ll2float_rn(lq) * (1.0f / kLFix) * (inv_rms / pscale) + p.logit_bias[tid];
            route_select(sm, v, p.forced_idx, E, K, p.err);
            SPROF(2);
            // ── weight requests (the shared expert's group made them at the top of the layer) ──
            if (!shared_slot) request_weights(ly);
            SPROF(3);
            prefetch_same_experts(rel);
        }
        // the copies are on their way: stage x, the softmax weights of the chosen experts, and what the end of
        // the layer needs from the layer's input
        stage_x(sm, norm_wb, hv, inv_rms);
        if (warp == grank) reinterpret_cast<float4*>(sm->hrow)[lane] = (slot == 0) ? hv : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (tid < kDnRows) sm->nwn[tid] = __uint_as_float((uint32_t)nwn_bits << 16);
        __syncthreads();  // x is staged for every warp
        SPROF(4);

        // ── gate/up + SwiGLU: two row pairs per warp (items warp and warp + 16); a lane holds the digits of one
        //    chunk of x in registers while it visits that chunk of all its rows ──
        int ok = 1;
        {
            const bool sg_now = shared_slot && warp == kDecWarps - 1;  // the gate score: one more row for one warp
            ok = wait_bar(&sm->bar_g[0], ph, p.err) ? 1 : 0;
            SPROF(10);
            ok = (ok && wait_bar(&sm->bar_g[1], ph, p.err)) ? 1 : 0;
            SPROF(11);
            float acc[2][2] = {{0.0f, 0.0f}, {0.0f, 0.0f}}, sg = 0.0f;
            if (ok) {
#pragma unroll
                for (int it = 0; it < 2; ++it) {
                    const int c = lane + 32 * it;
                    uint4 xe[3], xo[3];
#pragma unroll
                    for (int pl = 0; pl < 3; ++pl) {
                        xe[pl] = sm->xq[(pl * 2 + 0) * kChH + c];
                        xo[pl] = sm->xq[(pl * 2 + 1) * kChH + c];
                    }
                    const float sx = sm->sumx[c], dl = sm->xdl[c];
#pragma unroll
                    for (int k = 0; k < 2; ++k) {
                        const int t = warp + k * kBatch;
#pragma unroll
                        for (int a = 0; a < 2; ++a) {
                            const float sc = bf16_bits_to_f32(sm->gu_s[a][t][c >> 1]), bi = bf16_bits_to_f32(sm->gu_b[a][t][c >> 1]);
                            acc[k][a] += fmaf(sc * dl, dot32_regs(sm->gu_w[a][t][c], xe, xo), bi * sx);
                        }
                    }
                    if (sg_now) {
                        const float sc = bf16_bits_to_f32(sm->sg_s[c >> 1]), bi = bf16_bits_to_f32(sm->sg_b[c >> 1]);
                        sg += fmaf(sc * dl, dot32_regs(sm->sg_w[c], xe, xo), bi * sx);
                    }
                }
#pragma unroll
                for (int k = 0; k < 2; ++k) {
                    acc[k][0] = warp_sum(acc[k][0]);
                    acc[k][1] = warp_sum(acc[k][1]);
                }
                if (sg_now) sg = warp_sum(sg);
                if (lane == 0) {
                    sm->myact[warp] = swiglu(acc[0][0], acc[0][1]);
                    sm->myact[warp + kBatch] = swiglu(acc[1][0], acc[1][1]);
                    // sigmoid (reference src/math_util.rs:67-69) of the shared gate score
                    if (sg_now) sm->topw[K] = 1.0f / (1.0f + expf(-sg));
                }
            }
        }
        // this thread's part of the next layer's transposed router: into registers now, used at the end of the layer
        if (has_next) load_router_slice(rt, sm->tab[rel + 1].router_t, Ep, rt_row0, rt_e2);
        if (!__syncthreads_and(ok)) {
            if (tid == 0) atomicExch(p.err, 6u);
            alive = false;
            break;
        }
        SPROF(5);

        // ── this group's SwiGLU outputs: publish mine, gather all 512 ──
        {
            unsigned long long* grp = p.act_ll + (size_t)slot * kI;
            if (warp == 0) {
                const unsigned long long word = ((unsigned long long)epoch << 32) | (unsigned long long)__float_as_uint(sm->myact[lane]);
                asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(grp + item0 + lane), "l"(word) : "memory");
            }
            // while the group's outputs arrive: the softmax weights of the chosen experts (needed from the down phase on)
            route_weights(sm, v, E, K);  // ends with a CTA barrier
            if (blockIdx.x == 0 && warp == 0 && lane < K) {
                if (p.out_idx) p.out_idx[lane] = sm->topi[lane];
                if (p.out_w) p.out_w[lane] = sm->topw[lane];
            }
            // The readers poll the tagged words themselves: a word whose tag is the layer's epoch carries the value.
            // With sixteen CTAs per group a counter that says "everybody has published" costs one more L2 round trip
            // than it saves (measured: 474 -> 461 us per token without it).
            if (tid < kI / 4) {  // four whole warps: thread t takes values 4 t .. 4 t + 3
                unsigned long long q[4];
                long long t0 = 0;
                for (uint32_t it = 0; ok; ++it) {
                    asm volatile("ld.relaxed.gpu.global.v2.u64 {%0, %1}, [%2];" : "=l"(q[0]), "=l"(q[1]) : "l"(grp + 4 * tid) : "memory");
                    asm volatile("ld.relaxed.gpu.global.v2.u64 {%0, %1}, [%2];" : "=l"(q[2]), "=l"(q[3]) : "l"(grp + 4 * tid + 2) : "memory");
                    if ((unsigned int)(q[0] >> 32) == epoch && (unsigned int)(q[1] >> 32) == epoch &&
                        (unsigned int)(q[2] >> 32) == epoch && (unsigned int)(q[3] >> 32) == epoch)
                        break;
                    if ((it & 15u) == 15u) {
                        if (t0 == 0) t0 = clock64();
                        else if (clock64() - t0 > kWaitCycles) ok = 0;
                    }
                }
                ok = __all_sync(0xffffffffu, ok);  // the staging shuffles below need the whole warp
                if (ok) {
                    const float4 av = make_float4(__uint_as_float((unsigned int)q[0]), __uint_as_float((unsigned int)q[1]),
                                                  __uint_as_float((unsigned int)q[2]), __uint_as_float((unsigned int)q[3]));
                    const int c = tid >> 3, j = tid & 7;
                    stage_digits(sm->aq, sm->adl, kChI, c, j, av);
                    float sv = (av.x + av.y) + (av.z + av.w);
                    sv += __shfl_xor_sync(0xffffffffu, sv, 1);
                    sv += __shfl_xor_sync(0xffffffffu, sv, 2);
                    sv += __shfl_xor_sync(0xffffffffu, sv, 4);
                    if (j == 0) sm->suma[c] = sv;
                }
            }
            if (ok) ok = wait_bar(&sm->bar_d, ph, p.err) ? 1 : 0;
            if (!__syncthreads_and(ok)) {
                if (tid == 0) atomicExch(p.err, 4u);
                alive = false;
                break;
            }
        }
        SPROF(6);

        // ── down: eight output rows per warp, two at a time (half a warp per row, one chunk per lane) ──
        {
            const int sub = lane >> 4, c = lane & 15;
            const float wslot = sm->topw[slot];
            uint4 xe[3], xo[3];
#pragma unroll
            for (int q = 0; q < 3; ++q) {
                xe[q] = sm->aq[(q * 2 + 0) * kChI + c];
                xo[q] = sm->aq[(q * 2 + 1) * kChI + c];
            }
            const float dl = sm->adl[c], sa = sm->suma[c];
            float part[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int r = warp * 8 + 2 * i + sub;
                const float sc = bf16_bits_to_f32(sm->dn_s[r][c >> 1]), bi = bf16_bits_to_f32(sm->dn_b[r][c >> 1]);
                part[i] = fmaf(sc * dl, dot32_regs(sm->dn_w[r][c], xe, xo), bi * sa);
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                float s = part[i];
                s += __shfl_xor_sync(0xffffffffu, s, 8);
                s += __shfl_xor_sync(0xffffffffu, s, 4);
                s += __shfl_xor_sync(0xffffffffu, s, 2);
                s += __shfl_xor_sync(0xffffffffu, s, 1);
                if (c == 0) {
                    const int row = warp * 8 + 2 * i + sub;
                    const float mine = wslot * s;
                    const long long fx = __float2ll_rn(mine * kHFix);
                    unsigned long long* dst = p.hacc + (size_t)ph * kH + r0 + row;
                    asm volatile("red.relaxed.gpu.global.add.u64 [%0], %1;" ::"l"(dst), "l"(((unsigned long long)fx << 16) + 1ull) : "memory");
                    // this CTA's rows of (partial) h, times the next layer's norm weight: what the next router sees of them
                    sm->hn[row] = (mine + sm->hrow[row]) * sm->nwn[row];
                }
            }
        }
        __syncthreads();
        SPROF(7);
        if (has_next) {
            push_partial_logits(sm, rt, p.lacc + (size_t)((rel + 1) & 1) * kMaxE, E, Ep, inv_rms);
            pscale = inv_rms;
            __syncthreads();
        }
        if (tid == 0) asm volatile("red.relaxed.gpu.global.add.u64 [%0], %1;" ::"l"(p.hint), "l"(1ull) : "memory");
        SPROF(8);
    }

    // the first CTA collects the last layer's sums and writes the result
    if (alive && blockIdx.x == 0) {
        const int rel = n_layers - 1;
        long long unused = 0;
        if (read_acc(n_layers + 1, true, (n_layers + 1) & 1, false, 0, unused)) {
            reinterpret_cast<float4*>(p.h_out)[tid] = hv;
            // Leave the accumulators (hidden-state sets, then logit sets: one range) cleared for the next launch.  Nobody
            // reads or adds to them any more: every CTA has passed its last read, the last layer pushes no logits, and
            // the sums just read carried every contribution.  (A launch that fails leaves them to the host's reset.)
            for (int i = tid; i < 2 * kH + 2 * kMaxE; i += kDecThreads) p.hacc[i] = 0ull;
        } else if (tid == 0) {
            atomicExch(p.err, 3u);
        }
        SPROF(9);
    }
}

// ─── host side ──────────────────────────────────────────────────────────────

constexpr size_t kSlAccWords = 2 * kH + 2 * kMaxE;          // hidden-state sets, then logit sets
constexpr size_t kSlActWords = (size_t)kNSlots * kI;
constexpr size_t kSlHintWords = (size_t)(kNSlots + 2) * kHintStride;  // (unused group slots), the layer counter, the prefetch statistics

// Decides once per engine whether this device and model shape can use the kernel; never fatal.
int slots_decode_init(moe_engine* e) {
    e->dec_sl_ok = false;
    const moe_dims_t& d = e->dims;
    if (d.hidden != kH || d.inter != kI || d.shared_inter != kI || d.top_k != kMaxK || d.num_experts > 256) return MOE_OK;
    if (e->sm_count < kSG) return MOE_OK;
    const char* k = getenv("MOE_B200_DECODE_KERNEL");  // read once, at engine creation: "grid" keeps the grid-wide kernel
    if (k && strcmp(k, "grid") == 0) return MOE_OK;
    MOE_CUDA(cudaFuncSetAttribute(decode_slots_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(SlotSmem)));
    int per_sm = 0;
    MOE_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_slots_kernel, kDecThreads, sizeof(SlotSmem)));
    if (per_sm < 1) return MOE_OK;
    MOE_CUDA(cudaMalloc(&e->dec_sl_words, (kSlAccWords + kSlActWords + kSlHintWords) * sizeof(unsigned long long)));
    MOE_CUDA(cudaMemset(e->dec_sl_words, 0, (kSlAccWords + kSlActWords + kSlHintWords) * sizeof(unsigned long long)));
    e->dec_sl_hint_base = 0;
    e->dec_sl_epoch = 0;
    e->dec_sl_ok = true;
    {
        const char* v = getenv("MOE_B200_DECODE_PREFETCH");
        e->dec_sl_prefetch = v && atoi(v) != 0;
    }
    return MOE_OK;
}

void slots_decode_destroy(moe_engine* e) {
    if (e->dec_sl_words) cudaFree(e->dec_sl_words);
    e->dec_sl_words = nullptr;
    e->dec_sl_ok = false;
}

bool slots_decode_usable(const moe_engine* e, int l0, int l1) {
    if (!e->dec_sl_ok || l1 - l0 > kSlMaxLayers) return false;
    for (int l = l0; l < l1; ++l)
        if (!e->layers[l].router_is_bf16) return false;
    return true;
}

// After a failed device-side wait (and before the epoch counter would wrap): back to the state a launch expects.
int slots_decode_reset(moe_engine* e) {
    if (!e->dec_sl_ok) return MOE_OK;
    MOE_CUDA(cudaMemsetAsync(e->dec_sl_words, 0, (kSlAccWords + kSlActWords + kSlHintWords) * sizeof(unsigned long long), e->stream));
    e->dec_sl_hint_base = 0;
    e->dec_sl_epoch = 0;
    return MOE_OK;
}

// predictions checked / predictions right since the engine was created (zero unless MOE_B200_DECODE_PREFETCH=1)
int slots_decode_prefetch_stats(moe_engine* e, double* checks, double* hits) {
    *checks = *hits = 0.0;
    if (!e->dec_sl_ok || !e->dec_sl_prefetch) return MOE_OK;
    unsigned long long v[2] = {0ull, 0ull};
    const unsigned long long* src = e->dec_sl_words + kSlAccWords + kSlActWords + (size_t)kNSlots * kHintStride + kHintStride;
    MOE_CUDA(cudaMemcpyAsync(v, src, sizeof(v), cudaMemcpyDeviceToHost, e->stream));
    MOE_CUDA(cudaStreamSynchronize(e->stream));
    *checks = (double)v[0];
    *hits = (double)v[1];
    return MOE_OK;
}

int launch_decode_slots(moe_engine* e, int l0, int l1, const float* h_in, float* h_out, const float* logit_bias,
                        const int32_t* forced_idx, int32_t* out_idx, float* out_w, bool pdl) {
    MOE_REQUIRE(l0 >= 0 && l1 > l0 && l1 <= (int)e->layers.size() && l1 - l0 <= kSlMaxLayers, "decode: bad layer range [%d, %d)", l0, l1);
    MOE_REQUIRE((((uintptr_t)h_in) & 15) == 0 && (((uintptr_t)h_out) & 15) == 0, "decode: h must be 16-byte aligned");
    const int64_t launches_before = e->launches;
    const bool table_was_dirty = e->table_dirty;
    for (int l = l0; l < l1; ++l) {
        int rc = check_layer_ready(e, l);
        if (rc != MOE_OK) return rc;
        rc = ensure_router_t(e, l);
        if (rc != MOE_OK) return rc;
    }
    int rc = refresh_layer_table(e);
    if (rc != MOE_OK) return rc;
    // what the kernel reads ahead of its dependency wait was just rewritten on this stream: an ordinary launch this time
    if (e->launches != launches_before || table_was_dirty || e->table_dirty) pdl = false;
    if (e->dec_sl_epoch > 0xFFFF0000u - (unsigned int)(l1 - l0)) {
        rc = slots_decode_reset(e);  // tags must never repeat: start the epochs over on cleared buffers
        if (rc != MOE_OK) return rc;
    }
    SlotParams p{};
    p.layers = e->layers_dev;
    p.l0 = l0; p.l1 = l1;
    p.h_in = h_in; p.h_out = h_out;
    p.hacc = e->dec_sl_words;
    p.lacc = e->dec_sl_words + 2 * kH;
    p.act_ll = e->dec_sl_words + kSlAccWords;
    p.hint = e->dec_sl_words + kSlAccWords + kSlActWords + (size_t)kNSlots * kHintStride;
    p.hint_base = e->dec_sl_hint_base;
    p.epoch_base = e->dec_sl_epoch;
    p.logit_bias = logit_bias; p.forced_idx = forced_idx;
    p.out_idx = out_idx; p.out_w = out_w;
    p.err = e->dec_sync + 2;
    p.prof = e->dec_prof;
    p.E = e->dims.num_experts;
    p.lay = e->lay;
    p.prefetch_same = e->dec_sl_prefetch ? 1 : 0;
    p.pf_stats = e->dec_sl_words + kSlAccWords + kSlActWords + (size_t)kNSlots * kHintStride + kHintStride;
    // the accumulators start from zero: cleared at set-up and after an error by the host, at the end of every launch by
    // the kernel's first CTA (a memset per launch cost a single-layer call about two microseconds of stream time)
    e->dec_sl_hint_base += (unsigned long long)kSG * (unsigned long long)(l1 - l0 + 1);  // one push per layer and the prologue's
    e->dec_sl_epoch += (unsigned int)(l1 - l0);
    // A cooperative launch: every CTA resident, or the launch fails.  As a programmatic dependent (inside the whole-decoder
    // chain, and in single-layer calls) the kernel is launched the ordinary way instead, so that its CTAs can take their
    // SMs while the kernel before it drains (a cooperative grid waits for the whole device): its CTAs still all become
    // resident, because the kernels before it never wait for it and the kernels after it either are its programmatic
    // dependents, launched only once every CTA here has started, or ordinary launches that wait for its end.  Another
    // tenant holding SMs for good would end in the kernel's bounded waits and an error status, not in a hang.
    // MOE_B200_CHAIN_COOP=1 keeps the cooperative launch there too.
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(kSG);
    cfg.blockDim = dim3(kDecThreads);
    cfg.dynamicSmemBytes = sizeof(SlotSmem);
    cfg.stream = e->stream;
    cudaLaunchAttribute at[2];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    at[1].id = cudaLaunchAttributeCooperative;
    at[1].val.cooperative = 1;
    static const bool chain_coop = [] { const char* v = getenv("MOE_B200_CHAIN_COOP"); return v && atoi(v) != 0; }();
    cfg.attrs = pdl ? at : at + 1;
    cfg.numAttrs = pdl ? (chain_coop ? 2 : 1) : 1;
    MOE_CUDA(cudaLaunchKernelEx(&cfg, decode_slots_kernel, p));
    e->launches++;
    return MOE_OK;
}

}  // namespace moe
