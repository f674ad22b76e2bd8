// Stand-alone 4-bit dequant-matvec: y[r] = sum_c (nib*scale + bias) * x[c].
//
// Replaces dequant_matvec_4bit (reference src/math_util.rs:14-54) and the Metal
// kernel family dequant_matvec_4bit_* (reference src/engine/shaders.metal:74-3409).
// HBM-bound: 0.5625 B of weights per multiply-add.  One warp per output row; each
// lane issues 128-bit loads of 32 nibbles (half a group), dequantises in
// registers and reduces with warp shuffles.  x is staged into shared memory
// with one bulk (TMA) copy, then re-laid out chunk-transposed (see q4dot.cuh)
// together with the per-chunk sums the affine dequant needs.
#include "q4dot.cuh"
#include "stage.cuh"

namespace moe {

constexpr int kMvWarps = 8;

__global__ void __launch_bounds__(kMvWarps * 32)
matvec_int4_kernel(const uint32_t* __restrict__ w, const uint16_t* __restrict__ s,
                   const uint16_t* __restrict__ b, const float* __restrict__ x,
                   float* __restrict__ y, int rows, int cols, unsigned int* err_flag,
                   const float* __restrict__ residual) {  // nullable: y = W x + residual
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int nch = cols / 32;  // chunks per row
    float* raw = reinterpret_cast<float*>(smem_raw);                 // [cols]
    float4* xs = reinterpret_cast<float4*>(smem_raw + (size_t)cols * 4);  // [8][nch]
    float* sumx = reinterpret_cast<float*>(smem_raw + (size_t)cols * 8);  // [nch]
    __shared__ uint64_t bar;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    pdl_trigger();
    if (tid == 0) {
        mbar_init(&bar, 1);
        mbar_fence_init();
    }
    // nothing about the weights depends on x: ask for this warp's rows (L2) while the kernel that produces x still runs
    const int groups = cols / kGroup;
    const int row_first = blockIdx.x * kMvWarps + warp;
    {
        const int row = row_first + lane * (int)gridDim.x * kMvWarps;
        if (lane < 8 && row < rows) {
            const unsigned char* wr = reinterpret_cast<const unsigned char*>(w + (size_t)row * (cols / 8));
            for (int off = 0; off < cols / 2; off += 4096) prefetch_l2(wr + off, (uint32_t)min(4096, cols / 2 - off));
        }
    }
    __syncthreads();
    pdl_wait();
    if (tid == 0) {
        mbar_expect_tx(&bar, (uint32_t)cols * 4u);
        bulk_g2s(raw, x, (uint32_t)cols * 4u, &bar);
    }
    // the first two chunks of this warp's first row do not depend on x: request them before waiting for it
    uint4 pqa = make_uint4(0, 0, 0, 0), pqb = pqa;
    uint16_t psa = 0, pba = 0, psb = 0, pbb = 0;
    if (row_first < rows) {
        const uint4* wrow = reinterpret_cast<const uint4*>(w + (size_t)row_first * (cols / 8));
        const uint16_t* srow = s + (size_t)row_first * groups;
        const uint16_t* brow = b + (size_t)row_first * groups;
        if (lane < nch) { pqa = ld_stream_u4(wrow + lane); psa = srow[lane >> 1]; pba = brow[lane >> 1]; }
        if (32 + lane < nch) { pqb = ld_stream_u4(wrow + 32 + lane); psb = srow[(32 + lane) >> 1]; pbb = brow[(32 + lane) >> 1]; }
    }
    // every thread observes the phase itself, so the copied bytes are visible to it
    const int ok = __syncthreads_and(mbar_wait(&bar, 0) ? 1 : 0);
    if (!ok) {
        if (tid == 0) atomicExch(err_flag, 1u);
        return;
    }
    // chunk-transposed copy + per-chunk sums
    for (int c = tid; c < nch; c += blockDim.x) {
        float sum = 0.0f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float4 v = reinterpret_cast<const float4*>(raw)[c * 8 + j];
            xs[j * nch + c] = v;
            sum += (v.x + v.y) + (v.z + v.w);
        }
        sumx[c] = sum;
    }
    __syncthreads();

    for (int row = row_first; row < rows; row += gridDim.x * kMvWarps) {
        const uint4* wrow = reinterpret_cast<const uint4*>(w + (size_t)row * (cols / 8));
        const uint16_t* srow = s + (size_t)row * groups;
        const uint16_t* brow = b + (size_t)row * groups;
        float acc = 0.0f;
        for (int c0 = 0; c0 < nch; c0 += 64) {
            // two chunks per lane in flight
            const int ca = c0 + lane, cb = c0 + 32 + lane;
            const bool va = ca < nch, vb = cb < nch;
            uint4 qa = make_uint4(0, 0, 0, 0), qb = qa;
            uint16_t sa = 0, ba = 0, sb = 0, bb = 0;
            if (row == row_first && c0 == 0) {
                qa = pqa; sa = psa; ba = pba;
                qb = pqb; sb = psb; bb = pbb;
            } else {
                if (va) { qa = ld_stream_u4(wrow + ca); sa = srow[ca >> 1]; ba = brow[ca >> 1]; }
                if (vb) { qb = ld_stream_u4(wrow + cb); sb = srow[cb >> 1]; bb = brow[cb >> 1]; }
            }
            if (va) {
                float4 xv[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) xv[j] = xs[j * nch + ca];
                acc += chunk_term(qa, xv, sumx[ca], sa, ba);
            }
            if (vb) {
                float4 xv[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) xv[j] = xs[j * nch + cb];
                acc += chunk_term(qb, xv, sumx[cb], sb, bb);
            }
        }
        acc = warp_sum(acc);
        if (lane == 0) y[row] = residual ? acc + residual[row] : acc;
    }
}

// ─── streaming variant for rows of 2,048 columns ────────────────────────────
// The hidden width of both reference models: gate/up rows, router rows, lm_head rows.  x is staged once per
// CTA (bulk copy, then three signed-byte digit planes per 32-element chunk as in the decode kernel: exact
// integer sums, activations kept to 23 bits relative to their chunk's maximum); every lane then keeps the
// planes of its own two chunks (one 64-column group) in registers for the whole kernel, so the row loop reads
// nothing but weights: two 128-bit loads and one scale/bias pair per lane and row, four rows in flight per warp.
constexpr int kSvCols = 2048;
constexpr int kSvWarps = 8;
constexpr int kSvUnroll = 4;

__global__ void __launch_bounds__(kSvWarps * 32, 2)
matvec_int4_stream_kernel(const uint32_t* __restrict__ w, const uint16_t* __restrict__ s, const uint16_t* __restrict__ b,
                          const float* __restrict__ x, float* __restrict__ y, int rows, unsigned int* err_flag,
                          const float* __restrict__ residual) {
    constexpr int nch = kSvCols / 32;
    __shared__ __align__(128) float raw[kSvCols];
    __shared__ __align__(16) uint4 xq[6 * nch];
    __shared__ float xdl[nch];
    __shared__ float sumx[nch];
    __shared__ uint64_t bar;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    pdl_trigger();
    if (tid == 0) {
        mbar_init(&bar, 1);
        mbar_fence_init();
    }
    // the weights do not depend on x: ask for this warp's first rows (L2) while the kernel that produces x still runs
    {
        const int row = blockIdx.x * kSvWarps + warp + lane * (int)gridDim.x * kSvWarps;
        if (lane < 16 && row < rows) {
            prefetch_l2(w + (size_t)row * (kSvCols / 8), kSvCols / 2);
            if (((reinterpret_cast<uintptr_t>(s) | reinterpret_cast<uintptr_t>(b)) & 15) == 0) {
                prefetch_l2(s + (size_t)row * (kSvCols / kGroup), kSvCols / kGroup * 2);
                prefetch_l2(b + (size_t)row * (kSvCols / kGroup), kSvCols / kGroup * 2);
            }
        }
    }
    __syncthreads();
    pdl_wait();
    if (tid == 0) {
        mbar_expect_tx(&bar, kSvCols * 4u);
        bulk_g2s(raw, x, kSvCols * 4u, &bar);
    }
    const int ok = __syncthreads_and(mbar_wait(&bar, 0) ? 1 : 0);
    if (!ok) {
        if (tid == 0) atomicExch(err_flag, 1u);
        return;
    }
#pragma unroll
    for (int it = 0; it < kSvCols / 4 / (kSvWarps * 32); ++it) {
        const int f = tid + it * kSvWarps * 32;  // float4 index: chunk f >> 3, part f & 7 (eight consecutive lanes per chunk)
        const float4 v = reinterpret_cast<const float4*>(raw)[f];
        stage_digits(xq, xdl, nch, f >> 3, f & 7, v);
        float sv = (v.x + v.y) + (v.z + v.w);
        sv += __shfl_xor_sync(0xffffffffu, sv, 1);
        sv += __shfl_xor_sync(0xffffffffu, sv, 2);
        sv += __shfl_xor_sync(0xffffffffu, sv, 4);
        if ((f & 7) == 0) sumx[f >> 3] = sv;
    }
    __syncthreads();
    // this lane's group: chunks 2 lane and 2 lane + 1
    uint4 xe[2][3], xo[2][3];
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int p = 0; p < 3; ++p) {
            xe[h][p] = xq[(p * 2 + 0) * nch + 2 * lane + h];
            xo[h][p] = xq[(p * 2 + 1) * nch + 2 * lane + h];
        }
    const float dl0 = xdl[2 * lane], dl1 = xdl[2 * lane + 1];
    const float sx = sumx[2 * lane] + sumx[2 * lane + 1];

    const int stride = gridDim.x * kSvWarps;
    for (int row0 = blockIdx.x * kSvWarps + warp; row0 < rows; row0 += stride * kSvUnroll) {
        uint4 q[kSvUnroll][2];
        uint16_t sc[kSvUnroll], bi[kSvUnroll];
#pragma unroll
        for (int u = 0; u < kSvUnroll; ++u) {
            const int row = row0 + u * stride;
            if (row < rows) {
                const uint4* wrow = reinterpret_cast<const uint4*>(w + (size_t)row * (kSvCols / 8)) + 2 * lane;
                q[u][0] = ld_stream_u4(wrow);
                q[u][1] = ld_stream_u4(wrow + 1);
                sc[u] = __ldg(s + (size_t)row * (kSvCols / kGroup) + lane);
                bi[u] = __ldg(b + (size_t)row * (kSvCols / kGroup) + lane);
            }
        }
#pragma unroll
        for (int u = 0; u < kSvUnroll; ++u) {
            const int row = row0 + u * stride;
            if (row < rows) {  // uniform per warp
                const float d = fmaf(dl0, dot32_regs(q[u][0], xe[0], xo[0]), dl1 * dot32_regs(q[u][1], xe[1], xo[1]));
                float acc = fmaf(bf16_bits_to_f32(sc[u]), d, bf16_bits_to_f32(bi[u]) * sx);
                acc = warp_sum(acc);
                if (lane == 0) y[row] = residual ? acc + residual[row] : acc;
            }
        }
    }
}

int matvec_prepare(moe_engine* e) {
    if (!e->matvec_attr_set) {  // a per-device function attribute: set once per engine
        MOE_CUDA(cudaFuncSetAttribute(matvec_int4_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 16384 * 8 + 2048));
        e->matvec_attr_set = true;
    }
    return MOE_OK;
}

int launch_matvec(moe_engine* e, const void* w, const void* s, const void* b, const float* x,
                  float* y, int32_t rows, int32_t cols) {
    return launch_matvec_res(e, w, s, b, x, y, rows, cols, nullptr);
}

int launch_matvec_res(moe_engine* e, const void* w, const void* s, const void* b, const float* x,
                      float* y, int32_t rows, int32_t cols, const float* residual, bool pdl) {
    MOE_REQUIRE(rows > 0 && cols > 0 && cols % kGroup == 0, "matvec: cols (%d) must be a positive multiple of 64", cols);
    MOE_REQUIRE(cols <= 16384, "matvec: cols (%d) above 16384 not supported", cols);
    MOE_REQUIRE((((uintptr_t)x) & 15) == 0 && (((uintptr_t)w) & 15) == 0, "matvec: x and w must be 16-byte aligned");
    if (cols == kSvCols && rows >= 4096) {
        // enough rows to stream: the register-resident variant
        int blocks = (rows + kSvWarps * kSvUnroll - 1) / (kSvWarps * kSvUnroll);
        const int cap = e->sm_count * 2;
        if (blocks > cap) blocks = cap;
        MOE_CUDA(launch_kernel(pdl, matvec_int4_stream_kernel, dim3(blocks), dim3(kSvWarps * 32), 0, e->stream, (const uint32_t*)w,
                               (const uint16_t*)s, (const uint16_t*)b, x, y, rows, e->dec_sync + 2, residual));
        e->launches++;
        return MOE_OK;
    }
    const size_t smem = (size_t)cols * 8 + (size_t)(cols / 32) * 4;
    int rc = matvec_prepare(e);
    if (rc) return rc;
    int blocks = (rows + kMvWarps - 1) / kMvWarps;
    // every CTA stages the whole x: with long rows fewer CTAs, each taking several rows per warp, amortise that better
    const int cap = e->sm_count * (cols >= 4096 ? 1 : 8);
    if (blocks > cap) blocks = cap;
    MOE_CUDA(launch_kernel(pdl, matvec_int4_kernel, dim3(blocks), dim3(kMvWarps * 32), smem, e->stream, (const uint32_t*)w,
                           (const uint16_t*)s, (const uint16_t*)b, x, y, rows, cols, e->dec_sync + 2, residual));
    e->launches++;
    return MOE_OK;
}

}  // namespace moe
