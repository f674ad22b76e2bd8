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
                   const uint16_t* __restrict__ b, const float* x,
                   float* __restrict__ y, int rows, int cols, unsigned int* err_flag,
                   const float* residual,  // nullable: y = W x + residual
                   // nullable: every head of hs_dim inputs is scaled by rsqrt(sum / hs_dim + 1e-6), its sum of squares being
                   // the total of the head's hs_parts entries of hs_ss (the RMS norm of a gated norm whose other factors the
                   // producer has applied already; hs_dim % 32 == 0)
                   const float* hs_ss, int hs_parts, int hs_dim,
                   int x_stride, int y_stride, int r_stride, int ss_stride) {  // per vector of a batched launch (blockIdx.y)
    x += (size_t)blockIdx.y * x_stride;
    y += (size_t)blockIdx.y * y_stride;
    if (residual) residual += (size_t)blockIdx.y * r_stride;
    if (hs_ss) hs_ss += (size_t)blockIdx.y * ss_stride;
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
    // Nothing about the weights depends on x.  Before waiting for it (and for the kernel that produces it), this warp
    // requests its first two rows' first 128 chunks into registers (rows of up to 4,096 columns: everything) and asks
    // the L2 for its later rows.
    const int groups = cols / kGroup;
    const int row_first = blockIdx.x * kMvWarps + warp;
    const int row_step = (int)gridDim.x * kMvWarps;
    constexpr int kPreRows = 2, kPreSlots = 4;  // chunk slot j of a lane is chunk 32 j + lane
    uint4 pq[kPreRows][kPreSlots];
    uint16_t ps[kPreRows][kPreSlots], pb[kPreRows][kPreSlots];
#pragma unroll
    for (int r = 0; r < kPreRows; ++r) {
        const int row = row_first + r * row_step;
#pragma unroll
        for (int j = 0; j < kPreSlots; ++j) {
            const int c = 32 * j + lane;
            pq[r][j] = make_uint4(0, 0, 0, 0);
            ps[r][j] = pb[r][j] = 0;
            if (row < rows && c < nch) {
                pq[r][j] = ld_stream_u4(reinterpret_cast<const uint4*>(w + (size_t)row * (cols / 8)) + c);
                ps[r][j] = s[(size_t)row * groups + (c >> 1)];
                pb[r][j] = b[(size_t)row * groups + (c >> 1)];
            }
        }
    }
    {
        const int row = row_first + (kPreRows + lane) * row_step;
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
    // the per-head scales of this thread's chunks (chunks tid and tid + 256: cols <= 16384), while x is on its way
    float inv_mine[2] = {1.0f, 1.0f};
    if (hs_ss) {
        const int cph = hs_dim / 32;  // chunks per head
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int c = tid + u * kMvWarps * 32;
            if (c < nch) {
                float tot = 0.0f;
                for (int k = 0; k < hs_parts; ++k) tot += hs_ss[(c / cph) * hs_parts + k];
                inv_mine[u] = 1.0f / sqrtf(tot / (float)hs_dim + 1e-6f);
            }
        }
    }
    // every thread observes the phase itself, so the copied bytes are visible to it
    const int ok = __syncthreads_and(mbar_wait(&bar, 0) ? 1 : 0);
    if (!ok) {
        if (tid == 0) atomicExch(err_flag, 1u);
        return;
    }
    if (hs_ss) {
        for (int c = tid, u = 0; c < nch; c += blockDim.x, ++u) {
            const float inv = u == 0 ? inv_mine[0] : inv_mine[1];
            float sum = 0.0f;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                float4 v = reinterpret_cast<const float4*>(raw)[c * 8 + j];
                v.x *= inv; v.y *= inv; v.z *= inv; v.w *= inv;
                xs[j * nch + c] = v;
                sum += (v.x + v.y) + (v.z + v.w);
            }
            sumx[c] = sum;
        }
    } else {
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
    }
    __syncthreads();

    int nrow = 0;
    for (int row = row_first; row < rows; row += row_step, ++nrow) {
        const uint4* wrow = reinterpret_cast<const uint4*>(w + (size_t)row * (cols / 8));
        const uint16_t* srow = s + (size_t)row * groups;
        const uint16_t* brow = b + (size_t)row * groups;
        float acc = 0.0f;
#pragma unroll 1
        for (int c0 = 0; c0 < nch; c0 += 64) {
            // two chunks per lane in flight
            const int ca = c0 + lane, cb = c0 + 32 + lane;
            const bool va = ca < nch, vb = cb < nch;
            uint4 qa = make_uint4(0, 0, 0, 0), qb = qa;
            uint16_t sa = 0, ba = 0, sb = 0, bb = 0;
            if (nrow < kPreRows && c0 < 32 * kPreSlots) {
                // (constant indices after unrolling the two cases, so the arrays stay in registers)
                if (nrow == 0) {
                    if (c0 == 0) { qa = pq[0][0]; sa = ps[0][0]; ba = pb[0][0]; qb = pq[0][1]; sb = ps[0][1]; bb = pb[0][1]; }
                    else         { qa = pq[0][2]; sa = ps[0][2]; ba = pb[0][2]; qb = pq[0][3]; sb = ps[0][3]; bb = pb[0][3]; }
                } else {
                    if (c0 == 0) { qa = pq[1][0]; sa = ps[1][0]; ba = pb[1][0]; qb = pq[1][1]; sb = ps[1][1]; bb = pb[1][1]; }
                    else         { qa = pq[1][2]; sa = ps[1][2]; ba = pb[1][2]; qb = pq[1][3]; sb = ps[1][3]; bb = pb[1][3]; }
                }
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
                          const float* x, float* __restrict__ y, int rows, unsigned int* err_flag,
                          const float* residual,
                          const uint16_t* __restrict__ norm_w,  // nullable: the input is rmsnorm(x) * norm_w (bf16), eps 1e-6
                          int x_stride, int y_stride, int r_stride) {  // per vector of a batched launch (blockIdx.y)
    x += (size_t)blockIdx.y * x_stride;
    y += (size_t)blockIdx.y * y_stride;
    if (residual) residual += (size_t)blockIdx.y * r_stride;
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
    // The weights do not depend on x.  Before waiting for it (and for the kernel that produces it) this warp requests
    // its first batch of rows into registers and asks the L2 for the rows after them.
    const int stride = gridDim.x * kSvWarps;
    const int row_first = blockIdx.x * kSvWarps + warp;
    uint4 q[kSvUnroll][2] = {};
    uint16_t sc[kSvUnroll] = {}, bi[kSvUnroll] = {};
    auto load_batch = [&](int row0) {
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
    };
    load_batch(row_first);
    {
        const int row = row_first + (kSvUnroll + lane) * stride;
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
    float inv_rms = 1.0f;
    if (norm_w) {  // rms_norm_bf16 (reference src/math_util.rs:282-288) folded in: every CTA norms the 2,048 inputs itself
        __shared__ float red[kSvWarps];
        float ss = 0.0f;
#pragma unroll
        for (int it = 0; it < kSvCols / 4 / (kSvWarps * 32); ++it) {
            const float4 v = reinterpret_cast<const float4*>(raw)[tid + it * kSvWarps * 32];
            ss = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, ss))));
        }
        ss = warp_sum(ss);
        if (lane == 0) red[warp] = ss;
        __syncthreads();
        float tot = 0.0f;
#pragma unroll
        for (int i = 0; i < kSvWarps; ++i) tot += red[i];
        inv_rms = 1.0f / sqrtf(tot / (float)kSvCols + 1e-6f);
    }
#pragma unroll
    for (int it = 0; it < kSvCols / 4 / (kSvWarps * 32); ++it) {
        const int f = tid + it * kSvWarps * 32;  // float4 index: chunk f >> 3, part f & 7 (eight consecutive lanes per chunk)
        float4 v = reinterpret_cast<const float4*>(raw)[f];
        if (norm_w) {
            const uint2 wb = __ldg(reinterpret_cast<const uint2*>(norm_w) + f);
            v.x = v.x * inv_rms * __uint_as_float(wb.x << 16);
            v.y = v.y * inv_rms * __uint_as_float(wb.x & 0xFFFF0000u);
            v.z = v.z * inv_rms * __uint_as_float(wb.y << 16);
            v.w = v.w * inv_rms * __uint_as_float(wb.y & 0xFFFF0000u);
        }
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

    for (int row0 = row_first; row0 < rows;) {
        float acc[kSvUnroll];
#pragma unroll
        for (int u = 0; u < kSvUnroll; ++u) {
            const float d = fmaf(dl0, dot32_regs(q[u][0], xe[0], xo[0]), dl1 * dot32_regs(q[u][1], xe[1], xo[1]));
            acc[u] = fmaf(bf16_bits_to_f32(sc[u]), d, bf16_bits_to_f32(bi[u]) * sx);
        }
        const int done0 = row0;
        row0 += stride * kSvUnroll;
        if (row0 < rows) load_batch(row0);  // the next batch is on its way while this one is reduced and stored
#pragma unroll
        for (int u = 0; u < kSvUnroll; ++u) {
            const int row = done0 + u * stride;
            if (row < rows) {  // uniform per warp
                const float a = warp_sum(acc[u]);
                if (lane == 0) y[row] = residual ? a + residual[row] : a;
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

// y = W (x scaled per head) + residual: head h of head_dim inputs is multiplied by rsqrt(sum_h / head_dim + 1e-6), sum_h being
// the total of ss[h * parts .. h * parts + parts): the last step of an RMS norm whose sums the producer left in `ss`
bool matvec_folds_head_scale(int32_t rows, int32_t cols, int32_t head_dim) {
    return !matvec_folds_norm(rows, cols) && head_dim > 0 && head_dim % 32 == 0 && cols % head_dim == 0 && cols <= 16384;
}
int launch_matvec_head_scaled(moe_engine* e, const void* w, const void* s, const void* b, const float* x, const float* ss,
                              int32_t parts, int32_t head_dim, float* y, int32_t rows, int32_t cols, const float* residual,
                              bool pdl, MvBatch mb) {
    MOE_REQUIRE(rows > 0 && cols > 0 && cols % kGroup == 0 && parts > 0 && matvec_folds_head_scale(rows, cols, head_dim),
                "matvec: cannot fold a norm of %d-element heads into a %d x %d product", head_dim, rows, cols);
    MOE_REQUIRE((((uintptr_t)x) & 15) == 0 && (((uintptr_t)w) & 15) == 0, "matvec: x and w must be 16-byte aligned");
    const size_t smem = (size_t)cols * 8 + (size_t)(cols / 32) * 4;
    int rc = matvec_prepare(e);
    if (rc) return rc;
    int blocks = (rows + kMvWarps - 1) / kMvWarps;
    const int cap = e->sm_count * (cols >= 4096 ? 1 : 8);
    if (blocks > cap) blocks = cap;
    MOE_REQUIRE(mb.n >= 1 && mb.n <= 65535, "matvec: %d vectors in one launch", mb.n);
    blocks = matvec_batch_blocks(e, blocks, mb.n);
    MOE_CUDA(launch_kernel(pdl, matvec_int4_kernel, dim3(blocks, mb.n), dim3(kMvWarps * 32), smem, e->stream, (const uint32_t*)w,
                           (const uint16_t*)s, (const uint16_t*)b, x, y, rows, cols, e->dec_sync + 2, residual, ss, parts, head_dim,
                           mb.x_stride, mb.y_stride, mb.r_stride, mb.ss_stride));
    e->launches++;
    return MOE_OK;
}

bool matvec_folds_norm(int32_t rows, int32_t cols) { return cols == kSvCols && rows >= 4096; }

// CTAs per vector of a batched launch: every CTA stages its vector once, so with many vectors fewer CTAs, each with more
// rows, spread that cost; about four CTAs per SM over the whole launch keep the device busy
int matvec_batch_blocks(const moe_engine* e, int blocks, int n) {
    if (n <= 1) return blocks;
    int per = (4 * e->sm_count + n - 1) / n;
    if (per < 8) per = 8;
    return blocks < per ? blocks : per;
}

int launch_matvec_res(moe_engine* e, const void* w, const void* s, const void* b, const float* x,
                      float* y, int32_t rows, int32_t cols, const float* residual, bool pdl, const void* norm_w, MvBatch mb) {
    MOE_REQUIRE(mb.n >= 1 && mb.n <= 65535, "matvec: %d vectors in one launch", mb.n);
    MOE_REQUIRE(rows > 0 && cols > 0 && cols % kGroup == 0, "matvec: cols (%d) must be a positive multiple of 64", cols);
    MOE_REQUIRE(cols <= 16384, "matvec: cols (%d) above 16384 not supported", cols);
    MOE_REQUIRE((((uintptr_t)x) & 15) == 0 && (((uintptr_t)w) & 15) == 0, "matvec: x and w must be 16-byte aligned");
    MOE_REQUIRE(!norm_w || (matvec_folds_norm(rows, cols) && (((uintptr_t)norm_w) & 7) == 0),
                "matvec: the input norm can only be folded into the streaming kernel (2048 columns, >= 4096 rows)");
    if (matvec_folds_norm(rows, cols)) {
        // enough rows to stream: the register-resident variant
        int blocks = (rows + kSvWarps * kSvUnroll - 1) / (kSvWarps * kSvUnroll);
        const int cap = e->sm_count * 2;
        if (blocks > cap) blocks = cap;
        blocks = matvec_batch_blocks(e, blocks, mb.n);
        MOE_CUDA(launch_kernel(pdl, matvec_int4_stream_kernel, dim3(blocks, mb.n), dim3(kSvWarps * 32), 0, e->stream, (const uint32_t*)w,
                               (const uint16_t*)s, (const uint16_t*)b, x, y, rows, e->dec_sync + 2, residual,
                               (const uint16_t*)norm_w, mb.x_stride, mb.y_stride, mb.r_stride));
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
    blocks = matvec_batch_blocks(e, blocks, mb.n);
    MOE_CUDA(launch_kernel(pdl, matvec_int4_kernel, dim3(blocks, mb.n), dim3(kMvWarps * 32), smem, e->stream, (const uint32_t*)w,
                           (const uint16_t*)s, (const uint16_t*)b, x, y, rows, cols, e->dec_sync + 2, residual,
                           (const float*)nullptr, 0, 0, mb.x_stride, mb.y_stride, mb.r_stride, 0));
    e->launches++;
    return MOE_OK;
}

}  // namespace moe
