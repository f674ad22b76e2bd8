// GPU packer: f32/bf16 rows -> 4-bit words + bf16 scale + bf16 bias per 64 columns.
//
// Bit-exact restatement of quant_f32_to_int4 (reference src/dtype.rs:102-135) and
// of the expert-blob assembly in process_experts_common (reference
// src/quantize/qwen35_moe/common.rs:300-345).  HBM-bound: 2 B (bf16) or 4 B (f32)
// read and 0.5625 B written per element.
//
// Mapping: one thread owns one 64-column group, so min, max, the two IEEE divisions
// and the 64 quantisations need no cross-lane traffic.  A warp first copies its 32
// consecutive groups (4 KB of bf16, 8 KB of f32) into shared memory with coalesced
// 16-byte asynchronous copies; a pitch of one extra 16-byte unit per group makes
// both the copy and each thread's reads of its own group bank-conflict free.  All
// f32 arithmetic uses the explicitly rounded intrinsics so the compiler cannot
// contract a multiply-add: the reference computes trunc((v - min) * (1 / scale) + 0.5)
// with separately rounded operations.  bf16 sources take min and max on packed
// pairs (exact: no rounding is involved in a comparison).
#include "common.cuh"

namespace moe {

// Division of a 31-bit unsigned number by a run-time constant without a divide:
// q = (umulhi(n, mul) + n) >> shift, with shift = ceil(log2 d) and mul = floor(2^32 (2^shift - d) / d) + 1
// (Granlund-Montgomery; exact for n < 2^31, where the sum cannot overflow).
struct FastDiv {
    uint32_t mul, shift, d;
};
static FastDiv make_fastdiv(uint32_t d) {
    FastDiv f{};
    f.d = d;
    uint32_t s = 0;
    while ((1ull << s) < d) ++s;
    f.shift = s;
    f.mul = (uint32_t)((((1ull << s) - d) << 32) / d) + 1u;
    return f;
}
__device__ __forceinline__ uint32_t fdiv(uint32_t n, const FastDiv& f) { return (__umulhi(n, f.mul) + n) >> f.shift; }

struct PackJob {
    const void* src;         // [n_rows, cols], rows contiguous
    int64_t n_rows;          // total source rows
    int32_t cols;
    int64_t rows_per_unit;   // source rows per expert (plain pack: n_rows)
    int64_t rows_per_mat;    // rows of one destination matrix inside a unit
    int64_t unit_stride;     // destination bytes between units (experts)
    uint8_t* w_base[2];      // destination of matrix m of unit 0
    uint8_t* s_base[2];
    uint8_t* b_base[2];
    FastDiv div_gpr, div_unit, div_mat;  // by groups per row, rows per unit, rows per matrix (filled at launch)
    int32_t w_aligned16;     // every word destination is 16-byte aligned (filled at launch)
};

constexpr int kPackWarps = 8;            // warps per CTA
constexpr int kPackGroupsPerWarp = 32;   // one group per lane

template <bool kSrcBf16>
constexpr int pack_smem_bytes() { return kPackWarps * kPackGroupsPerWarp * ((kSrcBf16 ? 8 : 16) + 1) * 16; }

__device__ __forceinline__ void pack_cp16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}

// trunc((v - min) * inv + 0.5) as the reference rounds it, clamped to a nibble.  Rust's `as i32` truncates,
// saturates and maps NaN to 0, then clamp(0, 15): the unsigned conversion already sends everything below zero
// (and NaN) to 0, so one minimum remains.
__device__ __forceinline__ uint32_t pack_quant(float v, float fbias, float inv_scale) {
    const float t = __fadd_rn(__fmul_rn(__fsub_rn(v, fbias), inv_scale), 0.5f);
    return min(__float2uint_rz(t), 15u);
}

template <bool kSrcBf16>
__global__ void __launch_bounds__(256) pack_int4_kernel(PackJob job) {
    constexpr int kUnits = kSrcBf16 ? 8 : 16;  // 16-byte units per group
    constexpr int kPitch = kUnits + 1;
    extern __shared__ uint4 pack_stage[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    uint4* stage = pack_stage + warp * (kPackGroupsPerWarp * kPitch);
    // 32-bit index arithmetic: the host splits jobs so that a launch covers fewer than 2^31 groups
    const uint32_t groups_per_row = (uint32_t)(job.cols / kGroup);
    const uint32_t total_groups = (uint32_t)job.n_rows * groups_per_row;
    const uint32_t g_first = (blockIdx.x * kPackWarps + warp) * kPackGroupsPerWarp;
    if (g_first >= total_groups) return;
    const uint32_t n_here = min((uint32_t)kPackGroupsPerWarp, total_groups - g_first);
    {
        // source rows are contiguous, so group gi starts at element gi * 64: the warp's groups are one byte range
        const uint4* src = reinterpret_cast<const uint4*>(job.src) + (size_t)g_first * kUnits;
        const uint32_t n_units = n_here * kUnits;
#pragma unroll
        for (int i = 0; i < kUnits; ++i) {
            const uint32_t c = i * 32 + lane;
            if (c < n_units) pack_cp16(smem_u32(stage + c + c / kUnits), src + c);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncwarp();
    }
    if ((uint32_t)lane >= n_here) return;
    const uint32_t gi = g_first + lane;
    uint4 raw[kUnits];
#pragma unroll
    for (int k = 0; k < kUnits; ++k) raw[k] = stage[lane * kPitch + k];

    float gmin, gmax;
    if (kSrcBf16) {
        __nv_bfloat162 mn = *reinterpret_cast<const __nv_bfloat162*>(&raw[0].x), mx = mn;
#pragma unroll
        for (int k = 0; k < kUnits; ++k) {
            const uint32_t r[4] = {raw[k].x, raw[k].y, raw[k].z, raw[k].w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const __nv_bfloat162 w = *reinterpret_cast<const __nv_bfloat162*>(&r[i]);
                mn = __hmin2(mn, w);
                mx = __hmax2(mx, w);
            }
        }
        const uint32_t mnb = *reinterpret_cast<const uint32_t*>(&mn), mxb = *reinterpret_cast<const uint32_t*>(&mx);
        gmin = fminf(__uint_as_float(mnb << 16), __uint_as_float(mnb & 0xFFFF0000u));  // bf16 -> f32 is exact
        gmax = fmaxf(__uint_as_float(mxb << 16), __uint_as_float(mxb & 0xFFFF0000u));
    } else {
        gmin = gmax = __uint_as_float(raw[0].x);
#pragma unroll
        for (int k = 0; k < kUnits; ++k) {
            const float f[4] = {__uint_as_float(raw[k].x), __uint_as_float(raw[k].y), __uint_as_float(raw[k].z), __uint_as_float(raw[k].w)};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                gmin = fminf(gmin, f[i]);
                gmax = fmaxf(gmax, f[i]);
            }
        }
    }
    if (gmax == gmin) gmax = __fadd_rn(gmin, 1.0f);
    const float fscale = __fdiv_rn(__fsub_rn(gmax, gmin), 15.0f);
    const float inv_scale = __fdiv_rn(1.0f, fscale);
    const float fbias = gmin;

    uint32_t words[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        uint32_t word = 0;
        if (kSrcBf16) {
            const uint32_t r[4] = {raw[k].x, raw[k].y, raw[k].z, raw[k].w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                // multiply-add nibble insert (the nibbles do not overlap): one instruction, off the ALU pipe
                word = pack_quant(__uint_as_float(r[i] << 16), fbias, inv_scale) * (1u << (8 * i)) + word;
                word = pack_quant(__uint_as_float(r[i] & 0xFFFF0000u), fbias, inv_scale) * (1u << (8 * i + 4)) + word;
            }
        } else {
            const uint4 a = raw[kSrcBf16 ? 0 : 2 * k], b = raw[kSrcBf16 ? 0 : 2 * k + 1];
            const float f[8] = {__uint_as_float(a.x), __uint_as_float(a.y), __uint_as_float(a.z), __uint_as_float(a.w),
                                __uint_as_float(b.x), __uint_as_float(b.y), __uint_as_float(b.z), __uint_as_float(b.w)};
#pragma unroll
            for (int n = 0; n < 8; ++n) word = pack_quant(f[n], fbias, inv_scale) * (1u << (4 * n)) + word;
        }
        words[k] = word;
    }

    // where this group goes: (row, group in row) -> (unit, matrix, row in matrix)
    const uint32_t row = fdiv(gi, job.div_gpr);
    const uint32_t g = gi - row * groups_per_row;
    const uint32_t unit = fdiv(row, job.div_unit);
    const uint32_t rr = row - unit * (uint32_t)job.rows_per_unit;
    const uint32_t m = fdiv(rr, job.div_mat);
    const uint32_t r = rr - m * (uint32_t)job.rows_per_mat;
    const int64_t uoff = (int64_t)unit * job.unit_stride;
    // selects, not indexing: a dynamically indexed kernel parameter would be copied to local memory
    uint8_t* const wdst = (m ? job.w_base[1] : job.w_base[0]) + uoff;
    uint8_t* const sdst = (m ? job.s_base[1] : job.s_base[0]) + uoff;
    uint8_t* const bdst = (m ? job.b_base[1] : job.b_base[0]) + uoff;
    const uint64_t gq = (uint64_t)r * groups_per_row + g;  // group index inside the destination matrix
    if (job.w_aligned16) {
        uint4* const wd = reinterpret_cast<uint4*>(wdst + gq * 32);
        wd[0] = make_uint4(words[0], words[1], words[2], words[3]);
        wd[1] = make_uint4(words[4], words[5], words[6], words[7]);
    } else {
        uint32_t* const wd = reinterpret_cast<uint32_t*>(wdst + gq * 32);
#pragma unroll
        for (int k = 0; k < 8; ++k) wd[k] = words[k];
    }
    reinterpret_cast<uint16_t*>(sdst)[gq] = f32_to_bf16_ref(fscale);
    reinterpret_cast<uint16_t*>(bdst)[gq] = f32_to_bf16_ref(fbias);
}

static int run_pack_one(moe_engine* e, const PackJob& job, int src_dtype);

// Splits a job at unit boundaries so that every launch covers fewer than 2^30 groups.
static int run_pack(moe_engine* e, const PackJob& job, int src_dtype) {
    const int64_t gpr = job.cols / kGroup;
    const int64_t limit_rows = ((int64_t)1 << 30) / gpr;
    if (job.n_rows <= limit_rows) return run_pack_one(e, job, src_dtype);
    const size_t esz = src_dtype == MOE_DT_BF16 ? 2 : 4;
    if (job.unit_stride == 0) {  // plain matrix: split by rows, advancing the three outputs
        for (int64_t r0 = 0; r0 < job.n_rows; r0 += limit_rows) {
            PackJob j = job;
            j.n_rows = job.n_rows - r0 < limit_rows ? job.n_rows - r0 : limit_rows;
            j.rows_per_unit = j.rows_per_mat = j.n_rows;
            j.src = (const uint8_t*)job.src + (size_t)r0 * job.cols * esz;
            for (int m = 0; m < 2; ++m) {
                j.w_base[m] = job.w_base[m] + (size_t)r0 * (job.cols / 2);
                j.s_base[m] = job.s_base[m] + (size_t)r0 * gpr * 2;
                j.b_base[m] = job.b_base[m] + (size_t)r0 * gpr * 2;
            }
            int rc = run_pack_one(e, j, src_dtype);
            if (rc) return rc;
        }
        return MOE_OK;
    }
    const int64_t units_per = limit_rows / job.rows_per_unit > 0 ? limit_rows / job.rows_per_unit : 1;
    const int64_t n_units = job.n_rows / job.rows_per_unit;
    for (int64_t u0 = 0; u0 < n_units; u0 += units_per) {
        PackJob j = job;
        const int64_t nu = n_units - u0 < units_per ? n_units - u0 : units_per;
        j.n_rows = nu * job.rows_per_unit;
        j.src = (const uint8_t*)job.src + (size_t)u0 * job.rows_per_unit * job.cols * esz;
        for (int m = 0; m < 2; ++m) {
            j.w_base[m] = job.w_base[m] + u0 * job.unit_stride;
            j.s_base[m] = job.s_base[m] + u0 * job.unit_stride;
            j.b_base[m] = job.b_base[m] + u0 * job.unit_stride;
        }
        int rc = run_pack_one(e, j, src_dtype);
        if (rc) return rc;
    }
    return MOE_OK;
}

static int run_pack_one(moe_engine* e, const PackJob& job_in, int src_dtype) {
    PackJob job = job_in;
    const int64_t total_groups = job.n_rows * (job.cols / kGroup);
    if (total_groups == 0) return MOE_OK;
    MOE_REQUIRE(job.rows_per_unit < (1ll << 31) && job.rows_per_mat < (1ll << 31) && job.rows_per_unit > 0 && job.rows_per_mat > 0,
                "pack: unit of %lld rows is too large", (long long)job.rows_per_unit);
    job.div_gpr = make_fastdiv((uint32_t)(job.cols / kGroup));
    job.div_unit = make_fastdiv((uint32_t)job.rows_per_unit);
    job.div_mat = make_fastdiv((uint32_t)job.rows_per_mat);
    MOE_REQUIRE(((uintptr_t)job.src & 15u) == 0, "pack: the source must be 16-byte aligned");
    job.w_aligned16 = (((uintptr_t)job.w_base[0] | (uintptr_t)job.w_base[1] | (uintptr_t)job.unit_stride) & 15u) == 0;
    const int64_t per_block = (int64_t)kPackWarps * kPackGroupsPerWarp;
    const int64_t blocks = (total_groups + per_block - 1) / per_block;
    MOE_REQUIRE(blocks < (1ll << 31), "pack: too many rows for one launch (%lld blocks)", (long long)blocks);
    if (src_dtype == MOE_DT_BF16) {
        pack_int4_kernel<true><<<(unsigned)blocks, 256, pack_smem_bytes<true>(), e->stream>>>(job);
    } else {
        // above the default 48 KB of dynamic shared memory
        MOE_CUDA(cudaFuncSetAttribute(pack_int4_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, pack_smem_bytes<false>()));
        pack_int4_kernel<false><<<(unsigned)blocks, 256, pack_smem_bytes<false>(), e->stream>>>(job);
    }
    e->launches++;
    MOE_CUDA(cudaGetLastError());
    return MOE_OK;
}

int launch_pack(moe_engine* e, const void* src, int src_dtype, int64_t rows, int32_t cols,
                int64_t /*src_row_stride*/, void* w, void* s, void* b) {
    PackJob job{};
    job.src = src;
    job.n_rows = rows;
    job.cols = cols;
    job.rows_per_unit = rows > 0 ? rows : 1;
    job.rows_per_mat = job.rows_per_unit;
    job.unit_stride = 0;
    job.w_base[0] = job.w_base[1] = (uint8_t*)w;
    job.s_base[0] = job.s_base[1] = (uint8_t*)s;
    job.b_base[0] = job.b_base[1] = (uint8_t*)b;
    return run_pack(e, job, src_dtype);
}

// gate_up [n, 2I, H] -> gate (rows 0..I) and up (rows I..2I); down [n, H, I].
int launch_pack_experts(moe_engine* e, const void* gate_up, const void* down, int src_dtype,
                        int32_t n_experts, void* blob) {
    const int H = e->dims.hidden, I = e->dims.inter;
    const moe_expert_layout_t& L = e->lay;
    uint8_t* base = (uint8_t*)blob;
    PackJob gu{};
    gu.src = gate_up;
    gu.n_rows = (int64_t)n_experts * 2 * I;
    gu.cols = H;
    gu.rows_per_unit = 2 * I;
    gu.rows_per_mat = I;
    gu.unit_stride = L.expert_size;
    gu.w_base[0] = base + L.gate_w; gu.s_base[0] = base + L.gate_s; gu.b_base[0] = base + L.gate_b;
    gu.w_base[1] = base + L.up_w;   gu.s_base[1] = base + L.up_s;   gu.b_base[1] = base + L.up_b;
    int rc = run_pack(e, gu, src_dtype);
    if (rc != MOE_OK) return rc;
    PackJob dn{};
    dn.src = down;
    dn.n_rows = (int64_t)n_experts * H;
    dn.cols = I;
    dn.rows_per_unit = H;
    dn.rows_per_mat = H;
    dn.unit_stride = L.expert_size;
    dn.w_base[0] = dn.w_base[1] = base + L.down_w;
    dn.s_base[0] = dn.s_base[1] = base + L.down_s;
    dn.b_base[0] = dn.b_base[1] = base + L.down_b;
    return run_pack(e, dn, src_dtype);
}

// ─── INT8 per-row codec (lm_head of the BQ4 scheme) ─────────────────────────
// quant_f32_to_int8 (reference src/dtype.rs:164-179), bit for bit: scale = max|v| / 127 (1/127 for an all-zero
// row), q = clamp(round(v * (1 / scale)), -127, 127) with round-half-away-from-zero; one warp per row, two passes.
template <bool kSrcBf16>
__global__ void __launch_bounds__(256) pack_int8_kernel(const void* __restrict__ src, int64_t rows, int32_t cols,
                                                        int8_t* __restrict__ q, float* __restrict__ scales) {
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (row >= rows) return;
    auto load = [&](int c) -> float {
        if (kSrcBf16) return bf16_bits_to_f32(reinterpret_cast<const uint16_t*>(src)[row * cols + c]);
        return reinterpret_cast<const float*>(src)[row * cols + c];
    };
    float mx = 0.0f;
    for (int c = lane; c < cols; c += 32) mx = fmaxf(mx, fabsf(load(c)));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    const float scale = mx > 0.0f ? __fdiv_rn(mx, 127.0f) : __fdiv_rn(1.0f, 127.0f);
    const float inv = __fdiv_rn(1.0f, scale);
    if (lane == 0) scales[row] = scale;
    for (int c = lane; c < cols; c += 32) {
        const float r = roundf(__fmul_rn(load(c), inv));
        const int v = max(-127, min(127, __float2int_rz(r)));  // saturating convert, NaN -> 0, like Rust's `as i32`
        q[row * cols + c] = (int8_t)v;
    }
}

int launch_pack_int8(moe_engine* e, const void* src, int src_dtype, int64_t rows, int32_t cols, void* q, void* scales) {
    if (rows == 0) return MOE_OK;
    const int64_t blocks = (rows + 7) / 8;
    MOE_REQUIRE(blocks < (1ll << 31), "pack_int8: too many rows");
    if (src_dtype == MOE_DT_BF16)
        pack_int8_kernel<true><<<(unsigned)blocks, 256, 0, e->stream>>>(src, rows, cols, (int8_t*)q, (float*)scales);
    else
        pack_int8_kernel<false><<<(unsigned)blocks, 256, 0, e->stream>>>(src, rows, cols, (int8_t*)q, (float*)scales);
    e->launches++;
    MOE_CUDA(cudaGetLastError());
    return MOE_OK;
}

}  // namespace moe
