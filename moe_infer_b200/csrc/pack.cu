// GPU packer: f32/bf16 rows -> 4-bit words + bf16 scale + bf16 bias per 64 columns.
//
// Bit-exact restatement of quant_f32_to_int4 (reference src/dtype.rs:102-135) and
// of the expert-blob assembly in process_experts_common (reference
// src/quantize/qwen35_moe/common.rs:300-345).  HBM-bound: 2 B (bf16) or 4 B (f32)
// read and 0.5625 B written per element.
//
// Mapping: eight consecutive lanes own one 64-column group; lane p of the eight
// owns word p (columns p*8 .. p*8+7).  Min/max cross the eight lanes with three
// xor-shuffles.  All f32 arithmetic uses the explicitly rounded intrinsics so the
// compiler cannot contract a multiply-add: the reference computes
// trunc((v - min) * (1 / scale) + 0.5) with separately rounded operations.
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
};

constexpr int kPackUnroll = 4;  // groups per 8-lane team: their loads are all issued before the first use

template <bool kSrcBf16>
__global__ void __launch_bounds__(256) pack_int4_kernel(PackJob job) {
    // 32-bit index arithmetic: the host splits jobs so that a launch covers fewer than 2^31 groups
    const uint32_t groups_per_row = (uint32_t)(job.cols / kGroup);
    const uint32_t total_groups = (uint32_t)job.n_rows * groups_per_row;
    // a team of 8 lanes takes kPackUnroll consecutive groups: gi0 .. gi0 + kPackUnroll - 1
    const uint32_t team = (blockIdx.x * blockDim.x + threadIdx.x) >> 3;
    const uint32_t gi0 = team * kPackUnroll;
    const int p = threadIdx.x & 7;
    // Lanes of one team are 8-aligned inside the warp and take the same branches,
    // so the shuffle mask names just this team's lanes.
    const unsigned gmask = 0xFFu << (threadIdx.x & 24);

    uint4 raw[kPackUnroll][kSrcBf16 ? 1 : 2];
#pragma unroll
    for (int u = 0; u < kPackUnroll; ++u) {
        const uint32_t gi = gi0 + u;
        if (gi < total_groups) {
            // source rows are contiguous, so group gi starts at element gi * 64
            if (kSrcBf16) {
                raw[u][0] = ld_stream_u4(reinterpret_cast<const uint16_t*>(job.src) + (size_t)gi * kGroup + p * 8);
            } else {
                const float* sp = reinterpret_cast<const float*>(job.src) + (size_t)gi * kGroup + p * 8;
                raw[u][0] = ld_stream_u4(sp);
                raw[u][kSrcBf16 ? 0 : 1] = ld_stream_u4(sp + 4);
            }
        }
    }
    // pass 1: widen, and reduce min / max over each group (8 lanes, three xor-shuffles)
    float v[kPackUnroll][8], gmin[kPackUnroll], gmax[kPackUnroll];
#pragma unroll
    for (int u = 0; u < kPackUnroll; ++u) {
        if (kSrcBf16) {
            const uint32_t r[4] = {raw[u][0].x, raw[u][0].y, raw[u][0].z, raw[u][0].w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                v[u][2 * i] = __uint_as_float(r[i] << 16);            // bf16 -> f32 is exact
                v[u][2 * i + 1] = __uint_as_float(r[i] & 0xFFFF0000u);
            }
        } else {
            const uint4 a = raw[u][0], b = raw[u][kSrcBf16 ? 0 : 1];
            v[u][0] = __uint_as_float(a.x); v[u][1] = __uint_as_float(a.y); v[u][2] = __uint_as_float(a.z); v[u][3] = __uint_as_float(a.w);
            v[u][4] = __uint_as_float(b.x); v[u][5] = __uint_as_float(b.y); v[u][6] = __uint_as_float(b.z); v[u][7] = __uint_as_float(b.w);
        }
        float vmin = v[u][0], vmax = v[u][0];
#pragma unroll
        for (int i = 1; i < 8; ++i) {
            vmin = fminf(vmin, v[u][i]);
            vmax = fmaxf(vmax, v[u][i]);
        }
#pragma unroll
        for (int o = 1; o < 8; o <<= 1) {
            vmin = fminf(vmin, __shfl_xor_sync(gmask, vmin, o));
            vmax = fmaxf(vmax, __shfl_xor_sync(gmask, vmax, o));
        }
        gmin[u] = vmin;
        gmax[u] = vmax;
    }
    // pass 2: the two IEEE divisions of a group are done once, by lane u of its team (lane u takes group u),
    // and handed to the other seven lanes by shuffle: a division costs a dozen instructions
    static_assert(kPackUnroll <= 8, "one lane of the team per unrolled group");
    float my_min = gmin[0], my_max = gmax[0];
#pragma unroll
    for (int u = 1; u < kPackUnroll; ++u)
        if (p == u) { my_min = gmin[u]; my_max = gmax[u]; }
    if (my_max == my_min) my_max = __fadd_rn(my_min, 1.0f);
    const float my_scale = __fdiv_rn(__fsub_rn(my_max, my_min), 15.0f);
    const float my_inv = __fdiv_rn(1.0f, my_scale);
    const int team_lane0 = threadIdx.x & 24;  // first lane of this team inside the warp
    // pass 3: quantise and store.  (row, group in row) of the first group by division, of the others by stepping.
    uint32_t row = fdiv(gi0, job.div_gpr);
    uint32_t g = gi0 - row * groups_per_row;
    // where a row's groups go: recomputed only when the row changes
    uint8_t *wdst = nullptr, *sdst = nullptr, *bdst = nullptr;  // destination matrices of this row, at its unit
    uint64_t gq0 = 0;                                            // index of the row's first group inside them
    auto locate = [&]() {
        const uint32_t unit = fdiv(row, job.div_unit);
        const uint32_t rr = row - unit * (uint32_t)job.rows_per_unit;
        const uint32_t m = fdiv(rr, job.div_mat);
        const uint32_t r = rr - m * (uint32_t)job.rows_per_mat;
        const int64_t uoff = (int64_t)unit * job.unit_stride;
        // selects, not indexing: a dynamically indexed kernel parameter would be copied to local memory
        wdst = (m ? job.w_base[1] : job.w_base[0]) + uoff;
        sdst = (m ? job.s_base[1] : job.s_base[0]) + uoff;
        bdst = (m ? job.b_base[1] : job.b_base[0]) + uoff;
        gq0 = (uint64_t)r * groups_per_row;
    };
    locate();
#pragma unroll
    for (int u = 0; u < kPackUnroll; ++u) {
        const float fscale = __shfl_sync(gmask, my_scale, team_lane0 + u);
        const float inv_scale = __shfl_sync(gmask, my_inv, team_lane0 + u);
        if (u > 0 && ++g == groups_per_row) { g = 0; ++row; locate(); }
        const uint32_t gi = gi0 + u;
        if (gi >= total_groups) continue;
        const float fbias = gmin[u];
        uint32_t word = 0;
#pragma unroll
        for (int n = 0; n < 8; ++n) {
            const float t = __fadd_rn(__fmul_rn(__fsub_rn(v[u][n], fbias), inv_scale), 0.5f);
            // Rust `as i32` truncates, saturates and maps NaN to 0, then clamp(0, 15): the unsigned conversion
            // already sends everything below zero (and NaN) to 0, so one minimum remains
            const uint32_t q = min(__float2uint_rz(t), 15u);
            word = q * (1u << (n * 4)) + word;  // multiply-add (the nibbles do not overlap): one instruction, off the ALU pipe
        }
        const uint64_t gq = gq0 + g;  // group index inside the destination matrix
        reinterpret_cast<uint32_t*>(wdst)[gq * 8 + p] = word;
        // lane 0 writes the scale, lane 1 the bias: one conversion and one store per lane
        const float sv = p == 0 ? fscale : fbias;
        uint8_t* const dst = p == 0 ? sdst : bdst;
        if (p < 2) reinterpret_cast<uint16_t*>(dst)[gq] = f32_to_bf16_ref(sv);
    }
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
    const int64_t threads = (total_groups + kPackUnroll - 1) / kPackUnroll * 8;
    const int64_t blocks = (threads + 255) / 256;
    MOE_REQUIRE(blocks < (1ll << 31), "pack: too many rows for one launch (%lld blocks)", (long long)blocks);
    if (src_dtype == MOE_DT_BF16)
        pack_int4_kernel<true><<<(unsigned)blocks, 256, 0, e->stream>>>(job);
    else
        pack_int4_kernel<false><<<(unsigned)blocks, 256, 0, e->stream>>>(job);
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
