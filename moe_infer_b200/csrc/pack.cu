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
};

template <bool kSrcBf16>
__global__ void __launch_bounds__(256) pack_int4_kernel(PackJob job) {
    const int groups_per_row = job.cols / kGroup;
    const int64_t total_groups = job.n_rows * groups_per_row;
    const int64_t gi = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 3;
    const int p = threadIdx.x & 7;
    if (gi >= total_groups) return;  // whole 8-lane groups leave together
    const int64_t row = gi / groups_per_row;
    const int g = (int)(gi - row * groups_per_row);

    float v[8];
    if (kSrcBf16) {
        const uint4 raw = *reinterpret_cast<const uint4*>(
            reinterpret_cast<const uint16_t*>(job.src) + row * job.cols + g * kGroup + p * 8);
        const uint32_t r[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            v[2 * i] = __uint_as_float(r[i] << 16);            // bf16 -> f32 is exact
            v[2 * i + 1] = __uint_as_float(r[i] & 0xFFFF0000u);
        }
    } else {
        const float4* sp = reinterpret_cast<const float4*>(
            reinterpret_cast<const float*>(job.src) + row * job.cols + g * kGroup + p * 8);
        const float4 a = sp[0], b = sp[1];
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
        v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    }

    float vmin = v[0], vmax = v[0];
#pragma unroll
    for (int i = 1; i < 8; ++i) {
        vmin = fminf(vmin, v[i]);
        vmax = fmaxf(vmax, v[i]);
    }
    // Lanes of one group are 8-aligned inside the warp; all 32 lanes of a warp
    // are either all in range or leave together only per 8-lane group, so the
    // shuffle mask names just this group's lanes.
    const unsigned gmask = 0xFFu << (threadIdx.x & 24);
#pragma unroll
    for (int o = 1; o < 8; o <<= 1) {
        vmin = fminf(vmin, __shfl_xor_sync(gmask, vmin, o));
        vmax = fmaxf(vmax, __shfl_xor_sync(gmask, vmax, o));
    }
    if (vmax == vmin) vmax = __fadd_rn(vmin, 1.0f);
    const float fscale = __fdiv_rn(__fsub_rn(vmax, vmin), 15.0f);
    const float fbias = vmin;
    const float inv_scale = __fdiv_rn(1.0f, fscale);

    uint32_t word = 0;
#pragma unroll
    for (int n = 0; n < 8; ++n) {
        const float t = __fadd_rn(__fmul_rn(__fsub_rn(v[n], fbias), inv_scale), 0.5f);
        int q = __float2int_rz(t);  // truncates, saturates, NaN -> 0: Rust `as i32`
        q = min(max(q, 0), 15);
        word |= ((uint32_t)q) << (n * 4);
    }

    const int64_t unit = row / job.rows_per_unit;
    const int64_t rr = row - unit * job.rows_per_unit;
    const int m = (int)(rr / job.rows_per_mat);
    const int64_t r = rr - m * job.rows_per_mat;
    const int64_t uoff = unit * job.unit_stride;
    // selects, not indexing: a dynamically indexed kernel parameter would be copied to local memory
    uint8_t* const wb = m ? job.w_base[1] : job.w_base[0];
    uint8_t* const sb = m ? job.s_base[1] : job.s_base[0];
    uint8_t* const bb = m ? job.b_base[1] : job.b_base[0];
    uint32_t* wp = reinterpret_cast<uint32_t*>(wb + uoff) + r * (job.cols / 8) + g * 8 + p;
    *wp = word;
    if (p == 0)
        reinterpret_cast<uint16_t*>(sb + uoff)[r * groups_per_row + g] = f32_to_bf16_ref(fscale);
    if (p == 1)
        reinterpret_cast<uint16_t*>(bb + uoff)[r * groups_per_row + g] = f32_to_bf16_ref(fbias);
}

static int run_pack(moe_engine* e, const PackJob& job, int src_dtype) {
    const int64_t total_groups = job.n_rows * (job.cols / kGroup);
    if (total_groups == 0) return MOE_OK;
    const int64_t threads = total_groups * 8;
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

}  // namespace moe
