// Seeded N(0, sigma^2) fill of a device buffer (f32 or bf16), for synthetic
// checkpoints in benchmarks and tests.  No counterpart in the reference (its
// inputs are real checkpoints); counter-based, so the values do not depend on
// the launch shape.
#include "common.cuh"

namespace moe {

__device__ __forceinline__ uint64_t mix64(uint64_t z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

// Elements 2i and 2i+1 come from one Box-Muller pair keyed by (seed, i).
template <bool kBf16>
__global__ void __launch_bounds__(256) synth_normal_kernel(void* dst, int64_t n, uint64_t seed, float sigma,
                                                           float outlier_frac, float outlier_value) {
    const int64_t pairs = (n + 1) / 2;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < pairs;
         i += (int64_t)gridDim.x * blockDim.x) {
        const uint64_t r = mix64(seed * 0xD1342543DE82EF95ull + (uint64_t)i);
        const float u1 = ((uint32_t)(r >> 40) + 1.0f) * (1.0f / 16777217.0f);  // (0, 1]
        const float u2 = (uint32_t)((r >> 8) & 0xFFFFFFu) * (1.0f / 16777216.0f);
        const float rad = sqrtf(-2.0f * logf(u1)) * sigma;
        float s, c;
        sincospif(2.0f * u2, &s, &c);
        float v[2] = {rad * c, rad * s};
        if (outlier_frac > 0.0f) {
            const uint64_t q = mix64(r ^ 0xA5A5A5A5A5A5A5A5ull);
#pragma unroll
            for (int k = 0; k < 2; ++k) {
                const uint32_t h = (uint32_t)(q >> (32 * k));
                if ((h >> 8) * (1.0f / 16777216.0f) < outlier_frac) v[k] = (h & 1u) ? outlier_value : -outlier_value;
            }
        }
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            const int64_t j = 2 * i + k;
            if (j < n) {
                if (kBf16) reinterpret_cast<__nv_bfloat16*>(dst)[j] = __float2bfloat16_rn(v[k]);
                else reinterpret_cast<float*>(dst)[j] = v[k];
            }
        }
    }
}

}  // namespace moe

using namespace moe;

extern "C" int moe_synth_normal_dev(moe_engine_t* e, void* dst_dev, int dtype, int64_t n, uint64_t seed, float sigma,
                                    float outlier_frac, float outlier_value) {
    MOE_REQUIRE(e && dst_dev, "null argument");
    MOE_REQUIRE(dtype == MOE_DT_F32 || dtype == MOE_DT_BF16, "synth: dtype must be f32 or bf16");
    MOE_REQUIRE(n >= 0, "synth: negative count");
    if (n == 0) return MOE_OK;
    const int blocks = e->sm_count * 8;
    if (dtype == MOE_DT_BF16)
        synth_normal_kernel<true><<<blocks, 256, 0, e->stream>>>(dst_dev, n, seed, sigma, outlier_frac, outlier_value);
    else
        synth_normal_kernel<false><<<blocks, 256, 0, e->stream>>>(dst_dev, n, seed, sigma, outlier_frac, outlier_value);
    e->launches++;
    MOE_CUDA(cudaGetLastError());
    return MOE_OK;
}
