/* Bench and test tooling exported by libmoe_b200.so next to the product ABI (include/moe_b200.h):
 * a seeded device-side fill, CUDA-event timing on the engine's stream and a launch counter.
 * None of these has a counterpart in the reference; no product path depends on them. */
#ifndef MOE_B200_BENCH_H
#define MOE_B200_BENCH_H

#include "moe_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

/* ── synthetic data ──────────────────────────────────────────────────────────
 * No counterpart in the reference (it reads real checkpoints): fills a device
 * buffer with seeded N(0, sigma^2) values, a fraction `outlier_frac` of them
 * replaced by +-outlier_value; f32 or bf16.  Used to build synthetic
 * checkpoints of the reference's shapes for benchmarks and full-size tests. */
int moe_synth_normal_dev(moe_engine_t* e, void* dst_dev, int dtype, int64_t n, uint64_t seed, float sigma,
                         float outlier_frac, float outlier_value);

/* CUDA-event timing on the engine's stream: elapsed milliseconds between
 * moe_timer_start and moe_timer_stop (stop waits for the stream). */
int moe_timer_start(moe_engine_t* e);
int moe_timer_stop(moe_engine_t* e, float* ms);
/* Number of kernels this library has launched on the engine since creation. */
int moe_launch_count(const moe_engine_t* e, int64_t* n);

#ifdef __cplusplus
}
#endif
#endif /* MOE_B200_BENCH_H */
