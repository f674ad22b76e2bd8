// The MTP block's attention half, batch-1 decode: one gated full-attention layer with per-head q/k RMS norm,
// partial interleaved RoPE and an f32 KV cache (reference src/engine/qwen35_moe/mtp.rs:58-225), wrapped around
// the MoE half that the decode kernel already runs (layer index num_layers), the token embedding and the head.
//
// Everything here is a matrix-vector product or smaller: HBM-bound streaming kernels and a few tiny ones.
// Projections are bf16 matrices in the BQ4 scheme (bq4.rs:25-32) and 4-bit triples in the INT4 scheme.
#include "common.cuh"
#include "stage.cuh"

namespace moe {

// ─── y = W x, W bf16 [rows, cols], f32 accumulate ────────────────────────────
// One warp per row, two rows in flight; a lane reads 16 bytes (8 weights) per step; x is staged in shared memory.
// 2 B per weight: bound by HBM bandwidth like the 4-bit matvec.
constexpr int kBfWarps = 8;

__global__ void __launch_bounds__(kBfWarps * 32) matvec_bf16_kernel(const uint16_t* __restrict__ w, const float* x,
                                                                   float* __restrict__ y, int rows, int cols,
                                                                   const float* residual,  // nullable: y = W x + residual
                                                                   const uint16_t* __restrict__ norm_w,  // nullable: x <- rmsnorm(x) * norm_w
                                                                   int x_stride, int y_stride, int r_stride) {  // per vector (blockIdx.y)
    extern __shared__ float xs[];
    x += (size_t)blockIdx.y * x_stride;
    y += (size_t)blockIdx.y * y_stride;
    if (residual) residual += (size_t)blockIdx.y * r_stride;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int stride = gridDim.x * kBfWarps * 2;
    pdl_trigger();
    // the weights do not depend on x: ask for this warp's rows (L2) while the kernel that produces x still runs
    if ((cols & 7) == 0) {
        const int r = (blockIdx.x * kBfWarps + warp) * 2 + (lane >> 1) * stride + (lane & 1);
        if (lane < 16 && r < rows) {
            const unsigned char* wr = reinterpret_cast<const unsigned char*>(w + (size_t)r * cols);
            for (int off = 0; off < cols * 2; off += 4096) prefetch_l2(wr + off, (uint32_t)min(4096, cols * 2 - off));
        }
    }
    // ... and the first 16-byte steps of its first row pair go into registers before x is waited for
    constexpr int kBfPre = 4;
    const int r_first = (blockIdx.x * kBfWarps + warp) * 2;
    uint4 pa[kBfPre], pb[kBfPre];
#pragma unroll
    for (int j = 0; j < kBfPre; ++j) {
        const int c = lane * 8 + j * 256;
        pa[j] = pb[j] = make_uint4(0, 0, 0, 0);
        if (r_first < rows && c < cols) {
            pa[j] = ld_stream_u4(w + (size_t)r_first * cols + c);
            pb[j] = ld_stream_u4(w + (size_t)(r_first + 1 < rows ? r_first + 1 : r_first) * cols + c);
        }
    }
    pdl_wait();
    float ss = 0.0f;
    for (int i = threadIdx.x; i < cols; i += blockDim.x) {
        const float v = x[i];
        xs[i] = v;
        ss = fmaf(v, v, ss);
    }
    if (norm_w) {  // rms_norm_bf16 (reference src/math_util.rs:282-288) folded in: every CTA norms the input itself
        __shared__ float red[kBfWarps];
        ss = warp_sum(ss);
        if (lane == 0) red[warp] = ss;
        __syncthreads();
        float tot = 0.0f;
#pragma unroll
        for (int i = 0; i < kBfWarps; ++i) tot += red[i];
        const float inv_rms = 1.0f / sqrtf(tot / (float)cols + 1e-6f);
        for (int i = threadIdx.x; i < cols; i += blockDim.x) xs[i] = xs[i] * inv_rms * bf16_bits_to_f32(norm_w[i]);
    }
    __syncthreads();
    for (int r0 = (blockIdx.x * kBfWarps + warp) * 2; r0 < rows; r0 += stride) {
        const bool two = r0 + 1 < rows;
        const uint16_t* wa = w + (size_t)r0 * cols;
        const uint16_t* wb = w + (size_t)(two ? r0 + 1 : r0) * cols;
        float a0 = 0.0f, a1 = 0.0f;
        auto step = [&](int c, const uint4 qa, const uint4 qb) {
            const float4 x0 = *reinterpret_cast<const float4*>(xs + c), x1 = *reinterpret_cast<const float4*>(xs + c + 4);
            const uint32_t ra[4] = {qa.x, qa.y, qa.z, qa.w}, rb[4] = {qb.x, qb.y, qb.z, qb.w};
            const float xv[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                a0 = fmaf(__uint_as_float(ra[i] << 16), xv[2 * i], a0);
                a0 = fmaf(__uint_as_float(ra[i] & 0xFFFF0000u), xv[2 * i + 1], a0);
                a1 = fmaf(__uint_as_float(rb[i] << 16), xv[2 * i], a1);
                a1 = fmaf(__uint_as_float(rb[i] & 0xFFFF0000u), xv[2 * i + 1], a1);
            }
        };
        int c = lane * 8;
        if (r0 == r_first) {
#pragma unroll
            for (int j = 0; j < kBfPre; ++j, c += 256)
                if (c < cols) step(c, pa[j], pb[j]);
        }
#pragma unroll 8
        for (; c < cols; c += 256) step(c, ld_stream_u4(wa + c), ld_stream_u4(wb + c));
        a0 = warp_sum(a0);
        a1 = warp_sum(a1);
        if (lane == 0) {
            y[r0] = residual ? a0 + residual[r0] : a0;
            if (two) y[r0 + 1] = residual ? a1 + residual[r0 + 1] : a1;
        }
    }
}

// ─── RMS norm of `rows` vectors of `dim` elements with one bf16 weight vector (rms_norm, mtp.rs:261-266) ─────
__global__ void __launch_bounds__(256) rms_norm_rows_kernel(const float* x, const uint16_t* __restrict__ w, int dim,
                                                            float* __restrict__ out) {
    __shared__ float red[8];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float* row = x + (size_t)blockIdx.x * dim;
    pdl_trigger();
    pdl_wait();
    float ss = 0.0f;
    for (int i = tid; i < dim; i += 256) ss = fmaf(row[i], row[i], ss);
    ss = warp_sum(ss);
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    float tot = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) tot += red[i];
    const float inv_rms = 1.0f / sqrtf(tot / (float)dim + 1e-6f);  // RMS_NORM_EPS
    for (int i = tid; i < dim; i += 256) out[(size_t)blockIdx.x * dim + i] = row[i] * inv_rms * bf16_bits_to_f32(w[i]);
}

// ─── per-head norm + RoPE of q and k, K/V cache append ───────────────────────────────────────────────────────
// Block h < num_heads: query head h -> q_out.  Block num_heads + j: key head j -> k_cache[pos], and value head j
// is copied to v_cache[pos].  Two conventions exist in the reference:
//   * the MTP block (mtp.rs:137-157, 268-303): the q projection is [all heads | all gates] (q_stride = head_dim) and
//     RoPE rotates the interleaved pairs (2i, 2i+1), i < rope_dim / 2;
//   * the main model's full-attention layers (src/math_util.rs:501-597): the q projection is [head, gate] per head
//     (q_stride = 2 * head_dim) and RoPE rotates the pairs (i, i + rope_dim / 2).
// Either way the angle of pair i is pos * theta^(-2i / rope_dim).
__global__ void __launch_bounds__(256) attn_prep_kernel(const float* q, int q_stride, int rope_half_split,
                                                        const float* k,
                                                        const float* v, const uint16_t* __restrict__ q_norm,
                                                        const uint16_t* __restrict__ k_norm, int num_heads, int num_kv_heads,
                                                        int head_dim, int rope_dim, int pos_value, const int* __restrict__ pos_ptr,
                                                        float theta, float* __restrict__ q_out,
                                                        float* __restrict__ k_cache, float* __restrict__ v_cache,
                                                        int tok_stride) {  // several tokens in one launch: blockIdx.y, consecutive positions
    pdl_trigger();
    pdl_wait();
    q += (size_t)blockIdx.y * tok_stride;
    k += (size_t)blockIdx.y * tok_stride;
    v += (size_t)blockIdx.y * tok_stride;
    q_out += (size_t)blockIdx.y * tok_stride;
    const int pos = (pos_ptr ? *pos_ptr : pos_value) + (int)blockIdx.y;  // a device-side position keeps the launch replayable (CUDA graph)
    extern __shared__ float hv[];  // the normed head
    __shared__ float red[8];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const bool is_q = (int)blockIdx.x < num_heads;
    const int h = is_q ? blockIdx.x : blockIdx.x - num_heads;
    const float* src = is_q ? q + (size_t)h * q_stride : k + (size_t)h * head_dim;
    const uint16_t* nw = is_q ? q_norm : k_norm;
    const size_t kv_dim = (size_t)num_kv_heads * head_dim;
    float* dst = is_q ? q_out + (size_t)h * head_dim : k_cache + (size_t)pos * kv_dim + (size_t)h * head_dim;
    float ss = 0.0f;
    for (int i = tid; i < head_dim; i += 256) ss = fmaf(src[i], src[i], ss);
    ss = warp_sum(ss);
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    float tot = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) tot += red[i];
    const float inv_rms = 1.0f / sqrtf(tot / (float)head_dim + 1e-6f);
    for (int i = tid; i < head_dim; i += 256) hv[i] = src[i] * inv_rms * bf16_bits_to_f32(nw[i]);
    __syncthreads();
    for (int i = tid; i < head_dim; i += 256) {
        float o = hv[i];
        if (i < rope_dim) {
            const int half = rope_dim >> 1;
            const int p = rope_half_split ? (i < half ? i : i - half) : (i >> 1);
            const bool second = rope_half_split ? (i >= half) : ((i & 1) != 0);
            const float freq = powf(theta, -2.0f * (float)p / (float)rope_dim);
            float sn, cs;
            sincosf((float)pos * freq, &sn, &cs);
            const float x0 = hv[rope_half_split ? p : 2 * p], x1 = hv[rope_half_split ? p + half : 2 * p + 1];
            o = second ? x0 * sn + x1 * cs : x0 * cs - x1 * sn;
        }
        dst[i] = o;
    }
    if (!is_q) {
        const float* vs = v + (size_t)h * head_dim;
        float* vd = v_cache + (size_t)pos * kv_dim + (size_t)h * head_dim;
        for (int i = tid; i < head_dim; i += 256) vd[i] = vs[i];
    }
}

// ─── attention of one query position over the cache, output gate (cpu_attention + gate, mtp.rs:160-169, 305-352) ─
// One CTA per query head.  Scores: a warp per cached position (lanes stride the head), scaled, max-subtracted,
// exponentiated, summed.  Values: the positions are dealt to the warps as well; a lane owns head elements lane, lane +
// 32, ... (coalesced rows of V), keeps several positions' loads in flight, and the warps' partial sums meet in shared
// memory.  out = attention * sigmoid(gate).
constexpr int kAttnWarps = 8;
constexpr int kAttnPerLane = 8;   // head_dim <= 256
constexpr int kAttnInflight = 4;  // positions a warp has in flight in the value pass

__global__ void __launch_bounds__(kAttnWarps * 32) attn_decode_kernel(const float* q, const float* k_cache,
                                                          const float* v_cache, const float* gate,
                                                          int gate_stride, int num_heads, int num_kv_heads, int head_dim, int seq_value,
                                                          const int* __restrict__ pos_ptr, float kq_scale, float* __restrict__ out,
                                                          int tok_stride) {  // several tokens in one launch: blockIdx.y, each over its own prefix
    pdl_trigger();
    pdl_wait();
    q += (size_t)blockIdx.y * tok_stride;
    gate += (size_t)blockIdx.y * tok_stride;
    out += (size_t)blockIdx.y * tok_stride;
    const int seq_len = (pos_ptr ? *pos_ptr + 1 : seq_value) + (int)blockIdx.y;
    extern __shared__ float sc[];  // [seq_len] scores, then [head_dim] the query head, then [warps][head_dim] partial outputs
    __shared__ float red[kAttnWarps];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int h = blockIdx.x, kv_h = h / (num_heads / num_kv_heads);
    const size_t kv_dim = (size_t)num_kv_heads * head_dim;
    float* qs = sc + seq_len;
    float* part = qs + head_dim;
    for (int i = tid; i < head_dim; i += kAttnWarps * 32) qs[i] = q[(size_t)h * head_dim + i];
    __syncthreads();
    float qreg[kAttnPerLane];
#pragma unroll
    for (int j = 0; j < kAttnPerLane; ++j) qreg[j] = lane + 32 * j < head_dim ? qs[lane + 32 * j] : 0.0f;
    float mx = -INFINITY;
    for (int t0 = warp; t0 < seq_len; t0 += kAttnWarps * kAttnInflight) {
        float kr[kAttnInflight][kAttnPerLane];
#pragma unroll
        for (int u = 0; u < kAttnInflight; ++u) {
            const int t = t0 + u * kAttnWarps;
            const float* row = k_cache + (size_t)t * kv_dim + (size_t)kv_h * head_dim;
#pragma unroll
            for (int j = 0; j < kAttnPerLane; ++j) kr[u][j] = (t < seq_len && lane + 32 * j < head_dim) ? row[lane + 32 * j] : 0.0f;
        }
#pragma unroll
        for (int u = 0; u < kAttnInflight; ++u) {
            const int t = t0 + u * kAttnWarps;
            float dot = 0.0f;
#pragma unroll
            for (int j = 0; j < kAttnPerLane; ++j) dot = fmaf(qreg[j], kr[u][j], dot);
            dot = warp_sum(dot) * kq_scale;
            if (t < seq_len) {
                if (lane == 0) sc[t] = dot;
                mx = fmaxf(mx, dot);
            }
        }
    }
    if (lane == 0) red[warp] = mx;
    __syncthreads();
    mx = red[0];
#pragma unroll
    for (int i = 1; i < kAttnWarps; ++i) mx = fmaxf(mx, red[i]);
    __syncthreads();
    float sum = 0.0f;
    for (int t = tid; t < seq_len; t += kAttnWarps * 32) {
        const float e = expf(sc[t] - mx);
        sc[t] = e;
        sum += e;
    }
    sum = warp_sum(sum);
    if (lane == 0) red[warp] = sum;
    __syncthreads();
    float tot = 0.0f;
#pragma unroll
    for (int i = 0; i < kAttnWarps; ++i) tot += red[i];
    // values: this warp's positions, kAttnInflight rows of V in flight
    float acc[kAttnPerLane];
#pragma unroll
    for (int j = 0; j < kAttnPerLane; ++j) acc[j] = 0.0f;
    for (int t0 = warp; t0 < seq_len; t0 += kAttnWarps * kAttnInflight) {
        float vr[kAttnInflight][kAttnPerLane];
#pragma unroll
        for (int u = 0; u < kAttnInflight; ++u) {
            const int t = t0 + u * kAttnWarps;
            const float* row = v_cache + (size_t)t * kv_dim + (size_t)kv_h * head_dim;
#pragma unroll
            for (int j = 0; j < kAttnPerLane; ++j) vr[u][j] = (t < seq_len && lane + 32 * j < head_dim) ? row[lane + 32 * j] : 0.0f;
        }
#pragma unroll
        for (int u = 0; u < kAttnInflight; ++u) {
            const int t = t0 + u * kAttnWarps;
            const float p = t < seq_len ? sc[t] / tot : 0.0f;
#pragma unroll
            for (int j = 0; j < kAttnPerLane; ++j) acc[j] = fmaf(p, vr[u][j], acc[j]);
        }
    }
#pragma unroll
    for (int j = 0; j < kAttnPerLane; ++j)
        if (lane + 32 * j < head_dim) part[warp * head_dim + lane + 32 * j] = acc[j];
    __syncthreads();
    for (int d = tid; d < head_dim; d += kAttnWarps * 32) {
        float a = 0.0f;
#pragma unroll
        for (int w = 0; w < kAttnWarps; ++w) a += part[w * head_dim + d];
        const float g = gate[(size_t)h * gate_stride + d];
        out[(size_t)h * head_dim + d] = a * (1.0f / (1.0f + expf(-g)));
    }
}


// ─── Gated DeltaNet (linear attention) layer, one token (src/engine/qwen35_moe/cpu.rs:218-347) ───────────────
// One CTA per value head does everything between the input projections and the output projection:
//   * causal depthwise conv over the last `ksize` inputs of its channels (its key head's q and k, its own v), then
//     SiLU (conv1d_step, src/math_util.rs:149-168; weights [channels][ksize] bf16).  The state is a ring of `ksize`
//     input rows indexed by position: tap k < ksize - 1 reads the input of step pos - (ksize - 1) + k, the new input
//     goes to row pos % ksize, which nobody reads in this step, so the value heads that share a key head (and write
//     the same values) do not race.  Rows never written hold zeros, as the reference's shifted state does at start;
//   * unweighted per-head RMS norm of q and k, q scaled by 1 / key_dim and k by 1 / sqrt(key_dim) (cpu.rs:277-299);
//   * decay exp(-exp(A_log) * softplus(a + dt_bias)) and input gate sigmoid(b) (compute_decay_beta, math_util.rs:401-416);
//   * the delta rule on the head's [value_dim, key_dim] state, one warp per row at a time: decay, read against k,
//     correct, read against q (gated_delta_net_step, math_util.rs:425-466); the state is read and written once;
//   * RMS norm of the head's outputs, SiLU gate from z, bf16 weight (gated_rms_norm, math_util.rs:472-493; no weight:
//     the outputs pass through, cpu.rs:329-336).
// Shared memory: q, k [key_dim], v, vals [value_dim].
constexpr int kLinThreads = 1024, kLinWarps = kLinThreads / 32;
constexpr int kLinRows = 4;    // state rows a warp has in flight
constexpr int kLinPerMax = 8; // state elements per lane and row: key_dim <= 256

template <int kLinPer>  // 4: key_dim <= 128, 8: key_dim <= 256
__global__ void __launch_bounds__(kLinThreads) lin_core_kernel(float* __restrict__ conv_ring, const float* qkv_in,
                                                       const uint16_t* __restrict__ conv_w, const float* z,
                                                       const float* alpha, const float* beta,
                                                       const float* __restrict__ a_log, const uint16_t* __restrict__ dt_bias,
                                                       const uint16_t* __restrict__ norm_w, float* __restrict__ state,
                                                       float* __restrict__ out, const int* __restrict__ pos_ptr, int total_key,
                                                       int conv_dim, int ksize, int k_heads_per_v, int key_dim, int value_dim) {
    extern __shared__ float lsm[];
    __shared__ float red[kLinWarps];
    float* qs = lsm;
    float* ks = qs + key_dim;
    float* vs = ks + key_dim;
    float* vals = vs + value_dim;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int h = blockIdx.x, kh = h / k_heads_per_v;
    pdl_trigger();
    // this head's recurrence state was last written a token ago: ask for it (L2) while the projections still run
    {
        const size_t bytes = (size_t)value_dim * key_dim * 4;
        const unsigned char* sp = reinterpret_cast<const unsigned char*>(state + (size_t)h * value_dim * key_dim);
        if ((bytes & 15) == 0 && (reinterpret_cast<uintptr_t>(state) & 15) == 0)
            for (size_t off = (size_t)tid * 4096; off < bytes; off += (size_t)kLinThreads * 4096)
                prefetch_l2(sp + off, (uint32_t)(bytes - off < 4096 ? bytes - off : 4096));
    }
    // ... and this warp's first group of state rows goes into registers right away: the loads are in flight through
    // the conv and the norms.  (The state was last written by this kernel a token ago.)
    float spre[kLinRows][kLinPer];
#pragma unroll
    for (int r = 0; r < kLinRows; ++r) {
        const int v = warp * kLinRows + r;
        const float* srow = state + ((size_t)h * value_dim + v) * key_dim;
#pragma unroll
        for (int j = 0; j < kLinPer; ++j) {
            const int i = lane + 32 * j;
            spre[r][j] = (v < value_dim && i < key_dim) ? srow[i] : 0.0f;
        }
    }
    // Everything else that does not come from the kernel before this one is requested now as well, so that after the
    // wait only one round of loads (this thread's projection outputs) stands between the kernel and its arithmetic:
    // the position, this thread's channel (conv taps and the ring rows they multiply: written in earlier steps), the
    // head's decay parameters and this thread's norm weight.
    const int pos = *pos_ptr;
    const int n_ch = 2 * key_dim + value_dim;
    auto channel_of = [&](int i) {
        return i < key_dim ? kh * key_dim + i
               : i < 2 * key_dim ? total_key + kh * key_dim + (i - key_dim)
                                 : 2 * total_key + h * value_dim + (i - 2 * key_dim);
    };
    constexpr int kFastK = 4;  // conv kernel sizes up to this take the preloaded path for a thread's first channel
    const bool fast_conv = conv_w != nullptr && ksize <= kFastK && tid < n_ch;
    const int c_mine = tid < n_ch ? channel_of(tid) : 0;
    float cw[kFastK], rv[kFastK];
#pragma unroll
    for (int k = 0; k < kFastK; ++k) {
        cw[k] = rv[k] = 0.0f;
        if (fast_conv && k < ksize) cw[k] = bf16_bits_to_f32(conv_w[(size_t)c_mine * ksize + k]);
        if (fast_conv && k < ksize - 1) {
            const int step = pos - (ksize - 1) + k;
            const int row = ((step % ksize) + ksize) % ksize;
            rv[k] = conv_ring[(size_t)row * conv_dim + c_mine];
        }
    }
    const float a_log_h = a_log ? a_log[h] : 0.0f;
    const float dt_bias_h = dt_bias ? bf16_bits_to_f32(dt_bias[h]) : 0.0f;
    const float nw_mine = (norm_w && tid < value_dim) ? bf16_bits_to_f32(norm_w[tid]) : 0.0f;
    pdl_wait();
    const float xin_mine = tid < n_ch ? qkv_in[c_mine] : 0.0f;
    const float z_mine = (norm_w && tid < value_dim) ? z[(size_t)h * value_dim + tid] : 0.0f;
    const float alpha_h = alpha[h], beta_h = beta[h];
    // 1. conv + SiLU of this head's channels, and the ring update
    for (int i = tid; i < n_ch; i += kLinThreads) {
        const int c = i == tid ? c_mine : channel_of(i);
        const float xin = i == tid ? xin_mine : qkv_in[c];
        float val = xin;
        if (conv_w) {
            float acc = 0.0f;
            if (i == tid && fast_conv) {
#pragma unroll
                for (int k = 0; k < kFastK; ++k)
                    if (k < ksize - 1) acc += rv[k] * cw[k];
                float w_last = cw[0];
#pragma unroll
                for (int k = 1; k < kFastK; ++k)
                    if (k == ksize - 1) w_last = cw[k];
                acc += xin * w_last;
            } else {
                for (int k = 0; k < ksize - 1; ++k) {
                    const int step = pos - (ksize - 1) + k;                   // the input this tap multiplies
                    const int row = ((step % ksize) + ksize) % ksize;         // rows of steps before the start hold zeros
                    acc += conv_ring[(size_t)row * conv_dim + c] * bf16_bits_to_f32(conv_w[(size_t)c * ksize + k]);
                }
                acc += xin * bf16_bits_to_f32(conv_w[(size_t)c * ksize + ksize - 1]);
            }
            val = acc / (1.0f + expf(-acc));  // silu (src/math_util.rs:71-75)
            conv_ring[(size_t)(pos % ksize) * conv_dim + c] = xin;
        }
        if (i < key_dim) qs[i] = val;
        else if (i < 2 * key_dim) ks[i - key_dim] = val;
        else vs[i - 2 * key_dim] = val;
    }
    __syncthreads();
    // 2. q / k norms
    float sq = 0.0f, sk = 0.0f;
    for (int i = tid; i < key_dim; i += kLinThreads) {
        sq = fmaf(qs[i], qs[i], sq);
        sk = fmaf(ks[i], ks[i], sk);
    }
    sq = warp_sum(sq);
    sk = warp_sum(sk);
    __shared__ float red2[kLinWarps];
    if (lane == 0) { red[warp] = sq; red2[warp] = sk; }
    __syncthreads();
    float tq = 0.0f, tk = 0.0f;
#pragma unroll
    for (int i = 0; i < kLinWarps; ++i) { tq += red[i]; tk += red2[i]; }
    const float inv_scale = 1.0f / sqrtf((float)key_dim);
    const float q_mul = (1.0f / sqrtf(tq / (float)key_dim + 1e-6f)) * inv_scale * inv_scale;
    const float k_mul = (1.0f / sqrtf(tk / (float)key_dim + 1e-6f)) * inv_scale;
    __syncthreads();  // red / red2 are reused below
    for (int i = tid; i < key_dim; i += kLinThreads) {
        qs[i] *= q_mul;
        ks[i] *= k_mul;
    }
    // 3. decay and input gate of this head
    const float a = expf(a_log_h);
    const float softplus = logf(1.0f + expf(alpha_h + dt_bias_h));
    const float g = expf(-a * softplus);
    const float bgate = 1.0f / (1.0f + expf(-beta_h));
    __syncthreads();
    // 4. the recurrence: a warp takes kLinRows consecutive rows at a time and requests all their state up front
    for (int v0 = warp * kLinRows; v0 < value_dim; v0 += kLinWarps * kLinRows) {
        float sreg[kLinRows][kLinPer];
#pragma unroll
        for (int r = 0; r < kLinRows; ++r) {
            const float* srow = state + ((size_t)h * value_dim + v0 + r) * key_dim;
#pragma unroll
            for (int j = 0; j < kLinPer; ++j) {
                const int i = lane + 32 * j;
                if (v0 == warp * kLinRows) sreg[r][j] = spre[r][j];  // the group requested at the top
                else sreg[r][j] = (v0 + r < value_dim && i < key_dim) ? srow[i] : 0.0f;
            }
        }
        float kv[kLinRows];
#pragma unroll
        for (int r = 0; r < kLinRows; ++r) {
            float acc = 0.0f;
#pragma unroll
            for (int j = 0; j < kLinPer; ++j) {
                const int i = lane + 32 * j;
                sreg[r][j] *= g;
                if (i < key_dim) acc = fmaf(sreg[r][j], ks[i], acc);
            }
            kv[r] = acc;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
#pragma unroll
            for (int r = 0; r < kLinRows; ++r) kv[r] += __shfl_xor_sync(0xffffffffu, kv[r], o);
        float ov[kLinRows];
#pragma unroll
        for (int r = 0; r < kLinRows; ++r) {
            const float delta = ((v0 + r < value_dim ? vs[v0 + r] : 0.0f) - kv[r]) * bgate;
            float* srow = state + ((size_t)h * value_dim + v0 + r) * key_dim;
            float acc = 0.0f;
#pragma unroll
            for (int j = 0; j < kLinPer; ++j) {
                const int i = lane + 32 * j;
                if (v0 + r < value_dim && i < key_dim) {
                    const float sn = sreg[r][j] + ks[i] * delta;
                    srow[i] = sn;
                    acc = fmaf(sn, qs[i], acc);
                }
            }
            ov[r] = acc;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
#pragma unroll
            for (int r = 0; r < kLinRows; ++r) ov[r] += __shfl_xor_sync(0xffffffffu, ov[r], o);
        if (lane == 0) {
#pragma unroll
            for (int r = 0; r < kLinRows; ++r)
                if (v0 + r < value_dim) vals[v0 + r] = ov[r];
        }
    }
    __syncthreads();
    // 5. gated RMS norm
    if (!norm_w) {
        for (int i = tid; i < value_dim; i += kLinThreads) out[(size_t)h * value_dim + i] = vals[i];
        return;
    }
    float ss = 0.0f;
    for (int i = tid; i < value_dim; i += kLinThreads) ss = fmaf(vals[i], vals[i], ss);
    ss = warp_sum(ss);
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    float tot = 0.0f;
#pragma unroll
    for (int i = 0; i < kLinWarps; ++i) tot += red[i];
    const float inv = 1.0f / sqrtf(tot / (float)value_dim + 1e-6f);
    for (int i = tid; i < value_dim; i += kLinThreads) {
        const float zv = i == tid ? z_mine : z[(size_t)h * value_dim + i];
        const float nw = i == tid ? nw_mine : bf16_bits_to_f32(norm_w[i]);
        out[(size_t)h * value_dim + i] = vals[i] * inv * (zv / (1.0f + expf(-zv))) * nw;
    }
}

// ─── the same layer with a head's state rows dealt to several small CTAs ────────────────────────────────────
// One CTA of 256 threads per (value head, block of 32 state rows): conv + SiLU of the key head's q and k channels (every
// CTA of the head repeats them; they write the same values into the ring) and of its own 32 v channels, the q / k
// norms, decay and gate, and the delta rule on its rows.  The rows of a head are independent of one another given q
// and k; only the gated RMS norm joins them (a sum over the head's outputs): every CTA applies the gate and the norm
// weight to its outputs and leaves its sum of squares beside them, and the output projection's kernel multiplies by the
// head's rsqrt(mean + eps) while it stages its input (launch_matvec_head_scaled).  Four times as many SMs work on the 2 MB of state, and a 256-thread CTA finds room on an SM
// while the projection before it still runs, so what it requests ahead of its wait really is ahead.
constexpr int kLpThreads = 256, kLpWarps = kLpThreads / 32;
constexpr int kLpRows = kLpWarps * kLinRows;  // 32 state rows per CTA
constexpr int kLpCh = 2;                      // channels a thread prepares ahead of the wait (the CTA's channels <= 512)
constexpr int kLpK = 4;                       // conv kernel sizes up to this take the prepared path

template <int kLinPer>  // 4: key_dim <= 128, 8: key_dim <= 256
__global__ void __launch_bounds__(kLpThreads) lin_part_kernel(float* __restrict__ conv_ring, const float* qkv_in,
                                                      const uint16_t* __restrict__ conv_w, const float* alpha,
                                                      const float* beta, const float* __restrict__ a_log,
                                                      const uint16_t* __restrict__ dt_bias, float* __restrict__ state,
                                                      const float* z, const uint16_t* __restrict__ norm_w,
                                                      float* __restrict__ out_gated, float* __restrict__ ss_part,
                                                      const int* __restrict__ pos_ptr, int total_key,
                                                      int conv_dim, int ksize, int k_heads_per_v, int key_dim, int value_dim,
                                                      int parts) {
    extern __shared__ float lsm[];
    __shared__ float red[kLpWarps], red2[kLpWarps];
    float* qs = lsm;
    float* ks = qs + key_dim;
    float* vs = ks + key_dim;  // [kLpRows]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int h = blockIdx.x / parts, part = blockIdx.x % parts, kh = h / k_heads_per_v;
    const int v_begin = part * kLpRows;
    const int nv = value_dim - v_begin < kLpRows ? value_dim - v_begin : kLpRows;
    pdl_trigger();
    // ahead of the wait: this warp's state rows, this thread's channels (taps and the ring rows they multiply), the
    // head's decay parameters
    float sreg[kLinRows][kLinPer];
#pragma unroll
    for (int r = 0; r < kLinRows; ++r) {
        const int v = warp * kLinRows + r;
        const float* srow = state + ((size_t)h * value_dim + v_begin + v) * key_dim;
#pragma unroll
        for (int j = 0; j < kLinPer; ++j) {
            const int i = lane + 32 * j;
            sreg[r][j] = (v < nv && i < key_dim) ? srow[i] : 0.0f;
        }
    }
    const int pos = *pos_ptr;
    const int n_ch = 2 * key_dim + nv;
    auto channel_of = [&](int i) {
        return i < key_dim ? kh * key_dim + i
               : i < 2 * key_dim ? total_key + kh * key_dim + (i - key_dim)
                                 : 2 * total_key + h * value_dim + v_begin + (i - 2 * key_dim);
    };
    const bool prepared = conv_w != nullptr && ksize <= kLpK;
    int c_mine[kLpCh];
    float cw[kLpCh][kLpK], rv[kLpCh][kLpK];
#pragma unroll
    for (int u = 0; u < kLpCh; ++u) {
        const int i = tid + u * kLpThreads;
        c_mine[u] = i < n_ch ? channel_of(i) : 0;
#pragma unroll
        for (int k = 0; k < kLpK; ++k) {
            cw[u][k] = rv[u][k] = 0.0f;
            if (prepared && i < n_ch && k < ksize) cw[u][k] = bf16_bits_to_f32(conv_w[(size_t)c_mine[u] * ksize + k]);
            if (prepared && i < n_ch && k < ksize - 1) {
                const int step = pos - (ksize - 1) + k;                   // the input this tap multiplies
                const int row = ((step % ksize) + ksize) % ksize;         // rows of steps before the start hold zeros
                rv[u][k] = conv_ring[(size_t)row * conv_dim + c_mine[u]];
            }
        }
    }
    const float a_log_h = a_log ? a_log[h] : 0.0f;
    const float dt_bias_h = dt_bias ? bf16_bits_to_f32(dt_bias[h]) : 0.0f;
    // lanes 0..3 of a warp finish one of its rows each: the row's norm weight now, its gate input after the wait
    const int v_fin = warp * kLinRows + (lane & (kLinRows - 1));
    const float nw_fin = (lane < kLinRows && v_fin < nv) ? bf16_bits_to_f32(norm_w[v_begin + v_fin]) : 0.0f;
    pdl_wait();
    const float z_fin = (lane < kLinRows && v_fin < nv) ? z[(size_t)h * value_dim + v_begin + v_fin] : 0.0f;
    float xin_mine[kLpCh];
#pragma unroll
    for (int u = 0; u < kLpCh; ++u) xin_mine[u] = tid + u * kLpThreads < n_ch ? qkv_in[c_mine[u]] : 0.0f;
    const float alpha_h = alpha[h], beta_h = beta[h];
    // 1. conv + SiLU (conv1d_step, src/math_util.rs:149-168) and the ring update
    for (int i = tid, u = 0; i < n_ch; i += kLpThreads, ++u) {
        const bool mine = u < kLpCh;
        int c = channel_of(i);
        float xin, val;
        if (mine) {
            // (constant indices: the arrays stay in registers)
            xin = u == 0 ? xin_mine[0] : xin_mine[1];
        } else {
            xin = qkv_in[c];
        }
        val = xin;
        if (conv_w) {
            float acc = 0.0f;
            if (mine && prepared) {
#pragma unroll
                for (int k = 0; k < kLpK; ++k)
                    if (k < ksize - 1) acc += (u == 0 ? rv[0][k] : rv[1][k]) * (u == 0 ? cw[0][k] : cw[1][k]);
                float w_last = u == 0 ? cw[0][0] : cw[1][0];
#pragma unroll
                for (int k = 1; k < kLpK; ++k)
                    if (k == ksize - 1) w_last = u == 0 ? cw[0][k] : cw[1][k];
                acc += xin * w_last;
            } else {
                for (int k = 0; k < ksize - 1; ++k) {
                    const int step = pos - (ksize - 1) + k;
                    const int row = ((step % ksize) + ksize) % ksize;
                    acc += conv_ring[(size_t)row * conv_dim + c] * bf16_bits_to_f32(conv_w[(size_t)c * ksize + k]);
                }
                acc += xin * bf16_bits_to_f32(conv_w[(size_t)c * ksize + ksize - 1]);
            }
            val = acc / (1.0f + expf(-acc));  // silu (src/math_util.rs:71-75)
            conv_ring[(size_t)(pos % ksize) * conv_dim + c] = xin;
        }
        if (i < key_dim) qs[i] = val;
        else if (i < 2 * key_dim) ks[i - key_dim] = val;
        else vs[i - 2 * key_dim] = val;
    }
    __syncthreads();
    // 2. q / k norms (cpu.rs:277-299)
    float sq = 0.0f, sk = 0.0f;
    for (int i = tid; i < key_dim; i += kLpThreads) {
        sq = fmaf(qs[i], qs[i], sq);
        sk = fmaf(ks[i], ks[i], sk);
    }
    sq = warp_sum(sq);
    sk = warp_sum(sk);
    if (lane == 0) { red[warp] = sq; red2[warp] = sk; }
    __syncthreads();
    float tq = 0.0f, tk = 0.0f;
#pragma unroll
    for (int i = 0; i < kLpWarps; ++i) { tq += red[i]; tk += red2[i]; }
    const float inv_scale = 1.0f / sqrtf((float)key_dim);
    const float q_mul = (1.0f / sqrtf(tq / (float)key_dim + 1e-6f)) * inv_scale * inv_scale;
    const float k_mul = (1.0f / sqrtf(tk / (float)key_dim + 1e-6f)) * inv_scale;
    // 3. decay and input gate of this head (compute_decay_beta, math_util.rs:401-416)
    const float a = expf(a_log_h);
    const float softplus = logf(1.0f + expf(alpha_h + dt_bias_h));
    const float g = expf(-a * softplus);
    const float bgate = 1.0f / (1.0f + expf(-beta_h));
    // 4. the delta rule on this warp's rows (gated_delta_net_step, math_util.rs:425-466); q and k are scaled as they are read
    float kv[kLinRows];
#pragma unroll
    for (int r = 0; r < kLinRows; ++r) {
        float acc = 0.0f;
#pragma unroll
        for (int j = 0; j < kLinPer; ++j) {
            const int i = lane + 32 * j;
            sreg[r][j] *= g;
            if (i < key_dim) acc = fmaf(sreg[r][j], ks[i] * k_mul, acc);
        }
        kv[r] = acc;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
#pragma unroll
        for (int r = 0; r < kLinRows; ++r) kv[r] += __shfl_xor_sync(0xffffffffu, kv[r], o);
    float ov[kLinRows];
#pragma unroll
    for (int r = 0; r < kLinRows; ++r) {
        const int v = warp * kLinRows + r;
        const float delta = ((v < nv ? vs[v] : 0.0f) - kv[r]) * bgate;
        float* srow = state + ((size_t)h * value_dim + v_begin + v) * key_dim;
        float acc = 0.0f;
#pragma unroll
        for (int j = 0; j < kLinPer; ++j) {
            const int i = lane + 32 * j;
            if (v < nv && i < key_dim) {
                const float sn = sreg[r][j] + (ks[i] * k_mul) * delta;
                srow[i] = sn;
                acc = fmaf(sn, qs[i] * q_mul, acc);
            }
        }
        ov[r] = acc;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
#pragma unroll
        for (int r = 0; r < kLinRows; ++r) ov[r] += __shfl_xor_sync(0xffffffffu, ov[r], o);
    // 5. gated RMS norm (math_util.rs:472-493) up to the head's 1 / rms, which needs the other CTAs' rows: the outputs go
    //    out times silu(z) and the norm weight, this CTA's sum of squares beside them, and the consumer scales by
    //    rsqrt(mean + eps) while it stages its input.  Every lane holds the warp's sums; lane r finishes row r.
    float mine = 0.0f, ss = 0.0f;
#pragma unroll
    for (int r = 0; r < kLinRows; ++r) {
        if (lane == r) mine = ov[r];
        if (warp * kLinRows + r < nv) ss = fmaf(ov[r], ov[r], ss);
    }
    if (lane < kLinRows && v_fin < nv)
        out_gated[(size_t)h * value_dim + v_begin + v_fin] = mine * (z_fin / (1.0f + expf(-z_fin))) * nw_fin;
    __syncthreads();  // red was read by every warp above
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    if (tid == 0) {
        float tot = 0.0f;
#pragma unroll
        for (int i = 0; i < kLpWarps; ++i) tot += red[i];
        ss_part[blockIdx.x] = tot;
    }
}

// ─── the same for a run of tokens: one launch, the state in registers from the first token to the last ──────
// A prompt's tokens go through a DeltaNet layer one after the other (each step needs the state the previous one left),
// but not as one launch per token: here a CTA keeps its rows of the state, and every thread the last conv inputs of its
// channels, in registers across the tokens; per token it reads the projection outputs (the next token's while this one
// computes), writes the gated outputs and its sum of squares, and updates the conv ring; the state goes back to memory
// once at the end.  Token t's buffers lie t * tok_stride floats after token 0's.  For conv kernels up to kLpK taps and at
// most kLpCh channels per thread (the host checks).
template <int kLinPer>
__global__ void __launch_bounds__(kLpThreads) lin_seq_kernel(float* __restrict__ conv_ring, const float* qkv_in,
                                                     const uint16_t* __restrict__ conv_w, const float* alpha,
                                                     const float* beta, const float* __restrict__ a_log,
                                                     const uint16_t* __restrict__ dt_bias, float* __restrict__ state,
                                                     const float* z, const uint16_t* __restrict__ norm_w,
                                                     float* __restrict__ out_gated, float* __restrict__ ss_part,
                                                     const int* __restrict__ pos_ptr, int total_key,
                                                     int conv_dim, int ksize, int k_heads_per_v, int key_dim, int value_dim,
                                                     int parts, int n_tok, int tok_stride) {
    extern __shared__ float lsm[];
    __shared__ float red[kLpWarps], red2[kLpWarps];
    float* qs = lsm;
    float* ks = qs + key_dim;
    float* vs = ks + key_dim;  // [kLpRows]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int h = blockIdx.x / parts, part = blockIdx.x % parts, kh = h / k_heads_per_v;
    const int v_begin = part * kLpRows;
    const int nv = value_dim - v_begin < kLpRows ? value_dim - v_begin : kLpRows;
    pdl_trigger();
    pdl_wait();
    float sreg[kLinRows][kLinPer];
#pragma unroll
    for (int r = 0; r < kLinRows; ++r) {
        const int v = warp * kLinRows + r;
        const float* srow = state + ((size_t)h * value_dim + v_begin + v) * key_dim;
#pragma unroll
        for (int j = 0; j < kLinPer; ++j) {
            const int i = lane + 32 * j;
            sreg[r][j] = (v < nv && i < key_dim) ? srow[i] : 0.0f;
        }
    }
    const int pos0 = *pos_ptr;
    const int n_ch = 2 * key_dim + nv;
    auto channel_of = [&](int i) {
        return i < key_dim ? kh * key_dim + i
               : i < 2 * key_dim ? total_key + kh * key_dim + (i - key_dim)
                                 : 2 * total_key + h * value_dim + v_begin + (i - 2 * key_dim);
    };
    int c_mine[kLpCh];
    float cw[kLpCh][kLpK], rv[kLpCh][kLpK];  // taps; the last ksize - 1 inputs of the channel, oldest first
    bool have[kLpCh];
#pragma unroll
    for (int u = 0; u < kLpCh; ++u) {
        const int i = tid + u * kLpThreads;
        have[u] = i < n_ch;
        c_mine[u] = have[u] ? channel_of(i) : 0;
#pragma unroll
        for (int k = 0; k < kLpK; ++k) {
            cw[u][k] = rv[u][k] = 0.0f;
            if (have[u] && k < ksize) cw[u][k] = bf16_bits_to_f32(conv_w[(size_t)c_mine[u] * ksize + k]);
            if (have[u] && k < ksize - 1) {
                const int step = pos0 - (ksize - 1) + k;
                const int row = ((step % ksize) + ksize) % ksize;
                rv[u][k] = conv_ring[(size_t)row * conv_dim + c_mine[u]];
            }
        }
    }
    const float a_decay = expf(a_log ? a_log[h] : 0.0f);
    const float dt_bias_h = dt_bias ? bf16_bits_to_f32(dt_bias[h]) : 0.0f;
    const int v_fin = warp * kLinRows + (lane & (kLinRows - 1));
    const bool fin = lane < kLinRows && v_fin < nv;
    const float nw_fin = fin ? bf16_bits_to_f32(norm_w[v_begin + v_fin]) : 0.0f;
    const float inv_scale = 1.0f / sqrtf((float)key_dim);
    // the first token's inputs
    float xin[kLpCh], xin_next[kLpCh] = {};
    float alpha_t = alpha[h], beta_t = beta[h], z_t = fin ? z[(size_t)h * value_dim + v_begin + v_fin] : 0.0f;
    float alpha_n = 0.0f, beta_n = 0.0f, z_n = 0.0f;
#pragma unroll
    for (int u = 0; u < kLpCh; ++u) xin[u] = have[u] ? qkv_in[c_mine[u]] : 0.0f;
    for (int t = 0; t < n_tok; ++t) {
        const size_t off = (size_t)t * tok_stride;
        if (t + 1 < n_tok) {  // the next token's inputs are on their way while this one computes
            const size_t offn = off + tok_stride;
#pragma unroll
            for (int u = 0; u < kLpCh; ++u) xin_next[u] = have[u] ? qkv_in[offn + c_mine[u]] : 0.0f;
            alpha_n = alpha[offn + h];
            beta_n = beta[offn + h];
            z_n = fin ? z[offn + (size_t)h * value_dim + v_begin + v_fin] : 0.0f;
        }
        const int pos = pos0 + t;
        // 1. conv + SiLU, ring update, the channel's window moves on
#pragma unroll
        for (int u = 0; u < kLpCh; ++u) {
            if (!have[u]) continue;
            const int i = tid + u * kLpThreads;
            float acc = 0.0f;
#pragma unroll
            for (int k = 0; k < kLpK; ++k)
                if (k < ksize - 1) acc += rv[u][k] * cw[u][k];
            float w_last = cw[u][0];
#pragma unroll
            for (int k = 1; k < kLpK; ++k)
                if (k == ksize - 1) w_last = cw[u][k];
            acc += xin[u] * w_last;
            const float val = acc / (1.0f + expf(-acc));
            conv_ring[(size_t)(pos % ksize) * conv_dim + c_mine[u]] = xin[u];
#pragma unroll
            for (int k = 0; k < kLpK - 1; ++k)
                if (k < ksize - 2) rv[u][k] = rv[u][k + 1];
#pragma unroll
            for (int k = 0; k < kLpK; ++k)
                if (k == ksize - 2) rv[u][k] = xin[u];
            if (i < key_dim) qs[i] = val;
            else if (i < 2 * key_dim) ks[i - key_dim] = val;
            else vs[i - 2 * key_dim] = val;
        }
        __syncthreads();
        // 2. q / k norms
        float sq = 0.0f, sk = 0.0f;
        for (int i = tid; i < key_dim; i += kLpThreads) {
            sq = fmaf(qs[i], qs[i], sq);
            sk = fmaf(ks[i], ks[i], sk);
        }
        sq = warp_sum(sq);
        sk = warp_sum(sk);
        if (lane == 0) { red[warp] = sq; red2[warp] = sk; }
        __syncthreads();
        float tq = 0.0f, tk = 0.0f;
#pragma unroll
        for (int i = 0; i < kLpWarps; ++i) { tq += red[i]; tk += red2[i]; }
        const float q_mul = (1.0f / sqrtf(tq / (float)key_dim + 1e-6f)) * inv_scale * inv_scale;
        const float k_mul = (1.0f / sqrtf(tk / (float)key_dim + 1e-6f)) * inv_scale;
        // 3. decay and input gate
        const float softplus = logf(1.0f + expf(alpha_t + dt_bias_h));
        const float g = expf(-a_decay * softplus);
        const float bgate = 1.0f / (1.0f + expf(-beta_t));
        // 4. the delta rule on this warp's rows
        float kv[kLinRows];
#pragma unroll
        for (int r = 0; r < kLinRows; ++r) {
            float acc = 0.0f;
#pragma unroll
            for (int j = 0; j < kLinPer; ++j) {
                const int i = lane + 32 * j;
                sreg[r][j] *= g;
                if (i < key_dim) acc = fmaf(sreg[r][j], ks[i] * k_mul, acc);
            }
            kv[r] = acc;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
#pragma unroll
            for (int r = 0; r < kLinRows; ++r) kv[r] += __shfl_xor_sync(0xffffffffu, kv[r], o);
        float ov[kLinRows];
#pragma unroll
        for (int r = 0; r < kLinRows; ++r) {
            const int v = warp * kLinRows + r;
            const float delta = ((v < nv ? vs[v] : 0.0f) - kv[r]) * bgate;
            float acc = 0.0f;
#pragma unroll
            for (int j = 0; j < kLinPer; ++j) {
                const int i = lane + 32 * j;
                if (v < nv && i < key_dim) {
                    sreg[r][j] = sreg[r][j] + (ks[i] * k_mul) * delta;
                    acc = fmaf(sreg[r][j], qs[i] * q_mul, acc);
                }
            }
            ov[r] = acc;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
#pragma unroll
            for (int r = 0; r < kLinRows; ++r) ov[r] += __shfl_xor_sync(0xffffffffu, ov[r], o);
        // 5. gate and norm weight, this CTA's sum of squares
        float mine = 0.0f, ss = 0.0f;
#pragma unroll
        for (int r = 0; r < kLinRows; ++r) {
            if (lane == r) mine = ov[r];
            if (warp * kLinRows + r < nv) ss = fmaf(ov[r], ov[r], ss);
        }
        if (fin) out_gated[off + (size_t)h * value_dim + v_begin + v_fin] = mine * (z_t / (1.0f + expf(-z_t))) * nw_fin;
        __syncthreads();  // red was read by every warp above; qs / ks / vs by the recurrence
        if (lane == 0) red[warp] = ss;
        __syncthreads();
        if (tid == 0) {
            float tot = 0.0f;
#pragma unroll
            for (int i = 0; i < kLpWarps; ++i) tot += red[i];
            ss_part[off + blockIdx.x] = tot;
        }
        __syncthreads();  // before the next token overwrites red and the shared q / k / v
#pragma unroll
        for (int u = 0; u < kLpCh; ++u) xin[u] = xin_next[u];
        alpha_t = alpha_n; beta_t = beta_n; z_t = z_n;
    }
#pragma unroll
    for (int r = 0; r < kLinRows; ++r) {
        const int v = warp * kLinRows + r;
        float* srow = state + ((size_t)h * value_dim + v_begin + v) * key_dim;
#pragma unroll
        for (int j = 0; j < kLinPer; ++j) {
            const int i = lane + 32 * j;
            if (v < nv && i < key_dim) srow[i] = sreg[r][j];
        }
    }
}

// ─── host side ──────────────────────────────────────────────────────────────

static size_t al256a(size_t v) { return (v + 255) / 256 * 256; }

static bool mtp_is_norm(int which) {
    return which == MOE_M_PRE_FC_NORM_HIDDEN || which == MOE_M_PRE_FC_NORM_EMBEDDING || which == MOE_M_INPUT_NORM ||
           which == MOE_M_Q_NORM || which == MOE_M_K_NORM || which == MOE_M_OUT_NORM;
}
static const char* mtp_tensor_name(int which) {
    static const char* names[] = {"mtp.pre_fc_norm_hidden", "mtp.pre_fc_norm_embedding", "mtp.fc", "mtp.layers.0.input_layernorm",
                                  "mtp.layers.0.self_attn.q_proj", "mtp.layers.0.self_attn.k_proj", "mtp.layers.0.self_attn.v_proj",
                                  "mtp.layers.0.self_attn.q_norm", "mtp.layers.0.self_attn.k_norm", "mtp.layers.0.self_attn.o_proj",
                                  "mtp.norm"};
    return (which >= 0 && which <= MOE_M_OUT_NORM) ? names[which] : "?";
}

void mtp_destroy(moe_engine* e) {
    MtpAttnState& m = e->mtp;
    for (int i = 0; i <= MOE_M_OUT_NORM; ++i) {
        if (m.norms[i]) cudaFree(m.norms[i]);
        if (m.proj[i].w) cudaFree(m.proj[i].w);
        m.norms[i] = nullptr;
        m.proj[i] = ProjTensor{};
    }
    if (m.k_cache) cudaFree(m.k_cache);
    if (m.v_cache) cudaFree(m.v_cache);
    if (m.work) cudaFree(m.work);
    if (m.id_dev) cudaFree(m.id_dev);
    m.k_cache = m.v_cache = m.work = nullptr;
    m.id_dev = nullptr;
    m.configured = false;
}

int mtp_configure(moe_engine* e, const moe_attn_dims_t* ad) {
    const moe_dims_t& d = e->dims;
    if (d.num_mtp_layers == 0) {
        set_error("model has no MTP block (mtp_num_hidden_layers == 0)");
        return MOE_ERR_STATE;
    }
    MOE_REQUIRE(ad->num_heads > 0 && ad->num_kv_heads > 0 && ad->num_heads % ad->num_kv_heads == 0,
                "attention heads (%d) must be a positive multiple of the key/value heads (%d)", ad->num_heads, ad->num_kv_heads);
    MOE_REQUIRE(ad->head_dim > 0 && ad->head_dim % 8 == 0 && ad->head_dim <= 32 * kAttnPerLane, "head_dim (%d) must be a multiple of 8 up to 256", ad->head_dim);
    MOE_REQUIRE(ad->rotary_dim >= 0 && ad->rotary_dim <= ad->head_dim && ad->rotary_dim % 2 == 0,
                "rotary_dim (%d) must be even and at most head_dim (%d)", ad->rotary_dim, ad->head_dim);
    MOE_REQUIRE(ad->max_seq > 0 && ad->max_seq <= 8192, "max_seq (%d) must be in 1..8192", ad->max_seq);
    MOE_REQUIRE((size_t)ad->num_heads * ad->head_dim <= 16384, "num_heads * head_dim above 16384 not supported");
    mtp_destroy(e);
    MtpAttnState& m = e->mtp;
    m.ad = *ad;
    const size_t kv_dim = (size_t)ad->num_kv_heads * ad->head_dim, q_dim = (size_t)ad->num_heads * ad->head_dim;
    MOE_CUDA(cudaMalloc(&m.k_cache, (size_t)ad->max_seq * kv_dim * 4));
    MOE_CUDA(cudaMalloc(&m.v_cache, (size_t)ad->max_seq * kv_dim * 4));
    // scratch: h, tok, concat [2H], cur, x, q [2 q_dim], k, v, qr, gated, o, cur2, y: each 256-byte aligned
    const size_t H = d.hidden;
    const size_t floats = 8 * al256a(H * 4) / 4 + al256a(2 * H * 4) / 4 + al256a(2 * q_dim * 4) / 4 + 2 * al256a(q_dim * 4) / 4 +
                          2 * al256a(kv_dim * 4) / 4;
    MOE_CUDA(cudaMalloc(&m.work, floats * 4));
    MOE_CUDA(cudaMalloc(&m.id_dev, 256));
    m.configured = true;
    e->mtp_pos = 0;
    return MOE_OK;
}

int mtp_load_tensor(moe_engine* e, int which, const void* w, const void* s, const void* b, int dtype) {
    MtpAttnState& m = e->mtp;
    const moe_dims_t& d = e->dims;
    MOE_REQUIRE(which >= 0 && which <= MOE_M_OUT_NORM, "unknown MTP tensor %d", which);
    if (!m.configured) {
        set_error("moe_mtp_configure must come before the MTP tensors");
        return MOE_ERR_STATE;
    }
    MOE_REQUIRE(w, "%s: null weight pointer", mtp_tensor_name(which));
    const int H = d.hidden, q_dim = m.ad.num_heads * m.ad.head_dim, kv_dim = m.ad.num_kv_heads * m.ad.head_dim;
    if (mtp_is_norm(which)) {
        MOE_REQUIRE(dtype == MOE_DT_BF16, "%s must be bf16", mtp_tensor_name(which));
        const size_t n = (which == MOE_M_Q_NORM || which == MOE_M_K_NORM) ? m.ad.head_dim : H;
        if (!m.norms[which]) MOE_CUDA(cudaMalloc(&m.norms[which], al256a(n * 2)));
        MOE_CUDA(cudaMemcpyAsync(m.norms[which], w, n * 2, cudaMemcpyHostToDevice, e->stream));
        MOE_CUDA(cudaStreamSynchronize(e->stream));
        return MOE_OK;
    }
    int rows = 0, cols = H;
    switch (which) {
        case MOE_M_FC: rows = H; cols = 2 * H; break;
        case MOE_M_Q_PROJ: rows = 2 * q_dim; break;
        case MOE_M_K_PROJ: case MOE_M_V_PROJ: rows = kv_dim; break;
        default: rows = H; cols = q_dim; break;  // o_proj
    }
    MOE_REQUIRE(dtype == MOE_DT_INT4 || (dtype == MOE_DT_BF16 && which != MOE_M_FC), "%s: dtype %d not supported here",
                mtp_tensor_name(which), dtype);
    MOE_REQUIRE(cols % 64 == 0, "%s: inner dimension %d must be a multiple of 64", mtp_tensor_name(which), cols);
    ProjTensor& t = m.proj[which];
    if (t.w) { cudaFree(t.w); t = ProjTensor{}; }
    t.dtype = dtype; t.rows = rows; t.cols = cols;
    if (dtype == MOE_DT_BF16) {
        const size_t bytes = (size_t)rows * cols * 2;
        MOE_CUDA(cudaMalloc(&t.w, bytes));
        MOE_CUDA(cudaMemcpyAsync(t.w, w, bytes, cudaMemcpyHostToDevice, e->stream));
    } else {
        MOE_REQUIRE(s && b, "%s: a 4-bit tensor needs scales and biases", mtp_tensor_name(which));
        const size_t wb = (size_t)rows * cols / 2, sb = (size_t)rows * (cols / 64) * 2;
        t.s_off = al256a(wb);
        t.b_off = t.s_off + al256a(sb);
        MOE_CUDA(cudaMalloc(&t.w, t.b_off + al256a(sb)));
        MOE_CUDA(cudaMemcpyAsync(t.w, w, wb, cudaMemcpyHostToDevice, e->stream));
        MOE_CUDA(cudaMemcpyAsync(t.w + t.s_off, s, sb, cudaMemcpyHostToDevice, e->stream));
        MOE_CUDA(cudaMemcpyAsync(t.w + t.b_off, b, sb, cudaMemcpyHostToDevice, e->stream));
    }
    MOE_CUDA(cudaStreamSynchronize(e->stream));
    t.loaded = true;
    return MOE_OK;
}

// y = W x (+ residual) for a projection stored as bf16 rows or as a 4-bit triple
// norm_w: the input is rmsnorm(x) * norm_w, applied inside the kernel (see proj_folds_norm)
static bool proj_folds_norm(const ProjTensor& t) { return t.dtype != MOE_DT_INT4 || matvec_folds_norm(t.rows, t.cols); }
static int proj_run(moe_engine* e, const ProjTensor& t, const float* x, float* y, const float* residual = nullptr, bool pdl = false,
                    const void* norm_w = nullptr, MvBatch mb = MvBatch{}) {
    if (t.dtype == MOE_DT_INT4)
        return launch_matvec_res(e, t.w, t.w + t.s_off, t.w + t.b_off, x, y, t.rows, t.cols, residual, pdl, norm_w, mb);
    if (!e->mtp.bf_attr_set) {
        MOE_CUDA(cudaFuncSetAttribute(matvec_bf16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 16384 * 4));
        e->mtp.bf_attr_set = true;
    }
    int blocks = (t.rows + kBfWarps * 2 - 1) / (kBfWarps * 2);
    if (blocks > e->sm_count * 2) blocks = e->sm_count * 2;  // one wave (two CTAs per SM): x is staged once per CTA
    blocks = matvec_batch_blocks(e, blocks, mb.n);
    MOE_CUDA(launch_kernel(pdl, matvec_bf16_kernel, dim3(blocks, mb.n), dim3(kBfWarps * 32), (size_t)t.cols * 4, e->stream,
                           reinterpret_cast<const uint16_t*>(t.w), x, y, t.rows, t.cols, residual, (const uint16_t*)norm_w,
                           mb.x_stride, mb.y_stride, mb.r_stride));
    e->launches++;
    return MOE_OK;
}

// One MTP step, enqueued on the engine's stream (the caller copies the logits out, synchronises, polls the error
// word and advances the position): h_host [hidden] and token_id in, logits_dev [vocab] (device) out.
int mtp_step(moe_engine* e, const float* h_host, int64_t token_id, float* logits_dev) {
    MtpAttnState& m = e->mtp;
    const moe_dims_t& d = e->dims;
    if (d.num_mtp_layers == 0) {
        set_error("model has no MTP block (mtp_num_hidden_layers == 0)");
        return MOE_ERR_STATE;
    }
    if (!m.configured) {
        set_error("the MTP block is not configured (moe_mtp_configure)");
        return MOE_ERR_STATE;
    }
    for (int i = 0; i < MOE_M_OUT_NORM; ++i) {  // mtp.norm may be absent: the model's final norm stands in (mtp.rs:209-216)
        const bool ok = mtp_is_norm(i) ? m.norms[i] != nullptr : m.proj[i].loaded;
        if (!ok) {
            set_error("the MTP block is not loaded (%s missing)", mtp_tensor_name(i));
            return MOE_ERR_STATE;
        }
    }
    MOE_REQUIRE(token_id >= 0 && token_id < d.vocab, "token id %lld outside [0, %d)", (long long)token_id, d.vocab);
    const int pos = (int)e->mtp_pos;
    if (pos >= m.ad.max_seq) {
        set_error("the MTP block's KV cache is full (%d positions)", m.ad.max_seq);
        return MOE_ERR_STATE;
    }
    const int H = d.hidden, nh = m.ad.num_heads, nkv = m.ad.num_kv_heads, hd = m.ad.head_dim;
    const size_t q_dim = (size_t)nh * hd, kv_dim = (size_t)nkv * hd;
    // carve the scratch
    float* p = m.work;
    auto take = [&](size_t n) { float* r = p; p += al256a(n * 4) / 4; return r; };
    float* h = take(H); float* tok = take(H); float* concat = take(2 * (size_t)H); float* cur = take(H); float* x = take(H);
    float* q = take(2 * q_dim); float* k = take(kv_dim); float* v = take(kv_dim); float* qr = take(q_dim); float* gated = take(q_dim);
    float* cur2 = take(H); float* y = take(H);
    cudaStream_t st = e->stream;
    MOE_CUDA(cudaMemcpyAsync(h, h_host, (size_t)H * 4, cudaMemcpyHostToDevice, st));
    MOE_CUDA(cudaMemcpyAsync(m.id_dev, &token_id, 8, cudaMemcpyHostToDevice, st));
    int rc = launch_embed(e, m.id_dev, 1, tok);
    if (rc) return rc;
    // From here every kernel is a programmatic dependent of the one before it (see pdl_wait: each waits before it reads what
    // an earlier kernel of the chain wrote, whichever that was); MOE_B200_ATTN_PDL=0 keeps the ordinary dependencies.
    static const bool pdl = [] { const char* v = getenv("MOE_B200_ATTN_PDL"); return !(v && atoi(v) == 0); }();
    // embedding first, hidden state second (mtp.rs:103-105)
    rms_norm_rows_kernel<<<1, 256, 0, st>>>(tok, m.norms[MOE_M_PRE_FC_NORM_EMBEDDING], H, concat);
    MOE_CUDA(launch_kernel(pdl, rms_norm_rows_kernel, dim3(1), dim3(256), 0, st, (const float*)h, (const uint16_t*)m.norms[MOE_M_PRE_FC_NORM_HIDDEN], H, concat + H));
    e->launches += 2;
    rc = proj_run(e, m.proj[MOE_M_FC], concat, cur, nullptr, pdl);
    if (rc) return rc;
    MOE_CUDA(launch_kernel(pdl, rms_norm_rows_kernel, dim3(1), dim3(256), 0, st, (const float*)cur, (const uint16_t*)m.norms[MOE_M_INPUT_NORM], H, x));
    e->launches++;
    if ((rc = proj_run(e, m.proj[MOE_M_Q_PROJ], x, q, nullptr, pdl))) return rc;
    if ((rc = proj_run(e, m.proj[MOE_M_K_PROJ], x, k, nullptr, pdl))) return rc;
    if ((rc = proj_run(e, m.proj[MOE_M_V_PROJ], x, v, nullptr, pdl))) return rc;
    MOE_CUDA(launch_kernel(pdl, attn_prep_kernel, dim3(nh + nkv), dim3(256), (size_t)hd * 4, st, (const float*)q, hd, 0, (const float*)k,
                           (const float*)v, (const uint16_t*)m.norms[MOE_M_Q_NORM], (const uint16_t*)m.norms[MOE_M_K_NORM], nh, nkv, hd,
                           m.ad.rotary_dim, pos, (const int*)nullptr, m.ad.rope_theta, qr, m.k_cache, m.v_cache, 0));
    const int seq = pos + 1;
    MOE_CUDA(launch_kernel(pdl, attn_decode_kernel, dim3(nh), dim3(kAttnWarps * 32), (size_t)(seq + hd * (1 + kAttnWarps)) * 4, st,
                           (const float*)qr, (const float*)m.k_cache, (const float*)m.v_cache, (const float*)(q + q_dim), hd, nh, nkv, hd,
                           seq, (const int*)nullptr, 1.0f / sqrtf((float)hd), gated, 0));
    e->launches += 2;
    if ((rc = proj_run(e, m.proj[MOE_M_O_PROJ], gated, cur2, cur, pdl))) return rc;  // + residual
    // the MoE half: post-attention norm, router, experts, shared expert, residual (layer index num_layers)
    if ((rc = launch_decode(e, d.num_layers, d.num_layers + 1, cur2, y, nullptr, nullptr, nullptr, nullptr, pdl))) return rc;
    if ((rc = launch_logits_norm(e, y, 1, logits_dev, m.norms[MOE_M_OUT_NORM]))) return rc;
    return MOE_OK;
}


// ─── the main layers' attention halves ──────────────────────────────────────

static const char* attn_tensor_name(int which) {
    static const char* names[] = {"input_layernorm", "self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "self_attn.q_norm",
                                  "self_attn.k_norm", "self_attn.o_proj", "linear_attn.in_proj_qkv", "linear_attn.in_proj_z",
                                  "linear_attn.in_proj_b", "linear_attn.in_proj_a", "linear_attn.conv1d", "linear_attn.A_log",
                                  "linear_attn.dt_bias", "linear_attn.norm", "linear_attn.out_proj"};
    return (which >= 0 && which <= MOE_A_OUT_PROJ) ? names[which] : "?";
}
static bool attn_is_proj(int which) {
    return which == MOE_A_Q_PROJ || which == MOE_A_K_PROJ || which == MOE_A_V_PROJ || which == MOE_A_O_PROJ ||
           which == MOE_A_IN_PROJ_QKV || which == MOE_A_IN_PROJ_Z || which == MOE_A_IN_PROJ_B || which == MOE_A_IN_PROJ_A ||
           which == MOE_A_OUT_PROJ;
}
static bool attn_role_is_full(int which) { return which >= MOE_A_Q_PROJ && which <= MOE_A_O_PROJ; }

static void attn_drop_graphs(moe_engine* e) {
    ModelAttnState& a = e->attn;
    for (cudaGraphExec_t g : a.graphs)
        if (g) cudaGraphExecDestroy(g);
    a.graphs.clear();
    a.graph_nodes.clear();
    a.graphs_valid = false;
}

__global__ void set_pos_kernel(int* p, int v) { *p = v; }

void attn_destroy(moe_engine* e) {
    ModelAttnState& a = e->attn;
    attn_drop_graphs(e);
    if (a.d_pos) cudaFree(a.d_pos);
    a.d_pos = nullptr;
    if (a.pos_table) cudaFree(a.pos_table);
    a.pos_table = nullptr;
    if (a.prefill_mid) cudaFree(a.prefill_mid);
    a.prefill_mid = nullptr;
    a.prefill_cap = 0;
    for (AttnLayerState& ls : a.layers) {
        for (int i = 0; i < 16; ++i) {
            if (ls.vec[i]) cudaFree(ls.vec[i]);
            if (ls.proj[i].w) cudaFree(ls.proj[i].w);
        }
        if (ls.fused.w) cudaFree(ls.fused.w);
        if (ls.k_cache) cudaFree(ls.k_cache);
        if (ls.v_cache) cudaFree(ls.v_cache);
        if (ls.conv_state) cudaFree(ls.conv_state);
        if (ls.ssm_state) cudaFree(ls.ssm_state);
    }
    a.layers.clear();
    if (a.work) cudaFree(a.work);
    a.work = nullptr;
    a.configured = false;
    a.pos = 0;
}

struct AttnSizes {
    size_t H, q_dim, kv_dim, total_key, total_value, conv_dim;
};
static AttnSizes attn_sizes(const moe_engine* e) {
    const moe_model_attn_dims_t& d = e->attn.d;
    AttnSizes z{};
    z.H = (size_t)e->dims.hidden;
    z.q_dim = (size_t)d.full.num_heads * d.full.head_dim;
    z.kv_dim = (size_t)d.full.num_kv_heads * d.full.head_dim;
    z.total_key = (size_t)d.lin_num_k_heads * d.lin_key_dim;
    z.total_value = (size_t)d.lin_num_v_heads * d.lin_value_dim;
    z.conv_dim = 2 * z.total_key + z.total_value;
    return z;
}

// floats of the stacked input projections' output: q|k|v of a full layer or qkv|z|b|a of a linear one
static size_t attn_proj_out_floats(const AttnSizes& z, size_t v_heads) {
    const size_t full = 2 * z.q_dim + 2 * z.kv_dim, lin = z.conv_dim + z.total_value + 2 * v_heads;
    return full > lin ? full : lin;
}

int attn_reset(moe_engine* e) {
    ModelAttnState& a = e->attn;
    if (!a.configured) return MOE_OK;
    const AttnSizes z = attn_sizes(e);
    for (AttnLayerState& ls : a.layers) {
        if (ls.full) continue;  // KV entries behind the position are never read
        MOE_CUDA(cudaMemsetAsync(ls.conv_state, 0, (size_t)a.d.conv_kernel * z.conv_dim * 4, e->stream));
        MOE_CUDA(cudaMemsetAsync(ls.ssm_state, 0, z.total_value * a.d.lin_key_dim * 4, e->stream));
    }
    a.pos = 0;
    return MOE_OK;
}

// One state tensor of one layer between the device and host memory (which: moe_state_tensor_t).
int attn_state_io(moe_engine* e, int layer, int which, float* host, int64_t floats, bool to_device) {
    ModelAttnState& a = e->attn;
    MOE_REQUIRE(a.configured, "the attention halves are not configured (moe_attn_configure)");
    MOE_REQUIRE(layer >= 0 && layer < (int)a.layers.size(), "layer %d outside [0, %d)", layer, (int)a.layers.size());
    const AttnSizes z = attn_sizes(e);
    AttnLayerState& ls = a.layers[layer];
    float* dev = nullptr;
    int64_t want = 0;
    switch (which) {
    case MOE_ST_K_CACHE:
    case MOE_ST_V_CACHE:
        MOE_REQUIRE(ls.full, "layer %d is a linear-attention layer: it has no KV cache", layer);
        MOE_REQUIRE(floats >= 0 && floats % (int64_t)z.kv_dim == 0 && floats <= (int64_t)a.d.full.max_seq * (int64_t)z.kv_dim,
                    "KV cache: %lld floats is not a whole number of positions of %zu, at most %d", (long long)floats, z.kv_dim,
                    a.d.full.max_seq);
        dev = which == MOE_ST_K_CACHE ? ls.k_cache : ls.v_cache;
        want = floats;
        break;
    case MOE_ST_CONV:
    case MOE_ST_SSM:
        MOE_REQUIRE(!ls.full, "layer %d is a full-attention layer: it has no conv / recurrence state", layer);
        dev = which == MOE_ST_CONV ? ls.conv_state : ls.ssm_state;
        want = which == MOE_ST_CONV ? (int64_t)a.d.conv_kernel * (int64_t)z.conv_dim : (int64_t)(z.total_value * a.d.lin_key_dim);
        MOE_REQUIRE(floats == want, "state tensor %d of layer %d holds %lld floats, not %lld", which, layer, (long long)want,
                    (long long)floats);
        break;
    default:
        MOE_REQUIRE(false, "unknown state tensor %d", which);
    }
    if (want == 0) return MOE_OK;
    MOE_REQUIRE(host != nullptr, "null host buffer");
    if (to_device)
        MOE_CUDA(cudaMemcpyAsync(dev, host, (size_t)want * 4, cudaMemcpyHostToDevice, e->stream));
    else
        MOE_CUDA(cudaMemcpyAsync(host, dev, (size_t)want * 4, cudaMemcpyDeviceToHost, e->stream));
    MOE_CUDA(cudaStreamSynchronize(e->stream));
    return MOE_OK;
}

size_t attn_state_bytes(const moe_engine* e) {
    const ModelAttnState& a = e->attn;
    if (!a.configured) return 0;
    const AttnSizes z = attn_sizes(e);
    const size_t per = (size_t)a.d.conv_kernel * z.conv_dim * 4 + z.total_value * a.d.lin_key_dim * 4;
    size_t n = 0;
    for (const AttnLayerState& ls : a.layers) n += ls.full ? 0 : per;
    return n;
}

int attn_state_copy(moe_engine* e, uint8_t* buf, bool save) {
    ModelAttnState& a = e->attn;
    const AttnSizes z = attn_sizes(e);
    const size_t cb = (size_t)a.d.conv_kernel * z.conv_dim * 4, sb = z.total_value * a.d.lin_key_dim * 4;
    size_t off = 0;
    for (AttnLayerState& ls : a.layers) {
        if (ls.full) continue;
        if (save) {
            MOE_CUDA(cudaMemcpyAsync(buf + off, ls.conv_state, cb, cudaMemcpyDeviceToDevice, e->stream));
            MOE_CUDA(cudaMemcpyAsync(buf + off + cb, ls.ssm_state, sb, cudaMemcpyDeviceToDevice, e->stream));
        } else {
            MOE_CUDA(cudaMemcpyAsync(ls.conv_state, buf + off, cb, cudaMemcpyDeviceToDevice, e->stream));
            MOE_CUDA(cudaMemcpyAsync(ls.ssm_state, buf + off + cb, sb, cudaMemcpyDeviceToDevice, e->stream));
        }
        off += cb + sb;
    }
    return MOE_OK;
}

int attn_configure(moe_engine* e, const moe_model_attn_dims_t* dims) {
    const moe_attn_dims_t& f = dims->full;
    MOE_REQUIRE(f.num_heads > 0 && f.num_kv_heads > 0 && f.num_heads % f.num_kv_heads == 0,
                "attention heads (%d) must be a positive multiple of the key/value heads (%d)", f.num_heads, f.num_kv_heads);
    MOE_REQUIRE(f.head_dim > 0 && f.head_dim % 8 == 0 && f.head_dim <= 32 * kAttnPerLane, "head_dim (%d) must be a multiple of 8 up to 256", f.head_dim);
    MOE_REQUIRE(f.rotary_dim >= 0 && f.rotary_dim <= f.head_dim && f.rotary_dim % 2 == 0,
                "rotary_dim (%d) must be even and at most head_dim (%d)", f.rotary_dim, f.head_dim);
    MOE_REQUIRE(f.max_seq > 0 && f.max_seq <= 8192, "max_seq (%d) must be in 1..8192", f.max_seq);
    MOE_REQUIRE(dims->lin_num_k_heads > 0 && dims->lin_num_v_heads > 0 && dims->lin_num_v_heads % dims->lin_num_k_heads == 0,
                "linear-attention value heads (%d) must be a positive multiple of the key heads (%d)", dims->lin_num_v_heads,
                dims->lin_num_k_heads);
    MOE_REQUIRE(dims->lin_key_dim > 0 && dims->lin_key_dim <= 32 * kLinPerMax && dims->lin_value_dim > 0 && dims->lin_value_dim <= 2048 &&
                    dims->conv_kernel >= 2 && dims->conv_kernel <= 16,
                "linear-attention dimensions out of range (key_dim <= %d, value_dim <= 2048, conv kernel 2..16)", 32 * kLinPerMax);
    MOE_REQUIRE(dims->full_attn_interval >= 1, "full_attention_interval must be at least 1");
    attn_destroy(e);
    ModelAttnState& a = e->attn;
    a.d = *dims;
    const AttnSizes z = attn_sizes(e);
    MOE_REQUIRE(z.q_dim % 64 == 0 && z.total_value % 64 == 0 && z.q_dim <= 16384 && z.total_value <= 16384,
                "attention widths must be multiples of 64 up to 16384");
    a.layers.resize((size_t)e->dims.num_layers);
    for (int l = 0; l < e->dims.num_layers; ++l) {
        AttnLayerState& ls = a.layers[l];
        ls.full = (l + 1) % dims->full_attn_interval == 0;
        if (ls.full) {
            MOE_CUDA(cudaMalloc(&ls.k_cache, (size_t)f.max_seq * z.kv_dim * 4));
            MOE_CUDA(cudaMalloc(&ls.v_cache, (size_t)f.max_seq * z.kv_dim * 4));
        } else {
            MOE_CUDA(cudaMalloc(&ls.conv_state, (size_t)dims->conv_kernel * z.conv_dim * 4));
            MOE_CUDA(cudaMalloc(&ls.ssm_state, z.total_value * dims->lin_key_dim * 4));
        }
    }
    // scratch of one step: h_mid, ping, pong, x [H]; the stacked projections' output;
    // vals, normed [max(q_dim, total_value)]; qr [q_dim]
    const size_t mid = z.q_dim > z.total_value ? z.q_dim : z.total_value;
    size_t bytes = 4 * al256a(z.H * 4) + al256a(attn_proj_out_floats(z, (size_t)dims->lin_num_v_heads) * 4) +
                   2 * al256a(mid * 4) + al256a(z.q_dim * 4);
    MOE_CUDA(cudaMalloc(&a.work, bytes));
    MOE_CUDA(cudaMalloc(&a.d_pos, 256));
    {
        // positions 0 .. max_seq - 1 as a device table: a launch that is not replayed takes its position from there
        std::vector<int> tab((size_t)dims->full.max_seq);
        for (int i = 0; i < dims->full.max_seq; ++i) tab[(size_t)i] = i;
        MOE_CUDA(cudaMalloc(&a.pos_table, tab.size() * sizeof(int)));
        MOE_CUDA(cudaMemcpy(a.pos_table, tab.data(), tab.size() * sizeof(int), cudaMemcpyHostToDevice));
    }
    // function attributes are set here, never between the launches of a layer (those are captured into graphs)
    MOE_CUDA(cudaFuncSetAttribute(matvec_bf16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 16384 * 4));
    e->mtp.bf_attr_set = true;
    int rc = matvec_prepare(e);
    if (rc) return rc;
    a.configured = true;
    return attn_reset(e);
}

int attn_load_tensor(moe_engine* e, int layer, int which, const void* w, const void* s, const void* b, int dtype) {
    ModelAttnState& a = e->attn;
    if (!a.configured) {
        set_error("moe_attn_configure must come before the attention tensors");
        return MOE_ERR_STATE;
    }
    MOE_REQUIRE(layer >= 0 && layer < e->dims.num_layers, "attention tensor: layer %d out of range", layer);
    MOE_REQUIRE(which >= 0 && which <= MOE_A_OUT_PROJ, "unknown attention tensor %d", which);
    MOE_REQUIRE(w, "%s: null weight pointer", attn_tensor_name(which));
    AttnLayerState& ls = a.layers[layer];
    attn_drop_graphs(e);  // captured launches hold the old pointers
    MOE_REQUIRE(which == MOE_A_INPUT_NORM || attn_role_is_full(which) == ls.full, "layer %d is a %s layer: it has no %s", layer,
                ls.full ? "full-attention" : "linear-attention", attn_tensor_name(which));
    const AttnSizes z = attn_sizes(e);
    const moe_model_attn_dims_t& d = a.d;
    if (!attn_is_proj(which)) {
        size_t bytes = 0;
        int want = MOE_DT_BF16;
        switch (which) {
            case MOE_A_INPUT_NORM: bytes = z.H * 2; break;
            case MOE_A_Q_NORM: case MOE_A_K_NORM: bytes = (size_t)d.full.head_dim * 2; break;
            case MOE_A_CONV1D: bytes = z.conv_dim * d.conv_kernel * 2; break;
            case MOE_A_A_LOG: bytes = (size_t)d.lin_num_v_heads * 4; want = MOE_DT_F32; break;
            case MOE_A_DT_BIAS: bytes = (size_t)d.lin_num_v_heads * 2; break;
            default: bytes = (size_t)d.lin_value_dim * 2; break;  // linear_attn.norm
        }
        MOE_REQUIRE(dtype == want, "%s must be %s", attn_tensor_name(which), want == MOE_DT_F32 ? "f32" : "bf16");
        if (!ls.vec[which]) MOE_CUDA(cudaMalloc(&ls.vec[which], al256a(bytes)));
        MOE_CUDA(cudaMemcpyAsync(ls.vec[which], w, bytes, cudaMemcpyHostToDevice, e->stream));
        MOE_CUDA(cudaStreamSynchronize(e->stream));
        return MOE_OK;
    }
    size_t rows = 0, cols = z.H;
    switch (which) {
        case MOE_A_Q_PROJ: rows = 2 * z.q_dim; break;
        case MOE_A_K_PROJ: case MOE_A_V_PROJ: rows = z.kv_dim; break;
        case MOE_A_O_PROJ: rows = z.H; cols = z.q_dim; break;
        case MOE_A_IN_PROJ_QKV: rows = z.conv_dim; break;
        case MOE_A_IN_PROJ_Z: rows = z.total_value; break;
        case MOE_A_IN_PROJ_B: case MOE_A_IN_PROJ_A: rows = (size_t)d.lin_num_v_heads; break;
        default: rows = z.H; cols = z.total_value; break;  // out_proj
    }
    MOE_REQUIRE(dtype == MOE_DT_INT4 || dtype == MOE_DT_BF16, "%s: dtype %d not supported", attn_tensor_name(which), dtype);
    ProjTensor& t = ls.proj[which];
    if (t.w) { cudaFree(t.w); t = ProjTensor{}; }
    t.dtype = dtype; t.rows = (int)rows; t.cols = (int)cols;
    if (dtype == MOE_DT_BF16) {
        MOE_CUDA(cudaMalloc(&t.w, rows * cols * 2));
        MOE_CUDA(cudaMemcpyAsync(t.w, w, rows * cols * 2, cudaMemcpyHostToDevice, e->stream));
    } else {
        MOE_REQUIRE(s && b, "%s: a 4-bit tensor needs scales and biases", attn_tensor_name(which));
        const size_t wb = rows * cols / 2, sb = rows * (cols / 64) * 2;
        t.s_off = al256a(wb);
        t.b_off = t.s_off + al256a(sb);
        MOE_CUDA(cudaMalloc(&t.w, t.b_off + al256a(sb)));
        MOE_CUDA(cudaMemcpyAsync(t.w, w, wb, cudaMemcpyHostToDevice, e->stream));
        MOE_CUDA(cudaMemcpyAsync(t.w + t.s_off, s, sb, cudaMemcpyHostToDevice, e->stream));
        MOE_CUDA(cudaMemcpyAsync(t.w + t.b_off, b, sb, cudaMemcpyHostToDevice, e->stream));
    }
    MOE_CUDA(cudaStreamSynchronize(e->stream));
    t.loaded = true;
    return MOE_OK;
}

// Stacks a layer's input projections row-wise into one tensor (same storage type and width required; otherwise the
// layer keeps its separate launches).  The originals stay loaded.
static int attn_fuse_layer(moe_engine* e, AttnLayerState& ls) {
    if (ls.fused.w) { cudaFree(ls.fused.w); ls.fused = ProjTensor{}; }
    const int full_parts[] = {MOE_A_Q_PROJ, MOE_A_K_PROJ, MOE_A_V_PROJ};
    const int lin_parts[] = {MOE_A_IN_PROJ_QKV, MOE_A_IN_PROJ_Z, MOE_A_IN_PROJ_B, MOE_A_IN_PROJ_A};
    const int* parts = ls.full ? full_parts : lin_parts;
    const int np = ls.full ? 3 : 4;
    size_t rows = 0;
    for (int i = 0; i < np; ++i) {
        const ProjTensor& t = ls.proj[parts[i]];
        if (!t.loaded || t.dtype != ls.proj[parts[0]].dtype || t.cols != ls.proj[parts[0]].cols) return MOE_OK;
        rows += (size_t)t.rows;
    }
    const int dtype = ls.proj[parts[0]].dtype;
    const size_t cols = (size_t)ls.proj[parts[0]].cols;
    ProjTensor f;
    f.dtype = dtype; f.rows = (int)rows; f.cols = (int)cols;
    if (dtype == MOE_DT_BF16) {
        MOE_CUDA(cudaMalloc(&f.w, rows * cols * 2));
        size_t off = 0;
        for (int i = 0; i < np; ++i) {
            const ProjTensor& t = ls.proj[parts[i]];
            MOE_CUDA(cudaMemcpyAsync(f.w + off, t.w, (size_t)t.rows * cols * 2, cudaMemcpyDeviceToDevice, e->stream));
            off += (size_t)t.rows * cols * 2;
        }
    } else {
        const size_t wb = rows * cols / 2, sb = rows * (cols / 64) * 2;
        f.s_off = al256a(wb);
        f.b_off = f.s_off + al256a(sb);
        MOE_CUDA(cudaMalloc(&f.w, f.b_off + al256a(sb)));
        size_t wo = 0, so = 0;
        for (int i = 0; i < np; ++i) {
            const ProjTensor& t = ls.proj[parts[i]];
            const size_t twb = (size_t)t.rows * cols / 2, tsb = (size_t)t.rows * (cols / 64) * 2;
            MOE_CUDA(cudaMemcpyAsync(f.w + wo, t.w, twb, cudaMemcpyDeviceToDevice, e->stream));
            MOE_CUDA(cudaMemcpyAsync(f.w + f.s_off + so, t.w + t.s_off, tsb, cudaMemcpyDeviceToDevice, e->stream));
            MOE_CUDA(cudaMemcpyAsync(f.w + f.b_off + so, t.w + t.b_off, tsb, cudaMemcpyDeviceToDevice, e->stream));
            wo += twb;
            so += tsb;
        }
    }
    MOE_CUDA(cudaStreamSynchronize(e->stream));
    f.loaded = true;
    ls.fused = f;
    return MOE_OK;
}

// One layer's attention half on one token: h (device, [H]) -> h_mid (device, [H]) = attention(h) + h.
// first_pdl: the layer's first kernel is itself a programmatic dependent of the kernel before it in the stream
// pos_ptr: where the kernels read the token's position (null: the engine's device-side position word)
// floats of one token's scratch as attn_layer_step carves it
static size_t attn_scratch_floats(const moe_engine* e) {
    const AttnSizes z = attn_sizes(e);
    const size_t mid_n = z.q_dim > z.total_value ? z.q_dim : z.total_value;
    return (al256a(z.H * 4) + al256a(attn_proj_out_floats(z, (size_t)e->attn.d.lin_num_v_heads) * 4) + 2 * al256a(mid_n * 4) +
            al256a(z.q_dim * 4)) / 4;
}
// whether a layer's projections can run over several tokens in one launch (attn_layer_step with batch > 1): stacked
// input projections with the input norm folded in
static bool attn_layer_batchable(const AttnLayerState& ls) { return ls.fused.loaded && proj_folds_norm(ls.fused); }

// whether a DeltaNet layer runs as 256-thread CTAs per block of state rows with the gated norm's 1/rms left to the output
// projection (lin_part_kernel), and whether a run of tokens can then go through it in one launch (lin_seq_kernel)
static bool attn_lin_split(const moe_engine* e, const AttnLayerState& ls) {
    const ModelAttnState& a = e->attn;
    const moe_model_attn_dims_t& d = a.d;
    const AttnSizes z = attn_sizes(e);
    const size_t mid_n = z.q_dim > z.total_value ? z.q_dim : z.total_value;
    const ProjTensor& op = ls.proj[MOE_A_OUT_PROJ];
    const int parts = (d.lin_value_dim + kLpRows - 1) / kLpRows;
    return a.lin_split && !ls.full && op.loaded && op.dtype == MOE_DT_INT4 && ls.vec[MOE_A_LIN_NORM] != nullptr &&
           matvec_folds_head_scale(op.rows, op.cols, d.lin_value_dim) && 2 * d.lin_key_dim + kLpRows <= kLpCh * kLpThreads &&
           (size_t)d.lin_num_v_heads * parts <= mid_n;
}
static bool attn_lin_seq_ok(const moe_engine* e, const AttnLayerState& ls) {
    return attn_lin_split(e, ls) && ls.vec[MOE_A_CONV1D] != nullptr && e->attn.d.conv_kernel <= kLpK && e->attn.d.conv_kernel >= 2;
}

constexpr int kPhProj = 1, kPhCore = 2, kPhOut = 4;
// phases: which of input projections / core (cache or state update, token-serial) / output projection + residual to run;
// batch > 1 (projection phases only, batchable layers): that many tokens in one launch, token t's h and h_mid rows
// hidden-size floats apart and its scratch tok_stride floats apart
static int attn_layer_step(moe_engine* e, int layer, const float* h, float* h_mid, float* scratch, bool first_pdl = false,
                           const int* pos_ptr = nullptr, int phases = kPhProj | kPhCore | kPhOut, int batch = 1,
                           size_t tok_stride = 0) {
    ModelAttnState& a = e->attn;
    AttnLayerState& ls = a.layers[layer];
    const moe_model_attn_dims_t& d = a.d;
    const AttnSizes z = attn_sizes(e);
    const int H = (int)z.H;
    const size_t Hv = (size_t)d.lin_num_v_heads;
    cudaStream_t st = e->stream;
    const int* posp = pos_ptr ? pos_ptr : a.d_pos;
    const size_t mid_n = z.q_dim > z.total_value ? z.q_dim : z.total_value;
    float* p = scratch;
    auto take = [&](size_t n) { float* r = p; p += al256a(n * 4) / 4; return r; };
    float* x = take(z.H);
    float* proj_out = take(attn_proj_out_floats(z, Hv));  // the stacked projections' output
    float* vals = take(mid_n); float* normed = take(mid_n);
    float* qr = take(z.q_dim);
    auto need = [&](int which) -> bool {
        const bool ok = attn_is_proj(which) ? ls.proj[which].loaded : ls.vec[which] != nullptr;
        if (!ok) set_error("layer %d: the attention half is not loaded (%s missing)", layer, attn_tensor_name(which));
        return ok;
    };
    if (!need(MOE_A_INPUT_NORM)) return MOE_ERR_STATE;
    // the input norm is folded into the stacked projection where its kernel can do that; a kernel of its own otherwise
    const bool fold = ls.fused.loaded && proj_folds_norm(ls.fused);
    const void* fold_w = fold ? ls.vec[MOE_A_INPUT_NORM] : nullptr;
    const float* proj_in = fold ? h : x;
    bool pdl = first_pdl && a.pdl;  // every kernel after the first may start ahead of its predecessor's end (see pdl_wait)
    MOE_REQUIRE(batch == 1 || fold, "layer %d: a batched step needs stacked projections", layer);
    const int core_n = batch;  // tokens of a full-attention core launch (the cache rows of all of them are written first)
    MvBatch mb_in{}, mb_out{};
    if (batch > 1) {
        mb_in.n = batch; mb_in.x_stride = H; mb_in.y_stride = (int)tok_stride;
        mb_out.n = batch; mb_out.x_stride = (int)tok_stride; mb_out.y_stride = H; mb_out.r_stride = H; mb_out.ss_stride = (int)tok_stride;
    }
    if (!fold && (phases & kPhProj)) {
        MOE_CUDA(launch_kernel(pdl, rms_norm_rows_kernel, dim3(1), dim3(256), 0, st, h, (const uint16_t*)ls.vec[MOE_A_INPUT_NORM], H, x));
        e->launches++;
        pdl = a.pdl;
    }
    int rc;
    if (ls.full) {
        for (int w : {MOE_A_Q_PROJ, MOE_A_K_PROJ, MOE_A_V_PROJ, MOE_A_Q_NORM, MOE_A_K_NORM, MOE_A_O_PROJ})
            if (!need(w)) return MOE_ERR_STATE;
        const int nh = d.full.num_heads, nkv = d.full.num_kv_heads, hd = d.full.head_dim;
        float* qb = proj_out;                  // [head, gate] per head
        float* kb = qb + 2 * z.q_dim;
        float* vb = kb + z.kv_dim;
        if (!(phases & kPhProj)) {
        } else if (ls.fused.loaded) {
            if ((rc = proj_run(e, ls.fused, proj_in, proj_out, nullptr, pdl, fold_w, mb_in))) return rc;
            pdl = a.pdl;
        } else {
            if ((rc = proj_run(e, ls.proj[MOE_A_Q_PROJ], x, qb, nullptr, pdl))) return rc;
            if ((rc = proj_run(e, ls.proj[MOE_A_K_PROJ], x, kb, nullptr, pdl))) return rc;
            if ((rc = proj_run(e, ls.proj[MOE_A_V_PROJ], x, vb, nullptr, pdl))) return rc;
        }
        if (phases & kPhCore) {
        MOE_CUDA(launch_kernel(pdl, attn_prep_kernel, dim3(nh + nkv, core_n), dim3(256), (size_t)hd * 4, st, qb, 2 * hd, 1, kb, vb,
                               (const uint16_t*)ls.vec[MOE_A_Q_NORM], (const uint16_t*)ls.vec[MOE_A_K_NORM], nh, nkv, hd,
                               d.full.rotary_dim, 0, posp, d.full.rope_theta, qr, ls.k_cache, ls.v_cache, (int)tok_stride));
        pdl = a.pdl;
        // the position is read on the device and the score buffer is sized for the whole cache: the launch never changes
        MOE_CUDA(launch_kernel(pdl, attn_decode_kernel, dim3(nh, core_n), dim3(kAttnWarps * 32), (size_t)(d.full.max_seq + hd * (1 + kAttnWarps)) * 4, st, qr, ls.k_cache,
                               ls.v_cache, qb + hd, 2 * hd, nh, nkv, hd, 0, posp, 1.0f / sqrtf((float)hd), vals, (int)tok_stride));
        e->launches += 2;
        pdl = a.pdl;
        }
        if ((phases & kPhOut) && (rc = proj_run(e, ls.proj[MOE_A_O_PROJ], vals, h_mid, h, pdl, nullptr, mb_out))) return rc;  // + residual
    } else {
        for (int w : {MOE_A_IN_PROJ_QKV, MOE_A_IN_PROJ_Z, MOE_A_IN_PROJ_B, MOE_A_IN_PROJ_A, MOE_A_OUT_PROJ})
            if (!need(w)) return MOE_ERR_STATE;
        float* qkv_raw = proj_out;
        float* zb = qkv_raw + z.conv_dim;
        float* bb = zb + z.total_value;
        float* ab = bb + Hv;
        if (!(phases & kPhProj)) {
        } else if (ls.fused.loaded) {
            if ((rc = proj_run(e, ls.fused, proj_in, proj_out, nullptr, pdl, fold_w, mb_in))) return rc;
            pdl = a.pdl;
        } else {
            if ((rc = proj_run(e, ls.proj[MOE_A_IN_PROJ_QKV], x, qkv_raw, nullptr, pdl))) return rc;
            if ((rc = proj_run(e, ls.proj[MOE_A_IN_PROJ_Z], x, zb, nullptr, pdl))) return rc;
            if ((rc = proj_run(e, ls.proj[MOE_A_IN_PROJ_B], x, bb, nullptr, pdl))) return rc;
            if ((rc = proj_run(e, ls.proj[MOE_A_IN_PROJ_A], x, ab, nullptr, pdl))) return rc;
        }
        // a head's state rows dealt to several small CTAs, the gated norm folded into the output projection's kernel,
        // where that kernel can do it; one large CTA per head doing everything otherwise
        const ProjTensor& op = ls.proj[MOE_A_OUT_PROJ];
        const int parts = (d.lin_value_dim + kLpRows - 1) / kLpRows;
        const bool split = attn_lin_split(e, ls);
        MOE_REQUIRE(batch == 1 || !(phases & kPhCore) || attn_lin_seq_ok(e, ls), "layer %d: its DeltaNet core runs one token at a time", layer);
        if (split) {
            auto* part_kernel = d.lin_key_dim <= 128 ? lin_part_kernel<4> : lin_part_kernel<8>;
            float* ss_part = normed;  // one sum of squares per CTA
            if ((phases & kPhCore) && batch > 1) {
                auto* seq_kernel = d.lin_key_dim <= 128 ? lin_seq_kernel<4> : lin_seq_kernel<8>;
                MOE_CUDA(launch_kernel(pdl, seq_kernel, dim3(d.lin_num_v_heads * parts), dim3(kLpThreads),
                                       (size_t)(2 * d.lin_key_dim + kLpRows) * 4, st, ls.conv_state, qkv_raw,
                                       (const uint16_t*)ls.vec[MOE_A_CONV1D], ab, bb, (const float*)ls.vec[MOE_A_A_LOG],
                                       (const uint16_t*)ls.vec[MOE_A_DT_BIAS], ls.ssm_state, zb, (const uint16_t*)ls.vec[MOE_A_LIN_NORM],
                                       vals, ss_part, posp, (int)z.total_key, (int)z.conv_dim, d.conv_kernel,
                                       d.lin_num_v_heads / d.lin_num_k_heads, d.lin_key_dim, d.lin_value_dim, parts, batch,
                                       (int)tok_stride));
                e->launches++;
                pdl = a.pdl;
            } else if (phases & kPhCore) {
            MOE_CUDA(launch_kernel(pdl, part_kernel, dim3(d.lin_num_v_heads * parts), dim3(kLpThreads),
                                   (size_t)(2 * d.lin_key_dim + kLpRows) * 4, st, ls.conv_state, qkv_raw,
                                   (const uint16_t*)ls.vec[MOE_A_CONV1D], ab, bb, (const float*)ls.vec[MOE_A_A_LOG],
                                   (const uint16_t*)ls.vec[MOE_A_DT_BIAS], ls.ssm_state, zb, (const uint16_t*)ls.vec[MOE_A_LIN_NORM],
                                   vals, ss_part, posp, (int)z.total_key, (int)z.conv_dim, d.conv_kernel,
                                   d.lin_num_v_heads / d.lin_num_k_heads, d.lin_key_dim, d.lin_value_dim, parts));
            e->launches++;
            pdl = a.pdl;
            }
            if ((phases & kPhOut) && (rc = launch_matvec_head_scaled(e, op.w, op.w + op.s_off, op.w + op.b_off, vals, ss_part, parts,
                                                                     d.lin_value_dim, h_mid, op.rows, op.cols, h, pdl, mb_out)))
                return rc;
            MOE_CUDA(cudaGetLastError());
            return MOE_OK;
        }
        const size_t lin_smem = (size_t)(2 * d.lin_key_dim + 2 * d.lin_value_dim) * 4;
        auto* lin_kernel = d.lin_key_dim <= 128 ? lin_core_kernel<4> : lin_core_kernel<8>;
        if (phases & kPhCore) {
        MOE_CUDA(launch_kernel(pdl, lin_kernel, dim3(d.lin_num_v_heads), dim3(kLinThreads), lin_smem, st, ls.conv_state, qkv_raw,
                               (const uint16_t*)ls.vec[MOE_A_CONV1D], zb, ab, bb, (const float*)ls.vec[MOE_A_A_LOG],
                               (const uint16_t*)ls.vec[MOE_A_DT_BIAS], (const uint16_t*)ls.vec[MOE_A_LIN_NORM], ls.ssm_state, normed,
                               posp, (int)z.total_key, (int)z.conv_dim, d.conv_kernel, d.lin_num_v_heads / d.lin_num_k_heads,
                               d.lin_key_dim, d.lin_value_dim));
        e->launches++;
        pdl = a.pdl;
        }
        if ((phases & kPhOut) && (rc = proj_run(e, ls.proj[MOE_A_OUT_PROJ], normed, h_mid, h, pdl, nullptr, mb_out))) return rc;  // + residual
    }
    MOE_CUDA(cudaGetLastError());
    return MOE_OK;
}

// Two ways to run a token's 160-odd kernels.  The default ("chain"): every kernel, the MoE kernels included, is launched
// from the host as a programmatic dependent of the one before it, so each becomes resident, requests its weights and only
// then waits for its input while its predecessor still runs (the host enqueues a token in about 0.4 ms, the device needs
// four times that).  MOE_B200_ATTN_CHAIN=0 selects the other: every layer's attention half captured (fixed pointers,
// position read on the device) into a CUDA graph, so a token costs one graph launch + the MoE launch per layer; the
// graph's kernels are chained in the same way, but the graph and the MoE kernel meet at ordinary stream dependencies.
// Inside a graph (and in the eager path alike) every kernel after the first is a programmatic dependent of the one
// before it: it becomes resident while its predecessor still runs, asks for its weights (L2 prefetch) and only then
// waits for the predecessor's results.  MOE_B200_ATTN_GRAPHS=0 keeps the eager launches, MOE_B200_ATTN_PDL=0 the
// ordinary dependencies.
static int attn_build_graphs(moe_engine* e, const float* const* layer_in, float* h_mid, float* scratch) {
    ModelAttnState& a = e->attn;
    attn_drop_graphs(e);
    const char* env = getenv("MOE_B200_ATTN_GRAPHS");
    const char* env_pdl = getenv("MOE_B200_ATTN_PDL");
    a.pdl = !(env_pdl && atoi(env_pdl) == 0);
    const char* env_chain = getenv("MOE_B200_ATTN_CHAIN");
    a.chain = a.pdl && !(env_chain && atoi(env_chain) == 0);
    const char* env_pre = getenv("MOE_B200_PREFILL_MIN");
    a.prefill_min = env_pre ? atoi(env_pre) : 4;  // 5.2 against 6.1 ms at 4 tokens, 6.3 against 9.2 ms at 6; 3 tokens and fewer lose
    if (a.prefill_min < 2) a.prefill_min = 1 << 30;  // 0 or 1: token by token always
    const char* env_split = getenv("MOE_B200_LIN_SPLIT");
    a.lin_split = !(env_split && atoi(env_split) == 0);
    const int L = e->dims.num_layers;
    a.graphs.assign((size_t)L, nullptr);
    a.graph_nodes.assign((size_t)L, 0);
    a.graphs_valid = true;
    for (AttnLayerState& ls : a.layers) {
        const int rc = attn_fuse_layer(e, ls);
        if (rc) return rc;
    }
    if ((env && atoi(env) == 0) || a.chain) return MOE_OK;
    for (int l = 0; l < L; ++l) {
        const int64_t before = e->launches;
        if (cudaStreamBeginCapture(e->stream, cudaStreamCaptureModeThreadLocal) != cudaSuccess) {
            cudaGetLastError();
            return MOE_OK;  // capture unavailable: eager launches
        }
        const int rc = attn_layer_step(e, l, layer_in[l], h_mid, scratch);
        cudaGraph_t g = nullptr;
        const cudaError_t ce = cudaStreamEndCapture(e->stream, &g);
        e->launches = before;  // nothing ran
        if (rc) {
            if (g) cudaGraphDestroy(g);
            attn_drop_graphs(e);
            return rc;  // a missing tensor: reported as in the eager path
        }
        if (ce != cudaSuccess || !g) {
            cudaGetLastError();
            continue;
        }
        size_t nodes = 0;
        cudaGraphGetNodes(g, nullptr, &nodes);
        cudaGraphExec_t ex = nullptr;
        if (cudaGraphInstantiate(&ex, g, 0) == cudaSuccess) {
            a.graphs[l] = ex;
            a.graph_nodes[l] = (int)nodes;
        } else {
            cudaGetLastError();
        }
        cudaGraphDestroy(g);
    }
    return MOE_OK;
}

// Several tokens at once (a prompt), layer by layer: the attention half of a layer runs token after token (its state
// carries from one to the next) with the layer's projections staying in L2 from the first token on, and the layer's MoE
// half then takes all the tokens in one batched call (launch_batched_layer: every expert's weights read once).  The same
// arithmetic as token by token, except that the MoE half of a batch above 48 tokens computes on bf16 operands
// (the grouped GEMMs) like any batched call.
static int attn_model_prefill(moe_engine* e, const float* emb_dev, int32_t n, float* out_dev, float* scratch) {
    ModelAttnState& a = e->attn;
    const size_t H = (size_t)e->dims.hidden;
    const int L = e->dims.num_layers;
    int rc = batch_reserve(e, n);   // its two [n, H] buffers hold the layers' outputs in turn
    if (rc) return rc;
    if (a.prefill_cap < n) {
        MOE_CUDA(cudaStreamSynchronize(e->stream));
        if (a.prefill_mid) cudaFree(a.prefill_mid);
        a.prefill_mid = nullptr;
        a.prefill_cap = 0;
        MOE_CUDA(cudaMalloc(&a.prefill_mid, (size_t)n * (H + attn_scratch_floats(e)) * 4));
        a.prefill_scratch = a.prefill_mid + (size_t)n * H;   // every token's own scratch (projection outputs, core outputs)
        a.prefill_cap = n;
    }
    const float* cur = emb_dev;
    const size_t S = attn_scratch_floats(e);
    for (int l = 0; l < L; ++l) {
        const AttnLayerState& ls = a.layers[l];
        if (attn_layer_batchable(ls)) {
            // the projections of all the tokens in one launch each (they depend on the layer's input only), the token-serial
            // core in between.  The DeltaNet kernel reads the layer's conv ring and recurrence state ahead of its dependency
            // wait, which is only safe once the previous token's kernel, which writes them, has completed: ordinary launches.
            // (The two attention kernels of a full-attention layer could chain from token to token, but a chain of hundreds of
            // tiny grids that all become resident and wait for one another ran at 26 us per kernel instead of 8.)
            if ((rc = attn_layer_step(e, l, cur, a.prefill_mid, a.prefill_scratch, false, nullptr, kPhProj, n, S))) return rc;
            if (ls.full || attn_lin_seq_ok(e, ls)) {
                // full attention: every token's K / V rows first, then every token's attention over its own prefix (two launches);
                // DeltaNet: one launch that keeps the state in registers from the first token to the last
                // (both wait for their predecessor before they touch anything: programmatic dependents of the projection)
                if ((rc = attn_layer_step(e, l, cur, a.prefill_mid, a.prefill_scratch, true, a.pos_table + a.pos, kPhCore, n, S))) return rc;
            } else {
                for (int t = 0; t < n; ++t)
                    if ((rc = attn_layer_step(e, l, cur + (size_t)t * H, a.prefill_mid + (size_t)t * H, a.prefill_scratch + (size_t)t * S,
                                              false, a.pos_table + a.pos + t, kPhCore)))
                        return rc;
            }
            if ((rc = attn_layer_step(e, l, cur, a.prefill_mid, a.prefill_scratch, true, nullptr, kPhOut, n, S))) return rc;
        } else {
            for (int t = 0; t < n; ++t)  // a token's first kernel the ordinary way, for the same reason
                if ((rc = attn_layer_step(e, l, cur + (size_t)t * H, a.prefill_mid + (size_t)t * H, scratch, false, a.pos_table + a.pos + t)))
                    return rc;
        }
        float* nxt = (l == L - 1) ? out_dev : ((l & 1) ? e->bw.h_b : e->bw.h_a);
        rc = launch_batched_layer(e, l, a.prefill_mid, n, nxt, nullptr, nullptr, nullptr, nullptr);
        if (rc) return rc;
        cur = nxt;
    }
    a.pos += n;
    return MOE_OK;
}

int attn_model_forward(moe_engine* e, const float* emb_dev, int32_t n, float* out_dev) {
    ModelAttnState& a = e->attn;
    if (!a.configured) {
        set_error("the attention halves are not configured (moe_attn_configure)");
        return MOE_ERR_STATE;
    }
    if (a.pos + n > a.d.full.max_seq) {
        set_error("the KV caches hold %d positions: %lld + %d tokens do not fit", a.d.full.max_seq, (long long)a.pos, n);
        return MOE_ERR_STATE;
    }
    const size_t H = (size_t)e->dims.hidden;
    const int L = e->dims.num_layers;
    float* h_mid = a.work;
    float* ping = a.work + al256a(H * 4) / 4;
    float* pong = ping + al256a(H * 4) / 4;
    float* scratch = pong + al256a(H * 4) / 4;
    // every layer reads from a fixed buffer: layer 0 from `pong` (the token's embedding is copied there), layer l > 0
    // from where layer l - 1's MoE half wrote (ping / pong alternate); the last layer writes the caller's row
    std::vector<const float*> layer_in((size_t)L);
    std::vector<float*> layer_out((size_t)L);
    for (int l = 0; l < L; ++l) {
        layer_in[l] = (l == 0) ? pong : layer_out[l - 1];
        layer_out[l] = (l & 1) ? pong : ping;
    }
    if (!a.graphs_valid) {
        int rc = attn_build_graphs(e, layer_in.data(), h_mid, scratch);
        if (rc) return rc;
    }
    if (a.chain && n >= a.prefill_min) return attn_model_prefill(e, emb_dev, n, out_dev, scratch);
    for (int t = 0; t < n; ++t) {
        // graphs read the position from a fixed word (set per token); plain launches from the table entry of the position
        const int* pos_ptr = a.chain ? a.pos_table + a.pos : nullptr;
        if (!pos_ptr) {
            set_pos_kernel<<<1, 1, 0, e->stream>>>(a.d_pos, (int)a.pos);
            e->launches++;
        }
        MOE_CUDA(cudaMemcpyAsync(pong, emb_dev + (size_t)t * H, H * 4, cudaMemcpyDeviceToDevice, e->stream));
        for (int l = 0; l < L; ++l) {
            int rc = MOE_OK;
            if (a.graphs[l]) {
                MOE_CUDA(cudaGraphLaunch(a.graphs[l], e->stream));
                e->launches += a.graph_nodes[l];
            } else {
                // chained: a layer's first kernel depends programmatically on the MoE kernel of the layer before it
                rc = attn_layer_step(e, l, layer_in[l], h_mid, scratch, a.chain && l > 0, pos_ptr);
            }
            if (rc) return rc;
            float* nxt = (l == L - 1) ? out_dev + (size_t)t * H : layer_out[l];
            rc = launch_decode(e, l, l + 1, h_mid, nxt, nullptr, nullptr, nullptr, nullptr, a.chain);
            if (rc) return rc;
        }
        a.pos++;
    }
    return MOE_OK;
}

}  // namespace moe
