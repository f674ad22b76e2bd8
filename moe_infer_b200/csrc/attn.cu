// The MTP block's attention half, batch-1 decode: one gated full-attention layer with per-head q/k RMS norm,
// partial interleaved RoPE and an f32 KV cache (reference src/engine/qwen35_moe/mtp.rs:58-225), wrapped around
// the MoE half that the decode kernel already runs (layer index num_layers), the token embedding and the head.
//
// Everything here is a matrix-vector product or smaller: HBM-bound streaming kernels and a few tiny ones.
// Projections are bf16 matrices in the BQ4 scheme (bq4.rs:25-32) and 4-bit triples in the INT4 scheme.
#include "common.cuh"

namespace moe {

// ─── y = W x, W bf16 [rows, cols], f32 accumulate ────────────────────────────
// One warp per row, two rows in flight; a lane reads 16 bytes (8 weights) per step; x is staged in shared memory.
// 2 B per weight: bound by HBM bandwidth like the 4-bit matvec.
constexpr int kBfWarps = 8;

__global__ void __launch_bounds__(kBfWarps * 32) matvec_bf16_kernel(const uint16_t* __restrict__ w, const float* __restrict__ x,
                                                                   float* __restrict__ y, int rows, int cols) {
    extern __shared__ float xs[];
    for (int i = threadIdx.x; i < cols; i += blockDim.x) xs[i] = x[i];
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int stride = gridDim.x * kBfWarps * 2;
    for (int r0 = (blockIdx.x * kBfWarps + warp) * 2; r0 < rows; r0 += stride) {
        const bool two = r0 + 1 < rows;
        const uint16_t* wa = w + (size_t)r0 * cols;
        const uint16_t* wb = w + (size_t)(two ? r0 + 1 : r0) * cols;
        float a0 = 0.0f, a1 = 0.0f;
        for (int c = lane * 8; c < cols; c += 256) {
            const uint4 qa = ld_stream_u4(wa + c), qb = ld_stream_u4(wb + c);
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
        }
        a0 = warp_sum(a0);
        a1 = warp_sum(a1);
        if (lane == 0) {
            y[r0] = a0;
            if (two) y[r0 + 1] = a1;
        }
    }
}

// ─── RMS norm of `rows` vectors of `dim` elements with one bf16 weight vector (rms_norm, mtp.rs:261-266) ─────
__global__ void __launch_bounds__(256) rms_norm_rows_kernel(const float* __restrict__ x, const uint16_t* __restrict__ w, int dim,
                                                            float* __restrict__ out) {
    __shared__ float red[8];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float* row = x + (size_t)blockIdx.x * dim;
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

// ─── per-head norm + RoPE of q and k, K/V cache append (mtp.rs:137-157) ──────────────────────────────────────
// Block h < num_heads: query head h -> q_out.  Block num_heads + j: key head j -> k_cache[pos], and value head j
// is copied to v_cache[pos].  RoPE rotates the interleaved pairs (2i, 2i+1), i < rope_dim / 2, by pos * theta^(-2i/rope_dim).
__global__ void __launch_bounds__(256) attn_prep_kernel(const float* __restrict__ q, const float* __restrict__ k,
                                                        const float* __restrict__ v, const uint16_t* __restrict__ q_norm,
                                                        const uint16_t* __restrict__ k_norm, int num_heads, int num_kv_heads,
                                                        int head_dim, int rope_dim, int pos, float theta, float* __restrict__ q_out,
                                                        float* __restrict__ k_cache, float* __restrict__ v_cache) {
    extern __shared__ float hv[];  // the normed head
    __shared__ float red[8];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const bool is_q = (int)blockIdx.x < num_heads;
    const int h = is_q ? blockIdx.x : blockIdx.x - num_heads;
    const float* src = (is_q ? q : k) + (size_t)h * head_dim;
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
            const int p = i >> 1;
            const float freq = powf(theta, -2.0f * (float)p / (float)rope_dim);
            float sn, cs;
            sincosf((float)pos * freq, &sn, &cs);
            const float x0 = hv[i & ~1], x1 = hv[i | 1];
            o = (i & 1) ? x0 * sn + x1 * cs : x0 * cs - x1 * sn;
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
// exponentiated, summed; values: a thread per output element adds score / sum * v over the positions (coalesced
// across the head).  out = attention * sigmoid(gate).
__global__ void __launch_bounds__(256) attn_decode_kernel(const float* __restrict__ q, const float* __restrict__ k_cache,
                                                          const float* __restrict__ v_cache, const float* __restrict__ gate,
                                                          int num_heads, int num_kv_heads, int head_dim, int seq_len,
                                                          float kq_scale, float* __restrict__ out) {
    extern __shared__ float sc[];  // [seq_len] scores, then [head_dim] the query head
    __shared__ float red[8];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int h = blockIdx.x, kv_h = h / (num_heads / num_kv_heads);
    const size_t kv_dim = (size_t)num_kv_heads * head_dim;
    float* qs = sc + seq_len;
    for (int i = tid; i < head_dim; i += 256) qs[i] = q[(size_t)h * head_dim + i];
    __syncthreads();
    float mx = -INFINITY;
    for (int t = warp; t < seq_len; t += 8) {
        const float* kr = k_cache + (size_t)t * kv_dim + (size_t)kv_h * head_dim;
        float dot = 0.0f;
        for (int d = lane; d < head_dim; d += 32) dot = fmaf(qs[d], kr[d], dot);
        dot = warp_sum(dot) * kq_scale;
        if (lane == 0) sc[t] = dot;
        mx = fmaxf(mx, dot);
    }
    if (lane == 0) red[warp] = mx;
    __syncthreads();
    mx = red[0];
#pragma unroll
    for (int i = 1; i < 8; ++i) mx = fmaxf(mx, red[i]);
    __syncthreads();
    float sum = 0.0f;
    for (int t = tid; t < seq_len; t += 256) {
        const float e = expf(sc[t] - mx);
        sc[t] = e;
        sum += e;
    }
    sum = warp_sum(sum);
    if (lane == 0) red[warp] = sum;
    __syncthreads();
    float tot = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) tot += red[i];
    for (int d = tid; d < head_dim; d += 256) {
        const float* vc = v_cache + (size_t)kv_h * head_dim + d;
        float acc = 0.0f;
        for (int t = 0; t < seq_len; ++t) acc = fmaf(sc[t] / tot, vc[(size_t)t * kv_dim], acc);
        const float g = gate[(size_t)h * head_dim + d];
        out[(size_t)h * head_dim + d] = acc * (1.0f / (1.0f + expf(-g)));
    }
}

__global__ void __launch_bounds__(256) add_rows_kernel(const float* __restrict__ a, const float* __restrict__ b, int n, float* __restrict__ out) {
    const int i = blockIdx.x * 256 + threadIdx.x;
    if (i < n) out[i] = a[i] + b[i];
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
    MOE_REQUIRE(ad->head_dim > 0 && ad->head_dim % 8 == 0 && ad->head_dim <= 1024, "head_dim (%d) must be a multiple of 8 up to 1024", ad->head_dim);
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

static int mtp_project(moe_engine* e, int which, const float* x, float* y) {
    MtpAttnState& m = e->mtp;
    const ProjTensor& t = m.proj[which];
    if (t.dtype == MOE_DT_INT4) return launch_matvec(e, t.w, t.w + t.s_off, t.w + t.b_off, x, y, t.rows, t.cols);
    if (!m.bf_attr_set) {
        MOE_CUDA(cudaFuncSetAttribute(matvec_bf16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 16384 * 4));
        m.bf_attr_set = true;
    }
    int blocks = (t.rows + kBfWarps * 2 - 1) / (kBfWarps * 2);
    if (blocks > e->sm_count * 4) blocks = e->sm_count * 4;
    matvec_bf16_kernel<<<blocks, kBfWarps * 32, (size_t)t.cols * 4, e->stream>>>(reinterpret_cast<const uint16_t*>(t.w), x, y, t.rows, t.cols);
    e->launches++;
    MOE_CUDA(cudaGetLastError());
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
    float* o = take(H); float* cur2 = take(H); float* y = take(H);
    cudaStream_t st = e->stream;
    MOE_CUDA(cudaMemcpyAsync(h, h_host, (size_t)H * 4, cudaMemcpyHostToDevice, st));
    MOE_CUDA(cudaMemcpyAsync(m.id_dev, &token_id, 8, cudaMemcpyHostToDevice, st));
    int rc = launch_embed(e, m.id_dev, 1, tok);
    if (rc) return rc;
    // embedding first, hidden state second (mtp.rs:103-105)
    rms_norm_rows_kernel<<<1, 256, 0, st>>>(tok, m.norms[MOE_M_PRE_FC_NORM_EMBEDDING], H, concat);
    rms_norm_rows_kernel<<<1, 256, 0, st>>>(h, m.norms[MOE_M_PRE_FC_NORM_HIDDEN], H, concat + H);
    e->launches += 2;
    rc = mtp_project(e, MOE_M_FC, concat, cur);
    if (rc) return rc;
    rms_norm_rows_kernel<<<1, 256, 0, st>>>(cur, m.norms[MOE_M_INPUT_NORM], H, x);
    e->launches++;
    if ((rc = mtp_project(e, MOE_M_Q_PROJ, x, q))) return rc;
    if ((rc = mtp_project(e, MOE_M_K_PROJ, x, k))) return rc;
    if ((rc = mtp_project(e, MOE_M_V_PROJ, x, v))) return rc;
    attn_prep_kernel<<<nh + nkv, 256, (size_t)hd * 4, st>>>(q, k, v, m.norms[MOE_M_Q_NORM], m.norms[MOE_M_K_NORM], nh, nkv, hd,
                                                          m.ad.rotary_dim, pos, m.ad.rope_theta, qr, m.k_cache, m.v_cache);
    const int seq = pos + 1;
    attn_decode_kernel<<<nh, 256, (size_t)(seq + hd) * 4, st>>>(qr, m.k_cache, m.v_cache, q + q_dim, nh, nkv, hd, seq,
                                                               1.0f / sqrtf((float)hd), gated);
    e->launches += 2;
    if ((rc = mtp_project(e, MOE_M_O_PROJ, gated, o))) return rc;
    add_rows_kernel<<<(H + 255) / 256, 256, 0, st>>>(o, cur, H, cur2);
    e->launches++;
    MOE_CUDA(cudaGetLastError());
    // the MoE half: post-attention norm, router, experts, shared expert, residual (layer index num_layers)
    if ((rc = launch_decode(e, d.num_layers, d.num_layers + 1, cur2, y, nullptr, nullptr, nullptr, nullptr))) return rc;
    if ((rc = launch_logits_norm(e, y, 1, logits_dev, m.norms[MOE_M_OUT_NORM]))) return rc;
    return MOE_OK;
}

}  // namespace moe
