/*
 * CPU oracle for the quantized-MoE hot path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C, the arithmetic of the reference project
 * fbundle/moe_infer (Rust) for the 4-bit MoE path.  It exists to check the CUDA
 * library and to be timed as the CPU baseline; nothing in the shipped library
 * links, loads or calls it.
 *
 * Every function names the reference lines it follows (paths are relative to
 * the reference project root).  Arithmetic is scalar f32 in the same order as
 * the reference; build with -O2 -ffp-contract=off and without -ffast-math so
 * that no multiply-add is contracted and no sum is re-associated.
 *
 * Parity status: the bf16 rounding, the dequantiser and the expert blob layout
 * are pinned against the reference's own Python (golden fixtures).  The packer
 * (orc_quant_int4) has no known-answer vector in the reference's tests
 * ("parity unpinned" for packed nibbles: pinned by source text only, plus the
 * reference's own loose round-trip test restated as a property).
 *
 * The *_mt entry points split independent output rows / tokens over POSIX
 * threads; each row is still accumulated sequentially, so results are
 * identical to the single-threaded functions.
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>

#define ORC_GROUP 64
#define ORC_MAX_K 8
#define ORC_MAX_THREADS 256

/* ─── a small parallel-for over [0, n) ─────────────────────────────────── */

typedef void (*orc_range_fn)(int begin, int end, void* ctx);
typedef struct { orc_range_fn fn; void* ctx; int begin, end; } orc_job_t;

static void* orc_job_run(void* p) {
    orc_job_t* j = (orc_job_t*)p;
    j->fn(j->begin, j->end, j->ctx);
    return NULL;
}

static int g_threads = 0;

int orc_num_threads(void) {
    if (g_threads > 0) return g_threads;
    long n = sysconf(_SC_NPROCESSORS_ONLN);
    if (n < 1) n = 1;
    if (n > ORC_MAX_THREADS) n = ORC_MAX_THREADS;
    return (int)n;
}

void orc_set_num_threads(int n) { g_threads = n > ORC_MAX_THREADS ? ORC_MAX_THREADS : n; }

/* Contiguous static split; the calling thread takes the first chunk. */
static void orc_par_for(int n, orc_range_fn fn, void* ctx, int threads) {
    if (threads > n) threads = n;
    if (threads <= 1) { fn(0, n, ctx); return; }
    pthread_t tid[ORC_MAX_THREADS];
    orc_job_t job[ORC_MAX_THREADS];
    int started[ORC_MAX_THREADS];
    for (int t = 0; t < threads; ++t) {
        job[t].fn = fn; job[t].ctx = ctx;
        job[t].begin = (int)((int64_t)n * t / threads);
        job[t].end = (int)((int64_t)n * (t + 1) / threads);
        started[t] = 0;
    }
    for (int t = 1; t < threads; ++t)
        started[t] = pthread_create(&tid[t], NULL, orc_job_run, &job[t]) == 0;
    orc_job_run(&job[0]);
    for (int t = 1; t < threads; ++t) {
        if (started[t]) pthread_join(tid[t], NULL);
        else orc_job_run(&job[t]);
    }
}

/* ─── bf16 ─────────────────────────────────────────────────────────────── */

/* src/dtype.rs:85-89.  The reference ANDs a 1-bit value with a multi-bit
 * value, so only bit 0 of the "sticky" term takes part: this is NOT
 * round-to-nearest-even.  round_up = bit15 & (bit0 | bit16). */
uint16_t orc_f32_to_bf16(float v) {
    uint32_t bits;
    memcpy(&bits, &v, 4);
    uint32_t round_up = ((bits >> 15) & 1u) & ((bits & 0x7FFFu) | ((bits >> 16) & 1u));
    return (uint16_t)((bits + (round_up << 16)) >> 16);
}

/* src/dtype.rs:96-98; src/math_util.rs:9-11 */
float orc_bf16_to_f32(uint16_t v) {
    uint32_t bits = ((uint32_t)v) << 16;
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

void orc_f32_to_bf16_n(const float* src, uint16_t* dst, size_t n) {
    for (size_t i = 0; i < n; ++i) dst[i] = orc_f32_to_bf16(src[i]);
}
void orc_bf16_to_f32_n(const uint16_t* src, float* dst, size_t n) {
    for (size_t i = 0; i < n; ++i) dst[i] = orc_bf16_to_f32(src[i]);
}

/* Rust `as i32` on an f32: truncates toward zero, saturates, NaN -> 0. */
static int32_t rust_f32_as_i32(float x) {
    if (x != x) return 0;
    if (x >= 2147483648.0f) return INT32_MAX;
    if (x <= -2147483648.0f) return INT32_MIN;
    return (int32_t)x;
}

/* Rust f32::min / f32::max: a NaN operand is ignored. */
static float rust_min(float a, float b) { return fminf(a, b); }
static float rust_max(float a, float b) { return fmaxf(a, b); }

/* ─── packer ───────────────────────────────────────────────────────────── */

/* src/dtype.rs:102-135 (quant_f32_to_int4).
 * vals [out_dim, in_dim] f32 -> packed u32 [out_dim, in_dim/8],
 * scales/biases bf16 [out_dim, in_dim/64]. */
void orc_quant_int4(const float* vals, int out_dim, int in_dim,
                    uint32_t* packed, uint16_t* scales, uint16_t* biases) {
    const int num_groups = in_dim / ORC_GROUP;
    const int words_per_row = in_dim / 8;
    for (int row = 0; row < out_dim; ++row) {
        const size_t row_base = (size_t)row * in_dim;
        for (int g = 0; g < num_groups; ++g) {
            const float* group = vals + row_base + (size_t)g * ORC_GROUP;
            float vmin = group[0], vmax = group[0];
            for (int i = 1; i < ORC_GROUP; ++i) {
                vmin = rust_min(vmin, group[i]);
                vmax = rust_max(vmax, group[i]);
            }
            if (vmax == vmin) vmax = vmin + 1.0f;
            const float fscale = (vmax - vmin) / 15.0f;
            const float fbias = vmin;
            const size_t s_idx = (size_t)row * num_groups + g;
            scales[s_idx] = orc_f32_to_bf16(fscale);
            biases[s_idx] = orc_f32_to_bf16(fbias);
            const float inv_scale = 1.0f / fscale;
            for (int p = 0; p < 8; ++p) {
                uint32_t word = 0;
                for (int n = 0; n < 8; ++n) {
                    float v = group[p * 8 + n];
                    float t = (v - fbias) * inv_scale;
                    t = t + 0.5f;
                    int32_t q = rust_f32_as_i32(t);
                    if (q < 0) q = 0;
                    if (q > 15) q = 15;
                    word |= (((uint32_t)q) & 0xFu) << (n * 4);
                }
                packed[(size_t)row * words_per_row + g * 8 + p] = word;
            }
        }
    }
}

/* Same packer fed bf16 input: the reference widens bf16 to f32 exactly
 * (src/safetensors.rs:133-142 -> src/dtype.rs:96-98) before quantising. */
void orc_quant_int4_bf16(const uint16_t* vals, int out_dim, int in_dim,
                         uint32_t* packed, uint16_t* scales, uint16_t* biases) {
    size_t n = (size_t)out_dim * in_dim;
    float* tmp = (float*)malloc(n * sizeof(float));
    orc_bf16_to_f32_n(vals, tmp, n);
    orc_quant_int4(tmp, out_dim, in_dim, packed, scales, biases);
    free(tmp);
}

/* src/dtype.rs:138-160 (int4_to_f32); same math as moe_infer/dequantize.py:42-63 */
void orc_dequant_int4(const uint32_t* packed, const uint16_t* scales, const uint16_t* biases,
                      int out_dim, int in_dim, float* result) {
    const int num_groups = in_dim / ORC_GROUP;
    const int words_per_row = in_dim / 8;
    for (int row = 0; row < out_dim; ++row) {
        for (int g = 0; g < num_groups; ++g) {
            float scale = orc_bf16_to_f32(scales[(size_t)row * num_groups + g]);
            float bias = orc_bf16_to_f32(biases[(size_t)row * num_groups + g]);
            size_t out_base = (size_t)row * in_dim + (size_t)g * ORC_GROUP;
            for (int p = 0; p < 8; ++p) {
                uint32_t word = packed[(size_t)row * words_per_row + g * 8 + p];
                for (int n = 0; n < 8; ++n) {
                    uint32_t nib = (word >> (n * 4)) & 0xFu;
                    result[out_base + p * 8 + n] = (float)nib * scale + bias;
                }
            }
        }
    }
}

/* ─── expert blob layout ───────────────────────────────────────────────── */

typedef struct {
    int64_t gate_w, gate_s, gate_b, up_w, up_s, up_b, down_w, down_s, down_b, expert_size;
} orc_layout_t;

/* src/engine/qwen35_moe/constants.rs:117-139 (expert_layout) */
void orc_expert_layout(int hd, int mi, int gs, orc_layout_t* L) {
    int64_t gate_w = (int64_t)mi * hd / 2;
    int64_t gate_sb = (int64_t)mi * (hd / gs) * 2;
    int64_t up_w = gate_w, up_sb = gate_sb;
    int64_t down_w = (int64_t)hd * mi / 2;
    int64_t down_sb = (int64_t)hd * (mi / gs) * 2;
    L->gate_w = 0;
    L->gate_s = gate_w;
    L->gate_b = gate_w + gate_sb;
    L->up_w = gate_w + 2 * gate_sb;
    L->up_s = L->up_w + up_w;
    L->up_b = L->up_s + up_sb;
    L->down_w = L->up_b + up_sb;
    L->down_s = L->down_w + down_w;
    L->down_b = L->down_s + down_sb;
    L->expert_size = L->down_b + down_sb;
}

/* src/quantize/qwen35_moe/common.rs:300-345: HF gate_up [E, 2I, H] (gate rows
 * 0..I, up rows I..2I) and down [E, H, I], both already widened to f32, ->
 * E blobs back to back in the order w,s,b x gate,up,down. */
void orc_pack_experts_layer(const float* gate_up, const float* down, int num_experts,
                            int inter, int hidden, uint8_t* blob) {
    orc_layout_t L;
    orc_expert_layout(hidden, inter, ORC_GROUP, &L);
    for (int e = 0; e < num_experts; ++e) {
        uint8_t* base = blob + (size_t)e * L.expert_size;
        const float* gate = gate_up + (size_t)e * 2 * inter * hidden;
        const float* up = gate + (size_t)inter * hidden;
        const float* dn = down + (size_t)e * hidden * inter;
        orc_quant_int4(gate, inter, hidden, (uint32_t*)(base + L.gate_w),
                       (uint16_t*)(base + L.gate_s), (uint16_t*)(base + L.gate_b));
        orc_quant_int4(up, inter, hidden, (uint32_t*)(base + L.up_w),
                       (uint16_t*)(base + L.up_s), (uint16_t*)(base + L.up_b));
        orc_quant_int4(dn, hidden, inter, (uint32_t*)(base + L.down_w),
                       (uint16_t*)(base + L.down_s), (uint16_t*)(base + L.down_b));
    }
}

/* ─── matvec and small math ────────────────────────────────────────────── */

/* src/math_util.rs:14-54 (dequant_matvec_4bit): f32 accumulate in column order. */
static void matvec_int4_rows(const uint32_t* w, const uint16_t* s, const uint16_t* b,
                             const float* x, float* out, int row0, int row1, int in_dim) {
    const int num_groups = in_dim / ORC_GROUP;
    const int packed_cols = in_dim / 8;
    for (int row = row0; row < row1; ++row) {
        float acc = 0.0f;
        const uint32_t* w_row = w + (size_t)row * packed_cols;
        const uint16_t* s_row = s + (size_t)row * num_groups;
        const uint16_t* b_row = b + (size_t)row * num_groups;
        for (int g = 0; g < num_groups; ++g) {
            float scale = orc_bf16_to_f32(s_row[g]);
            float bias = orc_bf16_to_f32(b_row[g]);
            for (int p = 0; p < 8; ++p) {
                uint32_t word = w_row[g * 8 + p];
                const float* xp = x + g * ORC_GROUP + p * 8;
                for (int n = 0; n < 8; ++n) {
                    uint32_t nib = (word >> (n * 4)) & 0xFu;
                    float w_val = (float)nib * scale + bias;
                    acc += w_val * xp[n];
                }
            }
        }
        out[row] = acc;
    }
}

void orc_matvec_int4(const uint32_t* w, const uint16_t* s, const uint16_t* b,
                     const float* x, float* out, int out_dim, int in_dim) {
    matvec_int4_rows(w, s, b, x, out, 0, out_dim, in_dim);
}

typedef struct {
    const uint32_t* w; const uint16_t* s; const uint16_t* b; const float* x; float* out; int in_dim;
} mv_ctx_t;

static void mv_range(int r0, int r1, void* p) {
    mv_ctx_t* c = (mv_ctx_t*)p;
    matvec_int4_rows(c->w, c->s, c->b, c->x, c->out, r0, r1, c->in_dim);
}

/* Rows split over threads; per-row arithmetic unchanged. */
void orc_matvec_int4_mt(const uint32_t* w, const uint16_t* s, const uint16_t* b,
                        const float* x, float* out, int out_dim, int in_dim) {
    mv_ctx_t c = { w, s, b, x, out, in_dim };
    orc_par_for(out_dim, mv_range, &c, orc_num_threads());
}

/* bf16-weight matvec: what src/engine/shaders.metal:2392 (matvec_bf16) computes
 * for the BQ4 router, stated as a sequential f32 sum. */
void orc_matvec_bf16(const uint16_t* w, const float* x, float* out, int out_dim, int in_dim) {
    for (int row = 0; row < out_dim; ++row) {
        float acc = 0.0f;
        const uint16_t* w_row = w + (size_t)row * in_dim;
        for (int c = 0; c < in_dim; ++c) acc += orc_bf16_to_f32(w_row[c]) * x[c];
        out[row] = acc;
    }
}

/* src/math_util.rs:67-69 */
float orc_sigmoid(float x) { return 1.0f / (1.0f + expf(-x)); }

/* src/math_util.rs:77-88 */
void orc_softmax(float* x, int n) {
    float max_val = -INFINITY;
    for (int i = 0; i < n; ++i) max_val = rust_max(max_val, x[i]);
    float sum = 0.0f;
    for (int i = 0; i < n; ++i) {
        x[i] = expf(x[i] - max_val);
        sum += x[i];
    }
    float inv = 1.0f / sum;
    for (int i = 0; i < n; ++i) x[i] *= inv;
}

/* src/math_util.rs:90-118: size-k min-heap; a later score replaces the root
 * only when strictly greater; the result stays in heap order (unsorted). */
void orc_topk(const float* scores, int n, int k, int32_t* indices, float* values) {
    for (int i = 0; i < n; ++i) {
        float score = scores[i];
        if (i < k) {
            int pos = i;
            while (pos > 0 && values[(pos - 1) / 2] > score) {
                values[pos] = values[(pos - 1) / 2];
                indices[pos] = indices[(pos - 1) / 2];
                pos = (pos - 1) / 2;
            }
            values[pos] = score;
            indices[pos] = i;
        } else if (score > values[0]) {
            values[0] = score;
            indices[0] = i;
            int pos = 0;
            for (;;) {
                int left = 2 * pos + 1, right = 2 * pos + 2, smallest = pos;
                if (left < k && values[left] < values[smallest]) smallest = left;
                if (right < k && values[right] < values[smallest]) smallest = right;
                if (smallest == pos) break;
                float tv = values[pos]; values[pos] = values[smallest]; values[smallest] = tv;
                int32_t ti = indices[pos]; indices[pos] = indices[smallest]; indices[smallest] = ti;
                pos = smallest;
            }
        }
    }
}

/* src/math_util.rs:120-126 */
void orc_normalize_weights(float* w, int k) {
    float sum = 0.0f;
    for (int i = 0; i < k; ++i) sum += w[i];
    if (sum > 0.0f) {
        float inv = 1.0f / sum;
        for (int i = 0; i < k; ++i) w[i] *= inv;
    }
}

/* src/engine/qwen35_moe/cpu.rs:78-85 (route_experts); gate_scores is overwritten
 * with the softmax probabilities. */
void orc_route_experts(float* gate_scores, int num_experts, int k, int32_t* indices, float* weights) {
    orc_softmax(gate_scores, num_experts);
    for (int i = 0; i < k; ++i) { indices[i] = 0; weights[i] = 0.0f; }
    orc_topk(gate_scores, num_experts, k, indices, weights);
    orc_normalize_weights(weights, k);
}

/* src/math_util.rs:254-259 */
void orc_swiglu(const float* gate, const float* up, float* out, int dim) {
    for (int i = 0; i < dim; ++i) {
        float silu_g = gate[i] / (1.0f + expf(-gate[i]));
        out[i] = silu_g * up[i];
    }
}

/* src/math_util.rs:282-288 with eps = 1e-6 (src/constants.rs:15) */
void orc_rms_norm_bf16(const float* x, const uint16_t* w_bf16, float* out, int dim, float eps) {
    float sum_sq = 0.0f;
    for (int i = 0; i < dim; ++i) sum_sq += x[i] * x[i];
    float inv_rms = 1.0f / sqrtf(sum_sq / (float)dim + eps);
    for (int i = 0; i < dim; ++i) out[i] = x[i] * inv_rms * orc_bf16_to_f32(w_bf16[i]);
}

/* ─── one MoE block ────────────────────────────────────────────────────── */

typedef struct {
    int32_t hidden, inter, shared_inter, num_experts, top_k;
} orc_dims_t;

typedef struct {
    const uint32_t* w;
    const uint16_t* s;
    const uint16_t* b;
} orc_q4_t;

typedef struct {
    const uint16_t* post_norm_w; /* bf16 [hidden]: post_attention_layernorm */
    const uint16_t* router_bf16; /* bf16 [E, hidden] (BQ4 scheme) or NULL */
    orc_q4_t router_q4;          /* INT4 scheme router when router_bf16 == NULL */
    orc_q4_t sh_gate, sh_up, sh_down; /* shared expert */
    orc_q4_t sgate;              /* shared_expert_gate, 1 x hidden */
    const uint8_t* experts;      /* E blobs of expert_size bytes */
} orc_layer_t;

/* One token through one MoE block.
 * src/engine/qwen35_moe/cpu.rs:187-205 (post-attention norm, router, shared
 * gate/up, scalar gate), :78-85 (routing), :398-483 (experts, shared expert,
 * combine).  logit_bias (nullable, [E]) is added to the router logits before
 * the softmax; forced_idx (nullable, [k]) replaces the top-k choice while the
 * weights are still the renormalised softmax probabilities of those experts.
 * Both are harness controls with no counterpart in the reference. */
static void moe_layer_token(const orc_dims_t* d, const orc_layer_t* ly, const float* h_mid,
                            float* h_out, int32_t* out_idx, float* out_w,
                            const float* logit_bias, const int32_t* forced_idx) {
    const int hd = d->hidden, mi = d->inter, si = d->shared_inter, E = d->num_experts, k = d->top_k;
    orc_layout_t L;
    orc_expert_layout(hd, mi, ORC_GROUP, &L);

    float* post = (float*)malloc(sizeof(float) * hd);
    float* scores = (float*)malloc(sizeof(float) * E);
    float* g = (float*)malloc(sizeof(float) * (mi > si ? mi : si));
    float* u = (float*)malloc(sizeof(float) * (mi > si ? mi : si));
    float* act = (float*)malloc(sizeof(float) * (mi > si ? mi : si));
    float* eout = (float*)malloc(sizeof(float) * (size_t)k * hd);
    float* sdown = (float*)malloc(sizeof(float) * hd);

    orc_rms_norm_bf16(h_mid, ly->post_norm_w, post, hd, 1e-6f);

    if (ly->router_bf16) orc_matvec_bf16(ly->router_bf16, post, scores, E, hd);
    else orc_matvec_int4(ly->router_q4.w, ly->router_q4.s, ly->router_q4.b, post, scores, E, hd);
    if (logit_bias) for (int e = 0; e < E; ++e) scores[e] += logit_bias[e];

    int32_t idx[ORC_MAX_K];
    float wts[ORC_MAX_K];
    orc_route_experts(scores, E, k, idx, wts);
    if (forced_idx) {
        for (int i = 0; i < k; ++i) { idx[i] = forced_idx[i]; wts[i] = scores[idx[i]]; }
        orc_normalize_weights(wts, k);
    }

    float sg_score = 0.0f;
    orc_matvec_int4(ly->sgate.w, ly->sgate.s, ly->sgate.b, post, &sg_score, 1, hd);

    for (int ki = 0; ki < k; ++ki) {
        const uint8_t* ex = ly->experts + (size_t)idx[ki] * L.expert_size;
        orc_matvec_int4((const uint32_t*)(ex + L.gate_w), (const uint16_t*)(ex + L.gate_s),
                        (const uint16_t*)(ex + L.gate_b), post, g, mi, hd);
        orc_matvec_int4((const uint32_t*)(ex + L.up_w), (const uint16_t*)(ex + L.up_s),
                        (const uint16_t*)(ex + L.up_b), post, u, mi, hd);
        orc_swiglu(g, u, act, mi);
        orc_matvec_int4((const uint32_t*)(ex + L.down_w), (const uint16_t*)(ex + L.down_s),
                        (const uint16_t*)(ex + L.down_b), act, eout + (size_t)ki * hd, hd, mi);
    }

    orc_matvec_int4(ly->sh_gate.w, ly->sh_gate.s, ly->sh_gate.b, post, g, si, hd);
    orc_matvec_int4(ly->sh_up.w, ly->sh_up.s, ly->sh_up.b, post, u, si, hd);
    orc_swiglu(g, u, act, si);
    orc_matvec_int4(ly->sh_down.w, ly->sh_down.s, ly->sh_down.b, act, sdown, hd, si);

    /* cpu.rs:465-480 */
    float shared_gate = orc_sigmoid(sg_score);
    for (int i = 0; i < hd; ++i) {
        float moe_sum = 0.0f;
        for (int ki = 0; ki < k; ++ki) moe_sum += wts[ki] * eout[(size_t)ki * hd + i];
        h_out[i] = h_mid[i] + moe_sum + shared_gate * sdown[i];
    }
    if (out_idx) for (int i = 0; i < k; ++i) out_idx[i] = idx[i];
    if (out_w) for (int i = 0; i < k; ++i) out_w[i] = wts[i];

    free(post); free(scores); free(g); free(u); free(act); free(eout); free(sdown);
}

typedef struct {
    const orc_dims_t* d; const orc_layer_t* ly; const float* h_mid; float* h_out;
    int32_t* out_idx; float* out_w; const float* logit_bias; const int32_t* forced_idx;
} tok_ctx_t;

static void tok_range(int t0, int t1, void* p) {
    tok_ctx_t* c = (tok_ctx_t*)p;
    const int hd = c->d->hidden, k = c->d->top_k;
    for (int t = t0; t < t1; ++t)
        moe_layer_token(c->d, c->ly, c->h_mid + (size_t)t * hd, c->h_out + (size_t)t * hd,
                        c->out_idx ? c->out_idx + (size_t)t * k : NULL,
                        c->out_w ? c->out_w + (size_t)t * k : NULL, c->logit_bias,
                        c->forced_idx ? c->forced_idx + (size_t)t * k : NULL);
}

/* n tokens through one MoE block; tokens are independent
 * (src/engine/qwen35_moe/fused_exp3.rs:216-276 routes and runs each token on
 * its own).  h_mid/h_out [n, hidden]; out_idx/out_w [n, k] nullable;
 * forced_idx [n, k] nullable.  threads <= 1 runs serially. */
void orc_moe_layer(const orc_dims_t* d, const orc_layer_t* ly, const float* h_mid, int n_tokens,
                   float* h_out, int32_t* out_idx, float* out_w,
                   const float* logit_bias, const int32_t* forced_idx, int threads) {
    const int hd = d->hidden, k = d->top_k;
    (void)hd; (void)k;
    tok_ctx_t c = { d, ly, h_mid, h_out, out_idx, out_w, logit_bias, forced_idx };
    orc_par_for(n_tokens, tok_range, &c, threads);
}

/* One token through one MoE block with the matvec rows split over threads
 * (the way a multi-core CPU would run batch-1 decode). */
void orc_moe_layer_decode_mt(const orc_dims_t* d, const orc_layer_t* ly, const float* h_mid,
                             float* h_out, int32_t* out_idx, float* out_w) {
    const int hd = d->hidden, mi = d->inter, si = d->shared_inter, E = d->num_experts, k = d->top_k;
    orc_layout_t L;
    orc_expert_layout(hd, mi, ORC_GROUP, &L);
    float* post = (float*)malloc(sizeof(float) * hd);
    float* scores = (float*)malloc(sizeof(float) * E);
    int mx = mi > si ? mi : si;
    float* g = (float*)malloc(sizeof(float) * mx);
    float* u = (float*)malloc(sizeof(float) * mx);
    float* act = (float*)malloc(sizeof(float) * mx);
    float* eout = (float*)malloc(sizeof(float) * (size_t)k * hd);
    float* sdown = (float*)malloc(sizeof(float) * hd);
    orc_rms_norm_bf16(h_mid, ly->post_norm_w, post, hd, 1e-6f);
    if (ly->router_bf16) {
        orc_matvec_bf16(ly->router_bf16, post, scores, E, hd);
    } else {
        orc_matvec_int4_mt(ly->router_q4.w, ly->router_q4.s, ly->router_q4.b, post, scores, E, hd);
    }
    int32_t idx[ORC_MAX_K];
    float wts[ORC_MAX_K];
    orc_route_experts(scores, E, k, idx, wts);
    float sg_score = 0.0f;
    orc_matvec_int4(ly->sgate.w, ly->sgate.s, ly->sgate.b, post, &sg_score, 1, hd);
    for (int ki = 0; ki < k; ++ki) {
        const uint8_t* ex = ly->experts + (size_t)idx[ki] * L.expert_size;
        orc_matvec_int4_mt((const uint32_t*)(ex + L.gate_w), (const uint16_t*)(ex + L.gate_s),
                           (const uint16_t*)(ex + L.gate_b), post, g, mi, hd);
        orc_matvec_int4_mt((const uint32_t*)(ex + L.up_w), (const uint16_t*)(ex + L.up_s),
                           (const uint16_t*)(ex + L.up_b), post, u, mi, hd);
        orc_swiglu(g, u, act, mi);
        orc_matvec_int4_mt((const uint32_t*)(ex + L.down_w), (const uint16_t*)(ex + L.down_s),
                           (const uint16_t*)(ex + L.down_b), act, eout + (size_t)ki * hd, hd, mi);
    }
    orc_matvec_int4_mt(ly->sh_gate.w, ly->sh_gate.s, ly->sh_gate.b, post, g, si, hd);
    orc_matvec_int4_mt(ly->sh_up.w, ly->sh_up.s, ly->sh_up.b, post, u, si, hd);
    orc_swiglu(g, u, act, si);
    orc_matvec_int4_mt(ly->sh_down.w, ly->sh_down.s, ly->sh_down.b, act, sdown, hd, si);
    float shared_gate = orc_sigmoid(sg_score);
    for (int i = 0; i < hd; ++i) {
        float moe_sum = 0.0f;
        for (int ki = 0; ki < k; ++ki) moe_sum += wts[ki] * eout[(size_t)ki * hd + i];
        h_out[i] = h_mid[i] + moe_sum + shared_gate * sdown[i];
    }
    if (out_idx) for (int i = 0; i < k; ++i) out_idx[i] = idx[i];
    if (out_w) for (int i = 0; i < k; ++i) out_w[i] = wts[i];
    free(post); free(scores); free(g); free(u); free(act); free(eout); free(sdown);
}


/* ─── the model head: embedding rows, final norm, lm_head ──────────────── */

/* quant_f32_to_int8: src/dtype.rs:164-179.  Per-row symmetric: scale = max|v| / 127 (1/127 for an
 * all-zero row), q = clamp(round(v * (1 / scale)), -127, 127); Rust's f32::round rounds half away
 * from zero, like roundf. */
void orc_quant_int8(const float* vals, int out_dim, int in_dim, int8_t* packed, float* scales) {
    for (int row = 0; row < out_dim; ++row) {
        const float* r = vals + (size_t)row * in_dim;
        float max_abs = 0.0f;
        for (int j = 0; j < in_dim; ++j) max_abs = rust_max(max_abs, fabsf(r[j]));
        const float scale = max_abs > 0.0f ? max_abs / 127.0f : 1.0f / 127.0f;
        scales[row] = scale;
        const float inv_scale = 1.0f / scale;
        int8_t* dst = packed + (size_t)row * in_dim;
        for (int j = 0; j < in_dim; ++j) {
            int32_t q = rust_f32_as_i32(roundf(r[j] * inv_scale));
            if (q < -127) q = -127;
            if (q > 127) q = 127;
            dst[j] = (int8_t)q;
        }
    }
}

/* matvec_int8 (src/engine/shaders.metal:2435-2471): out[row] = sum_col float(w) * scale * x, stated as a
 * sequential f32 sum in column order (the shader strides the columns over 32 lanes). */
static void matvec_int8_rows(const int8_t* w, const float* scales, const float* x, float* out, int r0, int r1, int in_dim) {
    for (int row = r0; row < r1; ++row) {
        const int8_t* w_row = w + (size_t)row * in_dim;
        const float scale = scales[row];
        float acc = 0.0f;
        for (int c = 0; c < in_dim; ++c) acc += (float)w_row[c] * scale * x[c];
        out[row] = acc;
    }
}
typedef struct { const int8_t* w; const float* scales; const float* x; float* out; int in_dim; } mv8_ctx;
static void mv8_range(int r0, int r1, void* p) {
    mv8_ctx* c = (mv8_ctx*)p;
    matvec_int8_rows(c->w, c->scales, c->x, c->out, r0, r1, c->in_dim);
}
void orc_matvec_int8(const int8_t* w, const float* scales, const float* x, float* out, int out_dim, int in_dim, int threads) {
    mv8_ctx c = {w, scales, x, out, in_dim};
    orc_par_for(out_dim, mv8_range, &c, threads);
}

/* embed_lookup: src/math_util.rs:205-236.  One row of the 4-bit embedding table, (nibble as f32) * scale + bias. */
void orc_embed_lookup(const uint32_t* w, const uint16_t* s, const uint16_t* b, int64_t token_id, int hidden, float* out) {
    const int num_groups = hidden / ORC_GROUP, packed_cols = hidden / 8, packed_per_group = ORC_GROUP / 8;
    const uint32_t* w_row = w + (size_t)token_id * packed_cols;
    const uint16_t* s_row = s + (size_t)token_id * num_groups;
    const uint16_t* b_row = b + (size_t)token_id * num_groups;
    for (int g = 0; g < num_groups; ++g) {
        const float scale = orc_bf16_to_f32(s_row[g]), bias = orc_bf16_to_f32(b_row[g]);
        const int base = g * ORC_GROUP;
        for (int p = 0; p < packed_per_group; ++p) {
            const uint32_t packed = w_row[g * packed_per_group + p];
            for (int n = 0; n < 8; ++n) {
                const uint32_t nibble = (packed >> (n * 4)) & 0xF;
                out[base + p * 8 + n] = (float)nibble * scale + bias;
            }
        }
    }
}

/* final_norm: src/math_util.rs:240-247.  hidden[i] *= inv_rms * w[i], in place. */
void orc_final_norm(float* hidden, const uint16_t* w, int dim, float eps) {
    float sum_sq = 0.0f;
    for (int i = 0; i < dim; ++i) sum_sq += hidden[i] * hidden[i];
    const float inv_rms = 1.0f / sqrtf(sum_sq / (float)dim + eps);
    for (int i = 0; i < dim; ++i) hidden[i] *= inv_rms * orc_bf16_to_f32(w[i]);
}

/* ─── MTP block: the attention half (reference src/engine/qwen35_moe/mtp.rs) ─── */

/* apply_rope: mtp.rs:285-303.  Interleaved pairs (2i, 2i+1) of the first rope_dim elements of every head. */
void orc_rope(const float* x, float* out, int num_heads, int head_dim, int rope_dim, int pos, float theta) {
    const float pos_f = (float)pos;
    for (int i = 0; i < num_heads * head_dim; ++i) out[i] = x[i];
    for (int h = 0; h < num_heads; ++h) {
        const int base = h * head_dim;
        for (int i = 0; i < rope_dim / 2; ++i) {
            const int idx = base + i * 2;
            const float freq = powf(theta, -2.0f * (float)i / (float)rope_dim);
            const float angle = pos_f * freq;
            const float sin_a = sinf(angle), cos_a = cosf(angle);
            const float x0 = x[idx], x1 = x[idx + 1];
            out[idx] = x0 * cos_a - x1 * sin_a;
            out[idx + 1] = x0 * sin_a + x1 * cos_a;
        }
    }
}

/* cpu_attention: mtp.rs:305-352.  q [num_heads * head_dim] against caches [seq_len, num_kv_heads * head_dim];
 * scores scaled, max-subtracted, exponentiated; each output element adds score / sum * v over the positions. */
void orc_attention(const float* q, const float* k_cache, const float* v_cache, int num_heads, int num_kv_heads,
                   int head_dim, int seq_len, float kq_scale, float* out) {
    const int kv_dim = num_kv_heads * head_dim, group_size = num_heads / num_kv_heads;
    float* scores = (float*)malloc(sizeof(float) * (size_t)seq_len);
    for (int h = 0; h < num_heads; ++h) {
        const int kv_h = h / group_size, q_off = h * head_dim;
        float max_score = -INFINITY;
        for (int t = 0; t < seq_len; ++t) {
            const float* kr = k_cache + (size_t)t * kv_dim + kv_h * head_dim;
            float dot = 0.0f;
            for (int d = 0; d < head_dim; ++d) dot += q[q_off + d] * kr[d];
            scores[t] = dot * kq_scale;
            max_score = rust_max(max_score, scores[t]);
        }
        float sum_exp = 0.0f;
        for (int t = 0; t < seq_len; ++t) {
            scores[t] = expf(scores[t] - max_score);
            sum_exp += scores[t];
        }
        for (int d = 0; d < head_dim; ++d) {
            float acc = 0.0f;
            for (int t = 0; t < seq_len; ++t) acc += scores[t] / sum_exp * v_cache[(size_t)t * kv_dim + kv_h * head_dim + d];
            out[q_off + d] = acc;
        }
    }
    free(scores);
}

/* ─── main-model attention layers (reference src/engine/qwen35_moe/cpu.rs:87-347, src/math_util.rs) ─── */

/* q_head_norm_rope / k_head_norm_rope: src/math_util.rs:501-597.  Per-head RMS norm with a bf16 weight, then RoPE on
 * the pairs (d, d + rotary_dim / 2).  src holds `num_heads` heads `stride` floats apart; out is dense. */
void orc_head_norm_rope_split(const float* src, int stride, const uint16_t* norm_w, float* out, int num_heads,
                              int head_dim, int rotary_dim, float rope_theta, int pos, float eps) {
    const int rot_half = rotary_dim / 2;
    for (int h = 0; h < num_heads; ++h) {
        const float* x = src + (size_t)h * stride;
        float* o = out + (size_t)h * head_dim;
        float sum_sq = 0.0f;
        for (int d = 0; d < head_dim; ++d) sum_sq += x[d] * x[d];
        const float inv_rms = 1.0f / sqrtf(sum_sq / (float)head_dim + eps);
        for (int d = 0; d < head_dim; ++d) {
            const float val = x[d] * inv_rms * orc_bf16_to_f32(norm_w[d]);
            if (d < rotary_dim) {
                const int pair = d < rot_half ? d : d - rot_half;
                const int other = d < rot_half ? d + rot_half : d - rot_half;
                const float theta = (float)pos * powf(rope_theta, -2.0f * (float)pair / (float)rotary_dim);
                const float pair_val = x[other] * inv_rms * orc_bf16_to_f32(norm_w[other]);
                const float cos_t = cosf(theta), sin_t = sinf(theta);
                o[d] = d < rot_half ? val * cos_t - pair_val * sin_t : pair_val * sin_t + val * cos_t;
            } else {
                o[d] = val;
            }
        }
    }
}

/* conv1d_step + the state shift that follows it: src/math_util.rs:149-168, cpu.rs:263-275. */
void orc_conv1d_step(float* conv_state, const float* x, const uint16_t* w, float* out, int channels, int ksize) {
    for (int c = 0; c < channels; ++c) {
        float acc = 0.0f;
        for (int k = 0; k < ksize - 1; ++k) acc += conv_state[(size_t)k * channels + c] * orc_bf16_to_f32(w[(size_t)c * ksize + k]);
        acc += x[c] * orc_bf16_to_f32(w[(size_t)c * ksize + ksize - 1]);
        out[c] = acc;
    }
    for (int c = 0; c < channels; ++c) out[c] = out[c] / (1.0f + expf(-out[c]));
    for (int k = 0; k + 2 < ksize; ++k) memcpy(conv_state + (size_t)k * channels, conv_state + (size_t)(k + 1) * channels, sizeof(float) * (size_t)channels);
    if (ksize >= 2) memcpy(conv_state + (size_t)(ksize - 2) * channels, x, sizeof(float) * (size_t)channels);
}

/* cpu.rs:277-299: unweighted per-head RMS norm of q and k, q scaled by inv_scale^2 and k by inv_scale. */
void orc_lin_qk_norm(float* qkv, int total_key, int num_k_heads, int key_dim) {
    const float inv_scale = 1.0f / sqrtf((float)key_dim);
    for (int h = 0; h < num_k_heads; ++h) {
        float* q = qkv + (size_t)h * key_dim;
        float* k = qkv + total_key + (size_t)h * key_dim;
        float q_sq = 0.0f, k_sq = 0.0f;
        for (int d = 0; d < key_dim; ++d) q_sq += q[d] * q[d];
        for (int d = 0; d < key_dim; ++d) k_sq += k[d] * k[d];
        const float q_inv = 1.0f / sqrtf(q_sq / (float)key_dim + 1e-6f), k_inv = 1.0f / sqrtf(k_sq / (float)key_dim + 1e-6f);
        for (int d = 0; d < key_dim; ++d) {
            q[d] = q[d] * q_inv * inv_scale * inv_scale;
            k[d] = k[d] * k_inv * inv_scale;
        }
    }
}

/* compute_decay_beta + gated_delta_net_step: src/math_util.rs:401-466. */
void orc_delta_step(float* state, const float* q, const float* k, const float* v, const float* alpha, const float* beta,
                    const float* a_log, const uint16_t* dt_bias, float* out, int num_v_heads, int k_heads_per_v,
                    int key_dim, int value_dim) {
    for (int h = 0; h < num_v_heads; ++h) {
        const float a = expf(a_log[h]);
        const float softplus = logf(1.0f + expf(alpha[h] + orc_bf16_to_f32(dt_bias[h])));
        const float g = expf(-a * softplus);
        const float bgate = 1.0f / (1.0f + expf(-beta[h]));
        const int kh = h / k_heads_per_v;
        const float* kk = k + (size_t)kh * key_dim;
        const float* qq = q + (size_t)kh * key_dim;
        for (int vi = 0; vi < value_dim; ++vi) {
            float* row = state + ((size_t)h * value_dim + vi) * key_dim;
            float kv_mem = 0.0f;
            for (int ki = 0; ki < key_dim; ++ki) {
                const float s = row[ki] * g;
                row[ki] = s;
                kv_mem += s * kk[ki];
            }
            const float delta = (v[(size_t)h * value_dim + vi] - kv_mem) * bgate;
            for (int ki = 0; ki < key_dim; ++ki) row[ki] += kk[ki] * delta;
            float o = 0.0f;
            for (int ki = 0; ki < key_dim; ++ki) o += row[ki] * qq[ki];
            out[(size_t)h * value_dim + vi] = o;
        }
    }
}

/* gated_rms_norm: src/math_util.rs:472-493. */
void orc_gated_rms_norm(const float* vals, const float* z, const uint16_t* w, float* out, int num_heads, int value_dim, float eps) {
    for (int h = 0; h < num_heads; ++h) {
        const float* x = vals + (size_t)h * value_dim;
        float sum_sq = 0.0f;
        for (int d = 0; d < value_dim; ++d) sum_sq += x[d] * x[d];
        const float inv_rms = 1.0f / sqrtf(sum_sq / (float)value_dim + eps);
        for (int d = 0; d < value_dim; ++d) {
            const float zv = z[(size_t)h * value_dim + d];
            out[(size_t)h * value_dim + d] = x[d] * inv_rms * (zv / (1.0f + expf(-zv))) * orc_bf16_to_f32(w[d]);
        }
    }
}
