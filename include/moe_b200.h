/*
 * moe_b200.h — C ABI of the B200 (sm_100a) quantized-MoE hot path.
 *
 * This is the boundary a host program (a Rust crate through `extern "C"`, a
 * Python module through ctypes, C++) binds to replace the 4-bit MoE path of
 * fbundle/moe_infer.  Each entry point names the reference interface it stands
 * in for (paths are relative to the reference project root).
 *
 * Conventions
 *  - Every function returns an int status: 0 (MOE_OK) on success, a negative
 *    moe_status_t otherwise; moe_last_error() returns a thread-local message.
 *    Nothing throws, aborts or exits across this boundary.
 *  - Handles are opaque.  An engine is bound to one CUDA device and, like the
 *    reference engine (`#[pyclass(unsendable)]`, &mut self), serves one caller
 *    thread at a time; there is no internal locking.
 *  - Pointers named *_host are host memory (pageable or pinned), pointers
 *    named *_dev are device memory on the engine's device.  Inputs are borrowed
 *    read-only for the duration of the call; outputs are caller-allocated.
 *  - All work is issued on the engine's own CUDA stream.  Host-pointer entry
 *    points return after the result is in the caller's buffer; *_dev entry
 *    points return after enqueueing (call moe_engine_sync to wait).
 *  - There is no CPU fallback: without a usable CUDA device every compute entry
 *    point fails with MOE_ERR_CUDA.
 */
#ifndef MOE_B200_H
#define MOE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct moe_engine moe_engine_t;

typedef enum {
    MOE_OK = 0,
    MOE_ERR_INVALID = -1,     /* bad argument / shape / config  (reference: MoEError::Config -> ValueError) */
    MOE_ERR_CUDA = -2,        /* CUDA runtime failure           (reference: MoEError::Metal  -> RuntimeError) */
    MOE_ERR_STATE = -3,       /* tensors not loaded yet, wrong call order */
    MOE_ERR_INTERRUPTED = -4, /* the caller's check callback returned non-zero ("interrupted") */
    MOE_ERR_DEVICE_WAIT = -5, /* a bounded device-side wait gave up; the context stays usable */
    MOE_ERR_UNSUPPORTED = -6,
    MOE_ERR_IO = -7           /* reference: MoEError::Io -> IOError */
} moe_status_t;

/* Tensor-selection scheme (src/quantize/qwen35_moe/bq4.rs:25-45, int4.rs:24-35):
 * both use the same 4-bit codec for experts; they differ in the router dtype. */
typedef enum { MOE_SCHEME_BQ4 = 0, MOE_SCHEME_INT4 = 1 } moe_scheme_t;

typedef enum { MOE_DT_F32 = 0, MOE_DT_BF16 = 1, MOE_DT_INT4 = 2, MOE_DT_INT8 = 3 } moe_dtype_t;

/* Non-expert tensors of one MoE block, by role.  Names in the reference's
 * weight manifest: `model.layers.{L}.post_attention_layernorm.weight`,
 * `…mlp.gate`, `…mlp.shared_expert.{gate,up,down}_proj`, `…mlp.shared_expert_gate`
 * (src/engine/qwen35_moe/cpu.rs:180-205, 453-463). */
typedef enum {
    MOE_T_POST_NORM = 0,   /* bf16 [hidden] */
    MOE_T_ROUTER = 1,      /* bf16 [E, hidden] (BQ4) or INT4 triple (INT4 scheme) */
    MOE_T_SHARED_GATE = 2, /* INT4 [shared_inter, hidden] */
    MOE_T_SHARED_UP = 3,   /* INT4 [shared_inter, hidden] */
    MOE_T_SHARED_DOWN = 4, /* INT4 [hidden, shared_inter] */
    MOE_T_SHARED_SGATE = 5 /* INT4 [1, hidden]: the shared expert's sigmoid scalar gate */
} moe_tensor_role_t;

/* Replaces the compile-time ModelConfig constants
 * (src/engine/qwen35_moe/constants.rs:146-241) and validate_config (:57-90). */
typedef struct {
    int32_t hidden;         /* 2048 */
    int32_t inter;          /* moe_intermediate_size, 512 */
    int32_t shared_inter;   /* shared_expert_intermediate_size, 512 */
    int32_t num_experts;    /* 256 (stripped test model: 4) */
    int32_t top_k;          /* num_active_experts, <= 8 (src/engine/qwen35_moe/metal_context.rs:564-577) */
    int32_t num_layers;     /* 40 */
    int32_t num_mtp_layers; /* 0 or 1; the MTP block's experts are layer index num_layers */
    int32_t group;          /* 64 (src/constants.rs GROUP_SIZE) */
    int32_t vocab;          /* carried for the caller; unused by the MoE path */
    int32_t scheme;         /* moe_scheme_t */
} moe_dims_t;

/* Byte offsets inside one packed expert
 * (src/engine/qwen35_moe/constants.rs:117-139 expert_layout). */
typedef struct {
    int64_t gate_w, gate_s, gate_b, up_w, up_s, up_b, down_w, down_s, down_b, expert_size;
} moe_expert_layout_t;

const char* moe_last_error(void);
const char* moe_version(void);

/* src/engine/qwen35_moe/constants.rs:117-139 */
int moe_expert_layout(int32_t hidden, int32_t inter, int32_t group, moe_expert_layout_t* out);

/* ── engine lifetime ─────────────────────────────────────────────────────────
 * Replaces MetalContext::new (src/engine/qwen35_moe/metal_context.rs:558-600):
 * device, stream, persistent workspace.  MOE_ERR_INVALID for top_k > 8 or
 * dimensions the kernels do not cover. */
int moe_engine_create(const moe_dims_t* dims, int device, moe_engine_t** out);
void moe_engine_destroy(moe_engine_t* e);
int moe_engine_sync(moe_engine_t* e);
int moe_engine_dims(const moe_engine_t* e, moe_dims_t* out);

/* ── resident expert store ───────────────────────────────────────────────────
 * Replaces ExpertFile::read_expert (src/model/expert.rs:29-66), ExpertCache
 * (src/engine/qwen35_moe/metal_context.rs:25-121) and the prefetch pool: every
 * `packed_experts/layer_NN.bin` is copied once into device memory and stays.
 * `bytes` must equal num_experts * expert_size. */
int moe_store_load_layer(moe_engine_t* e, int layer, const void* blob_host, size_t bytes);
/* Device address of a layer's resident blob, so that the GPU packer can write
 * it in place (allocates the layer if needed). */
int moe_store_layer_dev(moe_engine_t* e, int layer, void** blob_dev);
/* Marks a layer whose blob was written on the device as loaded. */
int moe_store_mark_loaded(moe_engine_t* e, int layer);
/* Non-expert tensors by role; replaces WeightFile lookups by name
 * (src/model/weights.rs:124-179).  dtype MOE_DT_BF16: `w` only; MOE_DT_INT4:
 * `w` u32 words, `s` bf16 scales, `b` bf16 biases.  Host pointers. */
int moe_store_load_tensor(moe_engine_t* e, int layer, int role, const void* w_host,
                          const void* s_host, const void* b_host, int dtype);
int moe_store_bytes(const moe_engine_t* e, size_t* resident_bytes);

/* ── packer ──────────────────────────────────────────────────────────────────
 * quant_f32_to_int4 (src/dtype.rs:102-135) with the reference's bf16 rounding
 * (src/dtype.rs:85-89); bit-exact.  src is f32 or bf16 [rows, cols]; cols % 64
 * == 0.  Device pointers; src must be 16-byte aligned (MOE_ERR_INVALID otherwise),
 * the outputs need only their element alignment (word stores are 16 bytes wide
 * when the destination allows it). */
int moe_pack_int4_dev(moe_engine_t* e, const void* src_dev, int src_dtype, int64_t rows, int32_t cols,
                      void* w_dev, void* s_dev, void* b_dev);
/* Same through host buffers (copies in, packs on the GPU, copies out). */
int moe_pack_int4_host(moe_engine_t* e, const void* src_host, int src_dtype, int64_t rows, int32_t cols,
                       void* w_host, void* s_host, void* b_host);
/* quant_f32_to_int8 (src/dtype.rs:164-179; encode_int8 src/dtype.rs:466-475): per-row symmetric INT8, the
 * BQ4 scheme's lm_head codec.  src f32/bf16 [rows, cols] -> q int8 [rows, cols] + scales f32 [rows]; bit-exact
 * with the reference (scale = max|v| / 127, round half away from zero, clamp to +-127). */
int moe_pack_int8_host(moe_engine_t* e, const void* src_host, int src_dtype, int64_t rows, int32_t cols,
                       void* q_host, void* scales_host);

/* process_experts_common (src/quantize/qwen35_moe/common.rs:300-345): HF
 * gate_up [E, 2I, H] and down [E, H, I] -> E packed experts back to back.
 * Device pointers; n_experts may be a sub-range (pointers pre-offset). */
int moe_pack_experts_dev(moe_engine_t* e, const void* gate_up_dev, const void* down_dev, int src_dtype,
                         int32_t n_experts, void* blob_dev);
int moe_pack_experts_host(moe_engine_t* e, const void* gate_up_host, const void* down_host, int src_dtype,
                          int32_t n_experts, void* blob_host);

/* ── single dequant-matvec ───────────────────────────────────────────────────
 * dequant_matvec_4bit (src/math_util.rs:14-54; Metal default
 * dequant_matvec_4bit_v4_nr4, src/engine/shaders.metal:2949).  x f32 [cols],
 * y f32 [rows]. */
int moe_matvec_int4_dev(moe_engine_t* e, const void* w_dev, const void* s_dev, const void* b_dev,
                        const float* x_dev, float* y_dev, int32_t rows, int32_t cols);
int moe_matvec_int4_host(moe_engine_t* e, const void* w_host, const void* s_host, const void* b_host,
                         const float* x_host, float* y_host, int32_t rows, int32_t cols);

/* ── one MoE block ───────────────────────────────────────────────────────────
 * post-attention RMS norm, router, top-k, routed experts, gated shared expert,
 * combine with the residual: CpuEngine pre_expert (tail) + route_experts +
 * post_expert (src/engine/qwen35_moe/cpu.rs:187-205, 78-85, 398-483);
 * GPU engines: op1 tail + route_experts + encode_post_expert
 * (src/engine/qwen35_moe/fused_exp1.rs:231-365, 734-856), batched:
 * encode_post_expert_at (src/engine/qwen35_moe/batched.rs:334-447).
 *   h_in, h_out   f32 [n_tokens, hidden]  (h_in is the reference's h_mid)
 *   logit_bias    f32 [E] added to router logits before softmax, or NULL
 *   forced_idx    int32 [n_tokens, top_k] replaces the top-k choice, or NULL
 *   out_idx/out_w [n_tokens, top_k] chosen experts and renormalised weights
 *                 (descending weight order), or NULL
 * n_tokens == 1 runs the decode (matvec) path, n_tokens > 1 the grouped path
 * (token-serial fallback inside the reference: fused_exp3.rs:169-171). */
int moe_layer_forward_host(moe_engine_t* e, int layer, const float* h_in_host, int32_t n_tokens,
                           float* h_out_host, const float* logit_bias_host,
                           const int32_t* forced_idx_host, int32_t* out_idx_host, float* out_w_host);
int moe_layer_forward_dev(moe_engine_t* e, int layer, const float* h_in_dev, int32_t n_tokens,
                          float* h_out_dev, const float* logit_bias_dev, const int32_t* forced_idx_dev,
                          int32_t* out_idx_dev, float* out_w_dev);

/* ── the layer stack behind forward_hidden / forward_hidden_batched ──────────
 * Engine::forward_hidden / forward_hidden_batched (src/engine.rs:45-63;
 * src/engine/qwen35_moe/fused_exp1.rs:937-984, fused_exp3.rs:155-319) with the
 * attention half of every block passed through (h_mid = h): for each layer
 * h <- moe_block(h).  emb/out f32 [n_tokens, hidden]; out is the hidden state
 * before the final norm (Engine::last_h_pre_norm).  batched == 0 walks the
 * tokens one by one through the decode path (the reference's token-serial
 * loop), batched != 0 runs all tokens per layer through the grouped path.
 * mtp != 0 keeps the last token's hidden state for moe_mtp_forward.  `check`
 * (nullable) is polled between tokens / layers like the reference's
 * SignalCheckFn (src/engine.rs:10); non-zero aborts with MOE_ERR_INTERRUPTED. */
typedef int (*moe_check_fn)(void* ctx);
int moe_forward_hidden_host(moe_engine_t* e, const float* emb_host, int32_t n_tokens, int batched, int mtp,
                            moe_check_fn check, void* check_ctx, float* out_host);
int moe_forward_hidden_dev(moe_engine_t* e, const float* emb_dev, int32_t n_tokens, int batched,
                           float* out_dev);
/* Engine::last_h_pre_norm (src/engine.rs:66-68): f32 [hidden] of the last token. */
int moe_last_h_pre_norm(moe_engine_t* e, float* out_host);

/* ── the model head: embedding rows, final norm, lm_head ─────────────────────
 * What surrounds the stack inside Engine::forward (src/python_bindings.rs:172-202):
 * embed_lookup (src/math_util.rs:205-236: one row of the 4-bit table model.embed_tokens per token),
 * final_norm (src/math_util.rs:240-247, model.norm.weight) and the lm_head matvec
 * (src/engine/qwen35_moe/fused_exp1.rs:390-393, 860-879): INT8 rows with one f32 scale per row in the BQ4
 * scheme (src/dtype.rs:164-179, src/engine/shaders.metal:2435-2471), a 4-bit triple in the INT4 scheme.
 * moe_head_load_tensor copies a host tensor into HBM:
 *   MOE_H_EMBED       INT4 [vocab, hidden]: w = u32 words, s/b = bf16 [vocab, hidden/64]
 *   MOE_H_FINAL_NORM  bf16 [hidden] (w only)
 *   MOE_H_LM_HEAD     MOE_DT_INT8: w = int8 [vocab, hidden], s = f32 [vocab];  MOE_DT_INT4: triple as above
 * moe_embed_lookup_*: ids int64 [n] -> f32 [n, hidden]; an id outside [0, vocab) is MOE_ERR_INVALID.
 * moe_logits_*: hidden f32 [n, hidden] (before the final norm) -> logits f32 [n, vocab].
 * moe_forward_host: Engine::forward / forward_batched: ids -> logits [n, vocab] through embedding, stack and head
 * (`batched`, `mtp`, `check` as for moe_forward_hidden_host); keeps the last token's pre-norm hidden state.
 * MOE_ERR_STATE when a tensor the call needs has not been loaded. */
typedef enum { MOE_H_EMBED = 0, MOE_H_FINAL_NORM = 1, MOE_H_LM_HEAD = 2 } moe_head_tensor_t;
int moe_head_load_tensor(moe_engine_t* e, int which, const void* w_host, const void* s_host, const void* b_host, int dtype);
int moe_embed_lookup_host(moe_engine_t* e, const int64_t* ids_host, int32_t n_tokens, float* out_host);
int moe_embed_lookup_dev(moe_engine_t* e, const int64_t* ids_dev, int32_t n_tokens, float* out_dev);
int moe_logits_host(moe_engine_t* e, const float* hidden_host, int32_t n_tokens, float* logits_host);
int moe_logits_dev(moe_engine_t* e, const float* hidden_dev, int32_t n_tokens, float* logits_dev);
int moe_forward_host(moe_engine_t* e, const int64_t* ids_host, int32_t n_tokens, int batched, int mtp,
                     moe_check_fn check, void* check_ctx, float* logits_host);

/* ── MTP block ───────────────────────────────────────────────────────────────
 * Engine::mtp_forward / mtp_reset / mtp_rollback (src/engine.rs:70-78;
 * src/engine/qwen35_moe/mtp.rs:58-225).  Only the block's MoE half
 * (mtp.rs:176-207, 381-517; experts = layer index num_layers) runs here; its
 * attention half is passed through.  `h_in_host` is the block input the caller
 * built from last_h_pre_norm and the token embedding (mtp.rs:85-110); out is
 * f32 [hidden].  MOE_ERR_STATE when num_mtp_layers == 0. */
int moe_mtp_forward_host(moe_engine_t* e, const float* h_in_host, float* h_out_host);
int moe_mtp_reset(moe_engine_t* e);
int moe_mtp_rollback(moe_engine_t* e, int64_t pos);
int moe_mtp_pos(const moe_engine_t* e, int64_t* pos);

/* ── MTP block, whole step ───────────────────────────────────────────────────
 * mtp_step (src/engine/qwen35_moe/mtp.rs:58-225): (hidden state before the final norm, previous token) -> logits.
 * embed the token; RMS-norm it and the hidden state with their own weights; concatenate (embedding first) and
 * project with mtp.fc; one gated full-attention block (input norm; q/k/v projections, q carrying the output gate
 * in its second half; per-head q/k RMS norm; interleaved RoPE on the first rotary_dim elements of every head; f32
 * KV cache of the block's own; softmax attention; sigmoid gate; o projection; residual); the MoE half (layer index
 * num_layers of the store: post-attention norm, router, experts, shared expert, residual); mtp.norm (or the model's
 * final norm when mtp.norm was not loaded); lm_head.  The position is the one moe_mtp_reset / moe_mtp_rollback
 * manage.  Norm weights are bf16; a projection is MOE_DT_BF16 ([out, in], BQ4 scheme, bq4.rs:25-32) or MOE_DT_INT4
 * (triple); mtp.fc is always MOE_DT_INT4 [hidden, 2 * hidden].  Host pointers.
 * moe_mtp_configure allocates the KV cache (max_seq positions; the reference's MAX_SEQ = 4096 is src/constants.rs:12)
 * and must come before the tensors.  MOE_ERR_STATE when the block has no MTP layer, a tensor is missing or the
 * cache is full. */
typedef struct {
    int32_t num_heads, num_kv_heads, head_dim, rotary_dim, max_seq;
    float rope_theta;
} moe_attn_dims_t;
typedef enum {
    MOE_M_PRE_FC_NORM_HIDDEN = 0, MOE_M_PRE_FC_NORM_EMBEDDING = 1, MOE_M_FC = 2, MOE_M_INPUT_NORM = 3,
    MOE_M_Q_PROJ = 4, MOE_M_K_PROJ = 5, MOE_M_V_PROJ = 6, MOE_M_Q_NORM = 7, MOE_M_K_NORM = 8, MOE_M_O_PROJ = 9,
    MOE_M_OUT_NORM = 10
} moe_mtp_tensor_t;
int moe_mtp_configure(moe_engine_t* e, const moe_attn_dims_t* attn);
int moe_mtp_load_tensor(moe_engine_t* e, int which, const void* w_host, const void* s_host, const void* b_host, int dtype);
int moe_mtp_step_host(moe_engine_t* e, const float* h_host, int64_t token_id, float* logits_host);

/* ── attention half of the 40 main layers, batch-1 decode ────────────────────
 * pre_expert_full / pre_expert_linear up to the residual (src/engine/qwen35_moe/cpu.rs:87-183, 218-347; the
 * Metal engines' op1, fused_exp1.rs:399-732): layer l is a gated full-attention layer when (l + 1) %
 * full_attn_interval == 0 (input norm; q/k/v projections, q carrying [head, gate] per head; per-head q/k RMS
 * norm; RoPE on the pairs (d, d + rotary_dim / 2); f32 KV cache; softmax attention; sigmoid gate; o projection;
 * residual) and a Gated DeltaNet layer otherwise (input norm; in_proj_qkv / z / b / a; causal depthwise conv
 * over the last conv_kernel inputs + SiLU; unweighted per-head q/k norm; decay and input gate from a, b, A_log,
 * dt_bias; delta-rule recurrence on a [v_heads, value_dim, key_dim] f32 state; gated RMS norm; out_proj;
 * residual).  Each attention half feeds the layer's MoE half (the decode kernel).  Up to three tokens run as that many
 * decode steps; four and more run layer by layer (projections, cache update and attention, the DeltaNet recurrence and the MoE
 * half each over all the tokens of the call; same results to the batched MoE path's accuracy).  moe_attn_configure allocates every layer's cache / state and resets the position; tensors
 * by role (norms, conv1d [channels, kernel], dt_bias: bf16; A_log: MOE_DT_F32; projections: MOE_DT_BF16 [out,
 * in] or MOE_DT_INT4 triple).  moe_model_forward_hidden_host: embeddings [n, hidden] -> hidden states before
 * the final norm [n, hidden] (then moe_logits_host); moe_model_forward_host: token ids -> logits [n, vocab].
 * MOE_ERR_STATE when a tensor is missing or the position reaches max_seq.  Host pointers. */
typedef struct {
    moe_attn_dims_t full;
    int32_t lin_num_k_heads, lin_num_v_heads, lin_key_dim, lin_value_dim, conv_kernel, full_attn_interval;
} moe_model_attn_dims_t;
typedef enum {
    MOE_A_INPUT_NORM = 0, MOE_A_Q_PROJ = 1, MOE_A_K_PROJ = 2, MOE_A_V_PROJ = 3, MOE_A_Q_NORM = 4, MOE_A_K_NORM = 5,
    MOE_A_O_PROJ = 6, MOE_A_IN_PROJ_QKV = 7, MOE_A_IN_PROJ_Z = 8, MOE_A_IN_PROJ_B = 9, MOE_A_IN_PROJ_A = 10,
    MOE_A_CONV1D = 11, MOE_A_A_LOG = 12, MOE_A_DT_BIAS = 13, MOE_A_LIN_NORM = 14, MOE_A_OUT_PROJ = 15
} moe_attn_tensor_t;
int moe_attn_configure(moe_engine_t* e, const moe_model_attn_dims_t* dims);
int moe_attn_load_tensor(moe_engine_t* e, int layer, int which, const void* w_host, const void* s_host,
                         const void* b_host, int dtype);
int moe_model_forward_hidden_host(moe_engine_t* e, const float* emb_host, int32_t n, float* out_host);
int moe_model_forward_host(moe_engine_t* e, const int64_t* ids_host, int32_t n, float* logits_host);
int moe_model_reset(moe_engine_t* e);
int moe_model_pos(const moe_engine_t* e, int64_t* pos);
/* Engine::snapshot / restore (src/engine.rs:84-105): the state a speculative decode rolls back to, i.e. the position,
 * the MTP position, last_h_pre_norm and the conv + recurrence state of every linear-attention layer (KV entries behind
 * the position are simply overwritten later).  The copy lives in device memory owned by the snapshot; restoring is
 * allowed any number of times, into the engine it was taken from, until moe_model_snapshot_free. */
typedef struct moe_snapshot moe_snapshot_t;
int moe_model_snapshot(moe_engine_t* e, moe_snapshot_t** out);
int moe_model_restore(moe_engine_t* e, const moe_snapshot_t* snap);
void moe_model_snapshot_free(moe_snapshot_t* snap);
/* Engine::download_cache / upload_cache and what Cache::save / load put on disk (src/engine.rs:64-79,
 * src/cache.rs:133-233): one state tensor of one layer, device -> host (to_device == 0) or host -> device.
 *   MOE_ST_K_CACHE / MOE_ST_V_CACHE (full-attention layers): the first floats / kv_dim positions, [position, kv_dim];
 *   MOE_ST_CONV (linear-attention layers): [conv_kernel, conv_dim], the input of step s in row s % conv_kernel (a ring;
 *       the reference keeps the last conv_kernel - 1 inputs oldest first, src/math_util.rs:149-168: row k of that
 *       layout is row (pos - (conv_kernel - 1) + k) mod conv_kernel here, zeros for steps before the start);
 *   MOE_ST_SSM: the recurrence state [v_heads, value_dim, key_dim].
 * `floats` must be the tensor's size (for the caches: a multiple of kv_dim, at most max_seq positions).  MOE_ERR_INVALID
 * for a tensor the layer does not have.  moe_model_set_pos moves the position the next decode step runs at (after an
 * upload; 0 <= pos <= max_seq). */
typedef enum { MOE_ST_K_CACHE = 0, MOE_ST_V_CACHE = 1, MOE_ST_CONV = 2, MOE_ST_SSM = 3 } moe_state_tensor_t;
int moe_model_state_host(moe_engine_t* e, int32_t layer, int32_t which, float* host, int64_t floats, int32_t to_device);
int moe_model_set_pos(moe_engine_t* e, int64_t pos);

/* ── telemetry ───────────────────────────────────────────────────────────────
 * set_record_telemetry / Engine::telemetry (src/engine.rs:13-23, 80-84); keys
 * follow the reference (`engine.total_ms`, `phase.route_cpu_ms`, ...).  Fills up
 * to *n entries; on return *n is the number available.  Key pointers stay
 * valid until the next call on the same engine.  With MOE_B200_DECODE_PREFETCH=1 in
 * the environment when the engine is created, the decode kernel requests the next
 * layer's copy of every chosen expert into L2 ahead of time (the reference's
 * predictor, src/engine/qwen35_moe/expert_prefetch.rs:95-135) and the keys
 * `prefetch.checks` / `prefetch.hits` count its predictions since creation. */
void moe_set_record_telemetry(int on);
int moe_get_record_telemetry(void);
int moe_telemetry_get(moe_engine_t* e, const char** keys, double* vals, int* n);

/* Fine-grained phase timing of the decode kernel, the device-side counterpart of
 * the reference's `phase.*` telemetry (src/engine/qwen35_moe/fused_exp5.rs:162-177).
 * With stamps == NULL: switches recording on (enable != 0) or off.  Otherwise
 * copies the SM-clock stamps of the last decode launch, [layer][*points_per_layer]
 * (12 per layer), taken by thread 0 of CTA 0.  The default (slot-grouped) kernel
 * stamps: 0 layer start; 1 residual and router sums of the previous layer read,
 * 1/rms known; 2 top-k done; 3 this CTA's weight slices requested; 4 input staged
 * as digit planes; 10 / 11 first / second half of the gate/up slices landed;
 * 5 gate/up rows and SwiGLU done; 6 the group's 512 SwiGLU values gathered and
 * staged, down slices landed; 7 down rows added to the residual sums; 8 this CTA's
 * share of the next layer's router logits added, layer counter bumped; 9 (last
 * layer only) result written.  The grid-wide fallback kernel stamps its own
 * twelve points in the same order of events (copies issued, landed, rows done,
 * barrier passed) for its three phases. */
int moe_decode_profile(moe_engine_t* e, int enable, int64_t* stamps, int max_layers, int* points_per_layer);

/* ── expert parallelism over the GPUs of one box ─────────────────────────────
 * No counterpart in the reference (single device).  One process per GPU; rank r
 * keeps experts [r*E/P, (r+1)*E/P) of every layer, the router, the shared expert
 * and the norms are replicated, and every rank brings its own tokens.  Token rows
 * travel through device buffers the ranks map from one another (CUDA IPC) with
 * plain peer stores; ranks meet through epoch flags with bounded waits.
 *   1. every rank: moe_ep_export -> one 64-byte handle
 *   2. the host program gathers the handles of all ranks, in rank order, by any
 *      means it has (MPI, torch.distributed, a pipe)
 *   3. every rank: moe_ep_init with the table of world * 64 bytes
 *   4. every rank calls moe_ep_layer_forward_dev / moe_ep_forward_hidden_dev for the
 *      same layer at the same point of its program (collective calls)
 * h_in/h_out are f32 [n_local, hidden] on the device; n_local <= max_tokens_per_rank
 * and may differ between ranks.  The expert store keeps the full-size allocation
 * per layer; a rank only needs valid bytes for the experts it owns. */
#define MOE_EP_HANDLE_BYTES 64
int moe_ep_export(moe_engine_t* e, int rank, int world, int32_t max_tokens_per_rank,
                  void* handle_out /* MOE_EP_HANDLE_BYTES */);
int moe_ep_init(moe_engine_t* e, const void* all_handles /* world * MOE_EP_HANDLE_BYTES */);
int moe_ep_finalize(moe_engine_t* e);
int moe_ep_layer_forward_dev(moe_engine_t* e, int layer, const float* h_in_dev, int32_t n_local, float* h_out_dev);
int moe_ep_forward_hidden_dev(moe_engine_t* e, const float* emb_dev, int32_t n_local, float* out_dev);

/* ── decode of one MoE block without any allocation ─────────────────────────
 * This entry point has no counterpart in the reference.  It exists for hosts
 * that must not let a library allocate device memory: a serving process whose
 * HBM is partitioned once at start-up and owned by its own pool, a plug-in inside
 * such a process, or a loop in which cudaMalloc / cudaFree (they synchronise the
 * device and can fail under fragmentation) are banned after initialisation.
 *
 * It needs no engine.  It computes what moe_layer_forward_dev computes for one
 * token (n_tokens == 1, no logit bias, no forced indices) from tensor pointers
 * the caller owns (all device memory, in the reference's byte layout), and
 * keeps its work areas (router logits, SwiGLU outputs, barrier words) in a
 * 40 KiB array that is part of the library image; every GPU that loads the
 * library holds that array until the process exits.
 *
 *  - Limits: hidden 2048, inter = shared_inter = 512, group 64, top_k <= 8,
 *    num_experts <= 512 (the array has room for 512 router logits); anything
 *    else is rejected with MOE_ERR_INVALID and a message.
 *  - It calls no cudaMalloc, cudaFree or other allocating routine.
 *  - The first call on a device looks up the array's device address and sets the
 *    kernel's shared-memory attribute (under a lock: two host threads may race
 *    on a device's first call); make that first call before any stream capture
 *    begins.
 *  - All calls on a device share the one array and it keeps the previous call's
 *    contents; the words that must start at zero are cleared on the given stream
 *    at every call.  Two calls that overlap on the same GPU (different streams,
 *    or different threads) race on the array: serialise them.
 *  - `cuda_stream` is a cudaStream_t (NULL = the default stream).  With wait == 0
 *    the call returns after enqueueing and NEVER reports a device-side
 *    bounded-wait failure: the error word stays in the array until the next call
 *    on that device clears it, so a caller that enqueues must ask
 *    moe_layer_decode_noalloc_status (below) before its next call if it wants to
 *    know.  With wait != 0 the call waits for the stream and reports such a
 *    failure as MOE_ERR_DEVICE_WAIT.
 *  - h_out_dev may be the same buffer as h_in_dev. */
typedef struct {
    const void* experts;     /* num_experts packed experts (moe_expert_layout), back to back */
    const void* post_norm;   /* bf16 [hidden] */
    const void* router_bf16; /* bf16 [E, hidden], or NULL to use the 4-bit router below */
    const void* router_w;    /* u32 [E, hidden/8] */
    const void* router_s;    /* bf16 [E, hidden/64] */
    const void* router_b;    /* bf16 [E, hidden/64] */
    const void* shared;      /* shared expert, same byte layout as one packed expert */
    const void* sgate_w;     /* shared_expert_gate: u32 [1, hidden/8] */
    const void* sgate_s;     /* bf16 [1, hidden/64] */
    const void* sgate_b;     /* bf16 [1, hidden/64] */
} moe_layer_ptrs_t;
int moe_layer_decode_noalloc(const moe_dims_t* dims, int device, const moe_layer_ptrs_t* layer_ptrs_dev,
                             const float* h_in_dev, float* h_out_dev, int32_t* out_idx_dev /* nullable */,
                             float* out_w_dev /* nullable */, void* cuda_stream, int wait);
/* No counterpart in the reference.  Waits for `cuda_stream` on `device` and reads the error word the last
 * moe_layer_decode_noalloc call on that device left in the array: *code == 0 and MOE_OK when every device-side
 * wait completed, the code and MOE_ERR_DEVICE_WAIT otherwise.  Allocates nothing.  For callers that enqueue
 * with wait == 0. */
int moe_layer_decode_noalloc_status(int device, void* cuda_stream, unsigned int* code);

/* ── plain device-memory helpers for hosts without a CUDA binding ──────────── */
int moe_dev_alloc(moe_engine_t* e, size_t bytes, void** out_dev);
int moe_dev_free(moe_engine_t* e, void* p_dev);
int moe_dev_upload(moe_engine_t* e, void* dst_dev, const void* src_host, size_t bytes);
int moe_dev_download(moe_engine_t* e, void* dst_host, const void* src_dev, size_t bytes);
int moe_dev_memset(moe_engine_t* e, void* dst_dev, int value, size_t bytes);
int moe_host_alloc_pinned(size_t bytes, void** out_host);
int moe_host_free_pinned(void* p_host);
#ifdef __cplusplus
}
#endif
#endif /* MOE_B200_H */
