// Shared declarations of the sm_100a MoE library: engine state, error plumbing,
// small device helpers.  Internal; the public surface is include/moe_b200.h.
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdio.h>
#include <map>
#include <string>
#include <vector>

#include "../../include/moe_b200.h"

namespace moe {

constexpr int kGroup = 64;  // weights per scale/bias pair (src/constants.rs GROUP_SIZE)
constexpr int kMaxK = 8;    // MAX_K (src/engine/qwen35_moe/metal_context.rs:564-577)

// ─── host-side error plumbing ───────────────────────────────────────────────
void set_error(const char* fmt, ...);
int cuda_fail(cudaError_t err, const char* what, const char* file, int line);

#define MOE_CUDA(call)                                                            \
    do {                                                                          \
        cudaError_t _e = (call);                                                  \
        if (_e != cudaSuccess) return moe::cuda_fail(_e, #call, __FILE__, __LINE__); \
    } while (0)

#define MOE_REQUIRE(cond, ...)              \
    do {                                    \
        if (!(cond)) {                      \
            moe::set_error(__VA_ARGS__);    \
            return MOE_ERR_INVALID;         \
        }                                   \
    } while (0)

// One 4-bit tensor on the device: u32 words, bf16 scales, bf16 biases.
struct Q4Dev {
    const uint32_t* w = nullptr;
    const uint16_t* s = nullptr;
    const uint16_t* b = nullptr;
};

// Device pointers of one MoE block, passed to kernels by value (in an array in
// device memory for the persistent decode kernel).
struct LayerDev {
    const uint8_t* experts;      // E * expert_size
    const uint16_t* post_norm;   // bf16 [H]
    const uint16_t* router_bf16; // bf16 [E, H] or nullptr
    Q4Dev router_q4;             // INT4-scheme router
    const uint8_t* shared;       // shared expert in expert-blob layout (hidden, shared_inter)
    Q4Dev sgate;                 // [1, H]
    const uint16_t* router_planes;  // batched path: router weights split into bf16 planes (see grouped.cu), or nullptr
    int router_nplanes;             // 1 (bf16 router) or 3 (4-bit router)
    const void* router_t;           // decode path: router transposed to [H][E] (bf16 bits, or f32 for a 4-bit router), or nullptr
};

struct LayerHost {
    uint8_t* experts = nullptr;
    uint8_t* aux = nullptr;   // one allocation holding every non-expert tensor
    bool experts_loaded = false;
    bool role_loaded[6] = {false, false, false, false, false, false};
    bool router_is_bf16 = true;
    uint8_t* planes = nullptr;   // router planes of the batched path, built on first use
    bool planes_valid = false;
    alignas(64) unsigned char planes_map[128] = {};  // tensor map (TMA descriptor) over the planes
    uint8_t* router_t = nullptr; // transposed router of the decode path, built on first use
    bool router_t_valid = false;
    LayerDev dev{};
};

// Work areas of the batched (grouped) path, sized for `capacity` tokens.
struct BatchWork {
    int32_t capacity = 0;          // tokens
    uint8_t* base = nullptr;       // one allocation holding everything below
    float* h_a = nullptr;          // [cap, H] ping (layer stack)
    float* h_b = nullptr;          // [cap, H] pong
    __nv_bfloat16* x = nullptr;    // [cap, H] normalised activations, bf16, K-interleaved
    __nv_bfloat16* x_mid = nullptr;  // [cap, H] second and third bf16 terms of x (x = x + x_mid + x_lo to 24 bits),
    __nv_bfloat16* x_lo = nullptr;   //          same order, for the f32-accurate router
    float* logits = nullptr;       // [logit_rows, E]: up to kRtMaxSplit slabs of partial sums
    int64_t logit_rows = 0;
    int32_t* topk_idx = nullptr;   // [cap, K]
    float* topk_w = nullptr;       // [cap, K]
    float* sgate = nullptr;        // [cap] sigmoid(shared gate score)
    int32_t* counts = nullptr;     // [E + 1] tokens per expert (+ shared); zeroed every layer
    int32_t* offsets = nullptr;    // [E + 2] exclusive scan
    int32_t* cursor = nullptr;     // [E + 1]
    int32_t* slot_token = nullptr; // [cap*K + cap] token of each expert-sorted slot
    int32_t* slot_of = nullptr;    // [cap*K] slot of (token, k)
    __nv_bfloat16* act = nullptr;  // [cap*K + cap, I] SwiGLU outputs, expert-sorted, K-interleaved
    __nv_bfloat16* o = nullptr;    // [cap*K + cap, H] down-projection outputs, expert-sorted
    int32_t* slot_expert = nullptr;  // [cap*K + cap] expert of each slot (E: the shared expert), written for small batches
    float* act32 = nullptr;        // [small*K + small, I] f32 SwiGLU outputs of the slot-wise FFN (small batches)
    int32_t* tile_list = nullptr;  // (expert, first slot, slots) per token tile
    int32_t* n_tiles = nullptr;
    int32_t max_tiles = 0;
    alignas(64) unsigned char x_map[128] = {};  // tensor map (TMA descriptor) over x, x_mid, x_lo as one [3 * cap, H] tensor
};

// Expert-parallel state: experts of every layer are split over `world` GPUs of one box;
// token rows travel through buffers the ranks map from one another (CUDA IPC).
constexpr int kEpMaxWorld = 8;
struct EpSym {                    // layout of the buffer every rank exports (byte offsets)
    size_t flags, counts, meta, xmap, memb, mwt, xrecv, oback, total;
};
struct EpState {
    bool ready = false;
    int rank = 0, world = 1, cap = 0;       // cap = max tokens per rank
    int slots_cap = 0;                      // world * cap * top_k rows a rank can receive
    EpSym sym{};
    uint8_t* local = nullptr;               // this rank's exported buffer
    uint8_t* peer[kEpMaxWorld] = {};        // every rank's buffer as mapped here (peer[rank] == local)
    unsigned int epoch = 0;
    uint8_t* work = nullptr;                // private work areas (one allocation)
    __nv_bfloat16* act = nullptr;           // [slots_cap + cap, I]
    __nv_bfloat16* o = nullptr;             // [slots_cap + cap, H]
    int32_t* tile_list = nullptr;
    int32_t* n_tiles = nullptr;
    int32_t* base_send = nullptr;           // [E] first slot of my rows of expert e at its owner
    int32_t* cursor = nullptr;              // [E]
    int32_t* total_recv = nullptr;          // rows received this layer
    unsigned int* done = nullptr;           // blocks finished (scatter / return kernels), rewound by the last one
    uint8_t* lead_mask = nullptr;           // [cap] bit k: (token, k) is the first of the token's experts on its GPU
    int max_tiles = 0;
};

// The model head: token embedding table, final norm weight, lm_head (head.cu).
struct HeadState {
    uint8_t* embed = nullptr;      // 4-bit table [vocab, hidden]: words, then scales at embed_s, biases at embed_b
    size_t embed_s = 0, embed_b = 0;
    uint16_t* final_norm = nullptr;  // bf16 [hidden]
    uint8_t* lm_head = nullptr;    // INT8 rows + f32 scales at lm_s, or 4-bit words + bf16 scales at lm_s + biases at lm_b
    size_t lm_s = 0, lm_b = 0, lm_bytes = 0;
    int lm_dtype = 0;
    bool embed_loaded = false, norm_loaded = false, lm_loaded = false, i8_attr_set = false;
    uint8_t* work = nullptr;       // normalised hidden states and token ids of a call, grown on demand
    float* x = nullptr;
    int64_t* ids = nullptr;
    int32_t cap = 0;
};

// The MTP block's attention half (attn.cu): tensors, KV cache and scratch.
struct ProjTensor {
    uint8_t* w = nullptr;          // bf16 [rows, cols], or 4-bit words followed by scales at s_off and biases at b_off
    size_t s_off = 0, b_off = 0;
    int dtype = 0, rows = 0, cols = 0;
    bool loaded = false;
};
struct MtpAttnState {
    moe_attn_dims_t ad{};
    bool configured = false;
    uint16_t* norms[11] = {};      // bf16 norm weights by moe_mtp_tensor_t (projection slots stay null)
    ProjTensor proj[11];           // projections by moe_mtp_tensor_t (norm slots stay unloaded)
    float* k_cache = nullptr;      // [max_seq, num_kv_heads * head_dim]
    float* v_cache = nullptr;
    float* work = nullptr;         // scratch vectors of one step
    int64_t* id_dev = nullptr;
    bool bf_attr_set = false;
};

// The attention half of the main layers (attn.cu): per-layer tensors and caches, one scratch area.
struct AttnLayerState {
    bool full = false;
    void* vec[16] = {};            // norm weights, conv1d, dt_bias (bf16) and A_log (f32) by moe_attn_tensor_t
    ProjTensor proj[16];           // projections by moe_attn_tensor_t
    float* k_cache = nullptr;      // full attention: [max_seq, kv_dim] each
    float* v_cache = nullptr;
    float* conv_state = nullptr;   // linear attention: ring of the last conv_kernel inputs, [conv_kernel, conv_dim], row = position % conv_kernel
    float* ssm_state = nullptr;    // linear attention: [v_heads, value_dim, key_dim]
    ProjTensor fused;              // the input projections stacked row-wise (q|k|v, or qkv|z|b|a): one launch instead of 3-4
};
struct ModelAttnState {
    moe_model_attn_dims_t d{};
    bool configured = false;
    std::vector<AttnLayerState> layers;
    float* work = nullptr;
    int64_t pos = 0;
    int* d_pos = nullptr;                    // the position as the kernels read it
    std::vector<cudaGraphExec_t> graphs;     // one captured attention half per layer (null: launch eagerly)
    std::vector<int> graph_nodes;            // kernels in each
    bool graphs_valid = false;
    bool pdl = true;                         // kernels of a layer's attention half start ahead of their predecessor's end
    bool chain = true;                       // no graphs: every kernel of a token, the MoE kernels included, is a programmatic dependent of the one before it
    int prefill_min = 4;                     // calls of at least this many tokens run layer by layer (MoE halves batched)
    int* pos_table = nullptr;                // positions 0 .. max_seq - 1 on the device
    float* prefill_mid = nullptr;            // [prefill_cap, H] attention outputs of a layer, all tokens
    float* prefill_scratch = nullptr;        // [prefill_cap] scratch areas, one per token (same allocation)
    int prefill_cap = 0;
    bool lin_split = true;                   // DeltaNet core as 256-thread CTAs per block of state rows (gated norm in the out projection)
};

}  // namespace moe

struct moe_engine {
    moe_dims_t dims{};
    int device = 0;
    int sm_count = 0;
    cudaStream_t stream = nullptr;
    cudaEvent_t ev0 = nullptr, ev1 = nullptr, ev2 = nullptr;
    moe_expert_layout_t lay{};         // routed experts
    moe_expert_layout_t shared_lay{};  // shared expert (hidden, shared_inter)
    std::vector<moe::LayerHost> layers;  // num_layers + num_mtp_layers
    moe::LayerDev* layers_dev = nullptr; // device copy of the LayerDev table
    bool table_dirty = true;
    size_t resident = 0;
    int64_t launches = 0;

    // decode (n = 1) work areas
    unsigned int* dec_sync = nullptr;      // grid barrier words + error flag
    unsigned long long* dec_act_ll = nullptr;  // fused decode kernel: tagged SwiGLU outputs
    long long* dec_acc = nullptr;          // fused decode kernel: fixed-point router accumulators, two sets
    unsigned int dec_epoch = 0;            // tags consumed so far (one per layer pass)
    unsigned long long* dec_hint = nullptr;    // fused decode kernel: count of CTAs whose outputs are written
    unsigned long long dec_hint_base = 0;
    unsigned long long* dec_h_ll = nullptr;    // fused decode kernel: tagged hidden state between layers
    long long* dec_prof = nullptr;         // per-phase clock stamps (off unless enabled)
    int dec_grid = 0;
    // slot-grouped decode kernel (decode_slots.cu)
    bool dec_sl_ok = false;                     // device and model shape fit it
    unsigned long long* dec_sl_words = nullptr; // accumulators, tagged SwiGLU outputs, counters (one allocation)
    unsigned long long dec_sl_hint_base = 0;
    bool dec_sl_prefetch = false;          // request the next layer's copy of a layer's experts into L2 (environment switch)
    unsigned int dec_sl_epoch = 0;
    bool matvec_attr_set = false;          // matvec kernel's shared-memory attribute set on this engine's device
    float* stage_host = nullptr;           // pinned staging [H] x 2, then 16 words (the device error word is read into the first)
    bool err_read_pending = false;         // a read of the error word is enqueued behind the current call's work
    std::vector<float> last_h;             // last_h_pre_norm
    int64_t mtp_pos = 0;

    moe::BatchWork bw;
    uint8_t* io_dev = nullptr;  // staging of the host-pointer entry points
    size_t io_cap = 0;

    // telemetry
    std::map<std::string, double> telemetry;
    std::vector<std::string> tel_keys;

    // expert parallelism
    moe::EpState ep;

    moe::HeadState head;
    moe::MtpAttnState mtp;
    moe::ModelAttnState attn;
};

namespace moe {

// Kernel launchers implemented in the .cu files; all enqueue on e->stream.
int launch_pack(moe_engine* e, const void* src, int src_dtype, int64_t rows, int32_t cols,
                int64_t src_row_stride, void* w, void* s, void* b);
int launch_pack_int8(moe_engine* e, const void* src, int src_dtype, int64_t rows, int32_t cols, void* q, void* scales);
int launch_pack_experts(moe_engine* e, const void* gate_up, const void* down, int src_dtype,
                        int32_t n_experts, void* blob);
// A matvec over several input vectors in one launch (grid.y = vector): element strides from one vector's buffers to the
// next one's; the default is one vector.  The weights are read again for every vector (from L2 when they fit).
struct MvBatch {
    int n = 1;
    int x_stride = 0, y_stride = 0, r_stride = 0, ss_stride = 0;  // input, output, residual, per-head sums
};
// sets the per-device function attributes of the matvec kernels (so that later launches can be captured into a graph)
int matvec_prepare(moe_engine* e);
// y = W x + residual (residual nullable; may not alias y)
int launch_matvec_res(moe_engine* e, const void* w, const void* s, const void* b, const float* x, float* y, int32_t rows,
                      int32_t cols, const float* residual, bool pdl = false, const void* norm_w = nullptr, MvBatch mb = MvBatch{});
// whether launch_matvec_res can apply rmsnorm(x) * norm_w (bf16 weights) to its input itself for this shape
bool matvec_folds_norm(int32_t rows, int32_t cols);
int matvec_batch_blocks(const moe_engine* e, int blocks, int n);
// y = W (x scaled per head) + residual: the last step of a per-head RMS norm (sums of squares left in `ss` by the producer,
// `parts` entries per head) folded into the kernel's staging
bool matvec_folds_head_scale(int32_t rows, int32_t cols, int32_t head_dim);
int launch_matvec_head_scaled(moe_engine* e, const void* w, const void* s, const void* b, const float* x, const float* ss,
                              int32_t parts, int32_t head_dim, float* y, int32_t rows, int32_t cols, const float* residual,
                              bool pdl, MvBatch mb = MvBatch{});
int launch_matvec(moe_engine* e, const void* w, const void* s, const void* b, const float* x,
                  float* y, int32_t rows, int32_t cols);
int decode_init(moe_engine* e);
void decode_destroy(moe_engine* e);
int decode_reset_after_error(moe_engine* e);
int ensure_router_t(moe_engine* e, int layer);
// Runs layers [l0, l1) on one token: h_in (device, [H]) -> h_out (device, [H]).
int launch_slot_ffn(moe_engine* e, const moe::LayerDev& ly, const float* h_in, int slots, const int32_t* slot_token,
                    const int32_t* slot_expert, float* act, void* o);
int launch_decode(moe_engine* e, int l0, int l1, const float* h_in, float* h_out,
                  const float* logit_bias, const int32_t* forced_idx, int32_t* out_idx, float* out_w, bool pdl = false);
int decode_profile_enable(moe_engine* e, bool on);
int decode_profile_read(moe_engine* e, long long* out, int max_layers, int* points);
int batch_reserve(moe_engine* e, int32_t n_tokens);
void batch_destroy(moe_engine* e);
int launch_batched_layer(moe_engine* e, int layer, const float* h_in, int32_t n, float* h_out,
                         const float* logit_bias, const int32_t* forced_idx, int32_t* out_idx,
                         float* out_w);
int ep_layer(moe_engine* e, int layer, const float* h_in, int32_t n_local, float* h_out);
int ep_alloc_work(moe_engine* e);
int head_load_tensor(moe_engine* e, int which, const void* w, const void* s, const void* b, int dtype);
int launch_embed(moe_engine* e, const int64_t* ids_dev, int32_t n, float* out_dev);
int launch_logits(moe_engine* e, const float* hidden_dev, int32_t n, float* logits_dev);
// the same with another norm weight (bf16 [hidden], device) in place of the model's final norm; null = the model's
int launch_logits_norm(moe_engine* e, const float* hidden_dev, int32_t n, float* logits_dev, const uint16_t* norm_w);
int mtp_configure(moe_engine* e, const moe_attn_dims_t* ad);
int mtp_load_tensor(moe_engine* e, int which, const void* w, const void* s, const void* b, int dtype);
int mtp_step(moe_engine* e, const float* h_host, int64_t token_id, float* logits_dev);
void mtp_destroy(moe_engine* e);
int attn_configure(moe_engine* e, const moe_model_attn_dims_t* dims);
int attn_load_tensor(moe_engine* e, int layer, int which, const void* w, const void* s, const void* b, int dtype);
// n decode steps with attention, enqueued: emb_dev [n, hidden] -> out_dev [n, hidden]; advances the position
int attn_model_forward(moe_engine* e, const float* emb_dev, int32_t n, float* out_dev);
int attn_reset(moe_engine* e);
// bytes of the linear-attention layers' conv + recurrence states (0 when attention is not configured), and a copy of
// them to (save) or from a device buffer of that size, enqueued on the engine's stream
size_t attn_state_bytes(const moe_engine* e);
int attn_state_io(moe_engine* e, int layer, int which, float* host, int64_t floats, bool to_device);
int attn_state_copy(moe_engine* e, uint8_t* buf, bool save);
void attn_destroy(moe_engine* e);
int head_reserve(moe_engine* e, int32_t n);
void head_destroy(moe_engine* e);
int refresh_layer_table(moe_engine* e);
int check_layer_ready(moe_engine* e, int layer);

#ifdef __CUDACC__
// ─── device helpers ─────────────────────────────────────────────────────────

__device__ __forceinline__ float bf16_bits_to_f32(uint16_t v) {
    return __uint_as_float(((uint32_t)v) << 16);
}

// The reference's f32 -> bf16 (src/dtype.rs:85-89): round_up = bit15 & (bit0 | bit16).
// Not round-to-nearest-even; reproduced bit for bit.
__device__ __forceinline__ uint16_t f32_to_bf16_ref(float v) {
    uint32_t bits = __float_as_uint(v);
    uint32_t round_up = ((bits >> 15) & 1u) & ((bits & 0x7FFFu) | ((bits >> 16) & 1u));
    return (uint16_t)((bits + (round_up << 16)) >> 16);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// 128-bit read-only streaming load (weights are read once per token).
__device__ __forceinline__ uint4 ld_stream_u4(const void* p) {
    uint4 r;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
                 : "l"(p));
    return r;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

// Programmatic dependent launch.  A kernel launched with the attribute (launch_kernel below, pdl = true) may start
// while the kernel before it in the stream is still running.  The rule every kernel of such a chain keeps: before
// pdl_wait() it touches only bytes that no kernel writes (weights) and its own shared memory; pdl_wait() returns once
// the preceding kernel has completed and its writes are visible, and since that kernel waited in the same way, so has
// everything before it.  pdl_trigger() lets the next kernel of the chain become resident; both are no-ops in a
// kernel launched the ordinary way.  A pointer to what an earlier kernel of the chain wrote must not be declared
// `const __restrict__`: the compiler then treats it as read-only for the whole kernel and may move its loads above
// the wait (seen: a kernel resident early read its predecessor's output buffer before that had been written).
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// 16 bytes of a predecessor's output, read where the code says (never moved above the wait)
__device__ __forceinline__ float4 ld_dep_f4(const float4* p) {
    float4 v;
    asm volatile("ld.global.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
#endif

// Kernel launch with or without the programmatic-dependent-launch attribute (see pdl_wait above).
template <typename... P, typename... A>
inline cudaError_t launch_kernel(bool pdl, void (*kernel)(P...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, A&&... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, P(args)...);
}

}  // namespace moe
