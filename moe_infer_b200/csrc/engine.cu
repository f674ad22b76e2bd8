// Engine lifetime, the HBM-resident expert store and the C ABI glue.
//
// Replaces the reference's device context and expert I/O
// (src/engine/qwen35_moe/metal_context.rs:25-182, 558-600; src/model/expert.rs:29-66)
// with: one CUDA stream, one allocation per layer holding all E packed experts,
// one allocation per layer for the non-expert tensors, and persistent work areas.
#include <stdarg.h>
#include <string.h>

#include <atomic>
#include <chrono>

#include "common.cuh"
#include "decode_common.cuh"

namespace moe {

static thread_local char g_err[1024] = "";
static std::atomic<int> g_record_telemetry{0};

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

int cuda_fail(cudaError_t err, const char* what, const char* file, int line) {
    set_error("CUDA error %d (%s) at %s:%d: %s", (int)err, cudaGetErrorString(err), file, line, what);
    return MOE_ERR_CUDA;
}

static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

static void layout(int hd, int mi, int gs, moe_expert_layout_t* L) {
    const int64_t gate_w = (int64_t)mi * hd / 2;
    const int64_t gate_sb = (int64_t)mi * (hd / gs) * 2;
    const int64_t down_w = (int64_t)hd * mi / 2;
    const int64_t down_sb = (int64_t)hd * (mi / gs) * 2;
    L->gate_w = 0;
    L->gate_s = gate_w;
    L->gate_b = gate_w + gate_sb;
    L->up_w = gate_w + 2 * gate_sb;
    L->up_s = L->up_w + gate_w;
    L->up_b = L->up_s + gate_sb;
    L->down_w = L->up_b + gate_sb;
    L->down_s = L->down_w + down_w;
    L->down_b = L->down_s + down_sb;
    L->expert_size = L->down_b + down_sb;
}

// Offsets of the non-expert tensors inside a layer's aux allocation.
struct AuxLayout {
    size_t post_norm, router, sgate_w, sgate_s, sgate_b, shared, total;
    size_t router_s, router_b;  // INT4-scheme router
};

static AuxLayout aux_layout(const moe_engine* e) {
    const moe_dims_t& d = e->dims;
    AuxLayout a{};
    size_t off = 0;
    a.post_norm = off; off = align_up(off + (size_t)d.hidden * 2, 256);
    a.router = off;
    // room for the larger (bf16) form; the INT4 form uses a prefix of it
    const size_t router_bf16 = (size_t)d.num_experts * d.hidden * 2;
    a.router_s = a.router + align_up((size_t)d.num_experts * d.hidden / 2, 256);
    a.router_b = a.router_s + align_up((size_t)d.num_experts * (d.hidden / d.group) * 2, 256);
    off = align_up(off + router_bf16, 256);
    a.sgate_w = off; off = align_up(off + (size_t)d.hidden / 2, 256);
    a.sgate_s = off; off = align_up(off + (size_t)(d.hidden / d.group) * 2, 256);
    a.sgate_b = off; off = align_up(off + (size_t)(d.hidden / d.group) * 2, 256);
    a.shared = off; off = align_up(off + (size_t)e->shared_lay.expert_size, 256);
    a.total = off;
    return a;
}

static int ensure_layer(moe_engine* e, int layer) {
    MOE_REQUIRE(layer >= 0 && layer < (int)e->layers.size(), "layer %d out of range [0, %d)", layer,
                (int)e->layers.size());
    LayerHost& lh = e->layers[layer];
    const moe_dims_t& d = e->dims;
    if (!lh.experts) {
        const size_t bytes = (size_t)d.num_experts * e->lay.expert_size;
        MOE_CUDA(cudaMalloc(&lh.experts, bytes));
        e->resident += bytes;
        e->table_dirty = true;
    }
    if (!lh.aux) {
        const AuxLayout a = aux_layout(e);
        MOE_CUDA(cudaMalloc(&lh.aux, a.total));
        MOE_CUDA(cudaMemset(lh.aux, 0, a.total));
        e->resident += a.total;
        e->table_dirty = true;
    }
    return MOE_OK;
}

int refresh_layer_table(moe_engine* e) {
    if (!e->table_dirty) return MOE_OK;
    const AuxLayout a = aux_layout(e);
    std::vector<LayerDev> tab(e->layers.size());
    for (size_t l = 0; l < e->layers.size(); ++l) {
        LayerHost& lh = e->layers[l];
        LayerDev dv{};
        dv.experts = lh.experts;
        if (lh.aux) {
            dv.post_norm = (const uint16_t*)(lh.aux + a.post_norm);
            if (lh.router_is_bf16) {
                dv.router_bf16 = (const uint16_t*)(lh.aux + a.router);
            } else {
                dv.router_bf16 = nullptr;
                dv.router_q4.w = (const uint32_t*)(lh.aux + a.router);
                dv.router_q4.s = (const uint16_t*)(lh.aux + a.router_s);
                dv.router_q4.b = (const uint16_t*)(lh.aux + a.router_b);
            }
            dv.shared = lh.aux + a.shared;
            dv.sgate.w = (const uint32_t*)(lh.aux + a.sgate_w);
            dv.sgate.s = (const uint16_t*)(lh.aux + a.sgate_s);
            dv.sgate.b = (const uint16_t*)(lh.aux + a.sgate_b);
        }
        dv.router_planes = lh.planes_valid ? (const uint16_t*)lh.planes : nullptr;
        dv.router_nplanes = lh.router_is_bf16 ? 1 : 3;
        dv.router_t = lh.router_t_valid ? lh.router_t : nullptr;
        lh.dev = dv;
        tab[l] = dv;
    }
    // stream-ordered so that kernels already queued keep the table they were given
    MOE_CUDA(cudaMemcpyAsync(e->layers_dev, tab.data(), tab.size() * sizeof(LayerDev), cudaMemcpyHostToDevice,
                             e->stream));
    MOE_CUDA(cudaStreamSynchronize(e->stream));
    e->table_dirty = false;
    return MOE_OK;
}

int check_layer_ready(moe_engine* e, int layer) {
    if (layer < 0 || layer >= (int)e->layers.size()) {
        set_error("layer %d out of range [0, %d)", layer, (int)e->layers.size());
        return MOE_ERR_INVALID;
    }
    const LayerHost& lh = e->layers[layer];
    if (!lh.experts_loaded) {
        set_error("layer %d: packed experts not loaded", layer);
        return MOE_ERR_STATE;
    }
    static const char* names[6] = {"post_attention_layernorm", "mlp.gate", "shared_expert.gate_proj",
                                   "shared_expert.up_proj", "shared_expert.down_proj", "shared_expert_gate"};
    for (int r = 0; r < 6; ++r)
        if (!lh.role_loaded[r]) {
            set_error("layer %d: tensor %s not loaded", layer, names[r]);
            return MOE_ERR_STATE;
        }
    return MOE_OK;
}

// Enqueues the read of the device error word into pinned memory behind everything the call has launched, so that the
// call's own synchronisation covers it (a separate copy + synchronise afterwards cost a host call about 10 us).
static void error_read_enqueue(moe_engine* e) {
    unsigned int* dst = reinterpret_cast<unsigned int*>(e->stage_host + 2 * (size_t)e->dims.hidden);
    if (cudaMemcpyAsync(dst, e->dec_sync + 2, sizeof(unsigned int), cudaMemcpyDeviceToHost, e->stream) == cudaSuccess)
        e->err_read_pending = true;
}

// Reads and clears the device error word; maps it to a status.
static int poll_device_error(moe_engine* e) {
    unsigned int flag = 0;
    if (e->err_read_pending) {
        e->err_read_pending = false;
        MOE_CUDA(cudaStreamSynchronize(e->stream));  // returns at once when the caller has synchronised already
        flag = *reinterpret_cast<volatile unsigned int*>(e->stage_host + 2 * (size_t)e->dims.hidden);
    } else {
        MOE_CUDA(cudaMemcpyAsync(&flag, e->dec_sync + 2, sizeof(flag), cudaMemcpyDeviceToHost, e->stream));
        MOE_CUDA(cudaStreamSynchronize(e->stream));
    }
    if (flag != 0) {
        cudaMemsetAsync(e->dec_sync, 0, 16 * sizeof(unsigned int), e->stream);
        cudaStreamSynchronize(e->stream);
        decode_reset_after_error(e);
        if (flag == 11u) {
            set_error("a token id is outside [0, %d); the result of the last call is invalid", e->dims.vocab);
            return MOE_ERR_INVALID;
        }
        if (flag == 10u) {
            set_error("forced_idx holds an expert index outside [0, %d); the result of the last call is invalid",
                      e->dims.num_experts);
            return MOE_ERR_INVALID;
        }
        set_error("a bounded device-side wait gave up (code %u); the result of the last call is invalid", flag);
        return MOE_ERR_DEVICE_WAIT;
    }
    return MOE_OK;
}

// Persistent device staging for the host-pointer entry points (grown on demand,
// so steady-state calls allocate nothing).
static int io_reserve(moe_engine* e, size_t bytes) {
    if (bytes <= e->io_cap) return MOE_OK;
    MOE_CUDA(cudaStreamSynchronize(e->stream));
    if (e->io_dev) cudaFree(e->io_dev);
    e->io_dev = nullptr;
    e->io_cap = 0;
    const size_t cap = align_up(bytes + bytes / 4, 1 << 20);
    MOE_CUDA(cudaMalloc(&e->io_dev, cap));
    e->io_cap = cap;
    return MOE_OK;
}

static void tel_add(moe_engine* e, const char* key, double v) {
    if (g_record_telemetry.load(std::memory_order_relaxed)) e->telemetry[key] += v;
}

// The reference's per-phase keys (src/engine/qwen35_moe/fused_exp5.rs:162-177, 249, 378, 401, 412), as they map onto
// one call here: the host time spent enqueueing the stack (the reference's command-buffer encoding of the MoE half),
// the host time spent waiting for the stream (its wait for the hidden state), and the device time of final norm +
// lm_head.  The CPU routing and expert-read costs the reference also reports do not exist on this path: 0.
using host_time_t = std::chrono::steady_clock::time_point;
static void tel_phases(moe_engine_t* e, host_time_t t0, host_time_t t1, host_time_t t2, double lm_head_ms) {
    tel_add(e, "phase.op2_encode_ms", std::chrono::duration<double, std::milli>(t1 - t0).count());
    tel_add(e, "phase.hidden_wait_ms", std::chrono::duration<double, std::milli>(t2 - t1).count());
    tel_add(e, "phase.lm_head_ms", lm_head_ms);
    tel_add(e, "phase.route_cpu_ms", 0.0);
    tel_add(e, "engine.expert_io_ms", 0.0);
    tel_add(e, "engine.routing_cpu_ms", 0.0);
}

}  // namespace moe

using namespace moe;

extern "C" {

const char* moe_last_error(void) { return g_err; }
const char* moe_version(void) { return "moe_b200 0.1 (sm_100a)"; }

int moe_expert_layout(int32_t hidden, int32_t inter, int32_t group, moe_expert_layout_t* out) {
    MOE_REQUIRE(out && hidden > 0 && inter > 0 && group > 0 && hidden % group == 0 && inter % group == 0,
                "expert_layout: hidden and inter must be positive multiples of group");
    layout(hidden, inter, group, out);
    return MOE_OK;
}

int moe_engine_create(const moe_dims_t* dims, int device, moe_engine_t** out) {
    MOE_REQUIRE(dims && out, "engine_create: null argument");
    *out = nullptr;
    const moe_dims_t& d = *dims;
    MOE_REQUIRE(d.group == kGroup, "group size must be %d (got %d)", kGroup, d.group);
    MOE_REQUIRE(d.hidden > 0 && d.hidden % 256 == 0, "hidden (%d) must be a positive multiple of 256", d.hidden);
    MOE_REQUIRE(d.inter > 0 && d.inter % kGroup == 0 && d.shared_inter > 0 && d.shared_inter % kGroup == 0,
                "inter (%d) and shared_inter (%d) must be positive multiples of 64", d.inter, d.shared_inter);
    MOE_REQUIRE(d.num_experts > 0, "num_experts must be positive");
    // K <= MAX_K and K <= num_experts (reference metal_context.rs:564-577)
    MOE_REQUIRE(d.top_k >= 1 && d.top_k <= kMaxK, "num_active_experts (%d) must be in 1..%d", d.top_k, kMaxK);
    MOE_REQUIRE(d.top_k <= d.num_experts, "num_active_experts (%d) exceeds num_experts (%d)", d.top_k, d.num_experts);
    MOE_REQUIRE(d.num_layers >= 1 && d.num_mtp_layers >= 0 && d.num_mtp_layers <= 1, "bad layer counts %d + %d",
                d.num_layers, d.num_mtp_layers);
    MOE_REQUIRE(d.scheme == MOE_SCHEME_BQ4 || d.scheme == MOE_SCHEME_INT4, "unknown scheme %d", d.scheme);

    int n_dev = 0;
    MOE_CUDA(cudaGetDeviceCount(&n_dev));
    MOE_REQUIRE(device >= 0 && device < n_dev, "device %d out of range (%d CUDA devices)", device, n_dev);
    MOE_CUDA(cudaSetDevice(device));
    cudaDeviceProp prop;
    MOE_CUDA(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10) {
        set_error("device %d is sm_%d%d; this library is built for sm_100a only", device, prop.major, prop.minor);
        return MOE_ERR_CUDA;
    }
    moe_engine* e = new moe_engine();
    e->dims = d;
    e->device = device;
    e->sm_count = prop.multiProcessorCount;
    layout(d.hidden, d.inter, d.group, &e->lay);
    layout(d.hidden, d.shared_inter, d.group, &e->shared_lay);
    e->layers.resize((size_t)d.num_layers + d.num_mtp_layers);
    for (auto& lh : e->layers) lh.router_is_bf16 = (d.scheme == MOE_SCHEME_BQ4);
    e->last_h.assign(d.hidden, 0.0f);
    int rc = MOE_OK;
    do {
        if (cudaStreamCreateWithFlags(&e->stream, cudaStreamNonBlocking) != cudaSuccess ||
            cudaEventCreate(&e->ev0) != cudaSuccess || cudaEventCreate(&e->ev1) != cudaSuccess || cudaEventCreate(&e->ev2) != cudaSuccess ||
            cudaMalloc(&e->layers_dev, e->layers.size() * sizeof(LayerDev)) != cudaSuccess) {
            rc = cuda_fail(cudaGetLastError(), "engine resources", __FILE__, __LINE__);
            break;
        }
        rc = decode_init(e);
    } while (0);
    if (rc != MOE_OK) {
        moe_engine_destroy(e);
        return rc;
    }
    *out = e;
    return MOE_OK;
}

void moe_engine_destroy(moe_engine_t* e) {
    if (!e) return;
    cudaSetDevice(e->device);
    if (e->stream) cudaStreamSynchronize(e->stream);
    for (auto& lh : e->layers) {
        if (lh.experts) cudaFree(lh.experts);
        if (lh.aux) cudaFree(lh.aux);
        if (lh.planes) cudaFree(lh.planes);
        if (lh.router_t) cudaFree(lh.router_t);
    }
    moe_ep_finalize(e);
    decode_destroy(e);
    batch_destroy(e);
    head_destroy(e);
    mtp_destroy(e);
    attn_destroy(e);
    if (e->layers_dev) cudaFree(e->layers_dev);
    if (e->io_dev) cudaFree(e->io_dev);
    if (e->ev0) cudaEventDestroy(e->ev0);
    if (e->ev1) cudaEventDestroy(e->ev1);
    if (e->ev2) cudaEventDestroy(e->ev2);
    if (e->stream) cudaStreamDestroy(e->stream);
    delete e;
}

int moe_engine_sync(moe_engine_t* e) {
    MOE_REQUIRE(e, "null engine");
    MOE_CUDA(cudaStreamSynchronize(e->stream));
    return poll_device_error(e);
}

int moe_engine_dims(const moe_engine_t* e, moe_dims_t* out) {
    MOE_REQUIRE(e && out, "null argument");
    *out = e->dims;
    return MOE_OK;
}

// ── store ────────────────────────────────────────────────────────────────────

int moe_store_load_layer(moe_engine_t* e, int layer, const void* blob_host, size_t bytes) {
    MOE_REQUIRE(e && blob_host, "null argument");
    const size_t want = (size_t)e->dims.num_experts * e->lay.expert_size;
    // the reference rejects a short read of an expert (src/model/expert.rs:36-41)
    MOE_REQUIRE(bytes == want, "layer %d: blob is %zu bytes, expected num_experts * expert_size = %zu", layer, bytes, want);
    int rc = ensure_layer(e, layer);
    if (rc != MOE_OK) return rc;
    MOE_CUDA(cudaMemcpyAsync(e->layers[layer].experts, blob_host, bytes, cudaMemcpyHostToDevice, e->stream));
    MOE_CUDA(cudaStreamSynchronize(e->stream));
    e->layers[layer].experts_loaded = true;
    return MOE_OK;
}

int moe_store_layer_dev(moe_engine_t* e, int layer, void** blob_dev) {
    MOE_REQUIRE(e && blob_dev, "null argument");
    int rc = ensure_layer(e, layer);
    if (rc != MOE_OK) return rc;
    *blob_dev = e->layers[layer].experts;
    return MOE_OK;
}

int moe_store_mark_loaded(moe_engine_t* e, int layer) {
    MOE_REQUIRE(e && layer >= 0 && layer < (int)e->layers.size() && e->layers[layer].experts,
                "layer %d has no device blob", layer);
    e->layers[layer].experts_loaded = true;
    return MOE_OK;
}

int moe_store_load_tensor(moe_engine_t* e, int layer, int role, const void* w, const void* s, const void* b,
                          int dtype) {
    MOE_REQUIRE(e && w, "null argument");
    MOE_REQUIRE(role >= 0 && role <= MOE_T_SHARED_SGATE, "unknown tensor role %d", role);
    int rc = ensure_layer(e, layer);
    if (rc != MOE_OK) return rc;
    const moe_dims_t& d = e->dims;
    LayerHost& lh = e->layers[layer];
    const AuxLayout a = aux_layout(e);
    const moe_expert_layout_t& S = e->shared_lay;
    auto up = [&](size_t off, const void* src, size_t bytes) -> int {
        MOE_CUDA(cudaMemcpyAsync(lh.aux + off, src, bytes, cudaMemcpyHostToDevice, e->stream));
        return MOE_OK;
    };
    auto up_q4 = [&](size_t ow, size_t os, size_t ob, int rows, int cols) -> int {
        MOE_REQUIRE(dtype == MOE_DT_INT4 && s && b, "role %d needs an INT4 triple (weight, scales, biases)", role);
        int r1 = up(ow, w, (size_t)rows * cols / 2);
        if (r1) return r1;
        r1 = up(os, s, (size_t)rows * (cols / d.group) * 2);
        if (r1) return r1;
        return up(ob, b, (size_t)rows * (cols / d.group) * 2);
    };
    switch (role) {
        case MOE_T_POST_NORM:
            MOE_REQUIRE(dtype == MOE_DT_BF16, "post-attention norm weight must be bf16");
            rc = up(a.post_norm, w, (size_t)d.hidden * 2);
            break;
        case MOE_T_ROUTER:
            if (dtype == MOE_DT_BF16) {
                rc = up(a.router, w, (size_t)d.num_experts * d.hidden * 2);
                lh.router_is_bf16 = true;
            } else {
                rc = up_q4(a.router, a.router_s, a.router_b, d.num_experts, d.hidden);
                lh.router_is_bf16 = false;
            }
            e->table_dirty = true;
            lh.planes_valid = false;  // rebuilt from the new router on the next batched call
            lh.router_t_valid = false;
            break;
        case MOE_T_SHARED_GATE:
            rc = up_q4(a.shared + S.gate_w, a.shared + S.gate_s, a.shared + S.gate_b, d.shared_inter, d.hidden);
            break;
        case MOE_T_SHARED_UP:
            rc = up_q4(a.shared + S.up_w, a.shared + S.up_s, a.shared + S.up_b, d.shared_inter, d.hidden);
            break;
        case MOE_T_SHARED_DOWN:
            rc = up_q4(a.shared + S.down_w, a.shared + S.down_s, a.shared + S.down_b, d.hidden, d.shared_inter);
            break;
        case MOE_T_SHARED_SGATE:
            rc = up_q4(a.sgate_w, a.sgate_s, a.sgate_b, 1, d.hidden);
            break;
    }
    if (rc != MOE_OK) return rc;
    MOE_CUDA(cudaStreamSynchronize(e->stream));
    lh.role_loaded[role] = true;
    // the decode kernel reads the router transposed: build that copy now, off the first token's path
    if (role == MOE_T_ROUTER) return ensure_router_t(e, layer);
    return MOE_OK;
}

int moe_store_bytes(const moe_engine_t* e, size_t* resident_bytes) {
    MOE_REQUIRE(e && resident_bytes, "null argument");
    *resident_bytes = e->resident;
    return MOE_OK;
}

// ── packer ───────────────────────────────────────────────────────────────────

static int check_pack_args(const void* src, int src_dtype, int64_t rows, int32_t cols) {
    MOE_REQUIRE(src, "pack: null source");
    MOE_REQUIRE(src_dtype == MOE_DT_F32 || src_dtype == MOE_DT_BF16, "pack: source dtype must be f32 or bf16");
    MOE_REQUIRE(rows >= 0 && cols > 0 && cols % kGroup == 0, "pack: cols (%d) must be a positive multiple of 64", cols);
    return MOE_OK;
}

int moe_pack_int4_dev(moe_engine_t* e, const void* src, int src_dtype, int64_t rows, int32_t cols, void* w,
                      void* s, void* b) {
    MOE_REQUIRE(e && w && s && b, "null argument");
    int rc = check_pack_args(src, src_dtype, rows, cols);
    if (rc) return rc;
    MOE_REQUIRE((((uintptr_t)src) & 15) == 0, "pack: source must be 16-byte aligned");
    return launch_pack(e, src, src_dtype, rows, cols, cols, w, s, b);
}

int moe_pack_int4_host(moe_engine_t* e, const void* src, int src_dtype, int64_t rows, int32_t cols, void* w,
                       void* s, void* b) {
    MOE_REQUIRE(e && w && s && b, "null argument");
    int rc = check_pack_args(src, src_dtype, rows, cols);
    if (rc) return rc;
    if (rows == 0) return MOE_OK;
    const size_t esz = src_dtype == MOE_DT_F32 ? 4 : 2;
    const size_t n = (size_t)rows * cols;
    const size_t wb = n / 2, sb = n / kGroup * 2;
    uint8_t* dsrc = nullptr;
    uint8_t* dout = nullptr;
    const size_t sb_al = align_up(sb, 256), wb_al = align_up(wb, 256);
    if (cudaMalloc(&dsrc, n * esz) != cudaSuccess || cudaMalloc(&dout, wb_al + 2 * sb_al) != cudaSuccess) {
        cudaFree(dsrc);
        return cuda_fail(cudaGetLastError(), "pack_int4_host: device staging", __FILE__, __LINE__);
    }
    rc = MOE_OK;
    do {
        if (cudaMemcpyAsync(dsrc, src, n * esz, cudaMemcpyHostToDevice, e->stream) != cudaSuccess) { rc = MOE_ERR_CUDA; break; }
        rc = launch_pack(e, dsrc, src_dtype, rows, cols, cols, dout, dout + wb_al, dout + wb_al + sb_al);
        if (rc) break;
        if (cudaMemcpyAsync(w, dout, wb, cudaMemcpyDeviceToHost, e->stream) != cudaSuccess ||
            cudaMemcpyAsync(s, dout + wb_al, sb, cudaMemcpyDeviceToHost, e->stream) != cudaSuccess ||
            cudaMemcpyAsync(b, dout + wb_al + sb_al, sb, cudaMemcpyDeviceToHost, e->stream) != cudaSuccess ||
            cudaStreamSynchronize(e->stream) != cudaSuccess)
            rc = MOE_ERR_CUDA;
    } while (0);
    if (rc == MOE_ERR_CUDA) cuda_fail(cudaGetLastError(), "pack_int4_host", __FILE__, __LINE__);
    cudaFree(dsrc);
    cudaFree(dout);
    return rc;
}

int moe_pack_int8_host(moe_engine_t* e, const void* src, int src_dtype, int64_t rows, int32_t cols, void* q, void* scales) {
    MOE_REQUIRE(e && src && q && scales, "null argument");
    MOE_REQUIRE(src_dtype == MOE_DT_F32 || src_dtype == MOE_DT_BF16, "pack: source dtype must be f32 or bf16");
    MOE_REQUIRE(rows >= 0 && cols > 0, "pack_int8: bad shape");
    if (rows == 0) return MOE_OK;
    const size_t esz = src_dtype == MOE_DT_F32 ? 4 : 2, n = (size_t)rows * cols;
    uint8_t* d = nullptr;
    const size_t so = align_up(n * esz, 256), qo = so + align_up(n, 256);
    MOE_CUDA(cudaMalloc(&d, qo + (size_t)rows * 4));
    int rc = MOE_OK;
    do {
        if (cudaMemcpyAsync(d, src, n * esz, cudaMemcpyHostToDevice, e->stream) != cudaSuccess) { rc = MOE_ERR_CUDA; break; }
        rc = launch_pack_int8(e, d, src_dtype, rows, cols, d + so, d + qo);
        if (rc) break;
        if (cudaMemcpyAsync(q, d + so, n, cudaMemcpyDeviceToHost, e->stream) != cudaSuccess ||
            cudaMemcpyAsync(scales, d + qo, (size_t)rows * 4, cudaMemcpyDeviceToHost, e->stream) != cudaSuccess ||
            cudaStreamSynchronize(e->stream) != cudaSuccess)
            rc = MOE_ERR_CUDA;
    } while (0);
    if (rc == MOE_ERR_CUDA) cuda_fail(cudaGetLastError(), "pack_int8_host", __FILE__, __LINE__);
    cudaFree(d);
    return rc;
}

int moe_pack_experts_dev(moe_engine_t* e, const void* gate_up, const void* down, int src_dtype, int32_t n_experts,
                         void* blob) {
    MOE_REQUIRE(e && gate_up && down && blob, "null argument");
    MOE_REQUIRE(src_dtype == MOE_DT_F32 || src_dtype == MOE_DT_BF16, "pack: source dtype must be f32 or bf16");
    MOE_REQUIRE(n_experts >= 0, "pack: negative expert count");
    MOE_REQUIRE((((uintptr_t)gate_up) & 15) == 0 && (((uintptr_t)down) & 15) == 0 && (((uintptr_t)blob) & 15) == 0,
                "pack: pointers must be 16-byte aligned");
    return launch_pack_experts(e, gate_up, down, src_dtype, n_experts, blob);
}

int moe_pack_experts_host(moe_engine_t* e, const void* gate_up, const void* down, int src_dtype, int32_t n_experts,
                          void* blob) {
    MOE_REQUIRE(e && gate_up && down && blob, "null argument");
    MOE_REQUIRE(src_dtype == MOE_DT_F32 || src_dtype == MOE_DT_BF16, "pack: source dtype must be f32 or bf16");
    MOE_REQUIRE(n_experts >= 0, "pack: negative expert count");
    if (n_experts == 0) return MOE_OK;
    const moe_dims_t& d = e->dims;
    const size_t esz = src_dtype == MOE_DT_F32 ? 4 : 2;
    const size_t gu_b = (size_t)n_experts * 2 * d.inter * d.hidden * esz;
    const size_t dn_b = (size_t)n_experts * d.hidden * d.inter * esz;
    const size_t out_b = (size_t)n_experts * e->lay.expert_size;
    uint8_t *dgu = nullptr, *ddn = nullptr, *dblob = nullptr;
    if (cudaMalloc(&dgu, gu_b) != cudaSuccess || cudaMalloc(&ddn, dn_b) != cudaSuccess ||
        cudaMalloc(&dblob, out_b) != cudaSuccess) {
        cudaFree(dgu); cudaFree(ddn);
        return cuda_fail(cudaGetLastError(), "pack_experts_host: device staging", __FILE__, __LINE__);
    }
    int rc = MOE_OK;
    do {
        if (cudaMemcpyAsync(dgu, gate_up, gu_b, cudaMemcpyHostToDevice, e->stream) != cudaSuccess ||
            cudaMemcpyAsync(ddn, down, dn_b, cudaMemcpyHostToDevice, e->stream) != cudaSuccess) { rc = MOE_ERR_CUDA; break; }
        rc = launch_pack_experts(e, dgu, ddn, src_dtype, n_experts, dblob);
        if (rc) break;
        if (cudaMemcpyAsync(blob, dblob, out_b, cudaMemcpyDeviceToHost, e->stream) != cudaSuccess ||
            cudaStreamSynchronize(e->stream) != cudaSuccess)
            rc = MOE_ERR_CUDA;
    } while (0);
    if (rc == MOE_ERR_CUDA) cuda_fail(cudaGetLastError(), "pack_experts_host", __FILE__, __LINE__);
    cudaFree(dgu); cudaFree(ddn); cudaFree(dblob);
    return rc;
}

// ── matvec ───────────────────────────────────────────────────────────────────

int moe_matvec_int4_dev(moe_engine_t* e, const void* w, const void* s, const void* b, const float* x, float* y,
                        int32_t rows, int32_t cols) {
    MOE_REQUIRE(e && w && s && b && x && y, "null argument");
    return launch_matvec(e, w, s, b, x, y, rows, cols);
}

int moe_matvec_int4_host(moe_engine_t* e, const void* w, const void* s, const void* b, const float* x, float* y,
                         int32_t rows, int32_t cols) {
    MOE_REQUIRE(e && w && s && b && x && y, "null argument");
    MOE_REQUIRE(rows > 0 && cols > 0 && cols % kGroup == 0, "matvec: cols (%d) must be a positive multiple of 64", cols);
    const size_t wb = align_up((size_t)rows * cols / 2, 256), sb = align_up((size_t)rows * (cols / kGroup) * 2, 256);
    const size_t xb = align_up((size_t)cols * 4, 256), yb = (size_t)rows * 4;
    uint8_t* d = nullptr;
    MOE_CUDA(cudaMalloc(&d, wb + 2 * sb + xb + yb));
    int rc = MOE_OK;
    do {
        if (cudaMemcpyAsync(d, w, (size_t)rows * cols / 2, cudaMemcpyHostToDevice, e->stream) != cudaSuccess ||
            cudaMemcpyAsync(d + wb, s, (size_t)rows * (cols / kGroup) * 2, cudaMemcpyHostToDevice, e->stream) != cudaSuccess ||
            cudaMemcpyAsync(d + wb + sb, b, (size_t)rows * (cols / kGroup) * 2, cudaMemcpyHostToDevice, e->stream) != cudaSuccess ||
            cudaMemcpyAsync(d + wb + 2 * sb, x, (size_t)cols * 4, cudaMemcpyHostToDevice, e->stream) != cudaSuccess) {
            rc = cuda_fail(cudaGetLastError(), "matvec_int4_host upload", __FILE__, __LINE__);
            break;
        }
        rc = launch_matvec(e, d, d + wb, d + wb + sb, (const float*)(d + wb + 2 * sb), (float*)(d + wb + 2 * sb + xb), rows, cols);
        if (rc) break;
        if (cudaMemcpyAsync(y, d + wb + 2 * sb + xb, yb, cudaMemcpyDeviceToHost, e->stream) != cudaSuccess ||
            cudaStreamSynchronize(e->stream) != cudaSuccess) {
            rc = cuda_fail(cudaGetLastError(), "matvec_int4_host download", __FILE__, __LINE__);
            break;
        }
        rc = poll_device_error(e);
    } while (0);
    cudaFree(d);
    return rc;
}

// ── one MoE block ────────────────────────────────────────────────────────────

// A single-layer decode call launches its kernel as a programmatic dependent of whatever kernel precedes it in the stream:
// back-to-back layer calls overlap the next call's launch, layer table and router fetch with the tail of the one before
// (16.5 -> 14.0 us per call; the kernel waits before it reads its input; a predecessor that never signals simply completes
// first).  Such a launch is an ordinary one, not a cooperative one (a cooperative grid only starts on a drained device):
// see launch_decode_slots for why its CTAs are co-resident all the same.  MOE_B200_DECODE_PDL=0: the cooperative launch.
// The whole-stack launches stay cooperative: one launch per token gains nothing from starting early (445 against 448 us).
static bool decode_pdl() {
    static const bool on = [] { const char* v = getenv("MOE_B200_DECODE_PDL"); return !(v && atoi(v) == 0); }();
    return on;
}

int moe_layer_forward_dev(moe_engine_t* e, int layer, const float* h_in, int32_t n, float* h_out,
                          const float* logit_bias, const int32_t* forced_idx, int32_t* out_idx, float* out_w) {
    MOE_REQUIRE(e && h_in && h_out, "null argument");
    MOE_REQUIRE(n >= 0, "negative token count");
    if (n == 0) return MOE_OK;
    if (n == 1) return launch_decode(e, layer, layer + 1, h_in, h_out, logit_bias, forced_idx, out_idx, out_w, decode_pdl());
    return launch_batched_layer(e, layer, h_in, n, h_out, logit_bias, forced_idx, out_idx, out_w);
}

int moe_layer_forward_host(moe_engine_t* e, int layer, const float* h_in, int32_t n, float* h_out,
                           const float* logit_bias, const int32_t* forced_idx, int32_t* out_idx, float* out_w) {
    MOE_REQUIRE(e && h_in && h_out, "null argument");
    MOE_REQUIRE(n >= 0, "negative token count");
    if (n == 0) return MOE_OK;
    const moe_dims_t& d = e->dims;
    if (forced_idx)
        for (size_t i = 0; i < (size_t)n * d.top_k; ++i)
            MOE_REQUIRE(forced_idx[i] >= 0 && forced_idx[i] < d.num_experts,
                        "forced_idx[%zu] = %d is outside [0, %d)", i, forced_idx[i], d.num_experts);
    const size_t hb = (size_t)n * d.hidden * 4;
    const size_t hb_al = align_up(hb, 256);
    const size_t lb = align_up((size_t)d.num_experts * 4, 256);
    const size_t kb = align_up((size_t)n * d.top_k * 4, 256);
    int rc = io_reserve(e, 2 * hb_al + lb + 3 * kb);
    if (rc) return rc;
    uint8_t* dv = e->io_dev;
    float* d_in = (float*)dv;
    float* d_out = (float*)(dv + hb_al);
    float* d_lb = (float*)(dv + 2 * hb_al);
    int32_t* d_fi = (int32_t*)(dv + 2 * hb_al + lb);
    int32_t* d_oi = (int32_t*)(dv + 2 * hb_al + lb + kb);
    float* d_ow = (float*)(dv + 2 * hb_al + lb + 2 * kb);
    do {
        cudaError_t ce = cudaMemcpyAsync(d_in, h_in, hb, cudaMemcpyHostToDevice, e->stream);
        if (ce == cudaSuccess && logit_bias)
            ce = cudaMemcpyAsync(d_lb, logit_bias, (size_t)d.num_experts * 4, cudaMemcpyHostToDevice, e->stream);
        if (ce == cudaSuccess && forced_idx)
            ce = cudaMemcpyAsync(d_fi, forced_idx, (size_t)n * d.top_k * 4, cudaMemcpyHostToDevice, e->stream);
        if (ce != cudaSuccess) { rc = cuda_fail(ce, "layer_forward_host upload", __FILE__, __LINE__); break; }
        rc = moe_layer_forward_dev(e, layer, d_in, n, d_out, logit_bias ? d_lb : nullptr, forced_idx ? d_fi : nullptr,
                                   d_oi, d_ow);
        if (rc) break;
        ce = cudaMemcpyAsync(h_out, d_out, hb, cudaMemcpyDeviceToHost, e->stream);
        if (ce == cudaSuccess && out_idx)
            ce = cudaMemcpyAsync(out_idx, d_oi, (size_t)n * d.top_k * 4, cudaMemcpyDeviceToHost, e->stream);
        if (ce == cudaSuccess && out_w)
            ce = cudaMemcpyAsync(out_w, d_ow, (size_t)n * d.top_k * 4, cudaMemcpyDeviceToHost, e->stream);
        if (ce == cudaSuccess) error_read_enqueue(e);
        if (ce == cudaSuccess) ce = cudaStreamSynchronize(e->stream);
        if (ce != cudaSuccess) { rc = cuda_fail(ce, "layer_forward_host download", __FILE__, __LINE__); break; }
        rc = poll_device_error(e);
    } while (0);
    return rc;
}

// ── the stack ────────────────────────────────────────────────────────────────

int moe_forward_hidden_dev(moe_engine_t* e, const float* emb, int32_t n, int batched, float* out) {
    MOE_REQUIRE(e && emb && out, "null argument");
    MOE_REQUIRE(n >= 0, "negative token count");
    if (n == 0) return MOE_OK;
    const moe_dims_t& d = e->dims;
    if (!batched || n == 1) {
        // the reference's token-serial loop (fused_exp1.rs:937-984): one persistent launch per token
        for (int t = 0; t < n; ++t) {
            int rc = launch_decode(e, 0, d.num_layers, emb + (size_t)t * d.hidden, out + (size_t)t * d.hidden, nullptr,
                                   nullptr, nullptr, nullptr);
            if (rc) return rc;
        }
        return MOE_OK;
    }
    int rc = batch_reserve(e, n);
    if (rc) return rc;
    const float* cur = emb;
    for (int l = 0; l < d.num_layers; ++l) {
        float* nxt = (l == d.num_layers - 1) ? out : ((l & 1) ? e->bw.h_b : e->bw.h_a);
        rc = launch_batched_layer(e, l, cur, n, nxt, nullptr, nullptr, nullptr, nullptr);
        if (rc) return rc;
        cur = nxt;
    }
    return MOE_OK;
}

// The stack over device buffers, polling the caller between tokens (decode path) or layers (grouped path):
// the reference polls once per layer (fused_exp1.rs:966-968).
static int run_stack_checked(moe_engine* e, const float* d_in, int32_t n, int batched, moe_check_fn check, void* check_ctx,
                             float* d_out) {
    const moe_dims_t& d = e->dims;
    if (!check) return moe_forward_hidden_dev(e, d_in, n, batched, d_out);
    int rc = MOE_OK;
    if (!batched || n == 1) {
        for (int t = 0; t < n && rc == MOE_OK; ++t) {
            if (check(check_ctx)) { set_error("interrupted"); return MOE_ERR_INTERRUPTED; }
            rc = launch_decode(e, 0, d.num_layers, d_in + (size_t)t * d.hidden, d_out + (size_t)t * d.hidden, nullptr, nullptr,
                               nullptr, nullptr);
        }
        return rc;
    }
    rc = batch_reserve(e, n);
    if (rc) return rc;
    const float* cur = d_in;
    for (int l = 0; l < d.num_layers; ++l) {
        if (check(check_ctx)) { set_error("interrupted"); return MOE_ERR_INTERRUPTED; }
        float* nxt = (l == d.num_layers - 1) ? d_out : ((l & 1) ? e->bw.h_b : e->bw.h_a);
        rc = launch_batched_layer(e, l, cur, n, nxt, nullptr, nullptr, nullptr, nullptr);
        if (rc) return rc;
        cur = nxt;
    }
    return MOE_OK;
}

int moe_forward_hidden_host(moe_engine_t* e, const float* emb, int32_t n, int batched, int mtp, moe_check_fn check,
                            void* check_ctx, float* out) {
    (void)mtp;
    MOE_REQUIRE(e && emb && out, "null argument");
    MOE_REQUIRE(n >= 0, "negative token count");
    if (n == 0) return MOE_OK;
    const moe_dims_t& d = e->dims;
    const bool rec = g_record_telemetry.load(std::memory_order_relaxed) != 0;
    cudaEvent_t t0 = e->ev0, t1 = e->ev1;
    const size_t hb = (size_t)n * d.hidden * 4;
    int rc = io_reserve(e, 2 * align_up(hb, 256));
    if (rc) return rc;
    float* d_in = (float*)e->io_dev;
    float* d_out = (float*)(e->io_dev + align_up(hb, 256));
    do {
        const auto host_t0 = std::chrono::steady_clock::now();
        if (rec) cudaEventRecord(t0, e->stream);
        cudaError_t ce = cudaMemcpyAsync(d_in, emb, hb, cudaMemcpyHostToDevice, e->stream);
        if (ce != cudaSuccess) { rc = cuda_fail(ce, "forward_hidden upload", __FILE__, __LINE__); break; }
        rc = run_stack_checked(e, d_in, n, batched, check, check_ctx, d_out);
        if (rc) break;
        ce = cudaMemcpyAsync(out, d_out, hb, cudaMemcpyDeviceToHost, e->stream);
        if (rec && ce == cudaSuccess) ce = cudaEventRecord(t1, e->stream);
        const auto host_t1 = std::chrono::steady_clock::now();
        if (ce == cudaSuccess) error_read_enqueue(e);
        if (ce == cudaSuccess) ce = cudaStreamSynchronize(e->stream);
        const auto host_t2 = std::chrono::steady_clock::now();
        if (ce != cudaSuccess) { rc = cuda_fail(ce, "forward_hidden download", __FILE__, __LINE__); break; }
        rc = poll_device_error(e);
        if (rc) break;
        memcpy(e->last_h.data(), out + (size_t)(n - 1) * d.hidden, (size_t)d.hidden * 4);
        if (rec) {
            float ms = 0.0f;
            cudaEventElapsedTime(&ms, t0, t1);
            tel_add(e, "engine.total_ms", ms);
            tel_add(e, "engine.tokens", n);
            tel_phases(e, host_t0, host_t1, host_t2, 0.0);
        }
    } while (0);
    if (rc == MOE_ERR_INTERRUPTED) cudaStreamSynchronize(e->stream);
    return rc;
}

// ── the model head ───────────────────────────────────────────────────────────

int moe_head_load_tensor(moe_engine_t* e, int which, const void* w, const void* s, const void* b, int dtype) {
    MOE_REQUIRE(e, "null engine");
    return head_load_tensor(e, which, w, s, b, dtype);
}

int moe_embed_lookup_dev(moe_engine_t* e, const int64_t* ids_dev, int32_t n, float* out_dev) {
    MOE_REQUIRE(e && ids_dev && out_dev, "null argument");
    MOE_REQUIRE(n >= 0, "negative token count");
    if (n == 0) return MOE_OK;
    return launch_embed(e, ids_dev, n, out_dev);
}

int moe_embed_lookup_host(moe_engine_t* e, const int64_t* ids, int32_t n, float* out) {
    MOE_REQUIRE(e && ids && out, "null argument");
    MOE_REQUIRE(n >= 0, "negative token count");
    if (n == 0) return MOE_OK;
    const size_t hb = (size_t)n * e->dims.hidden * 4;
    int rc = io_reserve(e, align_up(hb, 256));
    if (rc) return rc;
    rc = head_reserve(e, n);
    if (rc) return rc;
    MOE_CUDA(cudaMemcpyAsync(e->head.ids, ids, (size_t)n * 8, cudaMemcpyHostToDevice, e->stream));
    rc = launch_embed(e, e->head.ids, n, (float*)e->io_dev);
    if (rc) return rc;
    MOE_CUDA(cudaMemcpyAsync(out, e->io_dev, hb, cudaMemcpyDeviceToHost, e->stream));
    MOE_CUDA(cudaStreamSynchronize(e->stream));
    return poll_device_error(e);
}

int moe_logits_dev(moe_engine_t* e, const float* hidden_dev, int32_t n, float* logits_dev) {
    MOE_REQUIRE(e && hidden_dev && logits_dev, "null argument");
    MOE_REQUIRE(n >= 0, "negative token count");
    if (n == 0) return MOE_OK;
    return launch_logits(e, hidden_dev, n, logits_dev);
}

int moe_logits_host(moe_engine_t* e, const float* hidden, int32_t n, float* logits) {
    MOE_REQUIRE(e && hidden && logits, "null argument");
    MOE_REQUIRE(n >= 0, "negative token count");
    if (n == 0) return MOE_OK;
    const moe_dims_t& d = e->dims;
    const size_t hb = align_up((size_t)n * d.hidden * 4, 256), lb = (size_t)n * d.vocab * 4;
    int rc = io_reserve(e, hb + align_up(lb, 256));
    if (rc) return rc;
    float* d_h = (float*)e->io_dev;
    float* d_l = (float*)(e->io_dev + hb);
    MOE_CUDA(cudaMemcpyAsync(d_h, hidden, (size_t)n * d.hidden * 4, cudaMemcpyHostToDevice, e->stream));
    rc = launch_logits(e, d_h, n, d_l);
    if (rc) return rc;
    MOE_CUDA(cudaMemcpyAsync(logits, d_l, lb, cudaMemcpyDeviceToHost, e->stream));
    MOE_CUDA(cudaStreamSynchronize(e->stream));
    return poll_device_error(e);
}

int moe_forward_host(moe_engine_t* e, const int64_t* ids, int32_t n, int batched, int mtp, moe_check_fn check, void* check_ctx,
                     float* logits) {
    (void)mtp;
    MOE_REQUIRE(e && ids && logits, "null argument");
    MOE_REQUIRE(n >= 0, "negative token count");
    if (n == 0) return MOE_OK;
    const moe_dims_t& d = e->dims;
    const bool rec = g_record_telemetry.load(std::memory_order_relaxed) != 0;
    const size_t hb = align_up((size_t)n * d.hidden * 4, 256), lb = (size_t)n * d.vocab * 4;
    int rc = io_reserve(e, 2 * hb + align_up(lb, 256));
    if (rc) return rc;
    rc = head_reserve(e, n);
    if (rc) return rc;
    float* d_in = (float*)e->io_dev;
    float* d_out = (float*)(e->io_dev + hb);
    float* d_l = (float*)(e->io_dev + 2 * hb);
    do {
        const auto host_t0 = std::chrono::steady_clock::now();
        if (rec) cudaEventRecord(e->ev0, e->stream);
        cudaError_t ce = cudaMemcpyAsync(e->head.ids, ids, (size_t)n * 8, cudaMemcpyHostToDevice, e->stream);
        if (ce != cudaSuccess) { rc = cuda_fail(ce, "forward upload", __FILE__, __LINE__); break; }
        rc = launch_embed(e, e->head.ids, n, d_in);
        if (rc) break;
        rc = run_stack_checked(e, d_in, n, batched, check, check_ctx, d_out);
        if (rc) break;
        if (rec) cudaEventRecord(e->ev2, e->stream);
        rc = launch_logits(e, d_out, n, d_l);
        if (rc) break;
        if (rec) cudaEventRecord(e->ev1, e->stream);
        ce = cudaMemcpyAsync(logits, d_l, lb, cudaMemcpyDeviceToHost, e->stream);
        if (ce == cudaSuccess)
            ce = cudaMemcpyAsync(e->stage_host, d_out + (size_t)(n - 1) * d.hidden, (size_t)d.hidden * 4, cudaMemcpyDeviceToHost, e->stream);
        const auto host_t1 = std::chrono::steady_clock::now();
        if (ce == cudaSuccess) error_read_enqueue(e);
        if (ce == cudaSuccess) ce = cudaStreamSynchronize(e->stream);
        const auto host_t2 = std::chrono::steady_clock::now();
        if (ce != cudaSuccess) { rc = cuda_fail(ce, "forward download", __FILE__, __LINE__); break; }
        rc = poll_device_error(e);
        if (rc) break;
        memcpy(e->last_h.data(), e->stage_host, (size_t)d.hidden * 4);
        if (rec) {
            float ms = 0.0f, head_ms = 0.0f;
            cudaEventElapsedTime(&ms, e->ev0, e->ev1);
            cudaEventElapsedTime(&head_ms, e->ev2, e->ev1);
            tel_add(e, "engine.total_ms", ms);
            tel_add(e, "engine.tokens", n);
            tel_phases(e, host_t0, host_t1, host_t2, head_ms);
        }
    } while (0);
    if (rc == MOE_ERR_INTERRUPTED) cudaStreamSynchronize(e->stream);
    return rc;
}

int moe_last_h_pre_norm(moe_engine_t* e, float* out) {
    MOE_REQUIRE(e && out, "null argument");
    memcpy(out, e->last_h.data(), e->last_h.size() * sizeof(float));
    return MOE_OK;
}

// ── MTP ──────────────────────────────────────────────────────────────────────

int moe_mtp_forward_host(moe_engine_t* e, const float* h_in, float* h_out) {
    MOE_REQUIRE(e && h_in && h_out, "null argument");
    if (e->dims.num_mtp_layers == 0) {
        set_error("model has no MTP block (mtp_num_hidden_layers == 0)");
        return MOE_ERR_STATE;
    }
    int rc = moe_layer_forward_host(e, e->dims.num_layers, h_in, 1, h_out, nullptr, nullptr, nullptr, nullptr);
    if (rc == MOE_OK) e->mtp_pos++;
    return rc;
}

int moe_mtp_configure(moe_engine_t* e, const moe_attn_dims_t* attn) {
    MOE_REQUIRE(e && attn, "null argument");
    return mtp_configure(e, attn);
}

int moe_mtp_load_tensor(moe_engine_t* e, int which, const void* w, const void* s, const void* b, int dtype) {
    MOE_REQUIRE(e, "null engine");
    return mtp_load_tensor(e, which, w, s, b, dtype);
}

int moe_mtp_step_host(moe_engine_t* e, const float* h_host, int64_t token_id, float* logits_host) {
    MOE_REQUIRE(e && h_host && logits_host, "null argument");
    const size_t lb = (size_t)e->dims.vocab * 4;
    int rc = io_reserve(e, align_up(lb, 256));
    if (rc) return rc;
    float* logits_dev = reinterpret_cast<float*>(e->io_dev);
    rc = mtp_step(e, h_host, token_id, logits_dev);
    if (rc) {
        cudaStreamSynchronize(e->stream);  // the inputs are the caller's: nothing of theirs may still be in flight
        return rc;
    }
    MOE_CUDA(cudaMemcpyAsync(logits_host, logits_dev, lb, cudaMemcpyDeviceToHost, e->stream));
    error_read_enqueue(e);
    MOE_CUDA(cudaStreamSynchronize(e->stream));
    rc = poll_device_error(e);
    if (rc == MOE_OK) e->mtp_pos++;
    return rc;
}

int moe_attn_configure(moe_engine_t* e, const moe_model_attn_dims_t* dims) {
    MOE_REQUIRE(e && dims, "null argument");
    return attn_configure(e, dims);
}

int moe_attn_load_tensor(moe_engine_t* e, int layer, int which, const void* w, const void* s, const void* b, int dtype) {
    MOE_REQUIRE(e, "null engine");
    return attn_load_tensor(e, layer, which, w, s, b, dtype);
}

int moe_model_reset(moe_engine_t* e) {
    MOE_REQUIRE(e, "null engine");
    int rc = attn_reset(e);
    if (rc) return rc;
    MOE_CUDA(cudaStreamSynchronize(e->stream));
    return MOE_OK;
}

int moe_model_pos(const moe_engine_t* e, int64_t* pos) {
    MOE_REQUIRE(e && pos, "null argument");
    *pos = e->attn.pos;
    return MOE_OK;
}

struct moe_snapshot {
    moe_engine_t* owner = nullptr;
    int64_t pos = 0, mtp_pos = 0;
    std::vector<float> last_h;
    uint8_t* dev = nullptr;   // conv + recurrence states of the linear-attention layers, back to back
    size_t bytes = 0;
};

int moe_model_snapshot(moe_engine_t* e, moe_snapshot_t** out) {
    MOE_REQUIRE(e && out, "null argument");
    MOE_CUDA(cudaSetDevice(e->device));
    moe_snapshot* s = new moe_snapshot();
    s->owner = e;
    s->pos = e->attn.pos;
    s->mtp_pos = e->mtp_pos;
    s->last_h = e->last_h;
    s->bytes = attn_state_bytes(e);
    if (s->bytes) {
        cudaError_t ce = cudaMalloc(&s->dev, s->bytes);
        if (ce != cudaSuccess) { delete s; return cuda_fail(ce, "snapshot allocation", __FILE__, __LINE__); }
        int rc = attn_state_copy(e, s->dev, true);
        if (rc == MOE_OK && cudaStreamSynchronize(e->stream) != cudaSuccess) rc = MOE_ERR_CUDA;
        if (rc) { cudaFree(s->dev); delete s; return rc; }
    }
    *out = s;
    return MOE_OK;
}

int moe_model_restore(moe_engine_t* e, const moe_snapshot_t* s) {
    MOE_REQUIRE(e && s, "null argument");
    MOE_REQUIRE(s->owner == e && s->bytes == attn_state_bytes(e), "the snapshot was taken from another engine or configuration");
    if (s->bytes) {
        int rc = attn_state_copy(e, s->dev, false);
        if (rc) return rc;
        MOE_CUDA(cudaStreamSynchronize(e->stream));
    }
    e->attn.pos = s->pos;
    e->mtp_pos = s->mtp_pos;
    e->last_h = s->last_h;
    return MOE_OK;
}

void moe_model_snapshot_free(moe_snapshot_t* s) {
    if (!s) return;
    if (s->dev) cudaFree(s->dev);
    delete s;
}

int moe_model_state_host(moe_engine_t* e, int32_t layer, int32_t which, float* host, int64_t floats, int32_t to_device) {
    MOE_REQUIRE(e, "null engine");
    MOE_CUDA(cudaSetDevice(e->device));
    return attn_state_io(e, layer, which, host, floats, to_device != 0);
}

int moe_model_set_pos(moe_engine_t* e, int64_t pos) {
    MOE_REQUIRE(e, "null engine");
    MOE_REQUIRE(e->attn.configured, "the attention halves are not configured (moe_attn_configure)");
    MOE_REQUIRE(pos >= 0 && pos <= e->attn.d.full.max_seq, "position %lld outside [0, %d]", (long long)pos, e->attn.d.full.max_seq);
    e->attn.pos = pos;
    return MOE_OK;
}

// n decode steps with attention; ids != null: embed first and return logits, else emb in and hidden states out
static int model_forward(moe_engine_t* e, const int64_t* ids, const float* emb, int32_t n, float* out, bool logits) {
    MOE_REQUIRE(n >= 0, "negative token count");
    if (n == 0) return MOE_OK;
    const moe_dims_t& d = e->dims;
    const size_t hb = align_up((size_t)n * d.hidden * 4, 256), lb = logits ? align_up((size_t)n * d.vocab * 4, 256) : 0;
    int rc = io_reserve(e, 2 * hb + lb);
    if (rc) return rc;
    float* d_in = (float*)e->io_dev;
    float* d_out = (float*)(e->io_dev + hb);
    float* d_l = (float*)(e->io_dev + 2 * hb);
    const int64_t pos0 = e->attn.pos;
    const bool rec = g_record_telemetry.load(std::memory_order_relaxed) != 0;
    host_time_t host_t0{}, host_t1{};
    if (rec) host_t0 = std::chrono::steady_clock::now();
    do {
        if (ids) {
            if ((rc = head_reserve(e, n))) break;
            cudaError_t ce = cudaMemcpyAsync(e->head.ids, ids, (size_t)n * 8, cudaMemcpyHostToDevice, e->stream);
            if (ce != cudaSuccess) { rc = cuda_fail(ce, "model forward upload", __FILE__, __LINE__); break; }
            if ((rc = launch_embed(e, e->head.ids, n, d_in))) break;
        } else {
            cudaError_t ce = cudaMemcpyAsync(d_in, emb, (size_t)n * d.hidden * 4, cudaMemcpyHostToDevice, e->stream);
            if (ce != cudaSuccess) { rc = cuda_fail(ce, "model forward upload", __FILE__, __LINE__); break; }
        }
        if ((rc = attn_model_forward(e, d_in, n, d_out))) break;
        if (rec) host_t1 = std::chrono::steady_clock::now();  // everything is enqueued; the copies below wait for the stream
        cudaError_t ce;
        if (logits) {
            if ((rc = launch_logits(e, d_out, n, d_l))) break;
            ce = cudaMemcpyAsync(out, d_l, (size_t)n * d.vocab * 4, cudaMemcpyDeviceToHost, e->stream);
        } else {
            ce = cudaMemcpyAsync(out, d_out, (size_t)n * d.hidden * 4, cudaMemcpyDeviceToHost, e->stream);
        }
        if (ce == cudaSuccess)
            ce = cudaMemcpyAsync(e->stage_host, d_out + (size_t)(n - 1) * d.hidden, (size_t)d.hidden * 4, cudaMemcpyDeviceToHost, e->stream);
        if (ce == cudaSuccess) error_read_enqueue(e);
        if (ce == cudaSuccess) ce = cudaStreamSynchronize(e->stream);
        if (ce != cudaSuccess) { rc = cuda_fail(ce, "model forward download", __FILE__, __LINE__); break; }
        if ((rc = poll_device_error(e))) break;
        memcpy(e->last_h.data(), e->stage_host, (size_t)d.hidden * 4);
        if (rec) tel_phases(e, host_t0, host_t1, std::chrono::steady_clock::now(), 0.0);  // enqueue time, then the wait for the stream
    } while (0);
    if (rc) {
        cudaStreamSynchronize(e->stream);
        e->attn.pos = pos0;  // a failed call consumes no positions (the recurrence states may have moved: reset to reuse)
    }
    return rc;
}

int moe_model_forward_hidden_host(moe_engine_t* e, const float* emb, int32_t n, float* out) {
    MOE_REQUIRE(e && emb && out, "null argument");
    return model_forward(e, nullptr, emb, n, out, false);
}

int moe_model_forward_host(moe_engine_t* e, const int64_t* ids, int32_t n, float* logits) {
    MOE_REQUIRE(e && ids && logits, "null argument");
    return model_forward(e, ids, nullptr, n, logits, true);
}

int moe_mtp_reset(moe_engine_t* e) {
    MOE_REQUIRE(e, "null engine");
    e->mtp_pos = 0;
    return MOE_OK;
}

int moe_mtp_rollback(moe_engine_t* e, int64_t pos) {
    MOE_REQUIRE(e, "null engine");
    MOE_REQUIRE(pos >= 0, "negative position");
    if (pos < e->mtp_pos) e->mtp_pos = pos;
    return MOE_OK;
}

int moe_mtp_pos(const moe_engine_t* e, int64_t* pos) {
    MOE_REQUIRE(e && pos, "null argument");
    *pos = e->mtp_pos;
    return MOE_OK;
}

// ── telemetry ────────────────────────────────────────────────────────────────

void moe_set_record_telemetry(int on) { g_record_telemetry.store(on ? 1 : 0, std::memory_order_relaxed); }
int moe_get_record_telemetry(void) { return g_record_telemetry.load(std::memory_order_relaxed); }

int moe_telemetry_get(moe_engine_t* e, const char** keys, double* vals, int* n) {
    MOE_REQUIRE(e && n, "null argument");
    const int cap = *n;
    if (e->dec_sl_prefetch) {
        // the expert-prefetch predictor's record (the reference logs hits and misses of its own, expert_prefetch.rs:95-135)
        double checks = 0.0, hits = 0.0;
        int rc = slots_decode_prefetch_stats(e, &checks, &hits);
        if (rc) return rc;
        e->telemetry["prefetch.checks"] = checks;
        e->telemetry["prefetch.hits"] = hits;
    }
    e->tel_keys.clear();
    for (auto& kv : e->telemetry) e->tel_keys.push_back(kv.first);
    int i = 0;
    for (auto& kv : e->telemetry) {
        if (i < cap && keys && vals) {
            keys[i] = e->tel_keys[i].c_str();
            vals[i] = kv.second;
        }
        ++i;
    }
    *n = i;
    return MOE_OK;
}

// ── decode phase profile ─────────────────────────────────────────────────────

int moe_decode_profile(moe_engine_t* e, int enable, int64_t* stamps, int max_layers, int* points_per_layer) {
    MOE_REQUIRE(e, "null engine");
    if (!stamps) return decode_profile_enable(e, enable != 0);
    MOE_REQUIRE(points_per_layer && max_layers > 0, "null argument");
    return decode_profile_read(e, (long long*)stamps, max_layers, points_per_layer);
}

// ── device-memory helpers ────────────────────────────────────────────────────

int moe_dev_alloc(moe_engine_t* e, size_t bytes, void** out) {
    MOE_REQUIRE(e && out, "null argument");
    MOE_CUDA(cudaSetDevice(e->device));
    MOE_CUDA(cudaMalloc(out, bytes ? bytes : 1));
    return MOE_OK;
}
int moe_dev_free(moe_engine_t* e, void* p) {
    MOE_REQUIRE(e, "null engine");
    MOE_CUDA(cudaStreamSynchronize(e->stream));
    MOE_CUDA(cudaFree(p));
    return MOE_OK;
}
int moe_dev_upload(moe_engine_t* e, void* dst, const void* src, size_t bytes) {
    MOE_REQUIRE(e && (bytes == 0 || (dst && src)), "null argument");
    MOE_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, e->stream));
    MOE_CUDA(cudaStreamSynchronize(e->stream));
    return MOE_OK;
}
int moe_dev_download(moe_engine_t* e, void* dst, const void* src, size_t bytes) {
    MOE_REQUIRE(e && (bytes == 0 || (dst && src)), "null argument");
    MOE_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, e->stream));
    MOE_CUDA(cudaStreamSynchronize(e->stream));
    return MOE_OK;
}
int moe_dev_memset(moe_engine_t* e, void* dst, int value, size_t bytes) {
    MOE_REQUIRE(e && (bytes == 0 || dst), "null argument");
    MOE_CUDA(cudaMemsetAsync(dst, value, bytes, e->stream));
    return MOE_OK;
}
int moe_host_alloc_pinned(size_t bytes, void** out) {
    MOE_REQUIRE(out, "null argument");
    MOE_CUDA(cudaMallocHost(out, bytes ? bytes : 1));
    return MOE_OK;
}
int moe_host_free_pinned(void* p) {
    MOE_CUDA(cudaFreeHost(p));
    return MOE_OK;
}
int moe_timer_start(moe_engine_t* e) {
    MOE_REQUIRE(e, "null engine");
    MOE_CUDA(cudaEventRecord(e->ev0, e->stream));
    return MOE_OK;
}
int moe_timer_stop(moe_engine_t* e, float* ms) {
    MOE_REQUIRE(e && ms, "null argument");
    MOE_CUDA(cudaEventRecord(e->ev1, e->stream));
    MOE_CUDA(cudaEventSynchronize(e->ev1));
    MOE_CUDA(cudaEventElapsedTime(ms, e->ev0, e->ev1));
    return MOE_OK;
}
int moe_launch_count(const moe_engine_t* e, int64_t* n) {
    MOE_REQUIRE(e && n, "null argument");
    *n = e->launches;
    return MOE_OK;
}

}  // extern "C"
