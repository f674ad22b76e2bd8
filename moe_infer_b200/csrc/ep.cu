// Expert parallelism over the GPUs of one box: set-up of the buffers the ranks
// map from one another (CUDA IPC) and the collective entry points.  No counterpart
// in the reference, which drives a single device.  The per-layer kernels live in
// grouped.cu (ep_layer).
#include <string.h>

#include "common.cuh"

using namespace moe;

static size_t al256(size_t v) { return (v + 255) / 256 * 256; }

extern "C" {

int moe_ep_export(moe_engine_t* e, int rank, int world, int32_t max_tokens_per_rank, void* handle_out) {
    MOE_REQUIRE(e && handle_out, "null argument");
    const moe_dims_t& d = e->dims;
    MOE_REQUIRE(world >= 1 && world <= kEpMaxWorld && rank >= 0 && rank < world, "bad rank %d / world %d (at most %d ranks)",
                rank, world, kEpMaxWorld);
    MOE_REQUIRE(d.num_experts % world == 0, "num_experts (%d) must be divisible by the number of ranks (%d)", d.num_experts, world);
    MOE_REQUIRE(max_tokens_per_rank >= 1, "max_tokens_per_rank must be positive");
    MOE_REQUIRE(d.num_experts <= 1024, "expert parallel planning supports at most 1024 experts");
    EpState& ep = e->ep;
    MOE_REQUIRE(!ep.local, "moe_ep_export was already called on this engine");
    MOE_CUDA(cudaSetDevice(e->device));
    ep.rank = rank; ep.world = world; ep.cap = max_tokens_per_rank;
    ep.slots_cap = world * max_tokens_per_rank * d.top_k;
    size_t off = 0;
    auto take = [&](size_t bytes) { size_t o = off; off += al256(bytes); return o; };
    ep.sym.flags = take(kEpMaxWorld * 64);
    ep.sym.counts = take((size_t)world * d.num_experts * 4);
    // per received row: who sent it and where its result goes (16 B); which received row holds its
    // activations (a token is sent once per GPU, its experts there share the row); and, for the first
    // ("leader") row of a (token, GPU) pair, the rows and weights to combine before returning
    ep.sym.meta = take((size_t)ep.slots_cap * 16);
    ep.sym.xmap = take(((size_t)ep.slots_cap + ep.cap) * 4);
    ep.sym.memb = take((size_t)ep.slots_cap * 8 * 4);
    ep.sym.mwt = take((size_t)ep.slots_cap * 8 * 4);
    ep.sym.xrecv = take(((size_t)ep.slots_cap + ep.cap) * d.hidden * 2);
    ep.sym.oback = take((size_t)ep.cap * d.top_k * d.hidden * 2);
    ep.sym.total = off;
    MOE_CUDA(cudaMalloc(&ep.local, ep.sym.total));
    MOE_CUDA(cudaMemset(ep.local, 0, ep.sym.total));
    cudaIpcMemHandle_t h;
    MOE_CUDA(cudaIpcGetMemHandle(&h, ep.local));
    static_assert(sizeof(cudaIpcMemHandle_t) == MOE_EP_HANDLE_BYTES, "handle size");
    memcpy(handle_out, &h, sizeof(h));
    return MOE_OK;
}

int moe_ep_init(moe_engine_t* e, const void* all_handles) {
    MOE_REQUIRE(e && all_handles, "null argument");
    EpState& ep = e->ep;
    MOE_REQUIRE(ep.local && !ep.ready, "call moe_ep_export first (and moe_ep_init only once)");
    MOE_CUDA(cudaSetDevice(e->device));
    for (int r = 0; r < ep.world; ++r) {
        if (r == ep.rank) { ep.peer[r] = ep.local; continue; }
        cudaIpcMemHandle_t h;
        memcpy(&h, (const uint8_t*)all_handles + (size_t)r * MOE_EP_HANDLE_BYTES, sizeof(h));
        void* p = nullptr;
        MOE_CUDA(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
        ep.peer[r] = (uint8_t*)p;
    }
    int rc = ep_alloc_work(e);
    if (rc) return rc;
    MOE_CUDA(cudaStreamSynchronize(e->stream));
    ep.ready = true;
    return MOE_OK;
}

int moe_ep_finalize(moe_engine_t* e) {
    MOE_REQUIRE(e, "null engine");
    EpState& ep = e->ep;
    if (!ep.local) return MOE_OK;
    cudaSetDevice(e->device);
    cudaStreamSynchronize(e->stream);
    for (int r = 0; r < ep.world; ++r)
        if (r != ep.rank && ep.peer[r]) cudaIpcCloseMemHandle(ep.peer[r]);
    cudaFree(ep.local);
    if (ep.work) cudaFree(ep.work);
    ep = EpState{};
    return MOE_OK;
}

int moe_ep_layer_forward_dev(moe_engine_t* e, int layer, const float* h_in_dev, int32_t n_local, float* h_out_dev) {
    MOE_REQUIRE(e && h_in_dev && h_out_dev, "null argument");
    return ep_layer(e, layer, h_in_dev, n_local, h_out_dev);
}

int moe_ep_forward_hidden_dev(moe_engine_t* e, const float* emb_dev, int32_t n_local, float* out_dev) {
    MOE_REQUIRE(e && emb_dev && out_dev, "null argument");
    const int L = e->dims.num_layers;
    const float* cur = emb_dev;
    for (int l = 0; l < L; ++l) {
        float* nxt = (l == L - 1) ? out_dev : ((l & 1) ? e->bw.h_b : e->bw.h_a);
        int rc = ep_layer(e, l, cur, n_local, nxt);
        if (rc) return rc;
        cur = nxt;
    }
    return MOE_OK;
}

}  // extern "C"
