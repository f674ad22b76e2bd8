// Expert parallelism over the GPUs of one box (no counterpart in the reference,
// which drives a single device).
#include "common.cuh"

using namespace moe;

extern "C" {

int moe_ep_export(moe_engine_t* e, int32_t max_tokens_per_rank, void* handle_out) {
    (void)max_tokens_per_rank;
    MOE_REQUIRE(e && handle_out, "null argument");
    set_error("expert parallelism is not built yet");
    return MOE_ERR_UNSUPPORTED;
}

int moe_ep_init(moe_engine_t* e, int rank, int world, const void* all_handles) {
    (void)rank; (void)world;
    MOE_REQUIRE(e && all_handles, "null argument");
    set_error("expert parallelism is not built yet");
    return MOE_ERR_UNSUPPORTED;
}

int moe_ep_finalize(moe_engine_t* e) {
    MOE_REQUIRE(e, "null engine");
    return MOE_OK;
}

}  // extern "C"
