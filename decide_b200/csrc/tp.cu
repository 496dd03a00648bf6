// Tensor-parallel group of a context: one process per GPU, NCCL over NVLink / NVSwitch for the
// partial-sum exchange after each row-split projection.
//
// The reference has no collective; its precedent is the GPU + Neural-Engine split of each MLP, two
// partial down-projections added afterwards (crates/decide-engine/src/forward.rs:270-303, 1286-1309,
// kernels/ane.metal:10-18). Here the same partial-sum add runs over G GPUs: gate_up / in-projections
// split by output column (per head, per gate|up block), down / out-projections by input column, and
// an all-reduce of the fp32 [rows, hidden] partials replaces `x += partial * inv_scale`.
//
// NCCL is opened with dlopen at dc_tp_init, so the library has no load-time dependency on it: a
// single-GPU host never touches NCCL. The unique id is made on one rank and handed to the others
// by the host (a file, a socket, torch.distributed: whatever launched the ranks).
#include <dlfcn.h>

#include <cstdlib>
#include <cstring>

#include "common.cuh"

namespace {

// The few NCCL declarations used, unchanged since NCCL 2.10 (nccl.h: ncclUniqueId, ncclDataType_t, ncclRedOp_t).
struct NcclUniqueId {
    char internal[128];
};
typedef void* NcclComm;
constexpr int kNcclFloat32 = 7, kNcclFloat16 = 6, kNcclBfloat16 = 9;
constexpr int kNcclSum = 0;

struct NcclApi {
    void* lib = nullptr;
    int (*GetUniqueId)(NcclUniqueId*) = nullptr;
    int (*CommInitRank)(NcclComm*, int, NcclUniqueId, int) = nullptr;
    int (*AllReduce)(const void*, void*, size_t, int, int, NcclComm, cudaStream_t) = nullptr;
    int (*CommDestroy)(NcclComm) = nullptr;
    int (*CommAbort)(NcclComm) = nullptr;
    const char* (*GetErrorString)(int) = nullptr;
};

NcclApi* nccl_api(char* err, size_t err_len) {
    static NcclApi api;
    static bool tried = false;
    if (api.lib) return &api;
    if (tried) {
        if (err && err_len) snprintf(err, err_len, "NCCL could not be loaded earlier in this process");
        return nullptr;
    }
    tried = true;
    const char* names[] = {getenv("DECIDE_NCCL_LIB"), "libnccl.so.2", "libnccl.so"};
    void* lib = nullptr;
    for (const char* n : names) {
        if (n && *n && (lib = dlopen(n, RTLD_NOW | RTLD_GLOBAL))) break;
    }
    if (!lib) {
        if (err && err_len) snprintf(err, err_len, "cannot load libnccl.so.2 (set DECIDE_NCCL_LIB to its path): %s", dlerror());
        return nullptr;
    }
    auto sym = [&](const char* name) { return dlsym(lib, name); };
    api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(sym("ncclGetUniqueId"));
    api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(sym("ncclCommInitRank"));
    api.AllReduce = reinterpret_cast<decltype(api.AllReduce)>(sym("ncclAllReduce"));
    api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(sym("ncclCommDestroy"));
    api.CommAbort = reinterpret_cast<decltype(api.CommAbort)>(sym("ncclCommAbort"));
    api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(sym("ncclGetErrorString"));
    if (!api.GetUniqueId || !api.CommInitRank || !api.AllReduce || !api.CommDestroy || !api.GetErrorString) {
        if (err && err_len) snprintf(err, err_len, "the NCCL library lacks an expected symbol");
        return nullptr;
    }
    api.lib = lib;
    return &api;
}

}  // namespace

extern "C" {

int dc_tp_unique_id(void* id128, char* err, size_t err_len) {
    if (!id128) return DC_INVALID_ARG;
    NcclApi* api = nccl_api(err, err_len);
    if (!api) return DC_UNSUPPORTED;
    NcclUniqueId id;
    const int rc = api->GetUniqueId(&id);
    if (rc != 0) {
        if (err && err_len) snprintf(err, err_len, "ncclGetUniqueId: %s", api->GetErrorString(rc));
        return DC_CUDA_ERROR;
    }
    memcpy(id128, id.internal, sizeof id.internal);
    return DC_OK;
}

int dc_tp_init(dc_ctx* ctx, const void* id128, uint32_t world, uint32_t rank) {
    if (!ctx) return DC_INVALID_ARG;
    DC_REQUIRE(ctx, id128 && world >= 1 && rank < world, "dc_tp_init: rank %u of %u", rank, world);
    DC_REQUIRE(ctx, !ctx->tp_comm, "dc_tp_init: this context already belongs to a tensor-parallel group");
    if (world == 1) {
        ctx->tp_world = 1;
        ctx->tp_rank = 0;
        return DC_OK;
    }
    char err[256] = "";
    NcclApi* api = nccl_api(err, sizeof err);
    if (!api) return dc_fail(ctx, DC_UNSUPPORTED, "dc_tp_init: %s", err);
    cudaSetDevice(ctx->device);
    NcclUniqueId id;
    memcpy(id.internal, id128, sizeof id.internal);
    NcclComm comm = nullptr;
    const int rc = api->CommInitRank(&comm, static_cast<int>(world), id, static_cast<int>(rank));
    if (rc != 0) return dc_fail(ctx, DC_CUDA_ERROR, "dc_tp_init: ncclCommInitRank: %s", api->GetErrorString(rc));
    ctx->tp_comm = comm;
    ctx->tp_world = world;
    ctx->tp_rank = rank;
    if (const char* e = getenv("DECIDE_TP_EXCHANGE")) ctx->tp_exchange16 = strcmp(e, "16") == 0;
    return DC_OK;
}

int dc_tp_all_reduce_f32(dc_ctx* ctx, void* stream, float* buf, size_t n) {
    if (!ctx) return DC_INVALID_ARG;
    DC_REQUIRE(ctx, buf || n == 0, "dc_tp_all_reduce_f32: null buffer");
    if (ctx->tp_world <= 1 || n == 0) return DC_OK;
    NcclApi* api = nccl_api(nullptr, 0);
    if (!api || !ctx->tp_comm) return dc_fail(ctx, DC_INVALID_ARG, "dc_tp_all_reduce_f32: no tensor-parallel group (dc_tp_init)");
    const int rc = api->AllReduce(buf, buf, n, kNcclFloat32, kNcclSum, ctx->tp_comm, static_cast<cudaStream_t>(stream));
    if (rc != 0) return dc_fail(ctx, DC_CUDA_ERROR, "ncclAllReduce: %s", api->GetErrorString(rc));
    ctx->launches++;
    return DC_OK;
}

int dc_tp_all_reduce_16(dc_ctx* ctx, void* stream, void* buf, size_t n) {
    if (!ctx) return DC_INVALID_ARG;
    DC_REQUIRE(ctx, buf || n == 0, "dc_tp_all_reduce_16: null buffer");
    if (ctx->tp_world <= 1 || n == 0) return DC_OK;
    NcclApi* api = nccl_api(nullptr, 0);
    if (!api || !ctx->tp_comm) return dc_fail(ctx, DC_INVALID_ARG, "dc_tp_all_reduce_16: no tensor-parallel group (dc_tp_init)");
    const int rc = api->AllReduce(buf, buf, n, ctx->act_dtype == DC_ACT_F16 ? kNcclFloat16 : kNcclBfloat16, kNcclSum, ctx->tp_comm, static_cast<cudaStream_t>(stream));
    if (rc != 0) return dc_fail(ctx, DC_CUDA_ERROR, "ncclAllReduce: %s", api->GetErrorString(rc));
    ctx->launches++;
    return DC_OK;
}

int dc_tp_set_exchange_16bit(dc_ctx* ctx, uint32_t on) {
    if (!ctx) return DC_INVALID_ARG;
    ctx->tp_exchange16 = on != 0;
    return DC_OK;
}

uint32_t dc_tp_world(dc_ctx* ctx) { return ctx ? ctx->tp_world : 1; }
uint32_t dc_tp_rank(dc_ctx* ctx) { return ctx ? ctx->tp_rank : 0; }

void dc_tp_destroy(dc_ctx* ctx) {
    if (!ctx || !ctx->tp_comm) return;
    if (NcclApi* api = nccl_api(nullptr, 0)) {
        cudaSetDevice(ctx->device);
        api->CommDestroy(ctx->tp_comm);
    }
    ctx->tp_comm = nullptr;
    ctx->tp_world = 1;
    ctx->tp_rank = 0;
}

}  // extern "C"
