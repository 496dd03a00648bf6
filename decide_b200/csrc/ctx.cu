// Context lifetime, error latch, status word and workspace of libdecide_cuda.so.
// Plays the part of the reference's DecideDevice (crates/decide-metal/src/device.rs:55-130):
// device handle, "pipeline" state that must exist before a timed request, and nothing else.
#include <cstdlib>
#include <cstring>

#include "common.cuh"

int dc_fail(dc_ctx* ctx, int code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    if (ctx && ctx->last_error.empty()) ctx->last_error = buf;  // first error wins, as Run::fail (forward.rs:322-329)
    return code;
}

int dc_check_launch(dc_ctx* ctx, const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return dc_fail(ctx, DC_CUDA_ERROR, "%s: launch failed: %s", what, cudaGetErrorString(e));
    ctx->launches++;
    return DC_OK;
}

int dc_get_workspace(dc_ctx* ctx, size_t bytes, const char* who, void** out) {
    *out = nullptr;
    if (bytes <= ctx->workspace_bytes && ctx->workspace) {
        *out = ctx->workspace;
        return DC_OK;
    }
    if (ctx->workspace_frozen)
        return dc_fail(ctx, DC_INVALID_ARG, "%s: needs %zu bytes of scratch but the workspace is frozen at %zu (reserve more with dc_reserve_workspace before freezing)",
                       who, bytes, ctx->workspace_bytes);
    if (ctx->workspace) cudaFree(ctx->workspace);
    ctx->workspace = nullptr;
    ctx->workspace_bytes = 0;
    void* p = nullptr;
    if (cudaMalloc(&p, bytes ? bytes : 256) != cudaSuccess) {
        cudaGetLastError();
        return dc_fail(ctx, DC_CUDA_ERROR, "%s: cannot allocate %zu bytes of scratch", who, bytes);
    }
    ctx->allocs++;
    ctx->workspace = p;
    ctx->workspace_bytes = bytes ? bytes : 256;
    *out = p;
    return DC_OK;
}

static uint32_t impl_from_env(const char* name, bool* bad) {
    const char* v = getenv(name);
    if (!v || !*v || strcmp(v, "fast") == 0) return DC_IMPL_FAST;
    if (strcmp(v, "baseline") == 0) return DC_IMPL_BASELINE;
    *bad = true;
    return DC_IMPL_FAST;
}

extern "C" {

dc_ctx* dc_open(int device, char* err, size_t err_len) {
    auto say = [&](const char* msg, const char* detail) {
        if (err && err_len) snprintf(err, err_len, "%s%s%s", msg, detail ? ": " : "", detail ? detail : "");
    };
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0) {
        say("dc_open: no CUDA device (this library has no CPU path)", e != cudaSuccess ? cudaGetErrorString(e) : nullptr);
        cudaGetLastError();
        return nullptr;
    }
    if (device < 0 || device >= count) {
        say("dc_open: device index out of range", nullptr);
        return nullptr;
    }
    cudaDeviceProp prop;
    if ((e = cudaSetDevice(device)) != cudaSuccess || (e = cudaGetDeviceProperties(&prop, device)) != cudaSuccess) {
        say("dc_open: cannot select device", cudaGetErrorString(e));
        return nullptr;
    }
    if (prop.major != 10) {
        say("dc_open: the kernels are built for sm_100a (B200) only", prop.name);
        return nullptr;
    }
    dc_ctx* ctx = new dc_ctx();
    ctx->device = device;
    ctx->sm_count = prop.multiProcessorCount;
    ctx->smem_optin = static_cast<int>(prop.sharedMemPerBlockOptin);
    bool bad = false;
    ctx->gemm_impl = impl_from_env("DECIDE_GEMM", &bad);
    ctx->attn_impl = impl_from_env("DECIDE_ATTN", &bad);
    ctx->delta_impl = impl_from_env("DECIDE_DELTA", &bad);
    if (const char* d = getenv("DECIDE_DELTA_SPLIT")) {
        if (strcmp(d, "1") == 0) ctx->delta_split = 1;
        else if (strcmp(d, "3") == 0 || !*d) ctx->delta_split = 3;
        else bad = true;
    }
    for (int f = 0; f < 2; ++f) {
        const char* d = getenv(f ? "DECIDE_ATTN_ENGINE" : "DECIDE_DELTA_ENGINE");
        if (!d) continue;
        uint32_t& engine = f ? ctx->attn_engine : ctx->delta_engine;
        if (strcmp(d, "mma") == 0) engine = DC_ENGINE_MMA_SYNC;
        else if (strcmp(d, "tcgen05") == 0 || !*d) engine = DC_ENGINE_TCGEN05;
        else bad = true;
    }
    if (const char* a = getenv("DECIDE_ACT")) {
        if (strcmp(a, "bf16") == 0) ctx->act_dtype = DC_ACT_BF16;
        else if (strcmp(a, "f16") == 0 || !*a) ctx->act_dtype = DC_ACT_F16;
        else bad = true;
    }
    if (bad) {
        say("dc_open: DECIDE_GEMM / DECIDE_ATTN / DECIDE_DELTA must be `fast` or `baseline`, DECIDE_ACT `f16` or `bf16`, DECIDE_DELTA_SPLIT 1 or 3, DECIDE_ATTN_ENGINE / DECIDE_DELTA_ENGINE `tcgen05` or `mma`", nullptr);
        delete ctx;
        return nullptr;
    }
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !fn) {
        say("dc_open: cuTensorMapEncodeTiled not available", e != cudaSuccess ? cudaGetErrorString(e) : nullptr);
        delete ctx;
        return nullptr;
    }
    ctx->encode_tiled = reinterpret_cast<dc_encode_tiled_fn>(fn);
    if ((e = cudaMalloc(&ctx->status_dev, sizeof(int))) != cudaSuccess ||
        (e = cudaMemset(ctx->status_dev, 0, sizeof(int))) != cudaSuccess ||
        (e = cudaMallocHost(&ctx->status_host, sizeof(int))) != cudaSuccess) {
        say("dc_open: cannot allocate the status word", cudaGetErrorString(e));
        dc_close(ctx);
        return nullptr;
    }
    *ctx->status_host = 0;
    ctx->allocs += 2;
    const size_t ws = static_cast<size_t>(ctx->sm_count) * 128 * 256 * sizeof(float);
    if ((e = cudaMalloc(&ctx->gemm_part_ws, ws)) != cudaSuccess || (e = cudaMalloc(&ctx->gemm_part_cnt, ctx->sm_count * 4 * sizeof(int))) != cudaSuccess ||
        (e = cudaMemset(ctx->gemm_part_cnt, 0, ctx->sm_count * 4 * sizeof(int))) != cudaSuccess) {
        say("dc_open: cannot allocate the GEMM split workspace", cudaGetErrorString(e));
        dc_close(ctx);
        return nullptr;
    }
    ctx->allocs += 2;
    return ctx;
}

void dc_close(dc_ctx* ctx) {
    if (!ctx) return;
    cudaSetDevice(ctx->device);
    dc_tp_destroy(ctx);
    if (ctx->status_dev) cudaFree(ctx->status_dev);
    if (ctx->status_host) cudaFreeHost(ctx->status_host);
    if (ctx->workspace) cudaFree(ctx->workspace);
    if (ctx->gemm_part_ws) cudaFree(ctx->gemm_part_ws);
    if (ctx->gemm_part_cnt) cudaFree(ctx->gemm_part_cnt);
    delete ctx;
}

size_t dc_last_error(dc_ctx* ctx, char* buf, size_t len) {
    if (!ctx) return 0;
    size_t n = ctx->last_error.size();
    if (buf && len) {
        snprintf(buf, len, "%s", ctx->last_error.c_str());
    }
    ctx->last_error.clear();
    return n;
}

int dc_set_impl(dc_ctx* ctx, uint32_t family, uint32_t impl) {
    if (!ctx) return DC_INVALID_ARG;
    DC_REQUIRE(ctx, impl == DC_IMPL_FAST || impl == DC_IMPL_BASELINE, "dc_set_impl: impl %u is neither fast nor baseline", impl);
    switch (family) {
        case DC_FAMILY_GEMM: ctx->gemm_impl = impl; break;
        case DC_FAMILY_ATTN: ctx->attn_impl = impl; break;
        case DC_FAMILY_DELTA: ctx->delta_impl = impl; break;
        default: return dc_fail(ctx, DC_INVALID_ARG, "dc_set_impl: unknown family %u", family);
    }
    return DC_OK;
}

uint32_t dc_get_impl(dc_ctx* ctx, uint32_t family) {
    if (!ctx) return DC_IMPL_FAST;
    switch (family) {
        case DC_FAMILY_GEMM: return ctx->gemm_impl;
        case DC_FAMILY_ATTN: return ctx->attn_impl;
        case DC_FAMILY_DELTA: return ctx->delta_impl;
        default: return DC_IMPL_FAST;
    }
}

int dc_set_activation_dtype(dc_ctx* ctx, uint32_t act) {
    if (!ctx) return DC_INVALID_ARG;
    DC_REQUIRE(ctx, act == DC_ACT_BF16 || act == DC_ACT_F16, "dc_set_activation_dtype: unknown type %u", act);
    ctx->act_dtype = act;
    return DC_OK;
}

uint32_t dc_get_activation_dtype(dc_ctx* ctx) { return ctx ? ctx->act_dtype : DC_ACT_F16; }

int dc_set_delta_split(dc_ctx* ctx, uint32_t split) {
    if (!ctx) return DC_INVALID_ARG;
    DC_REQUIRE(ctx, split == 1 || split == 3, "dc_set_delta_split: %u is neither 1 nor 3", split);
    ctx->delta_split = split;
    return DC_OK;
}

int dc_set_engine(dc_ctx* ctx, uint32_t family, uint32_t engine) {
    if (!ctx) return DC_INVALID_ARG;
    DC_REQUIRE(ctx, engine == DC_ENGINE_MMA_SYNC || engine == DC_ENGINE_TCGEN05, "dc_set_engine: unknown engine %u", engine);
    switch (family) {
        case DC_FAMILY_ATTN: ctx->attn_engine = engine; break;
        case DC_FAMILY_DELTA: ctx->delta_engine = engine; break;
        case DC_FAMILY_GEMM:
            DC_REQUIRE(ctx, engine == DC_ENGINE_TCGEN05, "dc_set_engine: the GEMM has no mma.sync engine (its baseline is DC_IMPL_BASELINE)");
            break;
        default: return dc_fail(ctx, DC_INVALID_ARG, "dc_set_engine: unknown family %u", family);
    }
    return DC_OK;
}

int dc_check_status(dc_ctx* ctx, void* stream) {
    if (!ctx) return DC_INVALID_ARG;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    cudaError_t e = cudaMemcpyAsync(ctx->status_host, ctx->status_dev, sizeof(int), cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    if (e != cudaSuccess) return dc_fail(ctx, DC_CUDA_ERROR, "dc_check_status: %s", cudaGetErrorString(e));
    int code = *ctx->status_host;
    if (code != 0) {
        cudaMemsetAsync(ctx->status_dev, 0, sizeof(int), s);
        // a split GEMM that gave up leaves arrival counters of its tail tiles non-zero: the next one must start from zero
        cudaMemsetAsync(ctx->gemm_part_cnt, 0, ctx->sm_count * 4 * sizeof(int), s);
        cudaStreamSynchronize(s);
        if (code == DC_STATUS_POSITION_PAST_CACHE)
            return dc_fail(ctx, DC_INVALID_ARG, "attention: a query row's position lies at or past the cache length given as max_len; the results of this run are invalid");
        return dc_fail(ctx, DC_TIMEOUT, "a bounded device-side wait ran out (wait id %d); the results of this run are invalid", code);
    }
    return DC_OK;
}

uint64_t dc_launch_count(dc_ctx* ctx) { return ctx ? ctx->launches : 0; }

int dc_reserve_workspace(dc_ctx* ctx, size_t bytes) {
    if (!ctx) return DC_INVALID_ARG;
    void* p = nullptr;
    return dc_get_workspace(ctx, bytes, "dc_reserve_workspace", &p);
}

int dc_set_workspace_frozen(dc_ctx* ctx, uint32_t on) {
    if (!ctx) return DC_INVALID_ARG;
    ctx->workspace_frozen = on != 0;
    return DC_OK;
}

size_t dc_workspace_bytes(dc_ctx* ctx) { return ctx ? ctx->workspace_bytes : 0; }
uint64_t dc_alloc_count(dc_ctx* ctx) { return ctx ? ctx->allocs : 0; }
uint64_t dc_tmap_encode_count(dc_ctx* ctx) { return ctx ? ctx->tmap_encodes : 0; }
size_t dc_tmap_cache_size(dc_ctx* ctx) { return ctx ? ctx->tmaps.size() : 0; }

int dc_warm_up(dc_ctx* ctx) {
    if (!ctx) return DC_INVALID_ARG;
    cudaSetDevice(ctx->device);
    int rc = dc_gemm_warm(ctx);
    if (rc == DC_OK) rc = dc_attention_warm(ctx);
    if (rc == DC_OK) rc = dc_attention_tc_warm(ctx);
    if (rc == DC_OK) rc = dc_delta_chunk_warm(ctx);
    return rc;
}

int dc_sm_count(dc_ctx* ctx) { return ctx ? ctx->sm_count : 0; }

}  // extern "C"
