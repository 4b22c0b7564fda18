// Context, memory, stream, events and the RoPE denominator cache of libagention_b200.
#include <math.h>
#include <stdarg.h>
#include <string.h>

#include "agn_common.cuh"

int32_t agn_fail(agn_ctx *ctx, int32_t status, const char *fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    if (ctx) ctx->last_error = buf;
    return status;
}

extern "C" {

const char *agn_backend_name(void) { return "cuda-sm100a"; }

const char *agn_status_string(int32_t s) {
    switch (s) {
    case AGN_OK: return "ok";
    case AGN_EINVAL: return "invalid argument";
    case AGN_EUNSUPPORTED_DTYPE: return "unsupported tensor type";
    case AGN_ECUDA: return "CUDA error";
    case AGN_EOOB_ID: return "row index out of range";
    case AGN_ENOMEM: return "out of memory";
    case AGN_ETIMEOUT: return "device-side wait timed out";
    case AGN_EFORMAT: return "malformed GGUF data";
    case AGN_ENOTFOUND: return "not found";
    case AGN_EIO: return "file cannot be opened or mapped";
    default: return "unknown status";
    }
}

int32_t agn_ctx_create(int32_t device, agn_ctx **out) {
    if (!out) return AGN_EINVAL;
    *out = nullptr;
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || device < 0 || device >= n) {
        (void)cudaGetLastError();
        return AGN_ECUDA;  // no device: never fall back to a CPU path
    }
    agn_ctx *ctx = new agn_ctx();
    ctx->device = device;
    ctx->launches = 0;
    ctx->last_kernel = "";
    ctx->rope_next = 0;
    ctx->flags_dirty = false;
    ctx->d_flags = nullptr;
    ctx->h_flags = nullptr;
    ctx->d_rope_denom = nullptr;
    ctx->h_rope_denom = nullptr;
    ctx->own_stream = nullptr;
    ctx->d_scratch = nullptr;
    ctx->scratch_bytes = 0;
    ctx->host_pipe = nullptr;
    ctx->pdl = true;
    ctx->capturing = false;
    ctx->capture_launches0 = 0;
    ctx->capture_rope_slots = 0;
    ctx->tune_rms_vpt = 0;
    ctx->tune_rms_recip = 1;
    ctx->tune_get_rows_threads = 0;
    ctx->tune_softmax_vpt = 0;
    ctx->tune_softmax_cluster = 1;
    ctx->tune_softmax_warp16 = 0;
    ctx->tune_softmax_causal_pair = 1;
    ctx->tune_rms_q8k_bpw = 0;
    ctx->tune_moe_small_sort = 1;
    ctx->tune_get_rows_tma = 1;
    ctx->tune_silu_unroll = 4;
    ctx->tune_silu_threads = 256;
    ctx->tune_silu_small = 1;
    ctx->tune_kv_multi = 1;
    ctx->tune_rms_ring = 0;
    ctx->tune_rms_ring_ctas = 0;
    ctx->tune_rope_ring = 0;
    ctx->tune_rope_ring_ctas = 0;
    ctx->tune_get_rows_ring = 0;
    ctx->tune_get_rows_ring_ctas = 0;
    ctx->tune_softmax_ring = 0;
    ctx->tune_softmax_ring_ctas = 0;
    ctx->tune_ring_force = 0;
    ctx->tune_host_chunk_bytes = 0;
    ctx->tune_host_slots = 0;
    ctx->mbar_spin_limit = AGN_MBAR_SPIN_LIMIT_DEFAULT;
    ctx->test_idle_barrier_wait = 0;
    memset(ctx->rope_slots, 0, sizeof(ctx->rope_slots));
    const size_t rope_bytes = sizeof(float) * AGN_ROPE_CACHE_SLOTS * AGN_ROPE_MAX_HALF;
    bool ok = cudaSetDevice(device) == cudaSuccess &&
              cudaDeviceGetAttribute(&ctx->sm_count, cudaDevAttrMultiProcessorCount, device) == cudaSuccess &&
              cudaStreamCreateWithFlags(&ctx->own_stream, cudaStreamNonBlocking) == cudaSuccess &&
              cudaMalloc(&ctx->d_flags, 4 * sizeof(uint32_t)) == cudaSuccess &&
              cudaMemset(ctx->d_flags, 0, 4 * sizeof(uint32_t)) == cudaSuccess &&
              cudaHostAlloc(&ctx->h_flags, 4 * sizeof(uint32_t), cudaHostAllocDefault) == cudaSuccess &&
              cudaMalloc(&ctx->d_rope_denom, rope_bytes) == cudaSuccess &&
              cudaMalloc(&ctx->d_scratch, AGN_SCRATCH_BYTES) == cudaSuccess &&
              cudaHostAlloc(&ctx->h_rope_denom, rope_bytes, cudaHostAllocDefault) == cudaSuccess;
    if (!ok) {
        (void)cudaGetLastError();
        agn_ctx_destroy(ctx);
        return AGN_ECUDA;
    }
    ctx->scratch_bytes = AGN_SCRATCH_BYTES;
    ctx->stream = ctx->own_stream;
    *out = ctx;
    return AGN_OK;
}

int32_t agn_ctx_destroy(agn_ctx *ctx) {
    if (!ctx) return AGN_EINVAL;
    cudaSetDevice(ctx->device);
    agn_host_pipe_destroy(ctx);
    if (ctx->own_stream) {
        cudaStreamSynchronize(ctx->own_stream);
        cudaStreamDestroy(ctx->own_stream);
    }
    if (ctx->d_flags) cudaFree(ctx->d_flags);
    if (ctx->h_flags) cudaFreeHost(ctx->h_flags);
    if (ctx->d_rope_denom) cudaFree(ctx->d_rope_denom);
    if (ctx->h_rope_denom) cudaFreeHost(ctx->h_rope_denom);
    if (ctx->d_scratch) cudaFree(ctx->d_scratch);
    (void)cudaGetLastError();
    delete ctx;
    return AGN_OK;
}

const char *agn_last_error(agn_ctx *ctx) { return ctx ? ctx->last_error.c_str() : "null context"; }

int32_t agn_ctx_set_stream(agn_ctx *ctx, void *cuda_stream) {
    AGN_CHECK_CTX(ctx);
    ctx->stream = cuda_stream ? reinterpret_cast<cudaStream_t>(cuda_stream) : ctx->own_stream;
    return AGN_OK;
}

int32_t agn_ctx_get_stream(agn_ctx *ctx, void **cuda_stream) {
    AGN_CHECK_CTX(ctx);
    if (!cuda_stream) return agn_fail(ctx, AGN_EINVAL, "agn_ctx_get_stream: null out pointer");
    *cuda_stream = reinterpret_cast<void *>(ctx->stream);
    return AGN_OK;
}

uint64_t agn_ctx_launch_count(agn_ctx *ctx) { return ctx ? ctx->launches : 0; }
const char *agn_ctx_last_kernel(agn_ctx *ctx) { return ctx ? ctx->last_kernel : ""; }

int32_t agn_ctx_set_option(agn_ctx *ctx, const char *name, int64_t value) {
    AGN_CHECK_CTX(ctx);
    if (!name) return agn_fail(ctx, AGN_EINVAL, "agn_ctx_set_option: null name");
    if (strcmp(name, "pdl") == 0) {
        ctx->pdl = value != 0;
        return AGN_OK;
    }
    if (strcmp(name, "rms_vpt") == 0) {
        ctx->tune_rms_vpt = (int)value;
        return AGN_OK;
    }
    if (strcmp(name, "silu_unroll") == 0 && (value == 2 || value == 4 || value == 8)) {
        ctx->tune_silu_unroll = (int)value;
        return AGN_OK;
    }
    if (strcmp(name, "silu_threads") == 0 && (value == 128 || value == 256 || value == 512)) {
        ctx->tune_silu_threads = (int)value;
        return AGN_OK;
    }
    if (strcmp(name, "moe_small_sort") == 0) {
        ctx->tune_moe_small_sort = value != 0;
        return AGN_OK;
    }
    if (strcmp(name, "softmax_cluster") == 0) {
        ctx->tune_softmax_cluster = (int)value;
        return AGN_OK;
    }
    if (strcmp(name, "softmax_vpt") == 0) {
        ctx->tune_softmax_vpt = (int)value;
        return AGN_OK;
    }
    if (strcmp(name, "get_rows_tma") == 0) {
        ctx->tune_get_rows_tma = value != 0;
        return AGN_OK;
    }
    if (strcmp(name, "get_rows_threads") == 0) {
        ctx->tune_get_rows_threads = (int)value;
        return AGN_OK;
    }
    if (strcmp(name, "rms_recip") == 0) {
        ctx->tune_rms_recip = value != 0;
        return AGN_OK;
    }
    {
        struct { const char *name; int *field; int64_t lo, hi; } ints[] = {
            {"rms_ring", &ctx->tune_rms_ring, 0, 8},
            {"rms_ring_ctas", &ctx->tune_rms_ring_ctas, 0, 32},
            {"rope_ring", &ctx->tune_rope_ring, 0, 8},
            {"rope_ring_ctas", &ctx->tune_rope_ring_ctas, 0, 32},
            {"get_rows_ring", &ctx->tune_get_rows_ring, 0, 16},
            {"get_rows_ring_ctas", &ctx->tune_get_rows_ring_ctas, 0, 32},
            {"softmax_ring", &ctx->tune_softmax_ring, 0, 8},
            {"softmax_ring_ctas", &ctx->tune_softmax_ring_ctas, 0, 32},
            {"ring_force", &ctx->tune_ring_force, 0, 1},
            {"softmax_warp16", &ctx->tune_softmax_warp16, 0, 1},
            {"softmax_causal_pair", &ctx->tune_softmax_causal_pair, 0, 1},
            {"rms_q8k_bpw", &ctx->tune_rms_q8k_bpw, 0, 4},
            {"silu_small", &ctx->tune_silu_small, 0, 1},
            {"kv_multi", &ctx->tune_kv_multi, 0, 1},
            {"host_chunk_bytes", &ctx->tune_host_chunk_bytes, 0, 24 << 20},
            {"host_slots", &ctx->tune_host_slots, 0, 16},
            {"mbar_spin_limit", &ctx->mbar_spin_limit, 1, 1 << 30},
            {"test_idle_barrier_wait", &ctx->test_idle_barrier_wait, 0, 1},
        };
        for (auto &o : ints) {
            if (strcmp(name, o.name) != 0) continue;
            if (value < o.lo || value > o.hi)
                return agn_fail(ctx, AGN_EINVAL, "agn_ctx_set_option: %s=%lld outside [%lld, %lld]", name, (long long)value,
                                (long long)o.lo, (long long)o.hi);
            *o.field = (int)value;
            return AGN_OK;
        }
    }
    return agn_fail(ctx, AGN_EINVAL, "agn_ctx_set_option: unknown option '%s'", name);
}

int32_t agn_malloc(agn_ctx *ctx, size_t bytes, void **dptr) {
    AGN_CHECK_CTX(ctx);
    if (!dptr) return agn_fail(ctx, AGN_EINVAL, "agn_malloc: null out pointer");
    *dptr = nullptr;
    if (bytes == 0) return AGN_OK;
    if (ctx->capturing) return agn_fail(ctx, AGN_EINVAL, "agn_malloc: allocation would invalidate the open graph capture");
    AGN_CUDA(ctx, cudaSetDevice(ctx->device));
    cudaError_t e = cudaMalloc(dptr, bytes);
    if (e == cudaErrorMemoryAllocation) {
        (void)cudaGetLastError();
        return agn_fail(ctx, AGN_ENOMEM, "agn_malloc: %zu bytes not available on device %d", bytes, ctx->device);
    }
    AGN_CUDA(ctx, e);
    return AGN_OK;
}

int32_t agn_free(agn_ctx *ctx, void *dptr) {
    AGN_CHECK_CTX(ctx);
    if (!dptr) return AGN_OK;
    if (ctx->capturing) return agn_fail(ctx, AGN_EINVAL, "agn_free: freeing would invalidate the open graph capture");
    AGN_CUDA(ctx, cudaSetDevice(ctx->device));
    AGN_CUDA(ctx, cudaFree(dptr));
    return AGN_OK;
}

int32_t agn_host_alloc(agn_ctx *ctx, size_t bytes, void **hptr) {
    AGN_CHECK_CTX(ctx);
    if (!hptr) return agn_fail(ctx, AGN_EINVAL, "agn_host_alloc: null out pointer");
    *hptr = nullptr;
    if (bytes == 0) return AGN_OK;
    if (ctx->capturing) return agn_fail(ctx, AGN_EINVAL, "agn_host_alloc: allocation would invalidate the open graph capture");
    AGN_CUDA(ctx, cudaSetDevice(ctx->device));
    cudaError_t e = cudaHostAlloc(hptr, bytes, cudaHostAllocDefault);
    if (e == cudaErrorMemoryAllocation) {
        (void)cudaGetLastError();
        return agn_fail(ctx, AGN_ENOMEM, "agn_host_alloc: %zu pinned bytes not available", bytes);
    }
    AGN_CUDA(ctx, e);
    return AGN_OK;
}

int32_t agn_host_free(agn_ctx *ctx, void *hptr) {
    AGN_CHECK_CTX(ctx);
    if (!hptr) return AGN_OK;
    AGN_CUDA(ctx, cudaFreeHost(hptr));
    return AGN_OK;
}

int32_t agn_memcpy_h2d(agn_ctx *ctx, void *dst, const void *src, size_t bytes) {
    AGN_CHECK_CTX(ctx);
    if (bytes == 0) return AGN_OK;
    if (!dst || !src) return agn_fail(ctx, AGN_EINVAL, "agn_memcpy_h2d: null pointer");
    AGN_CUDA(ctx, cudaSetDevice(ctx->device));
    AGN_CUDA(ctx, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, ctx->stream));
    return AGN_OK;
}

int32_t agn_memcpy_d2h(agn_ctx *ctx, void *dst, const void *src, size_t bytes) {
    AGN_CHECK_CTX(ctx);
    if (bytes == 0) return AGN_OK;
    if (!dst || !src) return agn_fail(ctx, AGN_EINVAL, "agn_memcpy_d2h: null pointer");
    AGN_CUDA(ctx, cudaSetDevice(ctx->device));
    AGN_CUDA(ctx, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, ctx->stream));
    return AGN_OK;
}

int32_t agn_memset(agn_ctx *ctx, void *dst, int value, size_t bytes) {
    AGN_CHECK_CTX(ctx);
    if (bytes == 0) return AGN_OK;
    if (!dst) return agn_fail(ctx, AGN_EINVAL, "agn_memset: null pointer");
    AGN_CUDA(ctx, cudaSetDevice(ctx->device));
    AGN_CUDA(ctx, cudaMemsetAsync(dst, value, bytes, ctx->stream));
    return AGN_OK;
}

int32_t agn_sync(agn_ctx *ctx) {
    AGN_CHECK_CTX(ctx);
    if (ctx->capturing) return agn_fail(ctx, AGN_EINVAL, "agn_sync: not allowed while a graph capture is open");
    AGN_CUDA(ctx, cudaSetDevice(ctx->device));
    {
        const int32_t jrc = agn_host_pipe_join(ctx);  // the sync covers the downloads of host-slice ops
        if (jrc != AGN_OK) return jrc;
    }
    if (ctx->flags_dirty) {
        AGN_CUDA(ctx, cudaMemcpyAsync(ctx->h_flags, ctx->d_flags, sizeof(uint32_t), cudaMemcpyDeviceToHost, ctx->stream));
    }
    AGN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    if (ctx->flags_dirty) {
        ctx->flags_dirty = false;
        uint32_t f = ctx->h_flags[0];
        if (f) {
            AGN_CUDA(ctx, cudaMemsetAsync(ctx->d_flags, 0, sizeof(uint32_t), ctx->stream));
            AGN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
            if (f & AGN_FLAG_TIMEOUT)
                return agn_fail(ctx, AGN_ETIMEOUT, "a staging wait in a kernel gave up; outputs of that launch are invalid");
            // one bit per class of index, so the message names the op that met it
            std::string msg;
            if (f & AGN_FLAG_OOB_ID) msg += "get_rows: row index out of range (those output rows are zero); ";
            if (f & AGN_FLAG_OOB_EXPERT) msg += "gather_rows_by_expert: expert index out of range (those pairs are dropped); ";
            if (f & AGN_FLAG_OOB_SLOT) msg += "kv_write: position outside the cache (those tokens are not written); ";
            if (msg.empty()) msg = "a kernel reported an index out of range; ";
            msg.resize(msg.size() - 2);
            return agn_fail(ctx, AGN_EOOB_ID, "%s", msg.c_str());
        }
    }
    return AGN_OK;
}

int32_t agn_event_create(agn_ctx *ctx, agn_event **ev) {
    AGN_CHECK_CTX(ctx);
    if (!ev) return agn_fail(ctx, AGN_EINVAL, "agn_event_create: null out pointer");
    AGN_CUDA(ctx, cudaSetDevice(ctx->device));
    agn_event *e = new agn_event();
    cudaError_t ce = cudaEventCreate(&e->ev);
    if (ce != cudaSuccess) {
        delete e;
        AGN_CUDA(ctx, ce);
    }
    *ev = e;
    return AGN_OK;
}

int32_t agn_event_record(agn_ctx *ctx, agn_event *ev) {
    AGN_CHECK_CTX(ctx);
    if (!ev) return agn_fail(ctx, AGN_EINVAL, "agn_event_record: null event");
    AGN_CUDA(ctx, cudaSetDevice(ctx->device));
    {
        const int32_t jrc = agn_host_pipe_join(ctx);  // an event after a host-slice op covers its downloads
        if (jrc != AGN_OK) return jrc;
    }
    AGN_CUDA(ctx, cudaEventRecord(ev->ev, ctx->stream));
    return AGN_OK;
}

int32_t agn_event_elapsed_ms(agn_ctx *ctx, agn_event *start, agn_event *stop, float *ms) {
    AGN_CHECK_CTX(ctx);
    if (!start || !stop || !ms) return agn_fail(ctx, AGN_EINVAL, "agn_event_elapsed_ms: null argument");
    AGN_CUDA(ctx, cudaEventSynchronize(stop->ev));
    AGN_CUDA(ctx, cudaEventElapsedTime(ms, start->ev, stop->ev));
    return AGN_OK;
}

int32_t agn_event_destroy(agn_ctx *ctx, agn_event *ev) {
    AGN_CHECK_CTX(ctx);
    if (!ev) return AGN_OK;
    cudaEventDestroy(ev->ev);
    delete ev;
    return AGN_OK;
}

// `compute_rope_freq_scale` (src/model/llama/cpu_path.rs:34-40): absent / "" / "none" -> 1,
// "linear" -> 1 / max(factor or 1, 1e-6), anything else (e.g. "yarn") -> not applied.
int32_t agn_rope_freq_scale(const char *scaling_type, int32_t has_factor, float factor, float *scale) {
    if (!scale) return AGN_EINVAL;
    if (!scaling_type || scaling_type[0] == '\0' || strcmp(scaling_type, "none") == 0) {
        *scale = 1.0f;
        return AGN_OK;
    }
    if (strcmp(scaling_type, "linear") == 0) {
        float f = has_factor ? factor : 1.0f;
        if (!(f > 1e-6f)) f = 1e-6f;  // f32::max(1e-6); a NaN factor also ends up here
        *scale = 1.0f / f;
        return AGN_OK;
    }
    return AGN_ENOTFOUND;
}

size_t agn_type_size(int32_t dtype, size_t n) {
    // GgmlType::block_size / block_bytes / type_size, src/types.rs:88-168
    size_t bs, bb;
    switch (dtype) {
    case AGN_F32: bs = 1; bb = 4; break;
    case AGN_F16: case AGN_BF16: bs = 1; bb = 2; break;
    case AGN_Q8_0: bs = 32; bb = 34; break;
    case AGN_Q5_0: bs = 32; bb = 22; break;
    case AGN_Q5_K: bs = 256; bb = 176; break;
    case AGN_Q2_K: bs = 256; bb = 84; break;  // the codec's block, src/quant/q2_k.rs:24 (types.rs:137 lists 256)
    case AGN_Q4_K: bs = 256; bb = 144; break;
    case AGN_Q6_K: bs = 256; bb = 210; break;
    default: return 0;
    }
    return ((n + bs - 1) / bs) * bb;
}

}  // extern "C"

namespace {
__global__ void noop_kernel() { agn_pdl_prologue(); }
}  // namespace

struct agn_graph {
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    uint64_t kernels = 0;  // kernels recorded, added to the launch count at every replay
    uint32_t rope_slots = 0;  // rope table slots its kernels read: kept out of eviction until the graph is destroyed
};

// Records every op enqueued on the context's stream between begin and end into a CUDA graph
// instead of running it.  The decode loop (a fixed chain of small kernels per token) is
// launch-bound from any host language; one graph replay costs a fraction of a microsecond
// per kernel.  The RoPE table of a (theta, n_rot) pair must already exist (run the chain
// once before capturing it); agn_sync and memory allocation are not allowed inside.
extern "C" int32_t agn_graph_begin(agn_ctx *ctx) {
    AGN_CHECK_CTX(ctx);
    if (ctx->capturing) return agn_fail(ctx, AGN_EINVAL, "agn_graph_begin: a capture is already open");
    AGN_CUDA(ctx, cudaSetDevice(ctx->device));
    AGN_CUDA(ctx, cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal));
    ctx->capturing = true;
    ctx->capture_launches0 = ctx->launches;
    ctx->capture_rope_slots = 0;
    return AGN_OK;
}

extern "C" int32_t agn_graph_end(agn_ctx *ctx, agn_graph **out) {
    AGN_CHECK_CTX(ctx);
    if (!out) return agn_fail(ctx, AGN_EINVAL, "agn_graph_end: null out pointer");
    *out = nullptr;
    if (!ctx->capturing) return agn_fail(ctx, AGN_EINVAL, "agn_graph_end: no capture is open");
    ctx->capturing = false;
    agn_graph *g = new agn_graph();
    cudaError_t e = cudaStreamEndCapture(ctx->stream, &g->graph);
    if (e == cudaSuccess) e = cudaGraphInstantiate(&g->exec, g->graph, 0);
    if (e != cudaSuccess) {
        if (g->graph) cudaGraphDestroy(g->graph);
        delete g;
        (void)cudaGetLastError();
        return agn_fail(ctx, AGN_ECUDA, "agn_graph_end: %s", cudaGetErrorString(e));
    }
    g->kernels = ctx->launches - ctx->capture_launches0;
    g->rope_slots = ctx->capture_rope_slots;
    for (int sl = 0; sl < AGN_ROPE_CACHE_SLOTS; sl++)
        if (g->rope_slots & (1u << sl)) ctx->rope_slots[sl].graph_refs++;
    ctx->launches = ctx->capture_launches0;  // nothing ran yet
    *out = g;
    return AGN_OK;
}

extern "C" int32_t agn_graph_launch(agn_ctx *ctx, agn_graph *g) {
    AGN_CHECK_CTX(ctx);
    if (!g || !g->exec) return agn_fail(ctx, AGN_EINVAL, "agn_graph_launch: null graph");
    AGN_CUDA(ctx, cudaSetDevice(ctx->device));
    AGN_CUDA(ctx, cudaGraphLaunch(g->exec, ctx->stream));
    ctx->launches += g->kernels;
    return AGN_OK;
}

extern "C" int32_t agn_graph_destroy(agn_ctx *ctx, agn_graph *g) {
    AGN_CHECK_CTX(ctx);
    if (!g) return AGN_OK;
    for (int sl = 0; sl < AGN_ROPE_CACHE_SLOTS; sl++)
        if ((g->rope_slots & (1u << sl)) && ctx->rope_slots[sl].graph_refs > 0) ctx->rope_slots[sl].graph_refs--;
    if (g->exec) cudaGraphExecDestroy(g->exec);
    if (g->graph) cudaGraphDestroy(g->graph);
    delete g;
    (void)cudaGetLastError();
    return AGN_OK;
}

// One empty kernel on the context's stream: the launch-latency floor that the decode-shaped
// (launch-bound) measurements are compared with.
extern "C" int32_t agn_launch_noop(agn_ctx *ctx) {
    AGN_CHECK_CTX(ctx);
    AGN_CUDA(ctx, cudaSetDevice(ctx->device));
    agn_launch(ctx, noop_kernel, dim3(1), dim3(32), 0);
    AGN_LAUNCHED(ctx, "noop");
    return AGN_OK;
}

// The reference builds its sin/cos table from
//   freq = pos as f32 * freq_scale / theta.powf(2.0 * d as f32 / n_rot as f32)
// (src/model/llama/cpu_path.rs:107-112, :474-479).  Device powf differs from libm's by
// an ulp now and then, which at pos ~ 3e4 moves the angle by ~1e-3 rad.  The powf values
// are therefore produced here, once per (theta, n_rot), by the host libm, and the kernel
// only performs the IEEE multiply and divide.
int32_t agn_rope_table(agn_ctx *ctx, float theta, int32_t n_rot, const float **d_table) {
    const int half = n_rot / 2;
    if (half < 1 || half > AGN_ROPE_MAX_HALF)
        return agn_fail(ctx, AGN_EINVAL, "rope: n_rot=%d outside [2, %d]", n_rot, 2 * AGN_ROPE_MAX_HALF);
    uint32_t bits;
    memcpy(&bits, &theta, 4);
    for (int s = 0; s < AGN_ROPE_CACHE_SLOTS; s++) {
        const agn_rope_slot &sl = ctx->rope_slots[s];
        if (sl.used && sl.theta_bits == bits && sl.n_rot == n_rot) {
            if (ctx->capturing) ctx->capture_rope_slots |= 1u << s;
            *d_table = ctx->d_rope_denom + (size_t)s * AGN_ROPE_MAX_HALF;
            return AGN_OK;
        }
    }
    // Building a table copies from a pinned staging slot and may synchronise the stream: neither
    // can be recorded into a graph (a replay would re-copy whatever the staging slot holds by then).
    if (ctx->capturing)
        return agn_fail(ctx, AGN_EINVAL, "rope: the table for theta=%g n_rot=%d does not exist yet; run the op once before "
                        "recording it into a graph", (double)theta, n_rot);
    // round robin over the slots that no recorded graph points at
    int s = -1;
    for (int k = 0; k < AGN_ROPE_CACHE_SLOTS; k++) {
        const int c = (ctx->rope_next + k) % AGN_ROPE_CACHE_SLOTS;
        if (ctx->rope_slots[c].graph_refs == 0) { s = c; break; }
    }
    if (s < 0)
        return agn_fail(ctx, AGN_EINVAL, "rope: all %d (theta, n_rot) table slots are in use by recorded graphs", AGN_ROPE_CACHE_SLOTS);
    ctx->rope_next = (s + 1) % AGN_ROPE_CACHE_SLOTS;
    float *h = ctx->h_rope_denom + (size_t)s * AGN_ROPE_MAX_HALF;
    float *d = ctx->d_rope_denom + (size_t)s * AGN_ROPE_MAX_HALF;
    if (ctx->rope_slots[s].used) {
        // The pinned staging slot may still be the source of an in-flight copy.
        AGN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    }
    for (int i = 0; i < half; i++) h[i] = powf(theta, 2.0f * (float)i / (float)n_rot);
    AGN_CUDA(ctx, cudaMemcpyAsync(d, h, sizeof(float) * half, cudaMemcpyHostToDevice, ctx->stream));
    ctx->rope_slots[s].used = true;
    ctx->rope_slots[s].theta_bits = bits;
    ctx->rope_slots[s].n_rot = n_rot;
    *d_table = d;
    return AGN_OK;
}
