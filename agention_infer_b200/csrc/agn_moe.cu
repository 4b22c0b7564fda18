// MoE routing ops for token rows: router softmax + top-2, and the stable gather of the
// hidden rows by expert that feeds the per-expert SwiGLU.
//
// The reference does not implement an MoE forward pass; the semantics follow its design
// notes (docs/08-moe-routing.md:27-33, docs/05-inference-pipeline.md:271-317):
//   probs = softmax(router logits) ; pick the top-k experts ; weights = their probabilities,
//   not renormalised.
// Selection compares the logits (softmax is monotonic, so this is top-k by probability
// without depending on exp rounding); ties go to the lower expert index.
//
// gather_rows_by_expert is a stable counting sort of the 2T (token, slot) pairs by expert
// (order inside an expert: ascending token, slot 0 before slot 1) followed by a row copy:
//   1. count   : per chunk of 1024 pairs, a histogram over experts      -> scratch
//   2. scan    : exclusive scan over (expert, chunk)                    -> scratch, offsets
//   3. place   : stable rank of each pair inside its chunk (warp match + warp prefix)
//   4. gather  : out[dst] = x[src_token[dst]], 128-bit streaming copies (bound by HBM:
//                8 bytes per gathered element)
#include <math.h>
#include <stdarg.h>

#include "agn_common.cuh"

namespace {

constexpr int CHUNK = 1024;  // pairs per CTA in count/place
constexpr int MAX_EXPERTS = 64;

__global__ void __launch_bounds__(256)
router_top2_kernel(const float *__restrict__ logits, int64_t T, int E, int32_t *__restrict__ idx, float *__restrict__ w) {
    agn_pdl_prologue();
    const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= T) return;
    const float *l = logits + t * E;
    // softmax statistics in the reference's order: max by left fold, then sequential sum
    float m = -INFINITY;
    for (int e = 0; e < E; e++) m = fmaxf(m, l[e]);
    float sum = 0.0f;
    for (int e = 0; e < E; e++) sum += expf(l[e] - m);
    int b0 = 0;
    for (int e = 1; e < E; e++)
        if (l[e] > l[b0]) b0 = e;
    int b1 = -1;
    for (int e = 0; e < E; e++) {
        if (e == b0) continue;
        if (b1 < 0 || l[e] > l[b1]) b1 = e;
    }
    idx[2 * t] = b0;
    idx[2 * t + 1] = b1;
    w[2 * t] = expf(l[b0] - m) / sum;
    w[2 * t + 1] = b1 >= 0 ? expf(l[b1] - m) / sum : 0.0f;
}

__global__ void __launch_bounds__(CHUNK)
expert_count_kernel(const int32_t *__restrict__ idx, int64_t n_pairs, int E, int32_t *__restrict__ chunk_counts,
                    uint32_t *flags) {
    agn_pdl_prologue();
    __shared__ int cnt[MAX_EXPERTS];
    if (threadIdx.x < MAX_EXPERTS) cnt[threadIdx.x] = 0;
    __syncthreads();
    const int64_t i = (int64_t)blockIdx.x * CHUNK + threadIdx.x;
    if (i < n_pairs) {
        const int e = idx[i];
        if (e >= 0 && e < E) atomicAdd(&cnt[e], 1);
        else atomicOr(flags, AGN_FLAG_OOB_EXPERT);
    }
    __syncthreads();
    if (threadIdx.x < E) chunk_counts[(int64_t)blockIdx.x * E + threadIdx.x] = cnt[threadIdx.x];
}

// One CTA.  chunk_counts[c][e] -> exclusive position of (e, c) in expert-major order.
__global__ void __launch_bounds__(MAX_EXPERTS)
expert_scan_kernel(int32_t *__restrict__ chunk_counts, int n_chunks, int E, int32_t *__restrict__ offsets) {
    agn_pdl_prologue();
    __shared__ int total[MAX_EXPERTS + 1];
    const int e = threadIdx.x;
    if (e < E) {
        int run = 0;
        for (int c = 0; c < n_chunks; c++) {
            const int v = chunk_counts[(int64_t)c * E + e];
            chunk_counts[(int64_t)c * E + e] = run;
            run += v;
        }
        total[e] = run;
    }
    __syncthreads();
    if (e == 0) {
        int run = 0;
        for (int k = 0; k < E; k++) {
            const int v = total[k];
            total[k] = run;
            offsets[k] = run;
            run += v;
        }
        offsets[E] = run;
    }
    __syncthreads();
    if (e < E)
        for (int c = 0; c < n_chunks; c++) chunk_counts[(int64_t)c * E + e] += total[e];
}

__global__ void __launch_bounds__(CHUNK)
expert_place_kernel(const int32_t *__restrict__ idx, int64_t n_pairs, int E, const int32_t *__restrict__ chunk_base,
                    int32_t *__restrict__ src_token, int32_t *__restrict__ src_slot) {
    agn_pdl_prologue();
    __shared__ int warp_cnt[CHUNK / 32][MAX_EXPERTS];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int k = threadIdx.x; k < (CHUNK / 32) * MAX_EXPERTS; k += blockDim.x) (&warp_cnt[0][0])[k] = 0;
    __syncthreads();
    const int64_t i = (int64_t)blockIdx.x * CHUNK + threadIdx.x;
    int e = -1;
    if (i < n_pairs) {
        e = idx[i];
        if (e < 0 || e >= E) e = -1;
    }
    // lanes of this warp holding the same expert; the rank inside the warp keeps lane order
    const unsigned same = __match_any_sync(0xffffffffu, e);
    const int rank_in_warp = __popc(same & ((1u << lane) - 1u));
    if (e >= 0 && rank_in_warp == 0) warp_cnt[warp][e] = __popc(same);
    __syncthreads();
    if (e >= 0) {
        int before = 0;
        for (int w = 0; w < warp; w++) before += warp_cnt[w][e];
        const int dst = chunk_base[(int64_t)blockIdx.x * E + e] + before + rank_in_warp;
        src_token[dst] = (int32_t)(i >> 1);
        src_slot[dst] = (int32_t)(i & 1);
    }
}

// Up to SMALL_SORT_PAIRS pairs (decode and small prefill batches): the whole counting sort in ONE
// CTA and one launch (count, scan and place of the three-kernel path, plus the -1 fill of the slots
// that dropped pairs leave empty).  At this size three dependent launches and a memset cost more
// in launch latency than the sort itself (T = 64: 17.4 -> 9.3 us for sort + copy; T = 2048: 27.4 ->
// 22.9 us); from 8192 tokens on, one CTA is slower than the three grids (94 vs 90 us).  Warp w owns the contiguous segment
// [w * seg, (w + 1) * seg) of the pairs, so "warp order, then iteration order, then lane order" is
// pair order and the sort is stable.
constexpr int SMALL_SORT_PAIRS = 4096;
constexpr int SMALL_SORT_WARPS = 32;

__global__ void __launch_bounds__(SMALL_SORT_WARPS * 32)
expert_sort_small_kernel(const int32_t *__restrict__ idx, int n_pairs, int E, int32_t *__restrict__ offsets,
                         int32_t *__restrict__ src_token, int32_t *__restrict__ src_slot, uint32_t *flags) {
    agn_pdl_prologue();
    __shared__ int base[SMALL_SORT_WARPS][MAX_EXPERTS];  // counts, then running destination of (warp, expert)
    __shared__ int total[MAX_EXPERTS + 1];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int k = threadIdx.x; k < SMALL_SORT_WARPS * MAX_EXPERTS; k += blockDim.x) (&base[0][0])[k] = 0;
    __syncthreads();
    const int seg = ((n_pairs + SMALL_SORT_WARPS - 1) / SMALL_SORT_WARPS + 31) & ~31;  // a multiple of the warp size
    const int begin = warp * seg, end = min(begin + seg, n_pairs);
    bool bad = false;
    for (int i0 = begin; i0 < end; i0 += 32) {
        const int i = i0 + lane;
        int e = -1;
        if (i < end) {
            e = idx[i];
            if (e < 0 || e >= E) { e = -1; bad = true; }
        }
        const unsigned same = __match_any_sync(0xffffffffu, e);
        if (e >= 0 && (same & ((1u << lane) - 1u)) == 0) base[warp][e] += __popc(same);  // one lane per expert present
        __syncwarp();
    }
    if (bad) atomicOr(flags, AGN_FLAG_OOB_EXPERT);
    __syncthreads();
    if (threadIdx.x < E) {  // exclusive scan over the warps of one expert
        const int e = threadIdx.x;
        int run = 0;
        for (int w = 0; w < SMALL_SORT_WARPS; w++) {
            const int v = base[w][e];
            base[w][e] = run;
            run += v;
        }
        total[e] = run;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0;
        for (int k = 0; k < E; k++) {
            const int v = total[k];
            total[k] = run;
            offsets[k] = run;
            run += v;
        }
        total[E] = run;
        offsets[E] = run;
    }
    __syncthreads();
    for (int i0 = begin; i0 < end; i0 += 32) {
        const int i = i0 + lane;
        int e = -1;
        if (i < end) {
            e = idx[i];  // second touch: an L1 / L2 hit
            if (e < 0 || e >= E) e = -1;
        }
        const unsigned same = __match_any_sync(0xffffffffu, e);
        const int rank = __popc(same & ((1u << lane) - 1u));
        if (e >= 0) {
            const int dst = total[e] + base[warp][e] + rank;
            src_token[dst] = i >> 1;
            src_slot[dst] = i & 1;
        }
        __syncwarp();
        if (e >= 0 && rank == 0) base[warp][e] += __popc(same);
        __syncwarp();
    }
    // slots past the last placed pair belong to dropped pairs (expert out of range): mark them empty
    for (int k = total[E] + threadIdx.x; k < n_pairs; k += blockDim.x) src_token[k] = -1;
}

__global__ void __launch_bounds__(256)
gather_rows_kernel(const float *__restrict__ x, const int32_t *__restrict__ src_token, int64_t n_out, int64_t T,
                   int64_t H, float *__restrict__ out, int vec) {
    agn_pdl_prologue();
    const int64_t r = blockIdx.x;
    const int64_t t = src_token[r];
    if (t < 0 || t >= T) return;
    if (vec) {
        const float4 *s = reinterpret_cast<const float4 *>(x + t * H);
        float4 *d = reinterpret_cast<float4 *>(out + r * H);
        const int n4 = (int)(H >> 2);
        // four loads in flight per thread before the first store
        for (int base = threadIdx.x; base < n4; base += 4 * blockDim.x) {
            float4 v[4];
#pragma unroll
            for (int k = 0; k < 4; k++) {
                const int i = base + k * blockDim.x;
                v[k] = i < n4 ? __ldg(s + i) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int k = 0; k < 4; k++) {
                const int i = base + k * blockDim.x;
                if (i < n4) agn_st_stream(d + i, v[k]);
            }
        }
    } else {
        for (int64_t i = threadIdx.x; i < H; i += blockDim.x) out[r * H + i] = x[t * H + i];
    }
}

}  // namespace

size_t agn_gather_scratch_bytes(int64_t T, int32_t n_experts) {
    const int64_t n_chunks = (2 * T + CHUNK - 1) / CHUNK;
    return (size_t)n_chunks * (size_t)n_experts * sizeof(int32_t);
}

// Shared by the context-workspace entry point and any caller that brings its own scratch.
int32_t agn_gather_rows_by_expert_impl(agn_ctx *ctx, const float *x, const int32_t *idx, int64_t T, int64_t H,
                                       int32_t n_experts, float *out, int32_t *offsets, int32_t *src_token,
                                       int32_t *src_slot, int32_t *scratch) {
    const int64_t n_pairs = 2 * T;
    const int n_chunks = (int)((n_pairs + CHUNK - 1) / CHUNK);
    const int vec = (H % 4 == 0 && agn_aligned16(x) && agn_aligned16(out)) ? 1 : 0;
    if (n_pairs <= SMALL_SORT_PAIRS && ctx->tune_moe_small_sort) {
        agn_launch(ctx, expert_sort_small_kernel, dim3(1), dim3(SMALL_SORT_WARPS * 32), 0, idx, (int)n_pairs, n_experts, offsets,
                   src_token, src_slot, ctx->d_flags);
        AGN_LAUNCHED(ctx, "expert_sort_small");
        agn_launch(ctx, gather_rows_kernel, dim3((unsigned)n_pairs), dim3(256), 0, x, src_token, n_pairs, T, H, out, vec);
        AGN_LAUNCHED(ctx, "gather_rows");
        ctx->flags_dirty = true;
        return AGN_OK;
    }
    // pairs with an out-of-range expert are skipped by `place`; mark their slots as empty
    AGN_CUDA(ctx, cudaMemsetAsync(src_token, 0xFF, sizeof(int32_t) * (size_t)n_pairs, ctx->stream));
    agn_launch(ctx, expert_count_kernel, dim3(n_chunks), dim3(CHUNK), 0, idx, n_pairs, n_experts, scratch, ctx->d_flags);
    AGN_LAUNCHED(ctx, "expert_count");
    agn_launch(ctx, expert_scan_kernel, dim3(1), dim3(MAX_EXPERTS), 0, scratch, n_chunks, n_experts, offsets);
    AGN_LAUNCHED(ctx, "expert_scan");
    agn_launch(ctx, expert_place_kernel, dim3(n_chunks), dim3(CHUNK), 0, idx, n_pairs, n_experts, scratch, src_token, src_slot);
    AGN_LAUNCHED(ctx, "expert_place");
    agn_launch(ctx, gather_rows_kernel, dim3((unsigned)n_pairs), dim3(256), 0, x, src_token, n_pairs, T, H, out, vec);
    AGN_LAUNCHED(ctx, "gather_rows");
    ctx->flags_dirty = true;
    return AGN_OK;
}

extern "C" int32_t agn_router_top2_f32(agn_ctx *ctx, const float *logits, int64_t T, int32_t n_experts, int32_t *idx,
                                       float *w) {
    AGN_CHECK_CTX(ctx);
    if (T < 0 || n_experts < 2 || n_experts > 1024)
        return agn_fail(ctx, AGN_EINVAL, "router_top2: T=%lld n_experts=%d (need 2..1024)", (long long)T, n_experts);
    if (T == 0) return AGN_OK;
    if (!logits || !idx || !w) return agn_fail(ctx, AGN_EINVAL, "router_top2: null pointer");
    AGN_CUDA(ctx, cudaSetDevice(ctx->device));
    const int64_t blocks = (T + 255) / 256;
    if (blocks > 0x7fffffffLL) return agn_fail(ctx, AGN_EINVAL, "router_top2: T too large");
    agn_launch(ctx, router_top2_kernel, dim3((unsigned)blocks), dim3(256), 0, logits, T, n_experts, idx, w);
    AGN_LAUNCHED(ctx, "router_top2");
    return AGN_OK;
}

extern "C" int32_t agn_gather_rows_by_expert_f32(agn_ctx *ctx, const float *x, const int32_t *idx, int64_t T, int64_t H,
                                                 int32_t n_experts, float *out, int32_t *offsets, int32_t *src_token,
                                                 int32_t *src_slot) {
    AGN_CHECK_CTX(ctx);
    if (T < 0 || H <= 0 || n_experts < 1 || n_experts > MAX_EXPERTS)
        return agn_fail(ctx, AGN_EINVAL, "gather_rows_by_expert: T=%lld H=%lld n_experts=%d (need 1..%d)", (long long)T,
                        (long long)H, n_experts, MAX_EXPERTS);
    if (!offsets) return agn_fail(ctx, AGN_EINVAL, "gather_rows_by_expert: null offsets");
    AGN_CUDA(ctx, cudaSetDevice(ctx->device));
    if (T == 0) {
        AGN_CUDA(ctx, cudaMemsetAsync(offsets, 0, sizeof(int32_t) * (n_experts + 1), ctx->stream));
        return AGN_OK;
    }
    if (!x || !idx || !out || !src_token || !src_slot) return agn_fail(ctx, AGN_EINVAL, "gather_rows_by_expert: null pointer");
    if (2 * T > 0x7fffffffLL) return agn_fail(ctx, AGN_EINVAL, "gather_rows_by_expert: T too large");
    const size_t need = agn_gather_scratch_bytes(T, n_experts);
    if (need > ctx->scratch_bytes)
        return agn_fail(ctx, AGN_EINVAL, "gather_rows_by_expert: needs %zu bytes of workspace, the context holds %zu", need,
                        ctx->scratch_bytes);
    return agn_gather_rows_by_expert_impl(ctx, x, idx, T, H, n_experts, out, offsets, src_token, src_slot,
                                          static_cast<int32_t *>(ctx->d_scratch));
}

// ------------------------------------------------------------------------------------------
// Allocation-free variant of gather_rows_by_expert.
//
// Who needs it: a host that has handed the whole GPU to its own arena (an inference server
// that sizes its KV cache to all free memory has nothing left for cudaMalloc to give out),
// and a host that must not allocate inside its serving loop because cudaMalloc / cudaFree
// stall every stream of the device.  Such a host cannot create an agn_ctx either: context
// creation allocates the workspace this op normally uses.  This entry point therefore takes
// no context and gets its scratch from a fixed array that is part of the loaded library.
//
// The array lives in every GPU on which the library's device code has been loaded (with lazy
// module loading: from the first call on that device, which is why hosts make a T = 0 warm-up
// call at start-up) until the process exits; its size is the limit of the problem size (see
// AGN_NOALLOC_SCRATCH_BYTES).  All calls share it: it still
// holds the previous call's counts when the next call starts, and two calls that run on the
// GPU at the same time (different streams, no event between them) overwrite each other.
#define AGN_NOALLOC_SCRATCH_BYTES (256 * 1024)
// Word 0 of the header takes the count kernel's "expert index out of range" bit.  It is write-only
// here: no entry point reads it back (that would need a synchronisation); the kernel is shared
// with the context-based op, which does report the bit.  A dropped pair shows in the outputs instead.
#define AGN_NOALLOC_HEADER_BYTES 256
static __device__ __align__(256) unsigned char g_noalloc_scratch[AGN_NOALLOC_SCRATCH_BYTES];

namespace {
constexpr int NOALLOC_MAX_DEVICES = 64;
std::mutex g_noalloc_mutex;
void *g_noalloc_dev_ptr[NOALLOC_MAX_DEVICES] = {};

int32_t noalloc_fail(char *err, size_t err_len, int32_t status, const char *fmt, ...) {
    if (err && err_len) {
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(err, err_len, fmt, ap);
        va_end(ap);
    }
    return status;
}
}  // namespace

extern "C" int32_t agn_gather_rows_by_expert_noalloc_f32(void *cuda_stream, const float *x, const int32_t *idx, int64_t T,
                                                         int64_t H, int32_t n_experts, float *out, int32_t *offsets,
                                                         int32_t *src_token, int32_t *src_slot, char *err, size_t err_len) {
    if (err && err_len) err[0] = '\0';
    if (T < 0 || H <= 0 || n_experts < 1 || n_experts > MAX_EXPERTS)
        return noalloc_fail(err, err_len, AGN_EINVAL, "gather_rows_by_expert_noalloc: T=%lld H=%lld n_experts=%d (need 1..%d)",
                            (long long)T, (long long)H, n_experts, MAX_EXPERTS);
    if (!offsets || (T > 0 && (!x || !idx || !out || !src_token || !src_slot)))
        return noalloc_fail(err, err_len, AGN_EINVAL, "gather_rows_by_expert_noalloc: null pointer");
    if (2 * T > 0x7fffffffLL) return noalloc_fail(err, err_len, AGN_EINVAL, "gather_rows_by_expert_noalloc: T too large");
    const int64_t n_pairs = 2 * T;
    const int64_t n_chunks = (n_pairs + CHUNK - 1) / CHUNK;
    const size_t need = AGN_NOALLOC_HEADER_BYTES + (size_t)n_chunks * (size_t)n_experts * sizeof(int32_t);
    if (need > AGN_NOALLOC_SCRATCH_BYTES)
        return noalloc_fail(err, err_len, AGN_EINVAL,
                            "gather_rows_by_expert_noalloc: T=%lld with %d experts needs %zu bytes of scratch, the built-in "
                            "array holds %d (limit: ceil(2T/1024)*n_experts <= %d); use agn_gather_rows_by_expert_f32",
                            (long long)T, n_experts, need, AGN_NOALLOC_SCRATCH_BYTES,
                            (AGN_NOALLOC_SCRATCH_BYTES - AGN_NOALLOC_HEADER_BYTES) / 4);
    cudaStream_t stream = reinterpret_cast<cudaStream_t>(cuda_stream);
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= NOALLOC_MAX_DEVICES) {
        (void)cudaGetLastError();
        return noalloc_fail(err, err_len, AGN_ECUDA, "gather_rows_by_expert_noalloc: no current CUDA device (%s)",
                            cudaGetErrorString(e));
    }
    // Set-up, once per device, with that device current: in host code the array's name is
    // only a handle; the address kernels can use comes from cudaGetSymbolAddress.  The stream
    // must belong to this (the current) device.
    void *scratch = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_noalloc_mutex);
        if (!g_noalloc_dev_ptr[dev]) {
            void *p = nullptr;
            e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
            if (e != cudaSuccess || !p) {
                (void)cudaGetLastError();
                return noalloc_fail(err, err_len, AGN_ECUDA, "gather_rows_by_expert_noalloc: cudaGetSymbolAddress failed: %s",
                                    cudaGetErrorString(e));
            }
            g_noalloc_dev_ptr[dev] = p;
        }
        scratch = g_noalloc_dev_ptr[dev];
    }
#define NOALLOC_CUDA(call)                                                                                              \
    do {                                                                                                                \
        cudaError_t _e = (call);                                                                                        \
        if (_e != cudaSuccess) {                                                                                        \
            (void)cudaGetLastError();                                                                                   \
            return noalloc_fail(err, err_len, AGN_ECUDA, "gather_rows_by_expert_noalloc: %s failed: %s", #call,         \
                                cudaGetErrorString(_e));                                                                \
        }                                                                                                               \
    } while (0)
    if (T == 0) {
        NOALLOC_CUDA(cudaMemsetAsync(offsets, 0, sizeof(int32_t) * (n_experts + 1), stream));
        return AGN_OK;
    }
    uint32_t *flags = static_cast<uint32_t *>(scratch);
    int32_t *counts = reinterpret_cast<int32_t *>(static_cast<unsigned char *>(scratch) + AGN_NOALLOC_HEADER_BYTES);
    // What must start clean: the flag word (left over from an earlier call) and the slots of
    // dropped pairs.  The counts need no clearing: the count kernel overwrites every entry
    // that the scan and place kernels of this call read.
    NOALLOC_CUDA(cudaMemsetAsync(flags, 0, AGN_NOALLOC_HEADER_BYTES, stream));
    NOALLOC_CUDA(cudaMemsetAsync(src_token, 0xFF, sizeof(int32_t) * (size_t)n_pairs, stream));
    expert_count_kernel<<<(unsigned)n_chunks, CHUNK, 0, stream>>>(idx, n_pairs, n_experts, counts, flags);
    NOALLOC_CUDA(cudaPeekAtLastError());
    expert_scan_kernel<<<1, MAX_EXPERTS, 0, stream>>>(counts, (int)n_chunks, n_experts, offsets);
    NOALLOC_CUDA(cudaPeekAtLastError());
    expert_place_kernel<<<(unsigned)n_chunks, CHUNK, 0, stream>>>(idx, n_pairs, n_experts, counts, src_token, src_slot);
    NOALLOC_CUDA(cudaPeekAtLastError());
    const int vec = (H % 4 == 0 && agn_aligned16(x) && agn_aligned16(out)) ? 1 : 0;
    gather_rows_kernel<<<(unsigned)n_pairs, 256, 0, stream>>>(x, src_token, n_pairs, T, H, out, vec);
    NOALLOC_CUDA(cudaPeekAtLastError());
#undef NOALLOC_CUDA
    return AGN_OK;
}
