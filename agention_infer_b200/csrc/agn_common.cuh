// Shared internals of libagention_b200: context struct, error plumbing, device helpers.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include <map>
#include <mutex>
#include <string>
#include <tuple>

#include "agention_b200.h"

// Device-side error bits kernels may OR into agn_ctx::d_flags[0].
#define AGN_FLAG_OOB_ID 1u       // get_rows: token id >= n_rows
#define AGN_FLAG_TIMEOUT 2u      // a bounded staging wait gave up
#define AGN_FLAG_OOB_EXPERT 4u   // gather_rows_by_expert: expert index outside [0, n_experts)
#define AGN_FLAG_OOB_SLOT 8u     // kv_write / fused cache write: position outside [0, max_seq_len)

// Polls of an mbarrier before a staging wait gives up (a few hundred ms at most); the option
// "mbar_spin_limit" overrides it per context.
#define AGN_MBAR_SPIN_LIMIT_DEFAULT (1 << 22)

#define AGN_ROPE_CACHE_SLOTS 16
#define AGN_ROPE_MAX_HALF 512  // n_rot <= 1024
#define AGN_SCRATCH_BYTES (1u << 20)

struct agn_host_pipe;  // staging ring of the host-slice entry points (agn_host_ops.cu)

struct agn_rope_slot {
    uint32_t theta_bits;
    int32_t n_rot;
    bool used;
    int graph_refs;  // recorded graphs that point at this table (counted at agn_graph_end, released at agn_graph_destroy): never evicted while > 0
};

struct agn_ctx {
    int device;
    int sm_count;
    cudaStream_t own_stream;
    cudaStream_t stream;        // own_stream or an adopted one
    uint32_t *d_flags;          // [4] device error bits
    uint32_t *h_flags;          // pinned mirror
    float *d_rope_denom;        // [AGN_ROPE_CACHE_SLOTS][AGN_ROPE_MAX_HALF]
    float *h_rope_denom;        // pinned staging, same shape
    void *d_scratch;            // workspace for ops that need one (gather_rows_by_expert)
    size_t scratch_bytes;
    agn_host_pipe *host_pipe;   // created by the first host-slice call
    bool pdl;                   // launch kernels with programmatic stream serialization
    bool capturing;             // between agn_graph_begin and agn_graph_end
    uint64_t capture_launches0;
    uint32_t capture_rope_slots; // bit s: the open capture recorded a kernel that reads rope table slot s
    int tune_rms_vpt;           // 0 = automatic; 1/2/4/8 float4 per thread in rms_norm
    int tune_rms_recip;         // rms_norm multiplies by 1/rms instead of dividing each element (default 1)
    int tune_get_rows_threads;  // 0 = automatic
    int tune_moe_small_sort;    // 1 = up to 4096 (token, slot) pairs are sorted by one CTA in one launch (default)
    int tune_softmax_cluster;   // rows of 16K-128K entries: 1 = one thread-block cluster per row, CTAs of <= 512 threads
                                // (default); 2 = CTAs of <= 256 threads; 0 = no clusters
    int tune_rms_q8k_bpw;         // RMSNorm -> Q8_K: blocks of 256 values per warp (1, 2, 4); 0 = by row length
    int tune_softmax_causal_pair; // 1 (default): square causal matrices pair rows i and L-1-i in one CTA
    int tune_softmax_warp16;    // 1: rows of 1025-2048 entries run one warp per row (16 float4 per lane); 0: one CTA per row
    int tune_softmax_vpt;       // 0 = automatic (8 float4 per thread in the CTA-per-row kernel)
    int tune_get_rows_tma;      // stage the quantised row with one bulk asynchronous copy (TMA)
    int tune_silu_unroll;       // float4 pairs in flight per thread in silu_mul: 2, 4 (default) or 8
    int tune_silu_threads;      // 128, 256 (default) or 512
    int tune_kv_multi;          // 1 (default): kv_write packs four tokens per CTA for batches that fill the GPU that way
    int tune_silu_small;        // 1 (default): decode-sized inputs run one float4 pair per thread in 128-thread CTAs
    // Persistent kernels with a shared-memory row ring (rows staged by bulk asynchronous copies
    // ahead of the row being processed).  *_ring: 0 = never (default: on B200 the CTA-per-row
    // kernels measured 5-15 % faster at every batch size), 1 = a ring of the default depth for
    // batches large enough to keep it busy, >= 2 = that many slots; *_ring_ctas: resident CTAs per
    // SM (0 = as many as fit).
    int tune_rms_ring, tune_rms_ring_ctas;
    int tune_rope_ring, tune_rope_ring_ctas;
    int tune_get_rows_ring, tune_get_rows_ring_ctas;
    int tune_softmax_ring, tune_softmax_ring_ctas;
    int tune_host_slots;        // host-slice ops: slots of the staging ring (2..16, read when the ring is created; 0 = 8)
    int tune_host_chunk_bytes;  // host-slice ops: bytes of one staging chunk over all buffers (0 = a whole 24 MiB slot)
    int tune_ring_force;        // 1 = take the persistent form whenever it applies, however few rows (tests)
    int mbar_spin_limit;        // polls before a staging wait gives up
    int test_idle_barrier_wait; // test hook (0 in normal use): after its row has arrived, every CTA of get_rows also waits on a
                                // barrier that nothing ever signals, so that the bounded wait runs out and is reported
    agn_rope_slot rope_slots[AGN_ROPE_CACHE_SLOTS];
    int rope_next;
    bool flags_dirty;           // a kernel that can raise a flag ran since the last sync
    uint64_t launches;
    bool ring_launched;         // set by a launcher that took the persistent form (read right after the launch)
    const char *last_kernel;    // name given to AGN_LAUNCHED by the most recent launch (a string literal)
    std::string last_error;
};

struct agn_event {
    cudaEvent_t ev;
};

int32_t agn_fail(agn_ctx *ctx, int32_t status, const char *fmt, ...);
void agn_host_pipe_destroy(agn_ctx *ctx);
int32_t agn_host_pipe_join(agn_ctx *ctx);  // the context's stream waits for the host-slice downloads enqueued so far

// Device pointer to the powf(theta, 2d/n_rot) table, d < n_rot/2 (built on the host
// with libm the first time a (theta, n_rot) pair is seen).
int32_t agn_rope_table(agn_ctx *ctx, float theta, int32_t n_rot, const float **d_table);

#define AGN_CHECK_CTX(ctx) \
    do {                   \
        if (!(ctx)) return AGN_EINVAL; \
    } while (0)

#define AGN_CUDA(ctx, call)                                                            \
    do {                                                                               \
        cudaError_t _e = (call);                                                       \
        if (_e != cudaSuccess)                                                         \
            return agn_fail((ctx), AGN_ECUDA, "%s failed: %s (%s:%d)", #call,          \
                            cudaGetErrorString(_e), __FILE__, __LINE__);               \
    } while (0)

// After a kernel launch: count it and surface launch-configuration errors.
#define AGN_LAUNCHED(ctx, name)                                                        \
    do {                                                                               \
        (ctx)->launches++;                                                             \
        (ctx)->last_kernel = (name);                                                   \
        cudaError_t _e = cudaPeekAtLastError();                                        \
        if (_e != cudaSuccess) {                                                       \
            (void)cudaGetLastError();                                                  \
            return agn_fail((ctx), AGN_ECUDA, "launch of %s failed: %s", name,         \
                            cudaGetErrorString(_e));                                   \
        }                                                                              \
    } while (0)

static inline bool agn_aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
static inline bool agn_aligned(const void *p, int a) { return (reinterpret_cast<uintptr_t>(p) & (uintptr_t)(a - 1)) == 0; }

#ifdef __CUDACC__

// --- bulk asynchronous copies (TMA, 1-D, this CTA's own shared memory only; no multicast) -----------
// A copy needs 16-byte aligned source, destination and size; it completes on an mbarrier whose
// wait is bounded: after `limit` polls the caller raises AGN_FLAG_TIMEOUT and leaves.
__device__ __forceinline__ uint32_t agn_smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void agn_mbar_init(uint64_t *bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(agn_smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void agn_mbar_init_fence() { asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory"); }
__device__ __forceinline__ void agn_mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(agn_smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void agn_bulk_g2s(void *smem_dst, const void *gmem_src, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(
                     agn_smem_u32(smem_dst)),
                 "l"(gmem_src), "r"(bytes), "r"(agn_smem_u32(bar))
                 : "memory");
}
// true once the phase with the given parity has completed; false after `limit` polls
__device__ __forceinline__ bool agn_mbar_wait(uint64_t *bar, uint32_t parity, int limit) {
    const uint32_t b = agn_smem_u32(bar);
    for (int it = 0; it < limit; it++) {
        uint32_t done;
        asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
                     : "=r"(done)
                     : "r"(b), "r"(parity)
                     : "memory");
        if (done) return true;
    }
    return false;
}

// Programmatic dependent launch.  Every kernel of this library starts with
// agn_pdl_prologue(): it lets the next kernel in the stream be scheduled onto SMs as this
// grid's CTAs retire (hiding its launch latency), and it blocks until the previous grid has
// completed and flushed its writes, before the first global access of this one.
__device__ __forceinline__ void agn_pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void agn_pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void agn_pdl_prologue() {
    agn_pdl_launch_dependents();
    agn_pdl_wait();
}

template <typename... KArgs, typename... Args>
inline void agn_launch(agn_ctx *ctx, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ctx->pdl ? 1 : 0;
    (void)cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);  // errors surface in AGN_LAUNCHED
}

// The same with a thread-block cluster of cluster_x CTAs along x (grid.x must be a multiple of it).
template <typename... KArgs, typename... Args>
inline void agn_launch_cluster(agn_ctx *ctx, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, int cluster_x,
                               Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)cluster_x;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ctx->pdl ? 2 : 1;
    (void)cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);  // errors surface in AGN_LAUNCHED
}

// Resident CTAs per SM of a persistent kernel for a launch shape, asked of the runtime once per
// (device, kernel, threads, shared memory).  The first call for a (device, kernel) also opts the
// kernel in to the device's largest dynamic shared-memory size, once, so that later launches with
// any smaller or larger ring are all valid.
template <typename K>
inline int agn_ring_ctas_per_sm(agn_ctx *ctx, K kernel, int threads, size_t smem) {
    static std::mutex mu;
    static std::map<std::tuple<int, const void *, int, size_t>, int> cache;
    static std::map<std::tuple<int, const void *>, int> opted;  // value: the opt-in limit in bytes, 0 = failed
    std::lock_guard<std::mutex> lock(mu);
    const void *kp = reinterpret_cast<const void *>(kernel);
    auto o = opted.find(std::make_tuple(ctx->device, kp));
    if (o == opted.end()) {
        int lim = 0;
        cudaFuncAttributes fa;
        // the opt-in limit covers static + dynamic shared memory: ask for what the kernel's static part leaves
        if (cudaDeviceGetAttribute(&lim, cudaDevAttrMaxSharedMemoryPerBlockOptin, ctx->device) != cudaSuccess ||
            cudaFuncGetAttributes(&fa, kernel) != cudaSuccess || (lim -= (int)fa.sharedSizeBytes) <= 0 ||
            cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, lim) != cudaSuccess) {
            (void)cudaGetLastError();
            lim = 0;
        }
        o = opted.emplace(std::make_tuple(ctx->device, kp), lim).first;
    }
    if ((size_t)o->second < smem) return 0;
    const auto key = std::make_tuple(ctx->device, kp, threads, smem);
    auto f = cache.find(key);
    if (f != cache.end()) return f->second;
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, threads, smem) != cudaSuccess) {
        (void)cudaGetLastError();
        n = 0;
    }
    cache[key] = n;
    return n;
}

__device__ __forceinline__ float agn_warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Warp-wide maximum in one instruction (redux.sync.max.f32, sm_100a); a NaN operand is ignored, as
// fmaxf ignores it.  Every lane of the warp must take part.
__device__ __forceinline__ float agn_warp_max(float v) {
    float r;
    asm volatile("redux.sync.max.f32 %0, %1, 0xffffffff;" : "=f"(r) : "f"(v));
    return r;
}
// max(m, x, y, z, w) as two three-input maxima (sm_100); NaN operands are ignored.
__device__ __forceinline__ float agn_max_acc4(float m, float4 v) {
    float t;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(t) : "f"(m), "f"(v.x), "f"(v.y));
    asm("max.f32 %0, %1, %2, %3;" : "=f"(m) : "f"(t), "f"(v.z), "f"(v.w));
    return m;
}

// Activation storage.  The kernels compute in f32; activations are stored as f32 or, like the
// reference's default `Act` type (src/ops/mod.rs:36-45), as f16 (converted with round to
// nearest even on store, `Act::cast_from`).  ActVec<T> moves four consecutive activations:
// one 128-bit access for f32, one 64-bit access for f16.
template <typename T> struct ActVec;
template <> struct ActVec<float> {
    static constexpr int ALIGN = 16;
    static __device__ __forceinline__ float4 load(const float *p, int64_t vec) {
        return __ldcs(reinterpret_cast<const float4 *>(p) + vec);
    }
    static __device__ __forceinline__ void store(float *p, int64_t vec, float4 v) {
        __stcs(reinterpret_cast<float4 *>(p) + vec, v);
    }
    static __device__ __forceinline__ float load1(const float *p, int64_t i) { return p[i]; }
    static __device__ __forceinline__ void store1(float *p, int64_t i, float v) { p[i] = v; }
    // the same four activations from a staged row in shared memory
    static __device__ __forceinline__ float4 load_shared(const float *p, int vec) { return reinterpret_cast<const float4 *>(p)[vec]; }
};
#include <cuda_fp16.h>
template <> struct ActVec<__half> {
    static constexpr int ALIGN = 8;
    static __device__ __forceinline__ float4 load(const __half *p, int64_t vec) {
        const uint2 r = __ldcs(reinterpret_cast<const uint2 *>(p) + vec);
        const float2 a = __half22float2(*reinterpret_cast<const __half2 *>(&r.x));
        const float2 b = __half22float2(*reinterpret_cast<const __half2 *>(&r.y));
        return make_float4(a.x, a.y, b.x, b.y);
    }
    static __device__ __forceinline__ void store(__half *p, int64_t vec, float4 v) {
        const __half2 a = __floats2half2_rn(v.x, v.y), b = __floats2half2_rn(v.z, v.w);
        uint2 r;
        r.x = *reinterpret_cast<const uint32_t *>(&a);
        r.y = *reinterpret_cast<const uint32_t *>(&b);
        __stcs(reinterpret_cast<uint2 *>(p) + vec, r);
    }
    static __device__ __forceinline__ float load1(const __half *p, int64_t i) { return __half2float(p[i]); }
    static __device__ __forceinline__ void store1(__half *p, int64_t i, float v) { p[i] = __float2half_rn(v); }
    static __device__ __forceinline__ float4 load_shared(const __half *p, int vec) {
        const uint2 r = reinterpret_cast<const uint2 *>(p)[vec];
        const float2 a = __half22float2(*reinterpret_cast<const __half2 *>(&r.x));
        const float2 b = __half22float2(*reinterpret_cast<const __half2 *>(&r.y));
        return make_float4(a.x, a.y, b.x, b.y);
    }
};

#include <cuda_bf16.h>
// bf16 is an OUTPUT format only (a normed row handed to a matmul that takes bf16 operands).
template <> struct ActVec<__nv_bfloat16> {
    static constexpr int ALIGN = 8;
    static __device__ __forceinline__ float4 load(const __nv_bfloat16 *p, int64_t vec) {
        const uint2 r = __ldcs(reinterpret_cast<const uint2 *>(p) + vec);
        return make_float4(__uint_as_float(r.x << 16), __uint_as_float(r.x & 0xffff0000u), __uint_as_float(r.y << 16),
                           __uint_as_float(r.y & 0xffff0000u));
    }
    static __device__ __forceinline__ void store(__nv_bfloat16 *p, int64_t vec, float4 v) {
        const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
        uint2 r;
        r.x = *reinterpret_cast<const uint32_t *>(&a);
        r.y = *reinterpret_cast<const uint32_t *>(&b);
        __stcs(reinterpret_cast<uint2 *>(p) + vec, r);
    }
    static __device__ __forceinline__ float load1(const __nv_bfloat16 *p, int64_t i) { return __bfloat162float(p[i]); }
    static __device__ __forceinline__ void store1(__nv_bfloat16 *p, int64_t i, float v) { p[i] = __float2bfloat16_rn(v); }
};

// Packed f32x2 arithmetic (Blackwell: add / mul / fma .rn.f32x2, two IEEE round-to-nearest results
// per instruction, each the same bits as the scalar operation).  The row-wise kernels spend a
// third to a half of their instructions on element-wise float arithmetic; issuing it two at a
// time keeps them bound by memory rather than by instruction issue when the SM clock is low.
__device__ __forceinline__ float4 agn_mul4(float4 a, float4 b) {
    const float2 lo = __fmul2_rn(make_float2(a.x, a.y), make_float2(b.x, b.y));
    const float2 hi = __fmul2_rn(make_float2(a.z, a.w), make_float2(b.z, b.w));
    return make_float4(lo.x, lo.y, hi.x, hi.y);
}
__device__ __forceinline__ float4 agn_scale4(float4 a, float f) { return agn_mul4(a, make_float4(f, f, f, f)); }
// acc + (x^2, y^2) + (z^2, w^2) as two packed fused multiply-adds; acc holds two partial sums
__device__ __forceinline__ float2 agn_sum_sq4(float4 v, float2 acc) {
    return __ffma2_rn(make_float2(v.z, v.w), make_float2(v.z, v.w), __ffma2_rn(make_float2(v.x, v.y), make_float2(v.x, v.y), acc));
}

// Streaming (read-once / write-once) 128-bit accesses: keep them from displacing
// reusable lines (weights, tables) in L1/L2.
__device__ __forceinline__ float4 agn_ld_stream(const float4 *p) { return __ldcs(p); }
__device__ __forceinline__ void agn_st_stream(float4 *p, float4 v) { __stcs(p, v); }

#endif  // __CUDACC__
