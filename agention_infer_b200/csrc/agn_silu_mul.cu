// gate·up -> SiLU·mul (SwiGLU combine), HBM-streaming kernel.
//
// Reference: out = g / (1 + exp(-g)) * u   (src/model/llama/cpu_path.rs:228-229, :975-978;
// GPU twin src/ops/kernels_wgpu.rs:22-31).  12 algorithmic bytes per element, ~25 lane
// instructions: bound by HBM, so the kernel is nothing but 128-bit streaming loads with
// several of them in flight per thread, and 128-bit streaming stores.
#include "agn_common.cuh"
#include "agn_row_math.cuh"

namespace {

// Each CTA owns a contiguous tile of UNROLL * blockDim vectors of four activations; a thread
// issues all of its 2*UNROLL loads before the first use so that UNROLL*32 B (f32) per thread
// are in flight.
// T: storage type of gate and up; OT: storage type of the result (T, or a 16-bit type when the
// product feeds a matmul with half-precision operands).
template <typename T, typename OT, int UNROLL>
__global__ void __launch_bounds__(512)
silu_mul_vec4_kernel(const T *__restrict__ gate, const T *__restrict__ up, OT *__restrict__ out, int64_t n4) {
    agn_pdl_prologue();
    const int64_t tile = (int64_t)blockIdx.x * (UNROLL * blockDim.x);
    float4 g[UNROLL], u[UNROLL];
#pragma unroll
    for (int k = 0; k < UNROLL; k++) {
        const int64_t i = tile + k * blockDim.x + threadIdx.x;
        if (i < n4) {
            g[k] = ActVec<T>::load(gate, i);
            u[k] = ActVec<T>::load(up, i);
        }
    }
#pragma unroll
    for (int k = 0; k < UNROLL; k++) {
        const int64_t i = tile + k * blockDim.x + threadIdx.x;
        if (i < n4) ActVec<OT>::store(out, i, agn_silu_mul4(g[k], u[k]));
    }
}

// f16 storage: at 6 bytes per element the f32 kernel's instruction stream (IEEE division,
// full-range expf, one 64-bit access per four values) would bound the kernel, not HBM.  This
// variant moves eight values per 128-bit access and uses the hardware approximations
// (ex2.approx, rcp.approx: relative error ~2^-22), far below the 2^-11 rounding of the f16
// result.
__device__ __forceinline__ float silu_mul1_fast(float g, float u) { return __fdividef(g, 1.0f + __expf(-g)) * u; }

__device__ __forceinline__ uint32_t silu_mul_h2(uint32_t g, uint32_t u) {
    const float2 gf = __half22float2(*reinterpret_cast<const __half2 *>(&g));
    const float2 uf = __half22float2(*reinterpret_cast<const __half2 *>(&u));
    const __half2 r = __floats2half2_rn(silu_mul1_fast(gf.x, uf.x), silu_mul1_fast(gf.y, uf.y));
    return *reinterpret_cast<const uint32_t *>(&r);
}

template <int UNROLL>
__global__ void __launch_bounds__(512)
silu_mul_h8_kernel(const uint4 *__restrict__ gate, const uint4 *__restrict__ up, uint4 *__restrict__ out, int64_t n8) {
    agn_pdl_prologue();
    const int64_t tile = (int64_t)blockIdx.x * (UNROLL * blockDim.x);
    uint4 g[UNROLL], u[UNROLL];
#pragma unroll
    for (int k = 0; k < UNROLL; k++) {
        const int64_t i = tile + k * blockDim.x + threadIdx.x;
        if (i < n8) {
            g[k] = __ldcs(gate + i);
            u[k] = __ldcs(up + i);
        }
    }
#pragma unroll
    for (int k = 0; k < UNROLL; k++) {
        const int64_t i = tile + k * blockDim.x + threadIdx.x;
        if (i < n8) {
            uint4 o;
            o.x = silu_mul_h2(g[k].x, u[k].x);
            o.y = silu_mul_h2(g[k].y, u[k].y);
            o.z = silu_mul_h2(g[k].z, u[k].z);
            o.w = silu_mul_h2(g[k].w, u[k].w);
            __stcs(out + i, o);
        }
    }
}

// Tail (n % 4 elements) and unaligned buffers.
template <typename T, typename OT>
__global__ void silu_mul_scalar_kernel(const T *__restrict__ gate, const T *__restrict__ up, OT *__restrict__ out,
                                       int64_t begin, int64_t n) {
    agn_pdl_prologue();
    const int64_t i = begin + (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) ActVec<OT>::store1(out, i, agn_silu_mul1(ActVec<T>::load1(gate, i), ActVec<T>::load1(up, i)));
}

template <typename T, typename OT>
int32_t silu_mul_dispatch(agn_ctx *ctx, const T *gate, const T *up, OT *out, int64_t n) {
    if (n < 0) return agn_fail(ctx, AGN_EINVAL, "silu_mul: n=%lld < 0", (long long)n);
    if (n == 0) return AGN_OK;
    if (!gate || !up || !out) return agn_fail(ctx, AGN_EINVAL, "silu_mul: null pointer");
    AGN_CUDA(ctx, cudaSetDevice(ctx->device));
    int THREADS = ctx->tune_silu_threads, UNROLL = ctx->tune_silu_unroll;
    // Decode-sized inputs (a few token rows): with the streaming shape a row of 18944 values is five
    // CTAs whose threads each run sixteen expf + IEEE divisions back to back, which is a microsecond
    // of dependent arithmetic on five SMs.  One float4 pair per thread in 128-thread CTAs spreads
    // the same work over 37 CTAs per row; up to about two such CTAs per thread slot of the GPU this
    // is the faster shape, beyond it the deep-unrolled streaming shape takes over.
    if (ctx->tune_silu_small && n / 4 <= (int64_t)ctx->sm_count * 2048) {
        THREADS = 128;
        UNROLL = 1;
    }
    constexpr int A = ActVec<T>::ALIGN;
    int64_t done = 0;
    if (agn_aligned(gate, A) && agn_aligned(up, A) && agn_aligned(out, ActVec<OT>::ALIGN)) {
        const int64_t n4 = n / 4;
        if (n4 > 0) {
            const int64_t per_cta = (int64_t)THREADS * UNROLL;
            const int64_t blocks = (n4 + per_cta - 1) / per_cta;
            if (blocks > 0x7fffffffLL) return agn_fail(ctx, AGN_EINVAL, "silu_mul: n too large");
            if (UNROLL == 1) agn_launch(ctx, silu_mul_vec4_kernel<T, OT, 1>, dim3((unsigned)blocks), dim3(THREADS), 0, gate, up, out, n4);
            else if (UNROLL == 2) agn_launch(ctx, silu_mul_vec4_kernel<T, OT, 2>, dim3((unsigned)blocks), dim3(THREADS), 0, gate, up, out, n4);
            else if (UNROLL == 8) agn_launch(ctx, silu_mul_vec4_kernel<T, OT, 8>, dim3((unsigned)blocks), dim3(THREADS), 0, gate, up, out, n4);
            else agn_launch(ctx, silu_mul_vec4_kernel<T, OT, 4>, dim3((unsigned)blocks), dim3(THREADS), 0, gate, up, out, n4);
            AGN_LAUNCHED(ctx, "silu_mul_vec4");
        }
        done = n4 * 4;
    }
    if (done < n) {
        const int64_t rest = n - done;
        const int64_t blocks = (rest + THREADS - 1) / THREADS;
        if (blocks > 0x7fffffffLL) return agn_fail(ctx, AGN_EINVAL, "silu_mul: unaligned n too large");
        agn_launch(ctx, silu_mul_scalar_kernel<T, OT>, dim3((unsigned)blocks), dim3(THREADS), 0, gate, up, out, done, n);
        AGN_LAUNCHED(ctx, "silu_mul_scalar");
    }
    return AGN_OK;
}

}  // namespace

extern "C" int32_t agn_silu_mul_f32(agn_ctx *ctx, const float *gate, const float *up, float *out, int64_t n) {
    AGN_CHECK_CTX(ctx);
    return silu_mul_dispatch<float, float>(ctx, gate, up, out, n);
}

// f16 activation storage, f32 arithmetic: the reference's GPU `silu_mul` with `Act = f16`
// (src/ops/kernels_wgpu.rs:22-31).
extern "C" int32_t agn_silu_mul_f16(agn_ctx *ctx, const void *gate, const void *up, void *out, int64_t n) {
    AGN_CHECK_CTX(ctx);
    if (n < 0) return agn_fail(ctx, AGN_EINVAL, "silu_mul_f16: n=%lld < 0", (long long)n);
    if (n == 0) return AGN_OK;
    if (!gate || !up || !out) return agn_fail(ctx, AGN_EINVAL, "silu_mul_f16: null pointer");
    const __half *g = static_cast<const __half *>(gate), *u = static_cast<const __half *>(up);
    __half *o = static_cast<__half *>(out);
    int64_t done = 0;
    if (agn_aligned16(gate) && agn_aligned16(up) && agn_aligned16(out) && n >= 8) {
        AGN_CUDA(ctx, cudaSetDevice(ctx->device));
        const int64_t n8 = n / 8;
        constexpr int THREADS = 256, UNROLL = 4;
        const int64_t blocks = (n8 + THREADS * UNROLL - 1) / (THREADS * UNROLL);
        if (blocks > 0x7fffffffLL) return agn_fail(ctx, AGN_EINVAL, "silu_mul_f16: n too large");
        agn_launch(ctx, silu_mul_h8_kernel<UNROLL>, dim3((unsigned)blocks), dim3(THREADS), 0, reinterpret_cast<const uint4 *>(gate),
                   reinterpret_cast<const uint4 *>(up), reinterpret_cast<uint4 *>(out), n8);
        AGN_LAUNCHED(ctx, "silu_mul_h8");
        done = n8 * 8;
    }
    if (done == n) return AGN_OK;
    // the remainder (and unaligned buffers) through the generic kernels
    return silu_mul_dispatch<__half, __half>(ctx, g + done, u + done, o + done, n - done);
}

// f32 gate and up in, the product stored as f16 (out_dtype = AGN_F16) or bf16 (AGN_BF16): the f32
// result of agn_silu_mul_f32 rounded to nearest even, i.e. the operand the down projection takes
// when it runs in half precision (10 instead of 12 bytes per element on the kernel that dominates
// the layer's elementwise time).  No counterpart in the reference, whose `silu_mul` reads and
// writes the same `Act` type (src/ops/kernels_wgpu.rs:22-31).
extern "C" int32_t agn_silu_mul_f32_out16(agn_ctx *ctx, const float *gate, const float *up, void *out, int64_t n,
                                          int32_t out_dtype) {
    AGN_CHECK_CTX(ctx);
    if (out_dtype == AGN_F16) return silu_mul_dispatch<float, __half>(ctx, gate, up, static_cast<__half *>(out), n);
    if (out_dtype == AGN_BF16) return silu_mul_dispatch<float, __nv_bfloat16>(ctx, gate, up, static_cast<__nv_bfloat16 *>(out), n);
    return agn_fail(ctx, AGN_EUNSUPPORTED_DTYPE, "silu_mul_f32_out16: output type %d is neither f16 nor bf16", out_dtype);
}
