// gate·up -> SiLU·mul (SwiGLU combine), HBM-streaming kernel.
//
// Reference: out = g / (1 + exp(-g)) * u   (src/model/llama/cpu_path.rs:228-229, :975-978;
// GPU twin src/ops/kernels_wgpu.rs:22-31).  12 algorithmic bytes per element, ~25 lane
// instructions: bound by HBM, so the kernel is nothing but 128-bit streaming loads with
// several of them in flight per thread, and 128-bit streaming stores.
#include "agn_common.cuh"

namespace {

__device__ __forceinline__ float silu_mul1(float g, float u) {
    // IEEE division (-prec-div=true is nvcc's default; no fast-math anywhere).
    const float silu = g / (1.0f + expf(-g));
    return silu * u;
}

__device__ __forceinline__ float4 silu_mul4(float4 g, float4 u) {
    float4 o;
    o.x = silu_mul1(g.x, u.x);
    o.y = silu_mul1(g.y, u.y);
    o.z = silu_mul1(g.z, u.z);
    o.w = silu_mul1(g.w, u.w);
    return o;
}

// Each CTA owns a contiguous tile of UNROLL * blockDim vectors of four activations; a thread
// issues all of its 2*UNROLL loads before the first use so that UNROLL*32 B (f32) per thread
// are in flight.
template <typename T, int UNROLL>
__global__ void __launch_bounds__(512)
silu_mul_vec4_kernel(const T *__restrict__ gate, const T *__restrict__ up, T *__restrict__ out, int64_t n4) {
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
        if (i < n4) ActVec<T>::store(out, i, silu_mul4(g[k], u[k]));
    }
}

// Tail (n % 4 elements) and unaligned buffers.
template <typename T>
__global__ void silu_mul_scalar_kernel(const T *__restrict__ gate, const T *__restrict__ up, T *__restrict__ out,
                                       int64_t begin, int64_t n) {
    agn_pdl_prologue();
    const int64_t i = begin + (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) ActVec<T>::store1(out, i, silu_mul1(ActVec<T>::load1(gate, i), ActVec<T>::load1(up, i)));
}

template <typename T>
int32_t silu_mul_dispatch(agn_ctx *ctx, const T *gate, const T *up, T *out, int64_t n) {
    if (n < 0) return agn_fail(ctx, AGN_EINVAL, "silu_mul: n=%lld < 0", (long long)n);
    if (n == 0) return AGN_OK;
    if (!gate || !up || !out) return agn_fail(ctx, AGN_EINVAL, "silu_mul: null pointer");
    AGN_CUDA(ctx, cudaSetDevice(ctx->device));
    const int THREADS = ctx->tune_silu_threads, UNROLL = ctx->tune_silu_unroll;
    constexpr int A = ActVec<T>::ALIGN;
    int64_t done = 0;
    if (agn_aligned(gate, A) && agn_aligned(up, A) && agn_aligned(out, A)) {
        const int64_t n4 = n / 4;
        if (n4 > 0) {
            const int64_t per_cta = (int64_t)THREADS * UNROLL;
            const int64_t blocks = (n4 + per_cta - 1) / per_cta;
            if (blocks > 0x7fffffffLL) return agn_fail(ctx, AGN_EINVAL, "silu_mul: n too large");
            if (UNROLL == 2) agn_launch(ctx, silu_mul_vec4_kernel<T, 2>, dim3((unsigned)blocks), dim3(THREADS), 0, gate, up, out, n4);
            else if (UNROLL == 8) agn_launch(ctx, silu_mul_vec4_kernel<T, 8>, dim3((unsigned)blocks), dim3(THREADS), 0, gate, up, out, n4);
            else agn_launch(ctx, silu_mul_vec4_kernel<T, 4>, dim3((unsigned)blocks), dim3(THREADS), 0, gate, up, out, n4);
            AGN_LAUNCHED(ctx, "silu_mul_vec4");
        }
        done = n4 * 4;
    }
    if (done < n) {
        const int64_t rest = n - done;
        const int64_t blocks = (rest + THREADS - 1) / THREADS;
        if (blocks > 0x7fffffffLL) return agn_fail(ctx, AGN_EINVAL, "silu_mul: unaligned n too large");
        agn_launch(ctx, silu_mul_scalar_kernel<T>, dim3((unsigned)blocks), dim3(THREADS), 0, gate, up, out, done, n);
        AGN_LAUNCHED(ctx, "silu_mul_scalar");
    }
    return AGN_OK;
}

}  // namespace

extern "C" int32_t agn_silu_mul_f32(agn_ctx *ctx, const float *gate, const float *up, float *out, int64_t n) {
    AGN_CHECK_CTX(ctx);
    return silu_mul_dispatch<float>(ctx, gate, up, out, n);
}

// f16 activation storage, f32 arithmetic: the reference's GPU `silu_mul` with `Act = f16`
// (src/ops/kernels_wgpu.rs:22-31).
extern "C" int32_t agn_silu_mul_f16(agn_ctx *ctx, const void *gate, const void *up, void *out, int64_t n) {
    AGN_CHECK_CTX(ctx);
    return silu_mul_dispatch<__half>(ctx, static_cast<const __half *>(gate), static_cast<const __half *>(up),
                                     static_cast<__half *>(out), n);
}
