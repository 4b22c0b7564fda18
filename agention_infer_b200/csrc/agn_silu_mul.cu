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

// Each CTA owns a contiguous tile of UNROLL * blockDim float4; a thread issues all of its
// 2*UNROLL loads before the first use so that UNROLL*32 B per thread are in flight.
template <int UNROLL>
__global__ void __launch_bounds__(512)
silu_mul_vec4_kernel(const float4 *__restrict__ gate, const float4 *__restrict__ up,
                     float4 *__restrict__ out, int64_t n4) {
    agn_pdl_prologue();
    const int64_t tile = (int64_t)blockIdx.x * (UNROLL * blockDim.x);
    float4 g[UNROLL], u[UNROLL];
#pragma unroll
    for (int k = 0; k < UNROLL; k++) {
        const int64_t i = tile + k * blockDim.x + threadIdx.x;
        if (i < n4) {
            g[k] = agn_ld_stream(gate + i);
            u[k] = agn_ld_stream(up + i);
        }
    }
#pragma unroll
    for (int k = 0; k < UNROLL; k++) {
        const int64_t i = tile + k * blockDim.x + threadIdx.x;
        if (i < n4) agn_st_stream(out + i, silu_mul4(g[k], u[k]));
    }
}

// Tail (n % 4 elements) and unaligned buffers.
__global__ void silu_mul_scalar_kernel(const float *__restrict__ gate, const float *__restrict__ up,
                                       float *__restrict__ out, int64_t begin, int64_t n) {
    agn_pdl_prologue();
    const int64_t i = begin + (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = silu_mul1(gate[i], up[i]);
}

}  // namespace

extern "C" int32_t agn_silu_mul_f32(agn_ctx *ctx, const float *gate, const float *up, float *out, int64_t n) {
    AGN_CHECK_CTX(ctx);
    if (n < 0) return agn_fail(ctx, AGN_EINVAL, "silu_mul: n=%lld < 0", (long long)n);
    if (n == 0) return AGN_OK;
    if (!gate || !up || !out) return agn_fail(ctx, AGN_EINVAL, "silu_mul: null pointer");
    AGN_CUDA(ctx, cudaSetDevice(ctx->device));
    const int THREADS = ctx->tune_silu_threads, UNROLL = ctx->tune_silu_unroll;
    int64_t done = 0;
    if (agn_aligned16(gate) && agn_aligned16(up) && agn_aligned16(out)) {
        const int64_t n4 = n / 4;
        if (n4 > 0) {
            const int64_t per_cta = (int64_t)THREADS * UNROLL;
            const int64_t blocks = (n4 + per_cta - 1) / per_cta;
            if (blocks > 0x7fffffffLL) return agn_fail(ctx, AGN_EINVAL, "silu_mul: n too large");
            const float4 *g4 = reinterpret_cast<const float4 *>(gate), *u4 = reinterpret_cast<const float4 *>(up);
            float4 *o4 = reinterpret_cast<float4 *>(out);
            if (UNROLL == 2) agn_launch(ctx, silu_mul_vec4_kernel<2>, dim3((unsigned)blocks), dim3(THREADS), 0, g4, u4, o4, n4);
            else if (UNROLL == 8) agn_launch(ctx, silu_mul_vec4_kernel<8>, dim3((unsigned)blocks), dim3(THREADS), 0, g4, u4, o4, n4);
            else agn_launch(ctx, silu_mul_vec4_kernel<4>, dim3((unsigned)blocks), dim3(THREADS), 0, g4, u4, o4, n4);
            AGN_LAUNCHED(ctx, "silu_mul_vec4");
        }
        done = n4 * 4;
    }
    if (done < n) {
        const int64_t rest = n - done;
        const int64_t blocks = (rest + THREADS - 1) / THREADS;
        if (blocks > 0x7fffffffLL) return agn_fail(ctx, AGN_EINVAL, "silu_mul: unaligned n too large");
        agn_launch(ctx, silu_mul_scalar_kernel, dim3((unsigned)blocks), dim3(THREADS), 0, gate, up, out, done, n);
        AGN_LAUNCHED(ctx, "silu_mul_scalar");
    }
    return AGN_OK;
}
