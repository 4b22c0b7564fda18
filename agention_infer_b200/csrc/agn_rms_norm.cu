// RMSNorm and fused residual-add + RMSNorm over T token rows.
//
// Reference (src/model/llama/cpu_path.rs:67-74):
//   sum_sq = sum_i x[i]^2 ; rms = sqrt(sum_sq / n + eps) ; out[i] = (w[i] * x[i]) / rms
// and `launch_add_residual_rms_norm` (src/ops/wgpu_backend/resident.rs:240-266).
//
// 8 algorithmic bytes per element (16 for the residual form): bound by HBM.  One CTA owns
// one row and keeps it in registers between the sum-of-squares pass and the scaling pass,
// so x is read from HBM exactly once: thread i holds float4 number i + k*blockDim, k < VPT
// (coalesced 128-bit loads, all VPT issued before the first use).  The statistic is reduced
// by warp shuffles, then across warps through shared memory in a fixed order, which makes
// the result independent of scheduling.
#include "agn_common.cuh"

namespace {

// Sum over the CTA; every thread returns the same value.
__device__ __forceinline__ float block_sum(float v, float *smem) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = agn_warp_sum(v);
    if (lane == 0) smem[warp] = v;
    __syncthreads();
    float total = 0.0f;
    for (int w = 0; w < nwarps; w++) total += smem[w];
    __syncthreads();  // smem is reused by the next call
    return total;
}

// T: storage type of x, delta and new_x; OT: storage type of the normed output (T, or a 16-bit
// type for a row that feeds a matmul with half-precision operands).
template <typename T, typename OT, int VPT, bool RESIDUAL, bool RECIP>
__global__ void __launch_bounds__(1024)
rms_norm_rows_kernel(const T *__restrict__ x, const T *__restrict__ delta, const float4 *__restrict__ w,
                     T *__restrict__ new_x, OT *__restrict__ out, int n4, float n_f, float eps) {
    agn_pdl_prologue();
    __shared__ float red[32];
    const int64_t row = (int64_t)blockIdx.x * n4;  // in vectors of four activations
    float4 v[VPT];
#pragma unroll
    for (int k = 0; k < VPT; k++) {
        const int i = threadIdx.x + k * blockDim.x;
        if (i < n4) v[k] = ActVec<T>::load(x, row + i);
        else v[k] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    if (RESIDUAL) {
#pragma unroll
        for (int k = 0; k < VPT; k++) {
            const int i = threadIdx.x + k * blockDim.x;
            if (i < n4) {
                const float4 d = ActVec<T>::load(delta, row + i);
                v[k].x += d.x; v[k].y += d.y; v[k].z += d.z; v[k].w += d.w;
                ActVec<T>::store(new_x, row + i, v[k]);
                if (sizeof(T) == 2) {
                    // the reference's f16 kernel normalises the STORED new_x (re-read after the
                    // cast, src/ops/kernels_wgpu.rs:139,159): round through f16 here as well
                    v[k].x = __half2float(__float2half_rn(v[k].x)); v[k].y = __half2float(__float2half_rn(v[k].y));
                    v[k].z = __half2float(__float2half_rn(v[k].z)); v[k].w = __half2float(__float2half_rn(v[k].w));
                }
            }
        }
    }
    float ss = 0.0f;
#pragma unroll
    for (int k = 0; k < VPT; k++) ss += v[k].x * v[k].x + v[k].y * v[k].y + v[k].z * v[k].z + v[k].w * v[k].w;
    ss = block_sum(ss, red);
    const float rms = sqrtf(ss / n_f + eps);  // same operations as the reference: sum/n + eps
    const float inv = 1.0f / rms;
#pragma unroll
    for (int k = 0; k < VPT; k++) {
        const int i = threadIdx.x + k * blockDim.x;
        if (i < n4) {
            const float4 ww = __ldg(w + i);
            float4 o;
            if (RECIP) {
                o.x = ww.x * v[k].x * inv;
                o.y = ww.y * v[k].y * inv;
                o.z = ww.z * v[k].z * inv;
                o.w = ww.w * v[k].w * inv;
            } else {
                o.x = ww.x * v[k].x / rms;
                o.y = ww.y * v[k].y / rms;
                o.z = ww.z * v[k].z / rms;
                o.w = ww.w * v[k].w / rms;
            }
            ActVec<OT>::store(out, row + i, o);
        }
    }
}

// Any H, any alignment, rows too long for registers: two passes over the row, the second
// one served by L2 for rows that fit there.
template <typename T, typename OT, bool RESIDUAL>
__global__ void __launch_bounds__(1024)
rms_norm_rows_generic_kernel(const T *__restrict__ x, const T *__restrict__ delta, const float *__restrict__ w,
                             T *__restrict__ new_x, OT *__restrict__ out, int64_t H, float eps) {
    agn_pdl_prologue();
    __shared__ float red[32];
    const int64_t row = (int64_t)blockIdx.x * H;
    float ss = 0.0f;
    for (int64_t i = threadIdx.x; i < H; i += blockDim.x) {
        float v = ActVec<T>::load1(x, row + i);
        if (RESIDUAL) {
            v += ActVec<T>::load1(delta, row + i);
            ActVec<T>::store1(new_x, row + i, v);
            v = ActVec<T>::load1(new_x, row + i);
        }
        ss += v * v;
    }
    ss = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)H + eps);
    const T *src = RESIDUAL ? new_x : x;
    for (int64_t i = threadIdx.x; i < H; i += blockDim.x)
        ActVec<OT>::store1(out, row + i, w[i] * ActVec<T>::load1(src, row + i) * inv);
}

template <typename T, typename OT, int VPT, bool RESIDUAL>
void launch_vec(agn_ctx *ctx, const T *x, const T *delta, const float *w, T *new_x, OT *out, int64_t T_rows, int n4,
                float eps, int threads) {
    const float4 *w4 = reinterpret_cast<const float4 *>(w);
    if (ctx->tune_rms_recip)
        agn_launch(ctx, rms_norm_rows_kernel<T, OT, VPT, RESIDUAL, true>, dim3((unsigned)T_rows), dim3(threads), 0, x, delta, w4,
                   new_x, out, n4, (float)(n4 * 4), eps);
    else
        agn_launch(ctx, rms_norm_rows_kernel<T, OT, VPT, RESIDUAL, false>, dim3((unsigned)T_rows), dim3(threads), 0, x, delta, w4,
                   new_x, out, n4, (float)(n4 * 4), eps);
}

template <typename T, typename OT, bool RESIDUAL>
int32_t rms_norm_dispatch(agn_ctx *ctx, const T *x, const T *delta, const float *w, T *new_x, OT *out, int64_t T_rows,
                          int64_t H, float eps, const char *name) {
    if (T_rows < 0 || H <= 0) return agn_fail(ctx, AGN_EINVAL, "%s: T=%lld H=%lld", name, (long long)T_rows, (long long)H);
    if (T_rows == 0) return AGN_OK;
    if (!x || !w || !out || (RESIDUAL && (!delta || !new_x))) return agn_fail(ctx, AGN_EINVAL, "%s: null pointer", name);
    if (T_rows > 0x7fffffffLL) return agn_fail(ctx, AGN_EINVAL, "%s: T too large", name);
    AGN_CUDA(ctx, cudaSetDevice(ctx->device));
    constexpr int A = ActVec<T>::ALIGN;
    const bool vec_ok = (H % 4 == 0) && agn_aligned(x, A) && agn_aligned16(w) && agn_aligned(out, ActVec<OT>::ALIGN) &&
                        (!RESIDUAL || (agn_aligned(delta, A) && agn_aligned(new_x, A))) && H <= 32768;
    if (vec_ok) {
        const int n4 = (int)(H / 4);
        // Pick the smallest VPT in {1,2,4,8} that keeps the CTA at <= 256 threads when
        // possible: more rows resident per SM and more loads in flight per thread.
        int vpt = 1;
        while (vpt < 8 && (n4 + vpt - 1) / vpt > 256) vpt *= 2;
        if (ctx->tune_rms_vpt == 1 || ctx->tune_rms_vpt == 2 || ctx->tune_rms_vpt == 4 || ctx->tune_rms_vpt == 8) {
            vpt = ctx->tune_rms_vpt;
            while (vpt < 8 && (n4 + vpt - 1) / vpt > 1024) vpt *= 2;
        }
        int threads = (n4 + vpt - 1) / vpt;
        threads = ((threads + 31) / 32) * 32;
        if (threads > 1024) threads = 1024;
        switch (vpt) {
        case 1: launch_vec<T, OT, 1, RESIDUAL>(ctx, x, delta, w, new_x, out, T_rows, n4, eps, threads); break;
        case 2: launch_vec<T, OT, 2, RESIDUAL>(ctx, x, delta, w, new_x, out, T_rows, n4, eps, threads); break;
        case 4: launch_vec<T, OT, 4, RESIDUAL>(ctx, x, delta, w, new_x, out, T_rows, n4, eps, threads); break;
        default: launch_vec<T, OT, 8, RESIDUAL>(ctx, x, delta, w, new_x, out, T_rows, n4, eps, threads); break;
        }
        AGN_LAUNCHED(ctx, name);
    } else {
        int threads = H >= 1024 ? 256 : (int)(((H + 31) / 32) * 32);
        if (threads > 256) threads = 256;
        agn_launch(ctx, rms_norm_rows_generic_kernel<T, OT, RESIDUAL>, dim3((unsigned)T_rows), dim3(threads), 0, x, delta, w, new_x,
                   out, H, eps);
        AGN_LAUNCHED(ctx, name);
    }
    return AGN_OK;
}

}  // namespace

extern "C" int32_t agn_rms_norm_f32(agn_ctx *ctx, const float *x, const float *w, float *out,
                                    int64_t T, int64_t H, float eps) {
    AGN_CHECK_CTX(ctx);
    return rms_norm_dispatch<float, float, false>(ctx, x, nullptr, w, nullptr, out, T, H, eps, "rms_norm");
}

extern "C" int32_t agn_add_residual_rms_norm_f32(agn_ctx *ctx, const float *x, const float *delta,
                                                 const float *w, float *new_x, float *normed,
                                                 int64_t T, int64_t H, float eps) {
    AGN_CHECK_CTX(ctx);
    return rms_norm_dispatch<float, float, true>(ctx, x, delta, w, new_x, normed, T, H, eps, "add_residual_rms_norm");
}

// f16 activation storage (the reference's `Act = f16`, src/ops/kernels_wgpu.rs:79-163): x, delta,
// new_x and the output are f16, the weight is f32, the arithmetic is f32.
extern "C" int32_t agn_rms_norm_f16(agn_ctx *ctx, const void *x, const float *w, void *out, int64_t T, int64_t H, float eps) {
    AGN_CHECK_CTX(ctx);
    return rms_norm_dispatch<__half, __half, false>(ctx, static_cast<const __half *>(x), nullptr, w, nullptr, static_cast<__half *>(out),
                                            T, H, eps, "rms_norm_f16");
}

extern "C" int32_t agn_add_residual_rms_norm_f16(agn_ctx *ctx, const void *x, const void *delta, const float *w, void *new_x,
                                                 void *normed, int64_t T, int64_t H, float eps) {
    AGN_CHECK_CTX(ctx);
    return rms_norm_dispatch<__half, __half, true>(ctx, static_cast<const __half *>(x), static_cast<const __half *>(delta), w,
                                           static_cast<__half *>(new_x), static_cast<__half *>(normed), T, H, eps,
                                           "add_residual_rms_norm_f16");
}

// f32 rows in, normed row stored as f16 or bf16 (round to nearest even of the f32 result): the
// input a matmul with half-precision operands wants, written once instead of an f32 row plus a
// cast pass.  out_dtype is AGN_F16 or AGN_BF16.  No counterpart in the reference, whose norm
// kernels store `Act` in and out (src/ops/kernels_wgpu.rs:79-163); the residual stream (new_x)
// stays f32.
extern "C" int32_t agn_rms_norm_f32_out16(agn_ctx *ctx, const float *x, const float *w, void *out, int64_t T, int64_t H,
                                          float eps, int32_t out_dtype) {
    AGN_CHECK_CTX(ctx);
    if (out_dtype == AGN_F16)
        return rms_norm_dispatch<float, __half, false>(ctx, x, nullptr, w, nullptr, static_cast<__half *>(out), T, H, eps,
                                                       "rms_norm_out_f16");
    if (out_dtype == AGN_BF16)
        return rms_norm_dispatch<float, __nv_bfloat16, false>(ctx, x, nullptr, w, nullptr, static_cast<__nv_bfloat16 *>(out), T, H,
                                                              eps, "rms_norm_out_bf16");
    return agn_fail(ctx, AGN_EUNSUPPORTED_DTYPE, "rms_norm_f32_out16: output type %d is neither f16 nor bf16", out_dtype);
}

extern "C" int32_t agn_add_residual_rms_norm_f32_out16(agn_ctx *ctx, const float *x, const float *delta, const float *w,
                                                       float *new_x, void *normed, int64_t T, int64_t H, float eps,
                                                       int32_t out_dtype) {
    AGN_CHECK_CTX(ctx);
    if (out_dtype == AGN_F16)
        return rms_norm_dispatch<float, __half, true>(ctx, x, delta, w, new_x, static_cast<__half *>(normed), T, H, eps,
                                                      "add_residual_rms_norm_out_f16");
    if (out_dtype == AGN_BF16)
        return rms_norm_dispatch<float, __nv_bfloat16, true>(ctx, x, delta, w, new_x, static_cast<__nv_bfloat16 *>(normed), T, H,
                                                             eps, "add_residual_rms_norm_out_bf16");
    return agn_fail(ctx, AGN_EUNSUPPORTED_DTYPE, "add_residual_rms_norm_f32_out16: output type %d is neither f16 nor bf16", out_dtype);
}
