// Q8_K activation quantisation of token rows, alone and fused onto the ops that produce a
// matmul's input (RMSNorm, residual-add + RMSNorm, SiLU·mul).
//
// Reference: quantize_row_q8_k (src/quant/q8_k.rs:49-92), which WeightMap::matmul_into runs on the
// activation vector before the int8 dot products of a Q5_K tensor (src/model/mod.rs:381-386).
// Per block of 256 values (the last block of a row zero-padded):
//   max    = the value of largest magnitude, the first one on ties (strict `>` scan; NaN never wins)
//   iscale = -127 / max ;  d = 1 / iscale            (all-zero block: d = 0, q = 0)
//   q      = min(round_half_away(iscale * v) as i32, 127) as i8
//   bsums[g] = sum of q over the g-th group of 16
// and the three outputs are the parallel arrays of `Q8KRow` (:27-37): d [T, nb] f32,
// qs [T, nb * 256] i8, bsums [T, nb * 16] i16, nb = ceil(n / 256).
//
// Integer output, so the result is the reference's bit for bit: IEEE division and multiplication
// (no fused multiply-add: the product is rounded before it is rounded to an integer), rounding
// half away from zero, the saturating float -> i32 conversion Rust's `as` performs (which is what
// cvt.rzi.s32.f32 does, NaN -> 0) and the wrapping i32 -> i8 one.
//
// 4 bytes read and 1.14 written per value: bound by HBM.  One warp owns one block of 256 values,
// lane l holding values 4l..4l+3 and 128+4l..128+4l+3 (two coalesced 128-bit loads); the maximum
// is two warp-wide redux instructions, a group of 16 values is four neighbouring lanes, the
// quantised values leave as one 32-bit store per lane and half-block.  Fused onto RMSNorm the row
// keeps the thread mapping of rms_norm_rows_kernel (so that the normed values, and with them every
// output byte, are those of the two separate launches): there a half-block of 128 values is one
// warp's vector, and the two halves of a block meet through shared memory.
#include "agn_common.cuh"
#include "agn_row_math.cuh"

namespace {

constexpr int QK_K = 256;

// Warp-wide maximum / minimum of f32 values in one instruction (sm_100a); NaN operands are ignored
// (the result is NaN only when every lane holds one).
__device__ __forceinline__ float warp_max_f32(float v) {
    float r;
    asm volatile("redux.sync.max.f32 %0, %1, 0xffffffff;" : "=f"(r) : "f"(v));
    return r;
}
__device__ __forceinline__ float warp_min_f32(float v) {
    float r;
    asm volatile("redux.sync.min.f32 %0, %1, 0xffffffff;" : "=f"(r) : "f"(v));
    return r;
}

// The value of largest magnitude among the N float4 per lane that a warp holds, the first one in
// index order on ties (v[k] component c of lane l has index k*128 + 4*l + c), 0 when no value has
// a magnitude above 0.  Every lane returns the same value.
// Common case: largest and smallest value differ in magnitude, and the larger magnitude wins.
// Only when +a and -a are both present does the order of the elements matter; then the lowest
// index among the candidates decides.
template <int N>
__device__ __forceinline__ float q8k_first_max(const float4 (&v)[N], int lane) {
    float mx = -INFINITY, mn = INFINITY;  // fmaxf / fminf drop a NaN operand, as the scan's `av > amax` does
#pragma unroll
    for (int k = 0; k < N; k++) {
        mx = fmaxf(fmaxf(mx, v[k].x), fmaxf(fmaxf(v[k].y, v[k].z), v[k].w));
        mn = fminf(fminf(mn, v[k].x), fminf(fminf(v[k].y, v[k].z), v[k].w));
    }
    mx = warp_max_f32(mx);
    mn = warp_min_f32(mn);
    const float amax = fmaxf(mx, -mn);
    if (!(amax > 0.0f)) return 0.0f;
    if (mx != -mn) return mx > -mn ? mx : mn;
    uint32_t key = 0xffffffffu;  // (index << 1) | negative
#pragma unroll
    for (int k = N - 1; k >= 0; k--) {
        const uint32_t base = (uint32_t)(k * 128 + 4 * lane) << 1;
        if (fabsf(v[k].w) == amax) key = (base + 6u) | (v[k].w < 0.0f ? 1u : 0u);
        if (fabsf(v[k].z) == amax) key = (base + 4u) | (v[k].z < 0.0f ? 1u : 0u);
        if (fabsf(v[k].y) == amax) key = (base + 2u) | (v[k].y < 0.0f ? 1u : 0u);
        if (fabsf(v[k].x) == amax) key = base | (v[k].x < 0.0f ? 1u : 0u);
    }
    key = __reduce_min_sync(0xffffffffu, key);
    return (key & 1u) ? -amax : amax;
}

// Of two halves of a block (each with its own first-largest value), the block's: the earlier half
// wins a tie in magnitude.
__device__ __forceinline__ float q8k_combine_halves(float first_half, float second_half) {
    return fabsf(first_half) >= fabsf(second_half) ? first_half : second_half;
}

// min(round_half_away(iscale * v) as i32, 127).  Rounding half away from zero as
// trunc(p + copysign(0.5 - 2^-25, p)): exact for every f32 p (a p below k + 0.5 stays below the
// integer after the addition, k + 0.5 itself lands on it), three instructions instead of roundf's
// sequence.  The conversion saturates and sends NaN to 0, like Rust's `as i32`.
__device__ __forceinline__ int q8k_q1(float v, float iscale) {
    const float p = __fmul_rn(iscale, v);
    const float t = __fadd_rn(p, copysignf(__int_as_float(0x3effffff), p));
    return min(__float2int_rz(t), 127);
}

// Four values -> four bytes (`as i8` keeps the low byte), little-endian in value order.
__device__ __forceinline__ uint32_t q8k_q4(float4 v, float iscale) {
    const uint32_t a = (uint32_t)q8k_q1(v.x, iscale) & 0xffu, b = (uint32_t)q8k_q1(v.y, iscale) & 0xffu;
    const uint32_t c = (uint32_t)q8k_q1(v.z, iscale) & 0xffu, d = (uint32_t)q8k_q1(v.w, iscale) & 0xffu;
    return a | (b << 8) | (c << 16) | (d << 24);
}

// One lane's four bytes of a 128-value half-block: store them, and the sums of the eight groups
// of 16 (four neighbouring lanes each).  qs_half / bsums_half point at the half-block's outputs.
__device__ __forceinline__ void q8k_store_half(uint32_t packed, int lane, int8_t *qs_half, int16_t *bsums_half) {
    reinterpret_cast<uint32_t *>(qs_half)[lane] = packed;
    int s = __dp4a((int)packed, 0x01010101, 0);  // sum of the four signed bytes
    s += __shfl_xor_sync(0xffffffffu, s, 1);
    s += __shfl_xor_sync(0xffffffffu, s, 2);
    if ((lane & 3) == 0) bsums_half[lane >> 2] = (int16_t)s;
}

// A whole block held by one warp as two float4 per lane: scale, quantise, store.
__device__ __forceinline__ void q8k_block_from_warp(const float4 (&v)[2], int lane, float *d_out, int8_t *qs_block,
                                                    int16_t *bsums_block) {
    const float mx = q8k_first_max<2>(v, lane);
    float iscale = 0.0f, d = 0.0f;
    if (mx != 0.0f) {  // (uniform over the warp)
        iscale = -127.0f / mx;
        d = 1.0f / iscale;
    }
    // a block without a magnitude above 0 (zeros, NaN only) is written as zeros, d = 0
    if (lane == 0) *d_out = d;
    q8k_store_half(mx != 0.0f ? q8k_q4(v[0], iscale) : 0u, lane, qs_block, bsums_block);
    q8k_store_half(mx != 0.0f ? q8k_q4(v[1], iscale) : 0u, lane, qs_block + 128, bsums_block + 8);
}

// ---- rows of f32 values -> Q8_K ---------------------------------------------------------------

// One warp per block; block B of the launch is block B % nb of row B / nb.  VEC: rows are whole
// float4 (n % 4 == 0, x 16-byte aligned); otherwise element-wise loads.
template <bool VEC>
__global__ void __launch_bounds__(256)
quantize_rows_q8k_kernel(const float *__restrict__ x, int64_t n_blocks_total, int nb, int n, float *__restrict__ d,
                         int8_t *__restrict__ qs, int16_t *__restrict__ bsums) {
    agn_pdl_prologue();
    const int lane = threadIdx.x & 31;
    const int64_t B = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (B >= n_blocks_total) return;
    const int64_t row = B / nb;
    const int b = (int)(B - row * nb);
    const float *xr = x + row * (int64_t)n;
    float4 v[2];
#pragma unroll
    for (int k = 0; k < 2; k++) {
        const int e = b * QK_K + k * 128 + 4 * lane;  // first of the lane's four values
        if (VEC) {
            v[k] = e < n ? __ldcs(reinterpret_cast<const float4 *>(xr + e)) : make_float4(0.f, 0.f, 0.f, 0.f);
        } else {
            v[k].x = e + 0 < n ? xr[e + 0] : 0.0f;
            v[k].y = e + 1 < n ? xr[e + 1] : 0.0f;
            v[k].z = e + 2 < n ? xr[e + 2] : 0.0f;
            v[k].w = e + 3 < n ? xr[e + 3] : 0.0f;
        }
    }
    q8k_block_from_warp(v, lane, d + B, qs + B * QK_K, bsums + B * 16);
}

// ---- SiLU·mul -> Q8_K --------------------------------------------------------------------------

// gate and up are [T, I] with I % 256 == 0, so the blocks of all rows form one flat sequence.
__global__ void __launch_bounds__(256)
silu_mul_q8k_kernel(const float *__restrict__ gate, const float *__restrict__ up, int64_t n_blocks_total,
                    float *__restrict__ d, int8_t *__restrict__ qs, int16_t *__restrict__ bsums) {
    agn_pdl_prologue();
    const int lane = threadIdx.x & 31;
    const int64_t B = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (B >= n_blocks_total) return;
    const float4 *g4 = reinterpret_cast<const float4 *>(gate) + B * 64, *u4 = reinterpret_cast<const float4 *>(up) + B * 64;
    const float4 g0 = __ldcs(g4 + lane), g1 = __ldcs(g4 + 32 + lane);
    const float4 u0 = __ldcs(u4 + lane), u1 = __ldcs(u4 + 32 + lane);
    float4 v[2];
    v[0] = agn_silu_mul4(g0, u0);
    v[1] = agn_silu_mul4(g1, u1);
    q8k_block_from_warp(v, lane, d + B, qs + B * QK_K, bsums + B * 16);
}

// ---- RMSNorm (and residual add + RMSNorm) -> Q8_K ---------------------------------------------

// The load, residual and statistic part is rms_norm_rows_kernel's, with the same thread mapping
// (thread i holds float4 number i + k*blockDim): the normed values are the same bits.  Vector
// k of warp w is half-block k * nwarps + w of the row (H % 256 == 0, so a warp's vector is wholly
// inside the row or wholly outside); the first-largest value of each half goes through shared
// memory to the warp that holds the other half.
template <int VPT, bool RESIDUAL>
__global__ void __launch_bounds__(1024)
rms_norm_q8k_rows_kernel(const float *__restrict__ x, const float *__restrict__ delta, const float4 *__restrict__ w,
                         float *__restrict__ new_x, int n4, float inv_n, float eps, float *__restrict__ d,
                         int8_t *__restrict__ qs, int16_t *__restrict__ bsums) {
    agn_pdl_prologue();
    __shared__ float red[32];
    __shared__ float half_max[256];  // one per half-block of 128 values: rows of up to 32768 values
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int64_t row = (int64_t)blockIdx.x * n4;  // in vectors of four activations
    float4 v[VPT];
#pragma unroll
    for (int k = 0; k < VPT; k++) {
        const int i = threadIdx.x + k * blockDim.x;
        if (i < n4) v[k] = ActVec<float>::load(x, row + i);
        else v[k] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    if (RESIDUAL) {
#pragma unroll
        for (int k = 0; k < VPT; k++) {
            const int i = threadIdx.x + k * blockDim.x;
            if (i < n4) {
                const float4 dl = ActVec<float>::load(delta, row + i);
                v[k].x += dl.x; v[k].y += dl.y; v[k].z += dl.z; v[k].w += dl.w;
                ActVec<float>::store(new_x, row + i, v[k]);
            }
        }
    }
    float2 ss2 = make_float2(0.0f, 0.0f);
#pragma unroll
    for (int k = 0; k < VPT; k++) ss2 = agn_sum_sq4(v[k], ss2);
    const float ss = agn_block_sum(ss2.x + ss2.y, red);
    const float inv = agn_inv_rms(ss, inv_n, eps);
#pragma unroll
    for (int k = 0; k < VPT; k++) {
        const int i = threadIdx.x + k * blockDim.x;
        if (i < n4) {
            v[k] = agn_scale4(agn_mul4(__ldg(w + i), v[k]), inv);  // (w * x) * inv, as rms_norm_rows_kernel
            const float4 one[1] = {v[k]};
            const float m = q8k_first_max<1>(one, lane);
            if (lane == 0) half_max[k * nwarps + warp] = m;
        }
    }
    __syncthreads();
    const int64_t first_block = (int64_t)blockIdx.x * (n4 >> 6);  // the row's first block in d / qs / bsums
#pragma unroll
    for (int k = 0; k < VPT; k++) {
        const int i = threadIdx.x + k * blockDim.x;
        if (i < n4) {
            const int hb = k * nwarps + warp;
            const float mx = q8k_combine_halves(half_max[hb & ~1], half_max[hb | 1]);
            float iscale = 0.0f, dd = 0.0f;
            if (mx != 0.0f) {
                iscale = -127.0f / mx;
                dd = 1.0f / iscale;
            }
            const int64_t B = first_block + (hb >> 1);
            if ((hb & 1) == 0 && lane == 0) d[B] = dd;
            q8k_store_half(mx != 0.0f ? q8k_q4(v[k], iscale) : 0u, lane, qs + B * QK_K + (hb & 1) * 128,
                           bsums + B * 16 + (hb & 1) * 8);
        }
    }
}

int32_t check_outputs(agn_ctx *ctx, const char *name, const float *d, const int8_t *qs, const int16_t *bsums) {
    if (!d || !qs || !bsums) return agn_fail(ctx, AGN_EINVAL, "%s: null output pointer", name);
    if (!agn_aligned(d, 4) || !agn_aligned(qs, 4) || !agn_aligned(bsums, 2))
        return agn_fail(ctx, AGN_EINVAL, "%s: d and qs must be 4-byte aligned, bsums 2-byte aligned", name);
    return AGN_OK;
}

template <bool RESIDUAL>
int32_t rms_norm_q8k_dispatch(agn_ctx *ctx, const float *x, const float *delta, const float *w, float *new_x, int64_t T,
                              int64_t H, float eps, float *d, int8_t *qs, int16_t *bsums, const char *name) {
    if (T < 0 || H <= 0) return agn_fail(ctx, AGN_EINVAL, "%s: T=%lld H=%lld", name, (long long)T, (long long)H);
    if (H % QK_K != 0 || H > 32768)
        return agn_fail(ctx, AGN_EINVAL, "%s: H=%lld must be a multiple of 256 (whole Q8_K blocks) and at most 32768", name,
                        (long long)H);
    if (T == 0) return AGN_OK;
    if (!x || !w || (RESIDUAL && (!delta || !new_x))) return agn_fail(ctx, AGN_EINVAL, "%s: null pointer", name);
    if (T > 0x7fffffffLL) return agn_fail(ctx, AGN_EINVAL, "%s: T too large", name);
    if (int32_t st = check_outputs(ctx, name, d, qs, bsums)) return st;
    if (!agn_aligned16(x) || !agn_aligned16(w) || (RESIDUAL && (!agn_aligned16(delta) || !agn_aligned16(new_x))))
        return agn_fail(ctx, AGN_EINVAL, "%s: x, w, delta and new_x must be 16-byte aligned", name);
    AGN_CUDA(ctx, cudaSetDevice(ctx->device));
    const int n4 = (int)(H / 4);
    int vpt, threads;
    agn_rms_shape(ctx, n4, &vpt, &threads);
    const float4 *w4 = reinterpret_cast<const float4 *>(w);
    const float inv_n = 1.0f / (float)(n4 * 4);
    const dim3 grid((unsigned)T), block(threads);
    switch (vpt) {
    case 1: agn_launch(ctx, rms_norm_q8k_rows_kernel<1, RESIDUAL>, grid, block, 0, x, delta, w4, new_x, n4, inv_n, eps, d, qs, bsums); break;
    case 2: agn_launch(ctx, rms_norm_q8k_rows_kernel<2, RESIDUAL>, grid, block, 0, x, delta, w4, new_x, n4, inv_n, eps, d, qs, bsums); break;
    case 4: agn_launch(ctx, rms_norm_q8k_rows_kernel<4, RESIDUAL>, grid, block, 0, x, delta, w4, new_x, n4, inv_n, eps, d, qs, bsums); break;
    default: agn_launch(ctx, rms_norm_q8k_rows_kernel<8, RESIDUAL>, grid, block, 0, x, delta, w4, new_x, n4, inv_n, eps, d, qs, bsums); break;
    }
    AGN_LAUNCHED(ctx, name);
    return AGN_OK;
}

}  // namespace

extern "C" int64_t agn_q8_k_blocks(int64_t n) { return n <= 0 ? 0 : (n + QK_K - 1) / QK_K; }

extern "C" int32_t agn_quantize_rows_q8_k_f32(agn_ctx *ctx, const float *x, int64_t T, int64_t n, float *d, int8_t *qs,
                                              int16_t *bsums) {
    AGN_CHECK_CTX(ctx);
    if (T < 0 || n <= 0) return agn_fail(ctx, AGN_EINVAL, "quantize_rows_q8_k: T=%lld n=%lld", (long long)T, (long long)n);
    if (n > 0x7fffff00LL) return agn_fail(ctx, AGN_EINVAL, "quantize_rows_q8_k: n too large");
    if (T == 0) return AGN_OK;
    if (!x) return agn_fail(ctx, AGN_EINVAL, "quantize_rows_q8_k: null pointer");
    if (int32_t st = check_outputs(ctx, "quantize_rows_q8_k", d, qs, bsums)) return st;
    const int64_t nb = (n + QK_K - 1) / QK_K;
    if (T > INT64_MAX / nb) return agn_fail(ctx, AGN_EINVAL, "quantize_rows_q8_k: T * blocks overflows");
    const int64_t total = T * nb, ctas = (total + 7) / 8;
    if (ctas > 0x7fffffffLL) return agn_fail(ctx, AGN_EINVAL, "quantize_rows_q8_k: too many blocks for one launch");
    AGN_CUDA(ctx, cudaSetDevice(ctx->device));
    if (n % 4 == 0 && agn_aligned16(x))
        agn_launch(ctx, quantize_rows_q8k_kernel<true>, dim3((unsigned)ctas), dim3(256), 0, x, total, (int)nb, (int)n, d, qs, bsums);
    else
        agn_launch(ctx, quantize_rows_q8k_kernel<false>, dim3((unsigned)ctas), dim3(256), 0, x, total, (int)nb, (int)n, d, qs, bsums);
    AGN_LAUNCHED(ctx, "quantize_rows_q8_k");
    return AGN_OK;
}

extern "C" int32_t agn_rms_norm_q8_k_f32(agn_ctx *ctx, const float *x, const float *w, int64_t T, int64_t H, float eps,
                                         float *d, int8_t *qs, int16_t *bsums) {
    AGN_CHECK_CTX(ctx);
    return rms_norm_q8k_dispatch<false>(ctx, x, nullptr, w, nullptr, T, H, eps, d, qs, bsums, "rms_norm_q8_k");
}

extern "C" int32_t agn_add_residual_rms_norm_q8_k_f32(agn_ctx *ctx, const float *x, const float *delta, const float *w,
                                                      float *new_x, int64_t T, int64_t H, float eps, float *d, int8_t *qs,
                                                      int16_t *bsums) {
    AGN_CHECK_CTX(ctx);
    return rms_norm_q8k_dispatch<true>(ctx, x, delta, w, new_x, T, H, eps, d, qs, bsums, "add_residual_rms_norm_q8_k");
}

extern "C" int32_t agn_silu_mul_q8_k_f32(agn_ctx *ctx, const float *gate, const float *up, int64_t T, int64_t I, float *d,
                                         int8_t *qs, int16_t *bsums) {
    AGN_CHECK_CTX(ctx);
    if (T < 0 || I <= 0) return agn_fail(ctx, AGN_EINVAL, "silu_mul_q8_k: T=%lld I=%lld", (long long)T, (long long)I);
    if (I % QK_K != 0) return agn_fail(ctx, AGN_EINVAL, "silu_mul_q8_k: I=%lld must be a multiple of 256 (whole Q8_K blocks)", (long long)I);
    if (T == 0) return AGN_OK;
    if (!gate || !up) return agn_fail(ctx, AGN_EINVAL, "silu_mul_q8_k: null pointer");
    if (int32_t st = check_outputs(ctx, "silu_mul_q8_k", d, qs, bsums)) return st;
    if (!agn_aligned16(gate) || !agn_aligned16(up)) return agn_fail(ctx, AGN_EINVAL, "silu_mul_q8_k: gate and up must be 16-byte aligned");
    const int64_t nb = I / QK_K;
    if (T > INT64_MAX / nb) return agn_fail(ctx, AGN_EINVAL, "silu_mul_q8_k: T * blocks overflows");
    const int64_t total = T * nb, ctas = (total + 7) / 8;
    if (ctas > 0x7fffffffLL) return agn_fail(ctx, AGN_EINVAL, "silu_mul_q8_k: too many blocks for one launch");
    AGN_CUDA(ctx, cudaSetDevice(ctx->device));
    agn_launch(ctx, silu_mul_q8k_kernel, dim3((unsigned)ctas), dim3(256), 0, gate, up, total, d, qs, bsums);
    AGN_LAUNCHED(ctx, "silu_mul_q8_k");
    return AGN_OK;
}
