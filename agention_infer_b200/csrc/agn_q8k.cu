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
// 4 bytes read and 1.14 written per value: bound by HBM, provided the instruction count stays
// near 120 per block and warp (it is 122).  One warp owns one block of 256 values, lane l holding values
// 4l..4l+3 and 128+4l..128+4l+3 (two coalesced 128-bit loads); the maximum is two warp-wide redux
// instructions, a group of 16 values is four neighbouring lanes, the quantised values leave as one
// 32-bit store per lane and half-block.  The fused kernels compute their f32 values with the
// functions the unfused kernels use and hand them to the same block routine.
#include "agn_common.cuh"
#include "agn_row_math.cuh"

namespace {

constexpr int QK_K = 256;

// Warp-wide minimum of f32 values in one instruction (sm_100a), the counterpart of agn_warp_max; NaN
// operands are ignored (the result is NaN only when every lane holds one).
__device__ __forceinline__ float warp_min_f32(float v) {
    float r;
    asm volatile("redux.sync.min.f32 %0, %1, 0xffffffff;" : "=f"(r) : "f"(v));
    return r;
}

// Three-input maximum / minimum (one instruction on sm_100); a NaN operand is ignored.
__device__ __forceinline__ float max3_f32(float a, float b, float c) {
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}
__device__ __forceinline__ float min3_f32(float a, float b, float c) {
    float r;
    asm("min.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
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
    float mx = -INFINITY, mn = INFINITY;  // max / min drop a NaN operand, as the scan's `av > amax` does
#pragma unroll
    for (int k = 0; k < N; k++) {
        mx = max3_f32(max3_f32(mx, v[k].x, v[k].y), v[k].z, v[k].w);
        mn = min3_f32(min3_f32(mn, v[k].x, v[k].y), v[k].z, v[k].w);
    }
    mx = agn_warp_max(mx);
    mn = warp_min_f32(mn);
    if (mx != -mn) return mx > -mn ? mx : mn;  // one sign holds the largest magnitude alone
    // +a and -a both present, nothing but zeros, or nothing but NaN (mx = -inf, mn = +inf)
    const float amax = mx;
    if (!(amax > 0.0f)) return 0.0f;
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

// q = min(round_half_away(iscale * v) as i32, 127) as i8.  Rounding half away from zero as
// trunc(p + copysign(0.5 - 2^-25, p)): exact for every f32 p (a p below k + 0.5 stays below the
// integer after the addition, k + 0.5 itself lands on it), three instructions instead of roundf's
// sequence.  The conversion saturates and sends NaN to 0, like Rust's `as i32`.
__device__ __forceinline__ int q8k_q1(float v, float iscale) {
    const float p = __fmul_rn(iscale, v);
    const float t = __fadd_rn(p, copysignf(__int_as_float(0x3effffff), p));
    return min(__float2int_rz(t), 127);
}

// Four values -> four bytes (`as i8` keeps the low byte), little-endian in value order: any iscale.
__device__ __forceinline__ uint32_t q8k_q4_general(float4 v, float iscale) {
    const uint32_t a = (uint32_t)q8k_q1(v.x, iscale) & 0xffu, b = (uint32_t)q8k_q1(v.y, iscale) & 0xffu;
    const uint32_t c = (uint32_t)q8k_q1(v.z, iscale) & 0xffu, d = (uint32_t)q8k_q1(v.w, iscale) & 0xffu;
    return a | (b << 8) | (c << 16) | (d << 24);
}

// The same for a FINITE iscale, which is every block whose largest magnitude is a normal number:
// then |iscale * v| <= 127 * (1 + 2^-23) for every finite v of the block (|v| <= |max|), a NaN or
// infinite product can only be NaN (iscale = -127 / inf = 0), so the rounded value lies in
// [-127, 127] or is 0: no clamp at 127 and no wrap can occur, and the two products / sums per
// instruction of the packed f32x2 forms and the saturating pack give the same bytes.
__device__ __forceinline__ uint32_t q8k_q4_finite(float4 v, float iscale) {
    const float2 is2 = make_float2(iscale, iscale);
    const float2 p01 = __fmul2_rn(make_float2(v.x, v.y), is2), p23 = __fmul2_rn(make_float2(v.z, v.w), is2);
    const float half = __int_as_float(0x3effffff);  // 0.5 - 2^-25
    const float2 t01 = __fadd2_rn(p01, make_float2(copysignf(half, p01.x), copysignf(half, p01.y)));
    const float2 t23 = __fadd2_rn(p23, make_float2(copysignf(half, p23.x), copysignf(half, p23.y)));
    const int a = __float2int_rz(t01.x), b = __float2int_rz(t01.y), c = __float2int_rz(t23.x), d = __float2int_rz(t23.y);
    uint32_t hi, all;  // cvt.pack: {sat8(first), sat8(second)} into the low half, the third operand's low half above it
    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(hi) : "r"(d), "r"(c), "r"(0));
    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(all) : "r"(b), "r"(a), "r"(hi));
    return all;
}

// iscale = -127 / max and d = 1 / iscale (both correctly rounded, as the reference's divisions); a
// block with nothing above 0 (mx = 0) has d = 0, and its iscale = -127 / 0 = -inf sends it down the
// general path below, where every product is NaN (0 * inf) and quantises to 0.
__device__ __forceinline__ void q8k_scales(float mx, float &iscale, float &d) {
    iscale = __fdiv_rn(-127.0f, mx);
    d = mx != 0.0f ? __frcp_rn(iscale) : 0.0f;
}

// The two float4 of a lane for one block -> their bytes.  (The branch is uniform over the block.)
__device__ __forceinline__ void q8k_q8(const float4 &v0, const float4 &v1, float iscale, uint32_t &p0, uint32_t &p1) {
    if (fabsf(iscale) < INFINITY) {
        p0 = q8k_q4_finite(v0, iscale);
        p1 = q8k_q4_finite(v1, iscale);
    } else {
        p0 = q8k_q4_general(v0, iscale);
        p1 = q8k_q4_general(v1, iscale);
    }
}

// A whole block held by one warp as two float4 per lane: scale, quantise, store, with the sums of
// the sixteen groups of 16 values (four neighbouring lanes each).  d_block: the block's scale;
// qs_lane: the lane's 32-bit word of the block's first half (qs32 + 64 * block + lane); bs_lane: the
// group sum of the lane's quad in the first half (bsums + 16 * block + lane / 4).
__device__ __forceinline__ void q8k_block_from_warp(const float4 (&v)[2], int lane, float *d_block, uint32_t *qs_lane,
                                                    int16_t *bs_lane) {
    const float mx = q8k_first_max<2>(v, lane);
    float iscale, d;
    q8k_scales(mx, iscale, d);
    if (lane == 0) *d_block = d;
    uint32_t p0, p1;
    q8k_q8(v[0], v[1], iscale, p0, p1);
    qs_lane[0] = p0;
    qs_lane[32] = p1;
    int s0 = __dp4a((int)p0, 0x01010101, 0), s1 = __dp4a((int)p1, 0x01010101, 0);  // sums of the four signed bytes
    s0 += __shfl_xor_sync(0xffffffffu, s0, 1);
    s1 += __shfl_xor_sync(0xffffffffu, s1, 1);
    s0 += __shfl_xor_sync(0xffffffffu, s0, 2);
    s1 += __shfl_xor_sync(0xffffffffu, s1, 2);
    if ((lane & 3) == 0) {
        bs_lane[0] = (int16_t)s0;
        bs_lane[8] = (int16_t)s1;
    }
}

// ---- rows of f32 values -> Q8_K ---------------------------------------------------------------

// One warp per block; block B of the launch is block B % nb of row B / nb.  VEC: rows are whole
// float4 (n % 4 == 0, x 16-byte aligned); otherwise element-wise loads.  FLAT: n % 256 == 0, so the
// blocks of all rows are one contiguous sequence and block B starts at x + 256 * B.
template <bool VEC, bool FLAT>
__global__ void __launch_bounds__(256)
quantize_rows_q8k_kernel(const float *__restrict__ x, int64_t n_blocks_total, int nb, int n, float *__restrict__ d,
                         int8_t *__restrict__ qs, int16_t *__restrict__ bsums) {
    agn_pdl_prologue();
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    const int64_t B0 = (int64_t)blockIdx.x * 8;  // the CTA's first block (256 threads: eight warps)
    if (B0 + warp >= n_blocks_total) return;
    float4 v[2];
    if (FLAT) {
        const float4 *xc = reinterpret_cast<const float4 *>(x) + B0 * 64;
        v[0] = __ldcs(xc + (warp * 64u + lane));
        v[1] = __ldcs(xc + (warp * 64u + 32u + lane));
    } else {
        const int64_t B = B0 + warp;
        int64_t row;
        int b;
        if (n_blocks_total <= 0x7fffffffLL) {  // 32-bit division when it is enough
            const uint32_t r32 = (uint32_t)B / (uint32_t)nb;
            row = r32;
            b = (int)((uint32_t)B - r32 * (uint32_t)nb);
        } else {
            row = B / nb;
            b = (int)(B - row * nb);
        }
        const float *xr = x + row * (int64_t)n;
#pragma unroll
        for (int k = 0; k < 2; k++) {
            const int e = b * QK_K + k * 128 + 4 * (int)lane;  // first of the lane's four values
            if (VEC) {
                v[k] = e < n ? __ldcs(reinterpret_cast<const float4 *>(xr + e)) : make_float4(0.f, 0.f, 0.f, 0.f);
            } else {
                v[k].x = e + 0 < n ? xr[e + 0] : 0.0f;
                v[k].y = e + 1 < n ? xr[e + 1] : 0.0f;
                v[k].z = e + 2 < n ? xr[e + 2] : 0.0f;
                v[k].w = e + 3 < n ? xr[e + 3] : 0.0f;
            }
        }
    }
    q8k_block_from_warp(v, (int)lane, d + B0 + warp, reinterpret_cast<uint32_t *>(qs) + B0 * 64 + (warp * 64u + lane),
                        bsums + B0 * 16 + (warp * 16u + (lane >> 2)));
}

// ---- SiLU·mul -> Q8_K --------------------------------------------------------------------------

// gate and up are [T, I] with I % 256 == 0, so the blocks of all rows form one flat sequence.
__global__ void __launch_bounds__(256)
silu_mul_q8k_kernel(const float *__restrict__ gate, const float *__restrict__ up, int64_t n_blocks_total,
                    float *__restrict__ d, int8_t *__restrict__ qs, int16_t *__restrict__ bsums) {
    agn_pdl_prologue();
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    const int64_t B0 = (int64_t)blockIdx.x * 8;  // the CTA's first block (256 threads: eight warps)
    if (B0 + warp >= n_blocks_total) return;
    const float4 *g4 = reinterpret_cast<const float4 *>(gate) + B0 * 64, *u4 = reinterpret_cast<const float4 *>(up) + B0 * 64;
    const uint32_t i = warp * 64u + lane;
    const float4 g0 = __ldcs(g4 + i), g1 = __ldcs(g4 + (i + 32u));
    const float4 u0 = __ldcs(u4 + i), u1 = __ldcs(u4 + (i + 32u));
    float4 v[2];
    v[0] = agn_silu_mul4(g0, u0);
    v[1] = agn_silu_mul4(g1, u1);
    q8k_block_from_warp(v, (int)lane, d + B0 + warp, reinterpret_cast<uint32_t *>(qs) + B0 * 64 + (warp * 64u + lane),
                        bsums + B0 * 16 + (warp * 16u + (lane >> 2)));
}

// ---- RMSNorm (and residual add + RMSNorm) -> Q8_K ---------------------------------------------

// One CTA per row, the row in registers between the sum of squares and the scaling as in
// rms_norm_rows_kernel, but with a warp owning whole blocks: warp w holds blocks w*BPW, w*BPW + 1, ...
// (BPW of them, two float4 per lane each), so a block's maximum, its two divisions and its group
// sums stay inside the warp and the CTA meets at one barrier only (the sum of squares).  That sum
// adds the same squares in another order than rms_norm_rows_kernel does, so the scale factor can
// differ from that kernel's in the last bit, and with it a quantised value here and there by one
// step.
// (Register cap: 32 keeps nine 224-thread CTAs — nine rows — per SM, which the residual form, with twice
// the loads in flight per row, is fastest with; the plain form gains a little from 40 and seven rows.)
template <int BPW, bool RESIDUAL, bool EXACT>
__global__ void __maxnreg__(BPW > 2 ? 64 : RESIDUAL ? 32 : 40)
rms_norm_q8k_blocks_kernel(const float *__restrict__ x, const float *__restrict__ delta, const float4 *__restrict__ w,
                           float *__restrict__ new_x, int nb, float inv_n, float eps, float *__restrict__ d,
                           int8_t *__restrict__ qs, int16_t *__restrict__ bsums) {
    agn_pdl_prologue();
    __shared__ float red[32];
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    // Warp w owns blocks w*BPW .. w*BPW + BPW-1: every access of the lane is one index (i0) plus a
    // compile-time offset.  EXACT: nb == BPW * nwarps, no block of any warp lies past the row.
    const uint32_t b0 = warp * BPW, i0 = b0 * 64u + lane;
    const int64_t row = (int64_t)blockIdx.x * nb * 64;  // in vectors of four activations
    const float4 *xr = reinterpret_cast<const float4 *>(x) + row + i0;
    float4 v[BPW][2];
#pragma unroll
    for (int j = 0; j < BPW; j++) {
#pragma unroll
        for (int h = 0; h < 2; h++)
            v[j][h] = (EXACT || b0 + j < (uint32_t)nb) ? __ldcs(xr + (j * 64 + h * 32)) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    if (RESIDUAL) {
        const float4 *dr = reinterpret_cast<const float4 *>(delta) + row + i0;
        float4 *nr = reinterpret_cast<float4 *>(new_x) + row + i0;
#pragma unroll
        for (int j = 0; j < BPW; j++) {
            if (EXACT || b0 + j < (uint32_t)nb) {
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    const float4 dl = __ldcs(dr + (j * 64 + h * 32));
                    v[j][h].x += dl.x; v[j][h].y += dl.y; v[j][h].z += dl.z; v[j][h].w += dl.w;
                    __stcs(nr + (j * 64 + h * 32), v[j][h]);
                }
            }
        }
    }
    float2 ss2 = make_float2(0.0f, 0.0f);
#pragma unroll
    for (int j = 0; j < BPW; j++) ss2 = agn_sum_sq4(v[j][1], agn_sum_sq4(v[j][0], ss2));
    // sum over the CTA: within the warp, then the per-warp sums (at most 32) by every warp again
    float ss = agn_warp_sum(ss2.x + ss2.y);
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    ss = agn_warp_sum(lane < nwarps ? red[lane] : 0.0f);
    const float inv = agn_inv_rms(ss, inv_n, eps);
    const int64_t first_block = (int64_t)blockIdx.x * nb;
    const float4 *wl = w + i0;
    float *d_warp = d + first_block + b0;
    uint32_t *qs_lane = reinterpret_cast<uint32_t *>(qs) + first_block * 64 + i0;
    int16_t *bs_lane = bsums + first_block * 16 + b0 * 16u + (lane >> 2);
#pragma unroll
    for (int j = 0; j < BPW; j++) {
        if (EXACT || b0 + j < (uint32_t)nb) {
            float4 o[2];
            o[0] = agn_scale4(agn_mul4(__ldg(wl + j * 64), v[j][0]), inv);  // (w * x) * inv
            o[1] = agn_scale4(agn_mul4(__ldg(wl + (j * 64 + 32)), v[j][1]), inv);
            q8k_block_from_warp(o, (int)lane, d_warp + j, qs_lane + j * 64, bs_lane + j * 16);
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
    const float4 *w4 = reinterpret_cast<const float4 *>(w);
    const float inv_n = 1.0f / (float)(n4 * 4);
    const dim3 grid((unsigned)T);
    // the fewest blocks per warp in {1, 2, 4} that keep the CTA at <= 8 warps when possible
    const int nb = (int)(H / QK_K);
    int bpw = 1;
    while (bpw < 4 && (nb + bpw - 1) / bpw > 8) bpw *= 2;
    if (ctx->tune_rms_q8k_bpw == 1 || ctx->tune_rms_q8k_bpw == 2 || ctx->tune_rms_q8k_bpw == 4) {
        bpw = ctx->tune_rms_q8k_bpw;
        while (bpw < 4 && (nb + bpw - 1) / bpw > 32) bpw *= 2;
    }
    const int nwarps = (nb + bpw - 1) / bpw;
    const dim3 block(32 * nwarps);
    const bool exact = nwarps * bpw == nb;
#define AGN_Q8K_LAUNCH(BPW)                                                                                              \
    do {                                                                                                                 \
        if (exact)                                                                                                       \
            agn_launch(ctx, rms_norm_q8k_blocks_kernel<BPW, RESIDUAL, true>, grid, block, 0, x, delta, w4, new_x, nb, inv_n, eps, \
                       d, qs, bsums);                                                                                    \
        else                                                                                                             \
            agn_launch(ctx, rms_norm_q8k_blocks_kernel<BPW, RESIDUAL, false>, grid, block, 0, x, delta, w4, new_x, nb, inv_n,     \
                       eps, d, qs, bsums);                                                                               \
    } while (0)
    switch (bpw) {
    case 1: AGN_Q8K_LAUNCH(1); break;
    case 2: AGN_Q8K_LAUNCH(2); break;
    default: AGN_Q8K_LAUNCH(4); break;
    }
#undef AGN_Q8K_LAUNCH
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
    const dim3 grid((unsigned)ctas), block(256);
    if (n % QK_K == 0 && agn_aligned16(x))
        agn_launch(ctx, quantize_rows_q8k_kernel<true, true>, grid, block, 0, x, total, (int)nb, (int)n, d, qs, bsums);
    else if (n % 4 == 0 && agn_aligned16(x))
        agn_launch(ctx, quantize_rows_q8k_kernel<true, false>, grid, block, 0, x, total, (int)nb, (int)n, d, qs, bsums);
    else
        agn_launch(ctx, quantize_rows_q8k_kernel<false, false>, grid, block, 0, x, total, (int)nb, (int)n, d, qs, bsums);
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
