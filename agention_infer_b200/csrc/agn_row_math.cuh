// Device arithmetic shared by the row kernels and by the kernels that fuse an activation
// quantiser onto them: one definition, so that a fused kernel produces the same bits as the
// separate launches.
#pragma once
#include "agn_common.cuh"

#ifdef __CUDACC__

// Sum over the CTA; every thread returns the same value.  Warp shuffles, then across warps
// through shared memory in a fixed order: the result does not depend on scheduling.  For a kernel
// that sums once per CTA: nothing writes smem again, so there is no barrier after the reads.
__device__ __forceinline__ float agn_block_sum_once(float v, float *smem) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = agn_warp_sum(v);
    if (lane == 0) smem[warp] = v;
    __syncthreads();
    float total = 0.0f;
    for (int w = 0; w < nwarps; w++) total += smem[w];
    return total;
}

// 1 / sqrt(ss / n + eps), the factor every element of the row is multiplied by.  Evaluated as
// rsqrt(ss * (1/n) + eps) with the hardware reciprocal square root (2 ulp): three instructions
// instead of the ~45 of two IEEE divisions and a square root, which every thread of the CTA would
// run while the row's stores wait.  Together with the multiplication by 1/n this moves a result
// by a few 1e-7 relative, inside the 1e-5 tolerance; infinities, zeros and NaN come out as they
// do from the exact sequence (rsqrt(inf) = 0, rsqrt(0) = inf).
__device__ __forceinline__ float agn_inv_rms(float ss, float inv_n, float eps) { return rsqrtf(__fmaf_rn(ss, inv_n, eps)); }

// silu(g) * u = g / (1 + exp(-g)) * u (src/model/llama/cpu_path.rs:228-229)
__device__ __forceinline__ float agn_silu_mul1(float g, float u) {
    // IEEE division (-prec-div=true is nvcc's default; no fast-math anywhere).
    const float silu = g / (1.0f + expf(-g));
    return silu * u;
}

__device__ __forceinline__ float4 agn_silu_mul4(float4 g, float4 u) {
    float4 o;
    o.x = agn_silu_mul1(g.x, u.x);
    o.y = agn_silu_mul1(g.y, u.y);
    o.z = agn_silu_mul1(g.z, u.z);
    o.w = agn_silu_mul1(g.w, u.w);
    return o;
}

// Q8_0 cache packing of four values of a block with the given scale (`KvDtype::pack`,
// src/model/mod.rs:574-583): q = (v / scale).round().clamp(-127, 127) as i8, NaN -> 0, as bytes.
// The reference divides every value by the scale (IEEE) and rounds half away from zero: ~25
// instructions per value.  Here the quotient is first approximated as v * rcp.approx(scale): within
// 1.5 * 2^-23 relative of the true quotient t, so within 3.1e-5 of fl(t) for |t| < 128.  If that
// approximation lies more than 1e-4 away from every k + 0.5, fl(t) rounds to the same integer, which
// is read off the mantissa of qa + 1.5 * 2^23 (round to nearest; exact ties never get here).  A lane with a
// value too close to a boundary, beyond +-127.25, or not finite (NaN value, infinite or subnormal
// scale) recomputes its four values the reference's way.  Same bytes for every input.
__device__ __forceinline__ void agn_q8_0_quant4(const float (&x)[4], float scale, uint32_t (&q)[4]) {
    float inv;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(inv) : "f"(scale));
    bool sure = true;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const float qa = __fmul_rn(x[i], inv);
        // 1.5 * 2^23 + round_to_nearest(qa) for |qa| < 2^22: the low mantissa bits are the integer in two's complement
        const float m = __fadd_rn(qa, 12582912.0f);
        const float g = __fsub_rn(qa, __fsub_rn(m, 12582912.0f));  // qa - round_to_nearest(qa), in [-0.5, 0.5]
        sure = sure && (fabsf(g) <= 0.4999f) && (fabsf(qa) < 127.25f);  // false for NaN
        q[i] = (uint32_t)__float_as_int(m) & 0xffu;
    }
    if (!sure) {
#pragma unroll
        for (int i = 0; i < 4; i++) {
            float r = roundf(__fdiv_rn(x[i], scale));
            r = (r != r) ? 0.0f : fminf(fmaxf(r, -127.0f), 127.0f);  // Rust's `NaN as i8` is 0 (a NaN value, or inf / inf)
            q[i] = (uint32_t)(unsigned char)(signed char)(int)r;
        }
    }
}

#endif  // __CUDACC__

// CTA shape of the register-resident RMSNorm kernels for a row of n4 vectors of four values:
// thread i holds vectors i + k * threads, k < vpt.  The smallest vpt in {1, 2, 4, 8} that keeps
// the CTA at <= 256 threads when possible: more rows resident per SM and more loads in flight per
// thread.  The `rms_vpt` option overrides it.
static inline void agn_rms_shape(const agn_ctx *ctx, int n4, int *vpt_out, int *threads_out) {
    int vpt = 1;
    while (vpt < 8 && (n4 + vpt - 1) / vpt > 256) vpt *= 2;
    if (ctx->tune_rms_vpt == 1 || ctx->tune_rms_vpt == 2 || ctx->tune_rms_vpt == 4 || ctx->tune_rms_vpt == 8) {
        vpt = ctx->tune_rms_vpt;
        while (vpt < 8 && (n4 + vpt - 1) / vpt > 1024) vpt *= 2;
    }
    int threads = (n4 + vpt - 1) / vpt;
    threads = ((threads + 31) / 32) * 32;
    if (threads > 1024) threads = 1024;
    *vpt_out = vpt;
    *threads_out = threads;
}
