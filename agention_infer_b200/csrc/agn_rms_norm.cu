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
//
// Batches with more rows than the GPU holds CTAs run as a persistent kernel
// (rms_norm_ring_kernel): a few CTAs per SM, each looping over rows blockIdx.x, blockIdx.x +
// gridDim.x, ..., with the rows ahead of the current one already on their way into a ring of
// shared-memory slots (one bulk asynchronous copy per row, issued by one thread, completing on
// the slot's mbarrier).  HBM reads of the next rows overlap the reduction and the stores of the
// current one, every SM gets the same number of rows to within one, and the per-CTA set-up
// (weight vector, barriers) is paid once per CTA instead of once per row.
#include "agn_common.cuh"
#include "agn_row_math.cuh"

namespace {

// (The sum of squares runs on fused multiply-adds, two per instruction (agn_sum_sq4): one rounding
// each; the reference's separate multiply and add differ from it by less than the reordering of
// the sum already does.)

// T: storage type of x, delta and new_x; OT: storage type of the normed output (T, or a 16-bit
// type for a row that feeds a matmul with half-precision operands).
// (Two CTAs of 1024 threads per SM as the launch bound caps the kernel at 32 registers for up to
// four float4 per thread, which is what keeps nine 224-thread CTAs — nine rows — resident per SM.)
template <typename T, typename OT, int VPT, bool RESIDUAL, bool RECIP>
__global__ void __launch_bounds__(1024, VPT <= 4 ? 2 : 1)
rms_norm_rows_kernel(const T *__restrict__ x, const T *__restrict__ delta, const float4 *__restrict__ w,
                     T *__restrict__ new_x, OT *__restrict__ out, int n4, float n_f, float inv_n, float eps) {
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
    float2 ss2 = make_float2(0.0f, 0.0f);
#pragma unroll
    for (int k = 0; k < VPT; k++) ss2 = agn_sum_sq4(v[k], ss2);
    float ss = agn_block_sum_once(ss2.x + ss2.y, red);
    const float rms = sqrtf(ss / n_f + eps);  // same operations as the reference: sum/n + eps (used by the dividing arm)
    const float inv = agn_inv_rms(ss, inv_n, eps);
#pragma unroll
    for (int k = 0; k < VPT; k++) {
        const int i = threadIdx.x + k * blockDim.x;
        if (i < n4) {
            const float4 ww = __ldg(w + i);
            float4 o;
            if (RECIP) {
                o = agn_scale4(agn_mul4(ww, v[k]), inv);  // (w * x) * inv, two roundings, as the scalar form
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

// Persistent form.  Shared memory: `slots` row slots (x row, then the delta row when RESIDUAL)
// followed by one mbarrier per slot.  Thread t owns float4 number t + k*blockDim of the row, as in
// the kernel above; its part of the weight vector stays in registers for the CTA's lifetime.
template <typename T, typename OT, int VPT, bool RESIDUAL>
__global__ void __launch_bounds__(1024)
rms_norm_ring_kernel(const T *__restrict__ x, const T *__restrict__ delta, const float4 *__restrict__ w,
                     T *__restrict__ new_x, OT *__restrict__ out, int64_t T_rows, int n4, float inv_n, float eps, int slots,
                     int spin_limit, uint32_t *flags) {
    extern __shared__ __align__(128) unsigned char ring[];
    __shared__ float red[2][32];
    const uint32_t row_bytes = (uint32_t)n4 * 4u * (uint32_t)sizeof(T);  // a multiple of 16 (checked by the host)
    const uint32_t slot_bytes = RESIDUAL ? 2u * row_bytes : row_bytes;
    uint64_t *full = reinterpret_cast<uint64_t *>(ring + (size_t)slots * slot_bytes);
    if (threadIdx.x == 0) {
        for (int s = 0; s < slots; s++) agn_mbar_init(&full[s], 1);
        agn_mbar_init_fence();
    }
    __syncthreads();
    agn_pdl_launch_dependents();
    agn_pdl_wait();  // global memory is touched from here on

    const int64_t first = blockIdx.x, stride = gridDim.x;
    const int n_my = first < T_rows ? (int)((T_rows - first + stride - 1) / stride) : 0;
    auto issue = [&](int j) {  // thread 0 only: row number j of this CTA into slot j % slots
        const int64_t row = (first + (int64_t)j * stride) * n4;  // in vectors of four activations
        unsigned char *dst = ring + (size_t)(j % slots) * slot_bytes;
        uint64_t *bar = &full[j % slots];
        agn_mbar_expect_tx(bar, slot_bytes);
        agn_bulk_g2s(dst, reinterpret_cast<const unsigned char *>(x) + row * (int64_t)(4 * sizeof(T)), row_bytes, bar);
        if (RESIDUAL)
            agn_bulk_g2s(dst + row_bytes, reinterpret_cast<const unsigned char *>(delta) + row * (int64_t)(4 * sizeof(T)), row_bytes, bar);
    };
    if (threadIdx.x == 0)
        for (int j = 0; j < slots && j < n_my; j++) issue(j);

    // the thread's part of the weight vector stays in registers (up to four float4; with eight,
    // 1024-thread CTAs would spill, so those re-read it from L1 per row)
    constexpr int WREG = VPT <= 4 ? VPT : 1;
    float4 ww[WREG];
    if (VPT <= 4) {
#pragma unroll
        for (int k = 0; k < WREG; k++) {
            const int i = threadIdx.x + k * blockDim.x;
            ww[k] = i < n4 ? __ldg(w + i) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;

    for (int it = 0; it < n_my; it++) {
        const int slot = it % slots;
        const int64_t row = (first + (int64_t)it * stride) * n4;
        const int failed = !agn_mbar_wait(&full[slot], (uint32_t)(it / slots) & 1u, spin_limit);
        const T *sx = reinterpret_cast<const T *>(ring + (size_t)slot * slot_bytes);
        float4 v[VPT];
#pragma unroll
        for (int k = 0; k < VPT; k++) {
            const int i = threadIdx.x + k * blockDim.x;
            v[k] = i < n4 ? ActVec<T>::load_shared(sx, i) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        if (RESIDUAL) {
            const T *sd = reinterpret_cast<const T *>(ring + (size_t)slot * slot_bytes + row_bytes);
#pragma unroll
            for (int k = 0; k < VPT; k++) {
                const int i = threadIdx.x + k * blockDim.x;
                if (i < n4) {
                    const float4 d = ActVec<T>::load_shared(sd, i);
                    v[k].x += d.x; v[k].y += d.y; v[k].z += d.z; v[k].w += d.w;
                }
            }
        }
        float2 ss2 = make_float2(0.0f, 0.0f);
        if (RESIDUAL && sizeof(T) == 2) {
            // the f16 residual form normalises the STORED new_x (see rms_norm_rows_kernel)
#pragma unroll
            for (int k = 0; k < VPT; k++) {
                float4 r;
                r.x = __half2float(__float2half_rn(v[k].x)); r.y = __half2float(__float2half_rn(v[k].y));
                r.z = __half2float(__float2half_rn(v[k].z)); r.w = __half2float(__float2half_rn(v[k].w));
                ss2 = agn_sum_sq4(r, ss2);
            }
        } else {
#pragma unroll
            for (int k = 0; k < VPT; k++) ss2 = agn_sum_sq4(v[k], ss2);
        }
        float ss = agn_warp_sum(ss2.x + ss2.y);
        float *r2 = red[it & 1];  // two sets: a warp may already write the next row's partial while another still sums this one's
        if (lane == 0) r2[warp] = ss;
        // partial sums visible; every thread has read its part of the slot; and one CTA-wide answer
        // to "did any thread's wait run out", so that all threads leave together
        if (__syncthreads_or(failed)) {
            // report it, give the copies still in flight one more bounded wait each (they target
            // this CTA's shared memory), and leave without storing the row
            if (threadIdx.x == 0) {
                atomicOr(flags, AGN_FLAG_TIMEOUT);
                for (int j = it; j < n_my && j < it + slots; j++) (void)agn_mbar_wait(&full[j % slots], (uint32_t)(j / slots) & 1u, spin_limit);
            }
            return;
        }
        if (threadIdx.x == 0 && it + slots < n_my) issue(it + slots);
        float total = 0.0f;
        for (int wi = 0; wi < nwarps; wi++) total += r2[wi];
        const float inv = agn_inv_rms(total, inv_n, eps);
#pragma unroll
        for (int k = 0; k < VPT; k++) {
            const int i = threadIdx.x + k * blockDim.x;
            if (i < n4) {
                float4 xv = v[k];
                if (RESIDUAL) {
                    ActVec<T>::store(new_x, row + i, xv);
                    if (sizeof(T) == 2) {
                        xv.x = __half2float(__float2half_rn(xv.x)); xv.y = __half2float(__float2half_rn(xv.y));
                        xv.z = __half2float(__float2half_rn(xv.z)); xv.w = __half2float(__float2half_rn(xv.w));
                    }
                }
                const float4 wk = VPT <= 4 ? ww[k < WREG ? k : 0] : __ldg(w + i);
                ActVec<OT>::store(out, row + i, agn_scale4(agn_mul4(wk, xv), inv));
            }
        }
    }
}

// Tries the persistent form; false = not applicable here (the caller launches the CTA-per-row kernel).
template <typename T, typename OT, int VPT, bool RESIDUAL>
bool launch_ring(agn_ctx *ctx, const T *x, const T *delta, const float *w, T *new_x, OT *out, int64_t T_rows, int n4, float eps,
                 int threads) {
    if (ctx->tune_rms_ring == 0) return false;
    const size_t row_bytes = (size_t)n4 * 4 * sizeof(T);
    const size_t slot_bytes = RESIDUAL ? 2 * row_bytes : row_bytes;
    if (row_bytes % 16 != 0 || !agn_aligned16(x) || (RESIDUAL && !agn_aligned16(delta))) return false;
    int slots = ctx->tune_rms_ring >= 2 ? ctx->tune_rms_ring : 3;
    if (slots > 8) slots = 8;
    while (slots > 2 && slots * slot_bytes + 64 > 100 * 1024) slots--;
    const size_t smem = slots * slot_bytes + 8 * (size_t)slots;
    if (smem > 200 * 1024) return false;
    auto kernel = rms_norm_ring_kernel<T, OT, VPT, RESIDUAL>;
    int per_sm = agn_ring_ctas_per_sm(ctx, kernel, threads, smem);
    if (per_sm < 1) return false;
    if (ctx->tune_rms_ring_ctas > 0 && ctx->tune_rms_ring_ctas < per_sm) per_sm = ctx->tune_rms_ring_ctas;
    int64_t grid = (int64_t)per_sm * ctx->sm_count;
    if (T_rows < 2 * grid && !ctx->tune_ring_force) return false;  // too few rows to keep a ring busy: one CTA per row is faster
    if (grid > T_rows) grid = T_rows;
    agn_launch(ctx, kernel, dim3((unsigned)grid), dim3(threads), smem, x, delta, reinterpret_cast<const float4 *>(w), new_x, out,
               T_rows, n4, 1.0f / (float)(n4 * 4), eps, slots, ctx->mbar_spin_limit, ctx->d_flags);
    ctx->flags_dirty = true;
    return true;
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
    ss = agn_block_sum_once(ss, red);
    const float inv = agn_inv_rms(ss, 1.0f / (float)H, eps);
    const T *src = RESIDUAL ? new_x : x;
    for (int64_t i = threadIdx.x; i < H; i += blockDim.x)
        ActVec<OT>::store1(out, row + i, w[i] * ActVec<T>::load1(src, row + i) * inv);
}

// Returns true when the persistent form was launched.
template <typename T, typename OT, int VPT, bool RESIDUAL>
bool launch_vec(agn_ctx *ctx, const T *x, const T *delta, const float *w, T *new_x, OT *out, int64_t T_rows, int n4,
                float eps, int threads) {
    const float4 *w4 = reinterpret_cast<const float4 *>(w);
    if (ctx->tune_rms_recip && launch_ring<T, OT, VPT, RESIDUAL>(ctx, x, delta, w, new_x, out, T_rows, n4, eps, threads)) return true;
    if (ctx->tune_rms_recip)
        agn_launch(ctx, rms_norm_rows_kernel<T, OT, VPT, RESIDUAL, true>, dim3((unsigned)T_rows), dim3(threads), 0, x, delta, w4,
                   new_x, out, n4, (float)(n4 * 4), 1.0f / (float)(n4 * 4), eps);
    else
        agn_launch(ctx, rms_norm_rows_kernel<T, OT, VPT, RESIDUAL, false>, dim3((unsigned)T_rows), dim3(threads), 0, x, delta, w4,
                   new_x, out, n4, (float)(n4 * 4), 1.0f / (float)(n4 * 4), eps);
    return false;
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
        int vpt, threads;
        agn_rms_shape(ctx, n4, &vpt, &threads);
        bool ring;
        switch (vpt) {
        case 1: ring = launch_vec<T, OT, 1, RESIDUAL>(ctx, x, delta, w, new_x, out, T_rows, n4, eps, threads); break;
        case 2: ring = launch_vec<T, OT, 2, RESIDUAL>(ctx, x, delta, w, new_x, out, T_rows, n4, eps, threads); break;
        case 4: ring = launch_vec<T, OT, 4, RESIDUAL>(ctx, x, delta, w, new_x, out, T_rows, n4, eps, threads); break;
        default: ring = launch_vec<T, OT, 8, RESIDUAL>(ctx, x, delta, w, new_x, out, T_rows, n4, eps, threads); break;
        }
        if (ring) AGN_LAUNCHED(ctx, "rms_norm_ring");
        else AGN_LAUNCHED(ctx, name);
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
