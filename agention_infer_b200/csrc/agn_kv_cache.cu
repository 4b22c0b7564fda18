// KV-cache write (pack) and read (unpack) for f16 and Q8_0 storage.
//
// Reference: `KvDtype::pack` / `unpack` (src/model/mod.rs:567-604), `KvCache::write`,
// `write_range` (:648-672) and `read_up_to` (:678-697); GPU twins `kv_cache_write` /
// `kv_cache_write_q8_0` (src/ops/kernels_wgpu.rs:566-698).  A cache holds, per layer,
// max_seq_len token slots of bytes_per_token = 2*hd (f16) or ceil(hd/32)*34 (Q8_0) bytes,
// hd = n_kv_heads * head_dim.
//
//   f16  : half::f16::from_f32 (round to nearest even) per element
//   Q8_0 : per 32 values: amax = max |v| ; scale = amax > 0 ? amax / 127 : 1 ;
//          store f16(scale) ; q = clamp(round(v / scale), -127, 127)   (round half away,
//          dividing by the f32 scale, not by the stored f16 one)
//
// Integer / byte outputs: bit-exact with the CPU code (f16 conversion by __float2half_rn; the
// division of every value by the scale through agn_q8_0_quant4, which takes the reference's IEEE
// division only where an approximate quotient could round differently).  Bound by HBM: 4 B read + 2 or 1.06 B written
// per element; eight lanes own one 32-value block (coalesced 128-bit loads, amax by three
// shuffles).
#include <cuda_fp16.h>
#include <math.h>

#include "agn_common.cuh"
#include "agn_row_math.cuh"

namespace {

struct KvArgs {
    const float *k, *v;
    unsigned char *k_cache, *v_cache;
    const int32_t *pos;
    int64_t T, hd, max_seq;
    int pos_start;
    int bytes_per_token;
    int words;  // Q8_0 in the GPU path's blocks of nine 32-bit words (f32 scale, offset-binary bytes)
    uint32_t *flags;
};

__device__ __forceinline__ int64_t kv_slot(const KvArgs &a, int64_t t) {
    const int64_t p = a.pos ? (int64_t)a.pos[t] : (int64_t)a.pos_start + t;
    return (p >= 0 && p < a.max_seq) ? p : -1;
}

// One CTA per (token, K or V): blockIdx.x = token, blockIdx.y = 0 (K) or 1 (V).  Eight lanes own
// one 32-value block (a float4 each), so a warp packs four blocks per pass.
__global__ void __launch_bounds__(256)
kv_write_q8_0_kernel(const KvArgs a) {
    agn_pdl_prologue();
    const int64_t t = blockIdx.x;
    const int lane8 = threadIdx.x & 7;
    const int nblk = (int)((a.hd + 31) >> 5);
    const float *src_row = (blockIdx.y ? a.v : a.k) + t * a.hd;
    const bool vec = (a.hd & 3) == 0 && ((reinterpret_cast<uintptr_t>(src_row) & 15) == 0);
    const int bpp = (int)(blockDim.x >> 3);  // blocks per pass
    const int e0 = lane8 * 4;
    // values of pass p, block b = p * bpp + (thread / 8): issued before the slot is known (below)
    auto load_pass = [&](int p, float (&x)[4]) {
        const int b = p * bpp + (int)(threadIdx.x >> 3);
        const int left = b < nblk ? (int)(a.hd - (int64_t)b * 32) : 0;  // elements of this (possibly partial) block
        const float *src = src_row + (int64_t)b * 32;
        x[0] = x[1] = x[2] = x[3] = 0.f;
        if (left > 0 && vec && e0 + 3 < left) {
            const float4 q = __ldcs(reinterpret_cast<const float4 *>(src + e0));
            x[0] = q.x; x[1] = q.y; x[2] = q.z; x[3] = q.w;
        } else if (left > 0) {
#pragma unroll
            for (int i = 0; i < 4; i++)
                if (e0 + i < left) x[i] = src[e0 + i];
        }
    };
    // The token's values do not depend on its position: their loads go out before the position load
    // returns, so the two memory latencies of this short kernel overlap instead of adding up.
    float x[4];
    load_pass(0, x);
    const int64_t slot = kv_slot(a, t);
    if (slot < 0) {  // same answer for the whole CTA
        if (threadIdx.x == 0) atomicOr(a.flags, AGN_FLAG_OOB_SLOT);
        return;
    }
    unsigned char *tok = (blockIdx.y ? a.v_cache : a.k_cache) + slot * a.bytes_per_token;
    // all lanes of a warp run the same number of passes (the shuffles below need them)
    const int passes = (nblk + bpp - 1) / bpp;
    for (int p = 0; p < passes; p++) {
        if (p > 0) load_pass(p, x);
        const int b = p * bpp + (int)(threadIdx.x >> 3);
        const bool on = b < nblk;
        const int left = on ? (int)(a.hd - (int64_t)b * 32) : 0;
        float amax = fmaxf(fmaxf(fabsf(x[0]), fabsf(x[1])), fmaxf(fabsf(x[2]), fabsf(x[3])));
#pragma unroll
        for (int o = 4; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        if (!on) continue;
        const float scale = amax > 0.0f ? __fdiv_rn(amax, 127.0f) : 1.0f;
        uint32_t q[4];
        agn_q8_0_quant4(x, scale, q);
        if (a.words) {  // nine aligned words per block; values past the row's end are 0, stored as byte 128
            uint32_t *blk32 = reinterpret_cast<uint32_t *>(tok + b * 36);
            if (lane8 == 0) blk32[0] = __float_as_uint(scale);
            blk32[1 + lane8] = (q[0] | (q[1] << 8) | (q[2] << 16) | (q[3] << 24)) ^ 0x80808080u;
            continue;
        }
        unsigned char *blk = tok + b * 34;
        if (lane8 == 0) *reinterpret_cast<uint16_t *>(blk) = __half_as_ushort(__float2half_rn(scale));
        if (e0 + 3 < left) {  // blocks are 2-byte aligned: two 16-bit stores
            *reinterpret_cast<uint16_t *>(blk + 2 + e0) = (uint16_t)(q[0] | (q[1] << 8));
            *reinterpret_cast<uint16_t *>(blk + 4 + e0) = (uint16_t)(q[2] | (q[3] << 8));
        } else {
#pragma unroll
            for (int i = 0; i < 4; i++)
                if (e0 + i < left) blk[2 + e0 + i] = q[i];
        }
    }
}

__global__ void __launch_bounds__(256)
kv_write_f16_kernel(const KvArgs a) {
    agn_pdl_prologue();
    const int64_t t = blockIdx.x;
    const float *src = (blockIdx.y ? a.v : a.k) + t * a.hd;
    unsigned char *cache = blockIdx.y ? a.v_cache : a.k_cache;
    // (a slot starts at a multiple of bytes_per_token from the cache base, so the alignment of the
    // destination is known before the position is)
    const bool vec = (a.hd & 3) == 0 && ((reinterpret_cast<uintptr_t>(src) & 15) == 0) &&
                     ((reinterpret_cast<uintptr_t>(cache) & 7) == 0) && (a.bytes_per_token & 7) == 0;
    const int n4 = (int)(a.hd >> 2);
    // The token's values do not depend on its position: the first load goes out before the position
    // load returns, so the two memory latencies of this short kernel overlap instead of adding up.
    float4 first = make_float4(0.f, 0.f, 0.f, 0.f);
    if (vec && (int)threadIdx.x < n4) first = __ldcs(reinterpret_cast<const float4 *>(src) + threadIdx.x);
    const int64_t slot = kv_slot(a, t);
    if (slot < 0) {
        if (threadIdx.x == 0) atomicOr(a.flags, AGN_FLAG_OOB_SLOT);
        return;
    }
    __half *dst = reinterpret_cast<__half *>(cache + slot * a.bytes_per_token);
    if (vec) {
        if ((int)threadIdx.x < n4) ActVec<__half>::store(dst, threadIdx.x, first);
        for (int i = threadIdx.x + blockDim.x; i < n4; i += blockDim.x)
            ActVec<__half>::store(dst, i, __ldcs(reinterpret_cast<const float4 *>(src) + i));
    } else {
        for (int i = threadIdx.x; i < (int)a.hd; i += blockDim.x) dst[i] = __float2half_rn(src[i]);
    }
}

// Batches of more than a few tokens: one CTA packs TPC consecutive tokens of K or of V.  Every
// thread owns float4 number threadIdx.x of each of them and issues all its loads (values and
// positions) before the first use, so a thread has TPC independent chains in flight instead of
// one and the launch has TPC times fewer CTAs: with a CTA per token this kernel moves 20 MB in
// about three rounds of short-lived CTAs whose whole life is one dependent chain of two memory
// latencies.  Needs whole 32-value blocks (hd % 32 == 0), hd / 4 <= 256 threads and 16-byte
// aligned rows (checked by the host).
template <bool Q8, int TPC>
__global__ void __launch_bounds__(256)
kv_write_multi_kernel(const KvArgs a) {
    agn_pdl_prologue();
    const int64_t t0 = (int64_t)blockIdx.x * TPC;
    const float *src = blockIdx.y ? a.v : a.k;
    unsigned char *cache = blockIdx.y ? a.v_cache : a.k_cache;
    const int n4 = (int)(a.hd >> 2);
    const bool lane_on = (int)threadIdx.x < n4;
    float4 x[TPC];
    int64_t p[TPC];
#pragma unroll
    for (int j = 0; j < TPC; j++) {
        const int64_t t = t0 + j;
        const bool on = t < a.T;
        x[j] = (on && lane_on) ? __ldcs(reinterpret_cast<const float4 *>(src + t * a.hd) + threadIdx.x) : make_float4(0.f, 0.f, 0.f, 0.f);
        p[j] = !on ? 0 : (a.pos ? (int64_t)a.pos[t] : (int64_t)a.pos_start + t);
    }
#pragma unroll
    for (int j = 0; j < TPC; j++) {
        if (t0 + j >= a.T) continue;  // past the last token: the same answer in every thread of the CTA
        const bool in_range = p[j] >= 0 && p[j] < a.max_seq;
        if (!in_range && threadIdx.x == 0) atomicOr(a.flags, AGN_FLAG_OOB_SLOT);
        unsigned char *tok = cache + (in_range ? p[j] : 0) * a.bytes_per_token;
        if (!Q8) {
            if (in_range && lane_on) ActVec<__half>::store(reinterpret_cast<__half *>(tok), threadIdx.x, x[j]);
        } else {
            // eight lanes hold one 32-value block; every lane of the warp takes part in the shuffles
            float amax = fmaxf(fmaxf(fabsf(x[j].x), fabsf(x[j].y)), fmaxf(fabsf(x[j].z), fabsf(x[j].w)));
#pragma unroll
            for (int o = 4; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
            if (in_range && lane_on) {
                const float scale = amax > 0.0f ? __fdiv_rn(amax, 127.0f) : 1.0f;
                const int lane8 = threadIdx.x & 7;
                const float xs[4] = {x[j].x, x[j].y, x[j].z, x[j].w};
                uint32_t q[4];
                agn_q8_0_quant4(xs, scale, q);
                if (a.words) {
                    uint32_t *blk32 = reinterpret_cast<uint32_t *>(tok + (size_t)(threadIdx.x >> 3) * 36);
                    if (lane8 == 0) blk32[0] = __float_as_uint(scale);
                    blk32[1 + lane8] = (q[0] | (q[1] << 8) | (q[2] << 16) | (q[3] << 24)) ^ 0x80808080u;
                } else {
                    unsigned char *blk = tok + (size_t)(threadIdx.x >> 3) * 34;
                    if (lane8 == 0) *reinterpret_cast<uint16_t *>(blk) = __half_as_ushort(__float2half_rn(scale));
                    *reinterpret_cast<uint16_t *>(blk + 2 + 4 * lane8) = (uint16_t)(q[0] | (q[1] << 8));
                    *reinterpret_cast<uint16_t *>(blk + 4 + 4 * lane8) = (uint16_t)(q[2] | (q[3] << 8));
                }
            }
        }
    }
}

// read positions [0, n_pos): one CTA per (position, K or V), four values per thread
__global__ void __launch_bounds__(256)
kv_read_kernel(const unsigned char *__restrict__ k_cache, const unsigned char *__restrict__ v_cache, int64_t n_pos, int64_t hd,
               int bytes_per_token, int q8, float *__restrict__ k_out, float *__restrict__ v_out) {
    agn_pdl_prologue();
    const int64_t p = blockIdx.x;
    const unsigned char *tok = (blockIdx.y ? v_cache : k_cache) + p * bytes_per_token;
    float *dst = (blockIdx.y ? v_out : k_out) + p * hd;
    const bool vec = (hd & 3) == 0 && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0) &&
                     (q8 || (reinterpret_cast<uintptr_t>(tok) & 7) == 0);
    if (vec) {
        for (int i = threadIdx.x; i < (int)(hd >> 2); i += blockDim.x) {
            float4 o;
            if (q8 == 2) {  // nine words per block: f32 scale, then offset-binary bytes (dequant_kv_q8_0, kernels_wgpu.rs:705-718)
                const int d = 4 * i;
                const uint32_t *blk = reinterpret_cast<const uint32_t *>(tok + (d >> 5) * 36);
                const float scale = __uint_as_float(blk[0]);
                const uint32_t wq = blk[1 + ((d & 31) >> 2)];
                o.x = __fmul_rn((float)(int)(wq & 0xff) - 128.0f, scale);
                o.y = __fmul_rn((float)(int)((wq >> 8) & 0xff) - 128.0f, scale);
                o.z = __fmul_rn((float)(int)((wq >> 16) & 0xff) - 128.0f, scale);
                o.w = __fmul_rn((float)(int)(wq >> 24) - 128.0f, scale);
            } else if (q8) {
                const int d = 4 * i;
                const unsigned char *blk = tok + (d >> 5) * 34;
                const float scale = __half2float(__ushort_as_half(*reinterpret_cast<const uint16_t *>(blk)));
                const uint32_t lo = *reinterpret_cast<const uint16_t *>(blk + 2 + (d & 31));
                const uint32_t hi = *reinterpret_cast<const uint16_t *>(blk + 4 + (d & 31));
                o.x = __fmul_rn((float)(signed char)(lo & 0xff), scale);
                o.y = __fmul_rn((float)(signed char)(lo >> 8), scale);
                o.z = __fmul_rn((float)(signed char)(hi & 0xff), scale);
                o.w = __fmul_rn((float)(signed char)(hi >> 8), scale);
            } else {
                o = ActVec<__half>::load(reinterpret_cast<const __half *>(tok), i);
            }
            __stcs(reinterpret_cast<float4 *>(dst) + i, o);
        }
    } else {
        for (int d = threadIdx.x; d < (int)hd; d += blockDim.x) {
            float val;
            if (q8 == 2) {
                const unsigned char *blk = tok + (d >> 5) * 36;
                val = __fmul_rn((float)(int)blk[4 + (d & 31)] - 128.0f, __uint_as_float(*reinterpret_cast<const uint32_t *>(blk)));
            } else if (q8) {
                const unsigned char *blk = tok + (d >> 5) * 34;
                const float scale = __half2float(__ushort_as_half(*reinterpret_cast<const uint16_t *>(blk)));
                val = __fmul_rn((float)(signed char)blk[2 + (d & 31)], scale);
            } else {
                val = __half2float(reinterpret_cast<const __half *>(tok)[d]);
            }
            dst[d] = val;
        }
    }
}

int kv_bytes_per_token(int32_t dtype, int64_t hd) {
    if (dtype == AGN_F16) return (int)(hd * 2);
    if (dtype == AGN_Q8_0) return (int)(((hd + 31) / 32) * 34);
    if (dtype == AGN_KV_Q8_0_WORDS) return (int)(((hd + 31) / 32) * 36);  // `words_per_token * 4`, gpu_resident.rs:276-277
    return 0;
}

}  // namespace

extern "C" int64_t agn_kv_bytes_per_token(int32_t kv_dtype, int64_t head_dim_kv) {
    return head_dim_kv > 0 ? kv_bytes_per_token(kv_dtype, head_dim_kv) : 0;
}

extern "C" int32_t agn_kv_write_f32(agn_ctx *ctx, int32_t kv_dtype, const float *k, const float *v, void *k_cache,
                                    void *v_cache, int64_t T, int64_t head_dim_kv, const int32_t *pos, int32_t pos_start,
                                    int64_t max_seq_len) {
    AGN_CHECK_CTX(ctx);
    const int bpt = head_dim_kv > 0 ? kv_bytes_per_token(kv_dtype, head_dim_kv) : 0;
    const bool words = kv_dtype == AGN_KV_Q8_0_WORDS;
    if (kv_dtype != AGN_F16 && kv_dtype != AGN_Q8_0 && !words)
        return agn_fail(ctx, AGN_EUNSUPPORTED_DTYPE, "kv_write: KV dtype %d is neither f16 (1), q8_0 (8) nor q8_0 in words (1008)", kv_dtype);
    if (T < 0 || head_dim_kv <= 0 || max_seq_len <= 0)
        return agn_fail(ctx, AGN_EINVAL, "kv_write: T=%lld head_dim_kv=%lld max_seq_len=%lld", (long long)T,
                        (long long)head_dim_kv, (long long)max_seq_len);
    if (T == 0) return AGN_OK;
    if (!k || !v || !k_cache || !v_cache) return agn_fail(ctx, AGN_EINVAL, "kv_write: null pointer");
    if ((reinterpret_cast<uintptr_t>(k_cache) | reinterpret_cast<uintptr_t>(v_cache)) & (words ? 3 : 1))
        return agn_fail(ctx, AGN_EINVAL, "kv_write: caches must be %d-byte aligned", words ? 4 : 2);
    AGN_CUDA(ctx, cudaSetDevice(ctx->device));
    KvArgs a;
    a.k = k; a.v = v; a.k_cache = static_cast<unsigned char *>(k_cache); a.v_cache = static_cast<unsigned char *>(v_cache);
    a.pos = pos; a.T = T; a.hd = head_dim_kv; a.max_seq = max_seq_len; a.pos_start = pos_start; a.bytes_per_token = bpt; a.words = words ? 1 : 0;
    a.flags = ctx->d_flags;
    // several tokens per CTA once there are enough tokens to fill the GPU that way
    constexpr int TPC = 4;
    const bool multi = ctx->tune_kv_multi && T >= 4 * TPC * (int64_t)ctx->sm_count && head_dim_kv % 32 == 0 && head_dim_kv <= 1024 &&
                       agn_aligned16(k) && agn_aligned16(v) &&
                       (kv_dtype != AGN_F16 || (agn_aligned(k_cache, 8) && agn_aligned(v_cache, 8)));
    if (multi) {
        if (T > 0x7fffffffLL) return agn_fail(ctx, AGN_EINVAL, "kv_write: too many rows");
        const int threads = (int)(((head_dim_kv / 4) + 31) / 32 * 32);
        const dim3 grid((unsigned)((T + TPC - 1) / TPC), 2);
        if (kv_dtype != AGN_F16) agn_launch(ctx, kv_write_multi_kernel<true, TPC>, grid, dim3(threads), 0, a);
        else agn_launch(ctx, kv_write_multi_kernel<false, TPC>, grid, dim3(threads), 0, a);
        ctx->flags_dirty = true;
        AGN_LAUNCHED(ctx, "kv_write_multi");
        return AGN_OK;
    }
    if (kv_dtype != AGN_F16) {
        if (T > 0x7fffffffLL) return agn_fail(ctx, AGN_EINVAL, "kv_write: too many rows");
        int threads = (int)(((head_dim_kv + 31) / 32) * 8);  // eight lanes per 32-value block
        threads = ((threads + 31) / 32) * 32;
        if (threads > 256) threads = 256;
        agn_launch(ctx, kv_write_q8_0_kernel, dim3((unsigned)T, 2), dim3(threads), 0, a);
    } else {
        if (T > 0x7fffffffLL) return agn_fail(ctx, AGN_EINVAL, "kv_write: too many rows");
        int threads = (int)(((head_dim_kv + 3) / 4 + 31) / 32 * 32);
        if (threads > 256) threads = 256;
        agn_launch(ctx, kv_write_f16_kernel, dim3((unsigned)T, 2), dim3(threads), 0, a);
    }
    ctx->flags_dirty = true;
    AGN_LAUNCHED(ctx, "kv_write");
    return AGN_OK;
}

extern "C" int32_t agn_kv_read_f32(agn_ctx *ctx, int32_t kv_dtype, const void *k_cache, const void *v_cache, int64_t n_pos,
                                   int64_t head_dim_kv, float *k_out, float *v_out) {
    AGN_CHECK_CTX(ctx);
    if (kv_dtype != AGN_F16 && kv_dtype != AGN_Q8_0 && kv_dtype != AGN_KV_Q8_0_WORDS)
        return agn_fail(ctx, AGN_EUNSUPPORTED_DTYPE, "kv_read: KV dtype %d is neither f16 (1), q8_0 (8) nor q8_0 in words (1008)", kv_dtype);
    if (kv_dtype == AGN_KV_Q8_0_WORDS && ((reinterpret_cast<uintptr_t>(k_cache) | reinterpret_cast<uintptr_t>(v_cache)) & 3))
        return agn_fail(ctx, AGN_EINVAL, "kv_read: caches must be 4-byte aligned");
    if (n_pos < 0 || head_dim_kv <= 0)
        return agn_fail(ctx, AGN_EINVAL, "kv_read: n_pos=%lld head_dim_kv=%lld", (long long)n_pos, (long long)head_dim_kv);
    if (n_pos == 0) return AGN_OK;
    if (!k_cache || !v_cache || !k_out || !v_out) return agn_fail(ctx, AGN_EINVAL, "kv_read: null pointer");
    AGN_CUDA(ctx, cudaSetDevice(ctx->device));
    if (n_pos > 0x7fffffffLL) return agn_fail(ctx, AGN_EINVAL, "kv_read: too many positions");
    int threads = (int)(((head_dim_kv + 3) / 4 + 31) / 32 * 32);
    if (threads > 256) threads = 256;
    agn_launch(ctx, kv_read_kernel, dim3((unsigned)n_pos, 2), dim3(threads), 0, static_cast<const unsigned char *>(k_cache),
               static_cast<const unsigned char *>(v_cache), n_pos, head_dim_kv, kv_bytes_per_token(kv_dtype, head_dim_kv),
               kv_dtype == AGN_Q8_0 ? 1 : kv_dtype == AGN_KV_Q8_0_WORDS ? 2 : 0, k_out, v_out);
    AGN_LAUNCHED(ctx, "kv_read");
    return AGN_OK;
}
