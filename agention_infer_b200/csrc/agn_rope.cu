// Rotary embedding and the fused per-head RMSNorm -> rotary embedding over T token rows.
//
// Reference: `qk_norm` (src/model/llama/cpu_path.rs:78-93), `rope` (:99-133),
// `rope_partial` (:461-496); GPU twins `launch_rope` / `launch_qk_norm_rope`
// (src/ops/wgpu_backend/resident.rs:326-353, :414-443).
//
//   norm : rms = sqrt(sum_d x[d]^2 / head_dim + eps) ; x[d] = (w[d] * x[d]) / rms
//   rope : freq = (pos * freq_scale) / powf(theta, 2d/n_rot) ; (sin, cos) of freq ;
//          NeoX pairs (d, d + n_rot/2):  x0' = x0*cos - x1*sin ; x1' = x0*sin + x1*cos
//
// 8 algorithmic bytes per element, in place: bound by HBM.  The sin/cos pair depends on
// (token, d) only, so it is computed once per token into shared memory and reused by all
// Q and K heads of that token (the reference's GPU kernel recomputes powf/sin/cos per
// (head, d) thread; at 6 TB/s that alone would saturate the SM's issue slots).
//
// Fast path (rope_heads_kernel): a group of W lanes owns one head, the head lives in
// registers (VPL float4 per lane), each group has SLOTS heads in flight so that every
// lane has SLOTS*VPL 128-bit loads outstanding before the first use.  The norm statistic
// is a shuffle reduction inside the group; the NeoX partner is fetched with one
// shuffle-xor (or is in the same lane for head_dim 256).  The intermediate normalised
// head never leaves registers.
#include "agn_common.cuh"

namespace {

constexpr int SLOTS = 4;

struct RopeArgs {
    float *q;
    float *k;
    const float *wq;
    const float *wk;
    const int32_t *pos;
    const float *denom;
    int64_t T;
    int n_q, n_kv, head_dim, n_rot;
    int pos_start;
    int tpc;  // tokens per CTA
    float freq_scale, eps;
};

// (cos, sin) of every (token of this CTA, d < half) into shared memory.
__device__ __forceinline__ void fill_sincos(const RopeArgs &a, float *s_cos, float *s_sin, int half) {
    const int64_t t0 = (int64_t)blockIdx.x * a.tpc;
    for (int i = threadIdx.x; i < a.tpc * half; i += blockDim.x) {
        const int tt = i / half, d = i - tt * half;
        const int64_t t = t0 + tt;
        if (t < a.T) {
            const int p = a.pos ? a.pos[t] : a.pos_start + (int)t;
            // pos as f32 * freq_scale / theta.powf(..): two IEEE roundings, as on the CPU
            const float freq = __fdiv_rn(__fmul_rn((float)p, a.freq_scale), a.denom[d]);
            float sn, cs;
            sincosf(freq, &sn, &cs);
            s_cos[i] = cs;
            s_sin[i] = sn;
        }
    }
}

template <int W, int VPL, int LAYOUT, bool NORM>
__global__ void __launch_bounds__(512)
rope_heads_kernel(const RopeArgs a) {
    extern __shared__ __align__(16) float smem[];
    const int half = a.n_rot >> 1;
    float *s_cos = smem;
    float *s_sin = smem + a.tpc * half;
    fill_sincos(a, s_cos, s_sin, half);
    __syncthreads();

    const int lane = threadIdx.x & (W - 1);
    const int group = threadIdx.x / W;
    const int n_groups = blockDim.x / W;
    const int n_heads = a.n_q + a.n_kv;
    const int rows = a.tpc * n_heads;  // head rows of this CTA
    const int hd4 = a.head_dim >> 2;
    const int hq = half >> 2;  // float4 per half (NeoX), n_rot/8
    const int64_t t0 = (int64_t)blockIdx.x * a.tpc;

    for (int base = 0; base < rows; base += n_groups * SLOTS) {
        float4 v[SLOTS][VPL];
        float *ptr[SLOTS];
        const float *wptr[SLOTS];
        int tok[SLOTS];
#pragma unroll
        for (int s = 0; s < SLOTS; s++) {
            const int hr = base + group + s * n_groups;
            const int tt = hr / n_heads, h = hr - tt * n_heads;
            const int64_t t = t0 + tt;
            const bool on = hr < rows && t < a.T;
            tok[s] = tt;
            ptr[s] = nullptr;
            wptr[s] = nullptr;
            if (on) {
                if (h < a.n_q) {
                    ptr[s] = a.q + (t * a.n_q + h) * (int64_t)a.head_dim;
                    wptr[s] = a.wq;
                } else {
                    ptr[s] = a.k + (t * a.n_kv + (h - a.n_q)) * (int64_t)a.head_dim;
                    wptr[s] = a.wk;
                }
            }
#pragma unroll
            for (int l = 0; l < VPL; l++) {
                const int i = lane + W * l;
                v[s][l] = (on && i < hd4) ? agn_ld_stream(reinterpret_cast<const float4 *>(ptr[s]) + i)
                                          : make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
#pragma unroll
        for (int s = 0; s < SLOTS; s++) {
            if (NORM) {
                float ss = 0.0f;
#pragma unroll
                for (int l = 0; l < VPL; l++)
                    ss += v[s][l].x * v[s][l].x + v[s][l].y * v[s][l].y + v[s][l].z * v[s][l].z + v[s][l].w * v[s][l].w;
#pragma unroll
                for (int o = W / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
                const float rms = sqrtf(ss / (float)a.head_dim + a.eps);
#pragma unroll
                for (int l = 0; l < VPL; l++) {
                    const int i = lane + W * l;
                    if (ptr[s] && i < hd4) {
                        const float4 ww = __ldg(reinterpret_cast<const float4 *>(wptr[s]) + i);
                        v[s][l].x = ww.x * v[s][l].x / rms;
                        v[s][l].y = ww.y * v[s][l].y / rms;
                        v[s][l].z = ww.z * v[s][l].z / rms;
                        v[s][l].w = ww.w * v[s][l].w / rms;
                    }
                }
            }
            const float *c_tab = s_cos + tok[s] * half;
            const float *s_tab = s_sin + tok[s] * half;
            if (LAYOUT == AGN_ROPE_NEOX) {
                if (VPL > 1 && hq == (W * VPL) / 2) {
                    // full rotation of a head wider than one float4 per lane: the partner
                    // float4 sits in the same lane, VPL/2 registers further on
#pragma unroll
                    for (int l = 0; l < VPL / 2; l++) {
                        const int i = lane + W * l;
                        if (ptr[s]) {
                            const float4 c = *reinterpret_cast<const float4 *>(c_tab + 4 * i);
                            const float4 sn = *reinterpret_cast<const float4 *>(s_tab + 4 * i);
                            const float4 x0 = v[s][l], x1 = v[s][l + VPL / 2];
                            v[s][l].x = x0.x * c.x - x1.x * sn.x;
                            v[s][l].y = x0.y * c.y - x1.y * sn.y;
                            v[s][l].z = x0.z * c.z - x1.z * sn.z;
                            v[s][l].w = x0.w * c.w - x1.w * sn.w;
                            v[s][l + VPL / 2].x = x0.x * sn.x + x1.x * c.x;
                            v[s][l + VPL / 2].y = x0.y * sn.y + x1.y * c.y;
                            v[s][l + VPL / 2].z = x0.z * sn.z + x1.z * c.z;
                            v[s][l + VPL / 2].w = x0.w * sn.w + x1.w * c.w;
                        }
                    }
                } else {
                    // hq is a power of two below W: the partner float4 is in lane ^ hq
                    const float4 mine = v[s][0];
                    float4 oth;
                    oth.x = __shfl_xor_sync(0xffffffffu, mine.x, hq);
                    oth.y = __shfl_xor_sync(0xffffffffu, mine.y, hq);
                    oth.z = __shfl_xor_sync(0xffffffffu, mine.z, hq);
                    oth.w = __shfl_xor_sync(0xffffffffu, mine.w, hq);
                    if (ptr[s] && lane < 2 * hq) {
                        const bool low = lane < hq;
                        const int i = low ? lane : lane - hq;
                        const float4 c = *reinterpret_cast<const float4 *>(c_tab + 4 * i);
                        const float4 sn = *reinterpret_cast<const float4 *>(s_tab + 4 * i);
                        if (low) {  // x0 = mine, x1 = oth
                            v[s][0].x = mine.x * c.x - oth.x * sn.x;
                            v[s][0].y = mine.y * c.y - oth.y * sn.y;
                            v[s][0].z = mine.z * c.z - oth.z * sn.z;
                            v[s][0].w = mine.w * c.w - oth.w * sn.w;
                        } else {  // x0 = oth, x1 = mine
                            v[s][0].x = oth.x * sn.x + mine.x * c.x;
                            v[s][0].y = oth.y * sn.y + mine.y * c.y;
                            v[s][0].z = oth.z * sn.z + mine.z * c.z;
                            v[s][0].w = oth.w * sn.w + mine.w * c.w;
                        }
                    }
                }
            } else {
                // pairs (2p, 2p+1): both members are in the same float4
#pragma unroll
                for (int l = 0; l < VPL; l++) {
                    const int i = lane + W * l;
                    if (ptr[s] && 4 * i < a.n_rot) {
                        const float2 c = *reinterpret_cast<const float2 *>(c_tab + 2 * i);
                        const float2 sn = *reinterpret_cast<const float2 *>(s_tab + 2 * i);
                        const float4 x = v[s][l];
                        v[s][l].x = x.x * c.x - x.y * sn.x;
                        v[s][l].y = x.x * sn.x + x.y * c.x;
                        v[s][l].z = x.z * c.y - x.w * sn.y;
                        v[s][l].w = x.z * sn.y + x.w * c.y;
                    }
                }
            }
#pragma unroll
            for (int l = 0; l < VPL; l++) {
                const int i = lane + W * l;
                // dims past n_rot are untouched by rope: skip the store unless normalised
                const bool touched = NORM || 4 * i < a.n_rot;
                if (ptr[s] && i < hd4 && touched) agn_st_stream(reinterpret_cast<float4 *>(ptr[s]) + i, v[s][l]);
            }
        }
    }
}

// Any even n_rot <= head_dim, any head_dim, any alignment: one warp per head, scalar
// accesses straight from global memory (second touch of an element is an L1/L2 hit).
template <int LAYOUT, bool NORM>
__global__ void __launch_bounds__(256)
rope_heads_generic_kernel(const RopeArgs a) {
    extern __shared__ __align__(16) float smem[];
    const int half = a.n_rot >> 1;
    float *s_cos = smem;
    float *s_sin = smem + half;  // tpc == 1
    fill_sincos(a, s_cos, s_sin, half);
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    const int n_heads = a.n_q + a.n_kv;
    const int64_t t = blockIdx.x;
    for (int h = warp; h < n_heads; h += n_warps) {
        float *x;
        const float *w;
        if (h < a.n_q) {
            x = a.q + (t * a.n_q + h) * (int64_t)a.head_dim;
            w = a.wq;
        } else {
            x = a.k + (t * a.n_kv + (h - a.n_q)) * (int64_t)a.head_dim;
            w = a.wk;
        }
        float rms = 1.0f;
        if (NORM) {
            float ss = 0.0f;
            for (int d = lane; d < a.head_dim; d += 32) ss += x[d] * x[d];
            ss = agn_warp_sum(ss);
            rms = sqrtf(ss / (float)a.head_dim + a.eps);
        }
        for (int d = lane; d < half; d += 32) {
            const int i0 = LAYOUT == AGN_ROPE_NEOX ? d : 2 * d;
            const int i1 = LAYOUT == AGN_ROPE_NEOX ? d + half : 2 * d + 1;
            float x0 = x[i0], x1 = x[i1];
            if (NORM) {
                x0 = w[i0] * x0 / rms;
                x1 = w[i1] * x1 / rms;
            }
            const float c = s_cos[d], sn = s_sin[d];
            x[i0] = x0 * c - x1 * sn;
            x[i1] = x0 * sn + x1 * c;
        }
        if (NORM)
            for (int d = a.n_rot + lane; d < a.head_dim; d += 32) x[d] = w[d] * x[d] / rms;
    }
}

template <int W, int VPL>
void launch_fast(const RopeArgs &a, bool norm, int layout, unsigned grid, int threads, size_t smem, cudaStream_t st) {
    if (layout == AGN_ROPE_NEOX) {
        if (norm) rope_heads_kernel<W, VPL, AGN_ROPE_NEOX, true><<<grid, threads, smem, st>>>(a);
        else rope_heads_kernel<W, VPL, AGN_ROPE_NEOX, false><<<grid, threads, smem, st>>>(a);
    } else {
        if (norm) rope_heads_kernel<W, VPL, AGN_ROPE_NORMAL, true><<<grid, threads, smem, st>>>(a);
        else rope_heads_kernel<W, VPL, AGN_ROPE_NORMAL, false><<<grid, threads, smem, st>>>(a);
    }
}

bool is_pow2(int v) { return v > 0 && (v & (v - 1)) == 0; }

int32_t rope_dispatch(agn_ctx *ctx, const char *name, float *q, float *k, const float *wq, const float *wk,
                      bool norm, int64_t T, int32_t n_q, int32_t n_kv, int32_t head_dim, float eps, int32_t n_rot,
                      const int32_t *pos, int32_t pos_start, float theta, float freq_scale, int32_t layout) {
    if (T < 0 || n_q < 0 || n_kv < 0 || n_q + n_kv <= 0 || head_dim <= 0)
        return agn_fail(ctx, AGN_EINVAL, "%s: T=%lld heads=%d+%d head_dim=%d", name, (long long)T, n_q, n_kv, head_dim);
    if (n_rot < 0 || n_rot > head_dim || (n_rot & 1))
        return agn_fail(ctx, AGN_EINVAL, "%s: n_rot=%d must be even and <= head_dim=%d", name, n_rot, head_dim);
    if (layout != AGN_ROPE_NEOX && layout != AGN_ROPE_NORMAL)
        return agn_fail(ctx, AGN_EINVAL, "%s: unknown layout %d", name, layout);
    if (T == 0) return AGN_OK;
    if ((n_q > 0 && !q) || (n_kv > 0 && !k)) return agn_fail(ctx, AGN_EINVAL, "%s: null activation pointer", name);
    if (norm && ((n_q > 0 && !wq) || (n_kv > 0 && !wk))) return agn_fail(ctx, AGN_EINVAL, "%s: null norm weight", name);
    if (!norm && n_rot == 0) return AGN_OK;  // nothing rotates
    if (T > 0x7fffffffLL) return agn_fail(ctx, AGN_EINVAL, "%s: T too large", name);
    AGN_CUDA(ctx, cudaSetDevice(ctx->device));

    RopeArgs a;
    a.q = q; a.k = k; a.wq = wq; a.wk = wk; a.pos = pos; a.T = T;
    a.n_q = n_q; a.n_kv = n_kv; a.head_dim = head_dim; a.n_rot = n_rot;
    a.pos_start = pos_start; a.freq_scale = freq_scale; a.eps = eps; a.tpc = 1;
    a.denom = nullptr;
    if (n_rot >= 2) {
        int32_t rc = agn_rope_table(ctx, theta, n_rot, &a.denom);
        if (rc != AGN_OK) return rc;
    }
    const int half = n_rot / 2;
    const int n_heads = n_q + n_kv;
    const int hd4 = head_dim / 4;

    // register fast path?
    int W = 8;
    while (W < 32 && W < hd4) W *= 2;
    const int VPL = (hd4 + W - 1) / W;
    const int hq = half / 4;
    bool fast = head_dim % 4 == 0 && (VPL == 1 || VPL == 2 || VPL == 4) && (n_q == 0 || agn_aligned16(q)) &&
                (n_kv == 0 || agn_aligned16(k)) &&
                (!norm || ((n_q == 0 || agn_aligned16(wq)) && (n_kv == 0 || agn_aligned16(wk))));
    if (fast && n_rot > 0) {
        if (layout == AGN_ROPE_NEOX)
            fast = half % 4 == 0 && ((VPL > 1 && hq == (W * VPL) / 2) || (is_pow2(hq) && hq < W));
        else
            fast = n_rot % 4 == 0;
    }
    if (fast) {
        // tokens per CTA: aim at 32 head rows per CTA, keep the sin/cos table small
        int tpc = 32 / n_heads;
        if (tpc < 1) tpc = 1;
        if (half > 0 && tpc * half > 2048) tpc = 2048 / half > 0 ? 2048 / half : 1;
        if ((int64_t)tpc > T) tpc = (int)T;
        a.tpc = tpc;
        const int rows = tpc * n_heads;
        int groups = (rows + SLOTS - 1) / SLOTS;
        int threads = groups * W;
        threads = ((threads + 31) / 32) * 32;
        if (threads > 512) threads = 512;
        const unsigned grid = (unsigned)((T + tpc - 1) / tpc);
        const size_t smem = sizeof(float) * 2 * (size_t)tpc * (half > 0 ? half : 1);
        if (W == 8) launch_fast<8, 1>(a, norm, layout, grid, threads, smem, ctx->stream);
        else if (W == 16) launch_fast<16, 1>(a, norm, layout, grid, threads, smem, ctx->stream);
        else if (VPL == 1) launch_fast<32, 1>(a, norm, layout, grid, threads, smem, ctx->stream);
        else if (VPL == 2) launch_fast<32, 2>(a, norm, layout, grid, threads, smem, ctx->stream);
        else launch_fast<32, 4>(a, norm, layout, grid, threads, smem, ctx->stream);
        AGN_LAUNCHED(ctx, name);
    } else {
        int threads = n_heads >= 8 ? 256 : 32 * n_heads;
        const size_t smem = sizeof(float) * 2 * (size_t)(half > 0 ? half : 1);
        if (layout == AGN_ROPE_NEOX) {
            if (norm) rope_heads_generic_kernel<AGN_ROPE_NEOX, true><<<(unsigned)T, threads, smem, ctx->stream>>>(a);
            else rope_heads_generic_kernel<AGN_ROPE_NEOX, false><<<(unsigned)T, threads, smem, ctx->stream>>>(a);
        } else {
            if (norm) rope_heads_generic_kernel<AGN_ROPE_NORMAL, true><<<(unsigned)T, threads, smem, ctx->stream>>>(a);
            else rope_heads_generic_kernel<AGN_ROPE_NORMAL, false><<<(unsigned)T, threads, smem, ctx->stream>>>(a);
        }
        AGN_LAUNCHED(ctx, name);
    }
    return AGN_OK;
}

}  // namespace

extern "C" int32_t agn_rope_f32(agn_ctx *ctx, float *x, int64_t T, int32_t n_heads, int32_t head_dim, int32_t n_rot,
                                const int32_t *pos, int32_t pos_start, float theta, float freq_scale, int32_t layout) {
    AGN_CHECK_CTX(ctx);
    return rope_dispatch(ctx, "rope", x, nullptr, nullptr, nullptr, false, T, n_heads, 0, head_dim, 0.0f, n_rot, pos,
                         pos_start, theta, freq_scale, layout);
}

extern "C" int32_t agn_rope_qk_f32(agn_ctx *ctx, float *q, float *k, int64_t T, int32_t n_q_heads, int32_t n_kv_heads,
                                   int32_t head_dim, int32_t n_rot, const int32_t *pos, int32_t pos_start, float theta,
                                   float freq_scale, int32_t layout) {
    AGN_CHECK_CTX(ctx);
    return rope_dispatch(ctx, "rope_qk", q, k, nullptr, nullptr, false, T, n_q_heads, n_kv_heads, head_dim, 0.0f, n_rot,
                         pos, pos_start, theta, freq_scale, layout);
}

extern "C" int32_t agn_qk_norm_rope_f32(agn_ctx *ctx, float *x, const float *w, int64_t T, int32_t n_heads,
                                        int32_t head_dim, float eps, int32_t n_rot, const int32_t *pos,
                                        int32_t pos_start, float theta, float freq_scale, int32_t layout) {
    AGN_CHECK_CTX(ctx);
    return rope_dispatch(ctx, "qk_norm_rope", x, nullptr, w, nullptr, true, T, n_heads, 0, head_dim, eps, n_rot, pos,
                         pos_start, theta, freq_scale, layout);
}

extern "C" int32_t agn_qk_norm_rope_qk_f32(agn_ctx *ctx, float *q, float *k, const float *wq, const float *wk, int64_t T,
                                           int32_t n_q_heads, int32_t n_kv_heads, int32_t head_dim, float eps,
                                           int32_t n_rot, const int32_t *pos, int32_t pos_start, float theta,
                                           float freq_scale, int32_t layout) {
    AGN_CHECK_CTX(ctx);
    return rope_dispatch(ctx, "qk_norm_rope_qk", q, k, wq, wk, true, T, n_q_heads, n_kv_heads, head_dim, eps, n_rot, pos,
                         pos_start, theta, freq_scale, layout);
}
