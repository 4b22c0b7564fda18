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
// registers (VPL float4 per lane, float4 number lane + W*l), each group has 2 or 4 heads
// in flight so that every lane has 8 or more 128-bit loads outstanding before the first
// use.  W is chosen so that the NeoX partner of a float4 is another register of the same
// lane (head_dim 128: W=8, VPL=4, partner two registers on), which needs no shuffle; the
// norm statistic is a log2(W)-step shuffle reduction inside the group.  The intermediate
// normalised head never leaves registers.
#include <cuda_fp16.h>

#include "agn_common.cuh"
#include "agn_row_math.cuh"

namespace {

struct RopeArgs {
    void *q;  // activations: float or __half, see the kernels' template parameter T
    void *k;
    const float *wq;
    const float *wk;
    const int32_t *pos;
    const float *denom;
    int64_t T;
    int n_q, n_kv, head_dim, n_rot;
    int pos_start;
    int tpc;  // tokens per CTA
    float freq_scale, eps;
    float inv_head_dim;  // 1 / head_dim, for the per-head mean square
    // fused KV-cache write (template parameter KV != 0): the rotated K heads and the V heads of the
    // token are packed into one layer's cache at slot pos (`KvCache::write`, src/model/mod.rs:648-672)
    const float *v;
    unsigned char *k_cache, *v_cache;
    int64_t max_seq;
    int bytes_per_token;
    int kv_words;  // Q8_0 cache blocks are the GPU path's nine 32-bit words instead of 34 bytes
    uint32_t *flags;
};

enum { KV_NONE = 0, KV_F16 = 1, KV_Q8_0 = 2 };

// Four values of a K or V head (float4 number i of the head) into the cache slot of the token.
// f16: `half::f16::from_f32` per element.  Q8_0 (`KvDtype::pack`, src/model/mod.rs:567-585): the
// eight lanes that hold one 32-value block (float4 numbers 8b .. 8b+7) share amax through three
// shuffles; scale = amax / 127 (1 if amax is 0), q = clamp(round(v / scale)).  Must be called by
// every lane of the warp (`on` = this lane holds data of a K / V row with a valid slot).
// words: the GPU path's block of nine 32-bit words (f32 scale, then offset-binary bytes, kernels_wgpu.rs:583-698)
// instead of the 34-byte block.
template <int KV>
__device__ __forceinline__ void kv_pack4(float4 x, bool on, unsigned char *tok_head, int i, int blocks_before, bool words) {
    if (KV == KV_F16) {
        if (on) ActVec<__half>::store(reinterpret_cast<__half *>(tok_head), i, x);
    } else if (KV == KV_Q8_0) {
        float amax = on ? fmaxf(fmaxf(fabsf(x.x), fabsf(x.y)), fmaxf(fabsf(x.z), fabsf(x.w))) : 0.0f;
#pragma unroll
        for (int o = 4; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        if (on) {
            const float scale = amax > 0.0f ? __fdiv_rn(amax, 127.0f) : 1.0f;
            const int lane8 = i & 7;
            const float xs[4] = {x.x, x.y, x.z, x.w};
            uint32_t q[4];
            agn_q8_0_quant4(xs, scale, q);
            if (words) {
                uint32_t *blk = reinterpret_cast<uint32_t *>(tok_head + (size_t)(blocks_before + (i >> 3)) * 36);
                if (lane8 == 0) blk[0] = __float_as_uint(scale);
                blk[1 + lane8] = (q[0] | (q[1] << 8) | (q[2] << 16) | (q[3] << 24)) ^ 0x80808080u;  // byte = q + 128
            } else {
                unsigned char *blk = tok_head + (size_t)(blocks_before + (i >> 3)) * 34;
                if (lane8 == 0) *reinterpret_cast<uint16_t *>(blk) = __half_as_ushort(__float2half_rn(scale));
                *reinterpret_cast<uint16_t *>(blk + 2 + 4 * lane8) = (uint16_t)(q[0] | (q[1] << 8));
                *reinterpret_cast<uint16_t *>(blk + 4 + 4 * lane8) = (uint16_t)(q[2] | (q[3] << 8));
            }
        }
    }
}

// With f16 storage the reference's fused kernel writes the normalised head to the f16 buffer
// and reads it back for the rotation (src/ops/kernels_wgpu.rs:296-316): the value that is
// rotated has been rounded to f16.  Keep that rounding (the data itself stays in registers).
template <typename T> __device__ __forceinline__ float act_round(float v) { return v; }
template <> __device__ __forceinline__ float act_round<__half>(float v) { return __half2float(__float2half_rn(v)); }

// (cos, sin) of every (token t0 + tt, d < half), tt < a.tpc, into shared memory.
__device__ __forceinline__ void fill_sincos(const RopeArgs &a, float *s_cos, float *s_sin, int half, int64_t t0) {
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

// How the rotated pairs map onto the registers of a lane (float4 number i = lane + W*l):
enum { MODE_NORMAL = 0,   // pairs (2p, 2p+1): both members inside one float4
       MODE_NEOX_K1 = 1,  // NeoX, n_rot/8 == W   : partner float4 is register l+1 of the same lane
       MODE_NEOX_K2 = 2,  // NeoX, n_rot/8 == 2*W : partner float4 is register l+2 of the same lane
       MODE_NEOX_SHFL = 3 // NeoX, n_rot/8 < W (power of two): partner is register 0 of lane ^ (n_rot/8)
};

// Norm (optional) and rotation of one head held in the registers of a lane group: float4 number
// lane + W*l of the head is v[l].  `rot`: the head is a Q or K row with data (V rows of the fused
// cache write and idle slots pass false; they still take part in the shuffles).
template <typename T, int W, int VPL, int MODE, bool NORM>
__device__ __forceinline__ void rope_head_math(float4 (&v)[VPL], bool rot, const float4 *wv, const float *c_tab,
                                               const float *s_tab, int lane, int hd4, int hq, float inv_head_dim, int n_rot, float eps) {
    if (NORM) {
        float2 ss2 = make_float2(0.0f, 0.0f);
#pragma unroll
        for (int l = 0; l < VPL; l++) ss2 = agn_sum_sq4(v[l], ss2);
        float ss = ss2.x + ss2.y;
#pragma unroll
        for (int o = W / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        // (w*x)/rms of the CPU path, evaluated as (w*x) * rsqrt(ss/hd + eps): the hardware reciprocal
        // square root (2 ulp) instead of two IEEE divisions and a square root per head row and lane;
        // a few 1e-7 relative from the CPU order, inside the 1e-5 tolerance
        const float inv = rsqrtf(__fmaf_rn(ss, inv_head_dim, eps));
#pragma unroll
        for (int l = 0; l < VPL; l++) {
            const int i = lane + W * l;
            if (rot && i < hd4) {
                const float4 ww = wv[i];  // shared memory (CTA-per-unit kernel) or global memory (persistent kernel)
                const float4 nx = agn_scale4(agn_mul4(ww, v[l]), inv);  // (w * x) * inv
                v[l].x = act_round<T>(nx.x);
                v[l].y = act_round<T>(nx.y);
                v[l].z = act_round<T>(nx.z);
                v[l].w = act_round<T>(nx.w);
            }
        }
    }
    if (MODE == MODE_NEOX_K1 || MODE == MODE_NEOX_K2) {
        constexpr int K = MODE == MODE_NEOX_K2 ? 2 : 1;
#pragma unroll
        for (int l = 0; l < K; l++) {
            if (l + K < VPL && rot) {
                const int i = lane + W * l;
                const float4 c = *reinterpret_cast<const float4 *>(c_tab + 4 * i);
                const float4 sn = *reinterpret_cast<const float4 *>(s_tab + 4 * i);
                const float4 x0 = v[l], x1 = v[(l + K) % VPL];
                float4 y0, y1;
                y0.x = x0.x * c.x - x1.x * sn.x;
                y0.y = x0.y * c.y - x1.y * sn.y;
                y0.z = x0.z * c.z - x1.z * sn.z;
                y0.w = x0.w * c.w - x1.w * sn.w;
                y1.x = x0.x * sn.x + x1.x * c.x;
                y1.y = x0.y * sn.y + x1.y * c.y;
                y1.z = x0.z * sn.z + x1.z * c.z;
                y1.w = x0.w * sn.w + x1.w * c.w;
                v[l] = y0;
                v[(l + K) % VPL] = y1;
            }
        }
    } else if (MODE == MODE_NEOX_SHFL) {
        const float4 mine = v[0];
        float4 oth;
        oth.x = __shfl_xor_sync(0xffffffffu, mine.x, hq);
        oth.y = __shfl_xor_sync(0xffffffffu, mine.y, hq);
        oth.z = __shfl_xor_sync(0xffffffffu, mine.z, hq);
        oth.w = __shfl_xor_sync(0xffffffffu, mine.w, hq);
        if (rot && lane < 2 * hq) {
            const bool low = lane < hq;
            const int i = low ? lane : lane - hq;
            const float4 c = *reinterpret_cast<const float4 *>(c_tab + 4 * i);
            const float4 sn = *reinterpret_cast<const float4 *>(s_tab + 4 * i);
            if (low) {  // x0 = mine, x1 = oth
                v[0].x = mine.x * c.x - oth.x * sn.x;
                v[0].y = mine.y * c.y - oth.y * sn.y;
                v[0].z = mine.z * c.z - oth.z * sn.z;
                v[0].w = mine.w * c.w - oth.w * sn.w;
            } else {  // x0 = oth, x1 = mine
                v[0].x = oth.x * sn.x + mine.x * c.x;
                v[0].y = oth.y * sn.y + mine.y * c.y;
                v[0].z = oth.z * sn.z + mine.z * c.z;
                v[0].w = oth.w * sn.w + mine.w * c.w;
            }
        }
    } else {
#pragma unroll
        for (int l = 0; l < VPL; l++) {
            const int i = lane + W * l;
            if (rot && 4 * i < n_rot) {
                const float2 c = *reinterpret_cast<const float2 *>(c_tab + 2 * i);
                const float2 sn = *reinterpret_cast<const float2 *>(s_tab + 2 * i);
                const float4 x = v[l];
                v[l].x = x.x * c.x - x.y * sn.x;
                v[l].y = x.x * sn.x + x.y * c.x;
                v[l].z = x.z * c.y - x.w * sn.y;
                v[l].w = x.z * sn.y + x.w * c.y;
            }
        }
    }
}

template <typename T, int W, int VPL, int MODE, bool NORM, int KV = KV_NONE>
__global__ void __launch_bounds__(256)
rope_heads_kernel(const RopeArgs a) {
    agn_pdl_launch_dependents();
    constexpr int NS = VPL == 4 ? 2 : 4;  // head rows in flight per lane group
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int half = a.n_rot >> 1;
    const int n_heads = a.n_q + a.n_kv + (KV != KV_NONE ? a.n_kv : 0);  // head rows per token: Q, K and (fused cache write) V
    const int rows = a.tpc * n_heads;  // head rows of this CTA
    // shared memory: row pointers | row meta (token in CTA, is-K flag) | cos | sin | (NORM) wq | wk
    T **s_ptr = reinterpret_cast<T **>(smem_raw);
    int *s_meta = reinterpret_cast<int *>(smem_raw + (size_t)rows * 8);
    float *s_cos = reinterpret_cast<float *>(smem_raw + (((size_t)rows * 12 + 15) & ~(size_t)15));
    float *s_sin = s_cos + a.tpc * half;
    float *s_wq = s_sin + a.tpc * half + ((4 - ((2 * a.tpc * half) & 3)) & 3);  // 16-byte aligned
    float *s_wk = s_wq + a.head_dim;
    const int64_t t0 = (int64_t)blockIdx.x * a.tpc;
    if (NORM) {
        // The norm weights are model parameters, not the previous kernel's output: they are staged
        // ahead of the dependency wait, so their load latency is off the critical path of a
        // decode-sized launch (a handful of CTAs whose whole life is one dependent chain).
        for (int d = threadIdx.x; d < a.head_dim; d += blockDim.x) {
            s_wq[d] = a.n_q > 0 ? a.wq[d] : 0.0f;
            s_wk[d] = a.n_kv > 0 ? a.wk[d] : 0.0f;
        }
    }

    // one integer division per head row per CTA, instead of one per lane and slot
    for (int hr = threadIdx.x; hr < rows; hr += blockDim.x) {
        const int tt = hr / n_heads, h = hr - tt * n_heads;
        const int64_t t = t0 + tt;
        T *p = nullptr;
        const int kind = h < a.n_q ? 0 : (h < a.n_q + a.n_kv ? 1 : 2);  // Q, K, V
        const int hk = kind == 0 ? 0 : h - a.n_q - (kind == 2 ? a.n_kv : 0);  // head index inside K / V
        if (t < a.T) {
            if (kind == 0) p = static_cast<T *>(a.q) + (t * a.n_q + h) * (int64_t)a.head_dim;
            else if (kind == 1) p = static_cast<T *>(a.k) + (t * a.n_kv + hk) * (int64_t)a.head_dim;
            else p = reinterpret_cast<T *>(const_cast<float *>(a.v)) + (t * a.n_kv + hk) * (int64_t)a.head_dim;  // read only
        }
        s_ptr[hr] = p;
        s_meta[hr] = tt | (kind << 16) | (hk << 18);
    }
    __syncthreads();
    // everything above used kernel parameters and shared memory only; global memory (which the
    // previous kernel of the stream may still be writing) is touched from here on
    agn_pdl_wait();

    const int lane = threadIdx.x & (W - 1);
    const int group = threadIdx.x / W;
    const int n_groups = blockDim.x / W;
    const int hd4 = a.head_dim >> 2;
    const int hq = half >> 2;  // float4 per rotated half (NeoX): n_rot/8

    for (int base = 0; base < rows; base += n_groups * NS) {
        float4 v[NS][VPL];
        T *ptr[NS];
        int meta[NS];
#pragma unroll
        for (int s = 0; s < NS; s++) {
            const int hr = base + group + s * n_groups;
            ptr[s] = hr < rows ? s_ptr[hr] : nullptr;
            meta[s] = hr < rows ? s_meta[hr] : 0;
#pragma unroll
            for (int l = 0; l < VPL; l++) {
                const int i = lane + W * l;
                v[s][l] = (ptr[s] && i < hd4) ? ActVec<T>::load(ptr[s], i) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
        if (base == 0) {
            // The sin/cos table is built while the HBM loads issued above are in flight.
            fill_sincos(a, s_cos, s_sin, half, (int64_t)blockIdx.x * a.tpc);
            __syncthreads();
        }
#pragma unroll
        for (int s = 0; s < NS; s++) {
            const int kind = (meta[s] >> 16) & 3;
            const float *c_tab = s_cos + (meta[s] & 0xffff) * half;
            const float *s_tab = s_sin + (meta[s] & 0xffff) * half;
            rope_head_math<T, W, VPL, MODE, NORM>(v[s], ptr[s] != nullptr && kind < 2,
                                                  reinterpret_cast<const float4 *>(kind == 1 ? s_wk : s_wq), c_tab, s_tab, lane, hd4, hq,
                                                  a.inv_head_dim, a.n_rot, a.eps);
#pragma unroll
            for (int l = 0; l < VPL; l++) {
                const int i = lane + W * l;
                // dims past n_rot are untouched by rope: skip the store unless normalised
                const bool touched = NORM || 4 * i < a.n_rot;
                if (ptr[s] && i < hd4 && touched && kind < 2) ActVec<T>::store(ptr[s], i, v[s][l]);
            }
            if (KV != KV_NONE) {
                // the rotated K head (still in registers) and the V head go into the token's cache slot
                const int hk = meta[s] >> 18;
                int64_t slot = -1;
                if (ptr[s] && kind >= 1) {
                    const int64_t t = t0 + (meta[s] & 0xffff);
                    const int64_t p = a.pos ? (int64_t)a.pos[t] : (int64_t)a.pos_start + t;
                    if (p >= 0 && p < a.max_seq) slot = p;
                    else if (lane == 0) atomicOr(a.flags, AGN_FLAG_OOB_SLOT);  // skipped and reported, never a fault
                }
                unsigned char *tok_head = nullptr;
                if (slot >= 0) {
                    tok_head = (kind == 1 ? a.k_cache : a.v_cache) + slot * a.bytes_per_token;
                    if (KV == KV_F16) tok_head += (size_t)hk * a.head_dim * 2;
                }
                const int blocks_before = hk * (a.head_dim >> 5);
#pragma unroll
                for (int l = 0; l < VPL; l++) {
                    const int i = lane + W * l;
                    kv_pack4<KV>(v[s][l], slot >= 0 && i < hd4, tok_head, i, blocks_before, a.kv_words != 0);
                }
            }
        }
    }
}

// Persistent form of rope_heads_kernel for large batches.  A unit is a.tpc consecutive tokens,
// i.e. one contiguous piece of q and one of k; a CTA loops over units blockIdx.x, blockIdx.x +
// gridDim.x, ... and the pieces of its next units are already on their way into a ring of
// shared-memory slots (two bulk asynchronous copies per unit, issued by one thread, completing
// on the slot's mbarrier).  Lane groups then read their heads from the slot instead of from
// global memory, rotate them in registers exactly as above and store them straight back to q / k.
// Shared memory: slots x [q piece | k piece] | mbarriers | per-row table | two sin/cos tables.
template <typename T, int W, int VPL, int MODE, bool NORM>
__global__ void __launch_bounds__(256)
rope_heads_ring_kernel(const RopeArgs a, int slots, int slot_bytes, int spin_limit) {
    constexpr int NS = VPL == 4 ? 2 : 4;
    extern __shared__ __align__(128) unsigned char ring_raw[];
    const int half = a.n_rot >> 1;
    const int n_heads = a.n_q + a.n_kv;
    const int rows_max = a.tpc * n_heads;
    const uint32_t q_tok_bytes = (uint32_t)a.n_q * a.head_dim * sizeof(T), k_tok_bytes = (uint32_t)a.n_kv * a.head_dim * sizeof(T);
    const uint32_t k_off = (uint32_t)a.tpc * q_tok_bytes;  // the k piece follows the largest q piece
    uint64_t *full = reinterpret_cast<uint64_t *>(ring_raw + (size_t)slots * slot_bytes);
    int *s_row = reinterpret_cast<int *>(full + slots);                      // [rows_max][2]: byte offset in the slot, meta
    float *s_tab = reinterpret_cast<float *>(s_row + 2 * rows_max + ((2 * rows_max) & 1) + 2);  // 16-byte aligned below
    s_tab = reinterpret_cast<float *>((reinterpret_cast<uintptr_t>(s_tab) + 15) & ~(uintptr_t)15);
    const int tab_stride = 2 * a.tpc * (half > 0 ? half : 1);  // floats per table: cos then sin
    if (threadIdx.x == 0) {
        for (int s = 0; s < slots; s++) agn_mbar_init(&full[s], 1);
        agn_mbar_init_fence();
    }
    for (int hr = threadIdx.x; hr < rows_max; hr += blockDim.x) {
        const int tt = hr / n_heads, h = hr - tt * n_heads;
        const bool is_k = h >= a.n_q;
        s_row[2 * hr] = is_k ? (int)(k_off + (uint32_t)tt * k_tok_bytes + (uint32_t)(h - a.n_q) * a.head_dim * sizeof(T))
                             : (int)((uint32_t)tt * q_tok_bytes + (uint32_t)h * a.head_dim * sizeof(T));
        s_row[2 * hr + 1] = tt | ((is_k ? 1 : 0) << 16);
    }
    __syncthreads();
    agn_pdl_launch_dependents();
    agn_pdl_wait();  // global memory is touched from here on

    const int64_t n_units = (a.T + a.tpc - 1) / a.tpc;
    const int64_t first = blockIdx.x, stride = gridDim.x;
    const int n_my = first < n_units ? (int)((n_units - first + stride - 1) / stride) : 0;
    unsigned char *qb = static_cast<unsigned char *>(a.q), *kb = static_cast<unsigned char *>(a.k);
    auto issue = [&](int j) {  // thread 0 only: unit number j of this CTA into slot j % slots
        const int64_t t0 = (first + (int64_t)j * stride) * a.tpc;
        const uint32_t ntok = (uint32_t)(a.T - t0 < a.tpc ? a.T - t0 : a.tpc);
        unsigned char *dst = ring_raw + (size_t)(j % slots) * slot_bytes;
        uint64_t *bar = &full[j % slots];
        agn_mbar_expect_tx(bar, ntok * (q_tok_bytes + k_tok_bytes));
        if (q_tok_bytes) agn_bulk_g2s(dst, qb + t0 * q_tok_bytes, ntok * q_tok_bytes, bar);
        if (k_tok_bytes) agn_bulk_g2s(dst + k_off, kb + t0 * k_tok_bytes, ntok * k_tok_bytes, bar);
    };
    int issued = 0;
    if (threadIdx.x == 0)
        for (; issued < slots - 1 && issued < n_my; issued++) issue(issued);

    const int lane = threadIdx.x & (W - 1);
    const int group = threadIdx.x / W;
    const int n_groups = blockDim.x / W;
    const int hd4 = a.head_dim >> 2;
    const int hq = half >> 2;

    int failed = 0;  // this thread's staging wait ran out
    for (int it = 0; it < n_my; it++) {
        const int slot = it % slots;
        const int64_t t0 = (first + (int64_t)it * stride) * a.tpc;
        const int ntok = (int)(a.T - t0 < a.tpc ? a.T - t0 : a.tpc);
        const int rows = ntok * n_heads;
        float *s_cos = s_tab + (it & 1) * tab_stride, *s_sin = s_cos + a.tpc * half;
        fill_sincos(a, s_cos, s_sin, half, t0);  // this unit's table, while its copies are in flight
        // table visible; every thread has finished reading the previous unit's slot; and one
        // CTA-wide answer to "did any thread's wait run out", so that all leave together
        if (__syncthreads_or(failed)) break;
        // the slot that the previous iteration emptied takes the unit slots - 1 ahead of this one
        if (threadIdx.x == 0 && issued < n_my) issue(issued++);
        if (!agn_mbar_wait(&full[slot], (uint32_t)(it / slots) & 1u, spin_limit)) {
            failed = 1;
            atomicOr(a.flags, AGN_FLAG_TIMEOUT);
            continue;  // the data did not arrive: store nothing; the CTA leaves at the next barrier
        }
        const unsigned char *sl = ring_raw + (size_t)slot * slot_bytes;
        for (int base = 0; base < rows; base += n_groups * NS) {
            float4 v[NS][VPL];
            int off[NS], meta[NS];
            bool live[NS];
#pragma unroll
            for (int s = 0; s < NS; s++) {
                const int hr = base + group + s * n_groups;
                live[s] = hr < rows;
                off[s] = live[s] ? s_row[2 * hr] : 0;
                meta[s] = live[s] ? s_row[2 * hr + 1] : 0;
#pragma unroll
                for (int l = 0; l < VPL; l++) {
                    const int i = lane + W * l;
                    v[s][l] = (live[s] && i < hd4) ? ActVec<T>::load_shared(reinterpret_cast<const T *>(sl + off[s]), i)
                                                   : make_float4(0.f, 0.f, 0.f, 0.f);
                }
            }
#pragma unroll
            for (int s = 0; s < NS; s++) {
                const bool is_k = (meta[s] >> 16) & 1;
                const float *c_tab = s_cos + (meta[s] & 0xffff) * half;
                const float *sn_tab = s_sin + (meta[s] & 0xffff) * half;
                rope_head_math<T, W, VPL, MODE, NORM>(v[s], live[s], reinterpret_cast<const float4 *>(is_k ? a.wk : a.wq), c_tab, sn_tab,
                                                      lane, hd4, hq, a.inv_head_dim, a.n_rot, a.eps);
                // the head's place in q / k: the slot holds the pieces in the same order as global memory
                T *dst = is_k ? reinterpret_cast<T *>(kb + t0 * k_tok_bytes + (off[s] - (int)k_off))
                              : reinterpret_cast<T *>(qb + t0 * q_tok_bytes + off[s]);
#pragma unroll
                for (int l = 0; l < VPL; l++) {
                    const int i = lane + W * l;
                    const bool touched = NORM || 4 * i < a.n_rot;
                    if (live[s] && i < hd4 && touched) ActVec<T>::store(dst, i, v[s][l]);
                }
            }
        }
    }
    if (__syncthreads_or(failed) && threadIdx.x == 0) {
        // a staging wait ran out (reported above): give every copy that may still be in flight
        // into this CTA's shared memory one more bounded wait before leaving
        for (int j = issued - slots > 0 ? issued - slots : 0; j < issued; j++)
            (void)agn_mbar_wait(&full[j % slots], (uint32_t)(j / slots) & 1u, spin_limit);
    }
}

// Any even n_rot <= head_dim, any head_dim, any alignment: one warp per head, scalar
// accesses straight from global memory (second touch of an element is an L1/L2 hit).
template <typename T, int LAYOUT, bool NORM>
__global__ void __launch_bounds__(256)
rope_heads_generic_kernel(const RopeArgs a) {
    agn_pdl_prologue();
    extern __shared__ __align__(16) float smem[];
    const int half = a.n_rot >> 1;
    float *s_cos = smem;
    float *s_sin = smem + half;  // tpc == 1
    fill_sincos(a, s_cos, s_sin, half, (int64_t)blockIdx.x * a.tpc);
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    const int n_heads = a.n_q + a.n_kv;
    const int64_t t = blockIdx.x;
    for (int h = warp; h < n_heads; h += n_warps) {
        T *x;
        const float *w;
        if (h < a.n_q) {
            x = static_cast<T *>(a.q) + (t * a.n_q + h) * (int64_t)a.head_dim;
            w = a.wq;
        } else {
            x = static_cast<T *>(a.k) + (t * a.n_kv + (h - a.n_q)) * (int64_t)a.head_dim;
            w = a.wk;
        }
        float inv = 1.0f;
        if (NORM) {
            float ss = 0.0f;
            for (int d = lane; d < a.head_dim; d += 32) {
                const float v = ActVec<T>::load1(x, d);
                ss += v * v;
            }
            ss = agn_warp_sum(ss);
            inv = 1.0f / sqrtf(ss / (float)a.head_dim + a.eps);
        }
        for (int d = lane; d < half; d += 32) {
            const int i0 = LAYOUT == AGN_ROPE_NEOX ? d : 2 * d;
            const int i1 = LAYOUT == AGN_ROPE_NEOX ? d + half : 2 * d + 1;
            float x0 = ActVec<T>::load1(x, i0), x1 = ActVec<T>::load1(x, i1);
            if (NORM) {
                x0 = act_round<T>(w[i0] * x0 * inv);
                x1 = act_round<T>(w[i1] * x1 * inv);
            }
            const float c = s_cos[d], sn = s_sin[d];
            ActVec<T>::store1(x, i0, x0 * c - x1 * sn);
            ActVec<T>::store1(x, i1, x0 * sn + x1 * c);
        }
        if (NORM)
            for (int d = a.n_rot + lane; d < a.head_dim; d += 32) ActVec<T>::store1(x, d, w[d] * ActVec<T>::load1(x, d) * inv);
    }
}

// Fused cache write: f32 activations, head_dim 128 (W = 8, VPL = 4) or 64 (W = 8, VPL = 2), the
// same-lane NeoX modes and the normal layout.  Everything else runs as two launches.
template <int W, int VPL, int MODE>
void launch_kv3(agn_ctx *ctx, const RopeArgs &a, bool norm, int kv, unsigned grid, int threads, size_t smem) {
    if (kv == KV_F16) {
        if (norm) agn_launch(ctx, rope_heads_kernel<float, W, VPL, MODE, true, KV_F16>, dim3(grid), dim3(threads), smem, a);
        else agn_launch(ctx, rope_heads_kernel<float, W, VPL, MODE, false, KV_F16>, dim3(grid), dim3(threads), smem, a);
    } else {
        if (norm) agn_launch(ctx, rope_heads_kernel<float, W, VPL, MODE, true, KV_Q8_0>, dim3(grid), dim3(threads), smem, a);
        else agn_launch(ctx, rope_heads_kernel<float, W, VPL, MODE, false, KV_Q8_0>, dim3(grid), dim3(threads), smem, a);
    }
}

bool launch_kv(agn_ctx *ctx, const RopeArgs &a, bool norm, int kv, int W, int VPL, int mode, unsigned grid, int threads, size_t smem) {
    if (W == 8 && VPL == 4 && mode == MODE_NEOX_K2) { launch_kv3<8, 4, MODE_NEOX_K2>(ctx, a, norm, kv, grid, threads, smem); return true; }
    if (W == 8 && VPL == 4 && mode == MODE_NORMAL) { launch_kv3<8, 4, MODE_NORMAL>(ctx, a, norm, kv, grid, threads, smem); return true; }
    if (W == 8 && VPL == 2 && mode == MODE_NEOX_K1) { launch_kv3<8, 2, MODE_NEOX_K1>(ctx, a, norm, kv, grid, threads, smem); return true; }
    if (W == 8 && VPL == 2 && mode == MODE_NORMAL) { launch_kv3<8, 2, MODE_NORMAL>(ctx, a, norm, kv, grid, threads, smem); return true; }
    return false;
}

// Persistent form for large batches; false = not applicable (the caller launches the CTA-per-unit kernel).
template <typename T, int W, int VPL, int MODE, bool NORM>
bool launch_ring4(agn_ctx *ctx, const RopeArgs &a, int threads) {
    const size_t q_tok = (size_t)a.n_q * a.head_dim * sizeof(T), k_tok = (size_t)a.n_kv * a.head_dim * sizeof(T);
    if (q_tok % 16 || k_tok % 16 || (a.n_q && !agn_aligned16(a.q)) || (a.n_kv && !agn_aligned16(a.k))) return false;
    const int slot_bytes = (int)(((size_t)a.tpc * (q_tok + k_tok) + 127) & ~(size_t)127);
    int slots = ctx->tune_rope_ring >= 2 ? ctx->tune_rope_ring : 3;
    while (slots > 2 && (size_t)slots * slot_bytes > 100 * 1024) slots--;
    const int half = a.n_rot >> 1, rows = a.tpc * (a.n_q + a.n_kv);
    const size_t smem = (size_t)slots * slot_bytes + 8 * (size_t)slots + 8 * (size_t)rows + 32 +
                        sizeof(float) * 4 * (size_t)a.tpc * (half > 0 ? half : 1);
    if (smem > 200 * 1024) return false;
    auto kernel = rope_heads_ring_kernel<T, W, VPL, MODE, NORM>;
    int per_sm = agn_ring_ctas_per_sm(ctx, kernel, threads, smem);
    if (per_sm < 1) return false;
    if (ctx->tune_rope_ring_ctas > 0 && ctx->tune_rope_ring_ctas < per_sm) per_sm = ctx->tune_rope_ring_ctas;
    int64_t grid = (int64_t)per_sm * ctx->sm_count;
    const int64_t n_units = (a.T + a.tpc - 1) / a.tpc;
    if (n_units < 2 * grid && !ctx->tune_ring_force) return false;  // too few units per CTA for a ring to pay
    if (grid > n_units) grid = n_units;
    agn_launch(ctx, kernel, dim3((unsigned)grid), dim3(threads), smem, a, slots, slot_bytes, ctx->mbar_spin_limit);
    ctx->flags_dirty = true;
    ctx->ring_launched = true;
    return true;
}

template <typename T, int W, int VPL, int MODE>
void launch_fast3(agn_ctx *ctx, const RopeArgs &a, bool norm, unsigned grid, int threads, size_t smem) {
    if (ctx->tune_rope_ring != 0 &&
        (norm ? launch_ring4<T, W, VPL, MODE, true>(ctx, a, threads) : launch_ring4<T, W, VPL, MODE, false>(ctx, a, threads)))
        return;
    if (norm) agn_launch(ctx, rope_heads_kernel<T, W, VPL, MODE, true>, dim3(grid), dim3(threads), smem, a);
    else agn_launch(ctx, rope_heads_kernel<T, W, VPL, MODE, false>, dim3(grid), dim3(threads), smem, a);
}

template <typename T, int W, int VPL>
bool launch_fast(agn_ctx *ctx, const RopeArgs &a, bool norm, int mode, unsigned grid, int threads, size_t smem) {
    switch (mode) {
    case MODE_NORMAL: launch_fast3<T, W, VPL, MODE_NORMAL>(ctx, a, norm, grid, threads, smem); return true;
    case MODE_NEOX_SHFL: launch_fast3<T, W, VPL, MODE_NEOX_SHFL>(ctx, a, norm, grid, threads, smem); return true;
    case MODE_NEOX_K1:
        if constexpr (VPL >= 2) { launch_fast3<T, W, VPL, MODE_NEOX_K1>(ctx, a, norm, grid, threads, smem); return true; }
        return false;
    case MODE_NEOX_K2:
        if constexpr (VPL >= 4) { launch_fast3<T, W, VPL, MODE_NEOX_K2>(ctx, a, norm, grid, threads, smem); return true; }
        return false;
    }
    return false;
}

bool is_pow2(int v) { return v > 0 && (v & (v - 1)) == 0; }

// What the fused cache write needs besides the rope arguments.
struct KvFuse {
    int kv;  // KV_F16 or KV_Q8_0
    int words;  // Q8_0 in the GPU path's 36-byte blocks
    const float *v;
    unsigned char *k_cache, *v_cache;
    int64_t max_seq;
    int bytes_per_token;
};

// kvf != nullptr: try to pack K (after the rotation) and V into the cache in the same launch;
// *fused tells the caller whether that happened (if not, only the rope ran).
template <typename AT>
int32_t rope_dispatch(agn_ctx *ctx, const char *name, AT *q, AT *k, const float *wq, const float *wk,
                      bool norm, int64_t T, int32_t n_q, int32_t n_kv, int32_t head_dim, float eps, int32_t n_rot,
                      const int32_t *pos, int32_t pos_start, float theta, float freq_scale, int32_t layout,
                      const KvFuse *kvf = nullptr, bool *fused = nullptr) {
    if (fused) *fused = false;
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
    a.inv_head_dim = 1.0f / (float)head_dim;
    a.denom = nullptr;
    a.v = nullptr; a.k_cache = nullptr; a.v_cache = nullptr; a.max_seq = 0; a.bytes_per_token = 0; a.kv_words = 0; a.flags = ctx->d_flags;
    if (n_rot >= 2) {
        int32_t rc = agn_rope_table(ctx, theta, n_rot, &a.denom);
        if (rc != AGN_OK) return rc;
    }
    const int half = n_rot / 2;
    const int n_heads = n_q + n_kv;
    const int hd4 = head_dim / 4;

    // Register fast path: a group of W lanes owns a head of W*VPL float4 (or fewer, with idle
    // lanes).  Prefer many registers per lane (VPL 4) so that the NeoX partner of a float4
    // is in the same lane and the per-head bookkeeping is amortised over more data.
    int W = 0, VPL = 0, mode = -1;
    const int hq = half / 4;
    constexpr int A = ActVec<AT>::ALIGN;
    bool fast = head_dim % 4 == 0 && (n_q == 0 || agn_aligned(q, A)) && (n_kv == 0 || agn_aligned(k, A)) &&
                (!norm || ((n_q == 0 || agn_aligned16(wq)) && (n_kv == 0 || agn_aligned16(wk))));
    if (fast) {
        static const int shapes[7][2] = {{8, 4}, {16, 4}, {32, 4}, {8, 2}, {8, 1}, {32, 2}, {32, 1}};
        bool found = false;
        for (int pass = 0; pass < 2 && !found; pass++) {
            for (int c = 0; c < 7 && !found; c++) {
                const int w = shapes[c][0], v = shapes[c][1];
                const bool exact = w * v == hd4;
                if (pass == 0 ? !exact : !(w == 32 && w * v >= hd4 && w * (v / 2) < hd4)) continue;
                int m = -1;
                if (n_rot == 0 || layout == AGN_ROPE_NORMAL) {
                    if (n_rot % 4 == 0) m = MODE_NORMAL;
                } else if (half % 4 == 0) {
                    if (hq == w && v >= 2) m = MODE_NEOX_K1;
                    else if (hq == 2 * w && v >= 4) m = MODE_NEOX_K2;
                    else if (is_pow2(hq) && 2 * hq <= w) m = MODE_NEOX_SHFL;
                }
                if (m >= 0) { W = w; VPL = v; mode = m; found = true; }
            }
        }
        fast = found;
    }
    bool kv_ok = false;
    // Q8_0 packing is division-heavy (an IEEE division and a rounding per value): on a handful of
    // tokens the one CTA that holds them is slower with it than a second small launch (T = 1: 4.2 vs
    // 4.1 us), so small batches fuse only the f16 cache.
    if (kvf && fast && sizeof(AT) == 4 && n_kv > 0 && W == 8 && (VPL == 4 || VPL == 2) && (kvf->kv == KV_F16 || T >= 512) &&
        (mode == MODE_NORMAL || mode == (VPL == 4 ? MODE_NEOX_K2 : MODE_NEOX_K1)) && agn_aligned16(kvf->v) &&
        (kvf->kv == KV_F16 ? (agn_aligned(kvf->k_cache, 8) && agn_aligned(kvf->v_cache, 8) && kvf->bytes_per_token % 8 == 0)
                           : (head_dim % 32 == 0 && agn_aligned(kvf->k_cache, kvf->words ? 4 : 2) &&
                              agn_aligned(kvf->v_cache, kvf->words ? 4 : 2)))) {
        kv_ok = true;
        a.v = kvf->v; a.k_cache = kvf->k_cache; a.v_cache = kvf->v_cache; a.max_seq = kvf->max_seq;
        a.bytes_per_token = kvf->bytes_per_token;
        a.kv_words = kvf->words;
    }
    if (fast) {
        // tokens per CTA: aim at 32 head rows per CTA, keep the sin/cos table small
        const int n_heads = n_q + n_kv + (kv_ok ? n_kv : 0);  // head rows per token (V rows only for the fused cache write)
        int tpc = 32 / n_heads;
        if (tpc < 1) tpc = 1;
        if (half > 0 && tpc * half > 2048) tpc = 2048 / half > 0 ? 2048 / half : 1;
        if ((int64_t)tpc > T) tpc = (int)T;
        a.tpc = tpc;
        const int rows = tpc * n_heads;
        const int ns = VPL == 4 ? 2 : 4;
        int groups = (rows + ns - 1) / ns;
        int threads = groups * W;
        threads = ((threads + 31) / 32) * 32;
        if (threads > 256) threads = 256;
        const unsigned grid = (unsigned)((T + tpc - 1) / tpc);
        const size_t smem = (((size_t)rows * 12 + 15) & ~(size_t)15) + sizeof(float) * 2 * (size_t)tpc * (half > 0 ? half : 1) + 16 +
                            (norm ? sizeof(float) * 2 * (size_t)head_dim : 0);
        bool ok = false;
        ctx->ring_launched = false;
        if (kv_ok) {
            ok = launch_kv(ctx, a, norm, kvf->kv, W, VPL, mode, grid, threads, smem);
            if (ok) {
                ctx->flags_dirty = true;
                if (fused) *fused = true;
            }
        } else if (W == 8 && VPL == 4) ok = launch_fast<AT, 8, 4>(ctx, a, norm, mode, grid, threads, smem);
        else if (W == 16 && VPL == 4) ok = launch_fast<AT, 16, 4>(ctx, a, norm, mode, grid, threads, smem);
        else if (W == 32 && VPL == 4) ok = launch_fast<AT, 32, 4>(ctx, a, norm, mode, grid, threads, smem);
        else if (W == 8 && VPL == 2) ok = launch_fast<AT, 8, 2>(ctx, a, norm, mode, grid, threads, smem);
        else if (W == 8 && VPL == 1) ok = launch_fast<AT, 8, 1>(ctx, a, norm, mode, grid, threads, smem);
        else if (W == 32 && VPL == 2) ok = launch_fast<AT, 32, 2>(ctx, a, norm, mode, grid, threads, smem);
        else if (W == 32 && VPL == 1) ok = launch_fast<AT, 32, 1>(ctx, a, norm, mode, grid, threads, smem);
        if (!ok) return agn_fail(ctx, AGN_EINVAL, "%s: internal dispatch error (W=%d VPL=%d mode=%d)", name, W, VPL, mode);
        if (ctx->ring_launched) AGN_LAUNCHED(ctx, norm ? "qk_norm_rope_ring" : "rope_ring");
        else AGN_LAUNCHED(ctx, name);
    } else {
        int threads = n_heads >= 8 ? 256 : 32 * n_heads;
        const size_t smem = sizeof(float) * 2 * (size_t)(half > 0 ? half : 1);
        if (layout == AGN_ROPE_NEOX) {
            if (norm) agn_launch(ctx, rope_heads_generic_kernel<AT, AGN_ROPE_NEOX, true>, dim3((unsigned)T), dim3(threads), smem, a);
            else agn_launch(ctx, rope_heads_generic_kernel<AT, AGN_ROPE_NEOX, false>, dim3((unsigned)T), dim3(threads), smem, a);
        } else {
            if (norm) agn_launch(ctx, rope_heads_generic_kernel<AT, AGN_ROPE_NORMAL, true>, dim3((unsigned)T), dim3(threads), smem, a);
            else agn_launch(ctx, rope_heads_generic_kernel<AT, AGN_ROPE_NORMAL, false>, dim3((unsigned)T), dim3(threads), smem, a);
        }
        AGN_LAUNCHED(ctx, name);
    }
    return AGN_OK;
}

}  // namespace

extern "C" int32_t agn_rope_f32(agn_ctx *ctx, float *x, int64_t T, int32_t n_heads, int32_t head_dim, int32_t n_rot,
                                const int32_t *pos, int32_t pos_start, float theta, float freq_scale, int32_t layout) {
    AGN_CHECK_CTX(ctx);
    return rope_dispatch<float>(ctx, "rope", x, nullptr, nullptr, nullptr, false, T, n_heads, 0, head_dim, 0.0f, n_rot, pos,
                         pos_start, theta, freq_scale, layout);
}

extern "C" int32_t agn_rope_qk_f32(agn_ctx *ctx, float *q, float *k, int64_t T, int32_t n_q_heads, int32_t n_kv_heads,
                                   int32_t head_dim, int32_t n_rot, const int32_t *pos, int32_t pos_start, float theta,
                                   float freq_scale, int32_t layout) {
    AGN_CHECK_CTX(ctx);
    return rope_dispatch<float>(ctx, "rope_qk", q, k, nullptr, nullptr, false, T, n_q_heads, n_kv_heads, head_dim, 0.0f, n_rot,
                         pos, pos_start, theta, freq_scale, layout);
}

extern "C" int32_t agn_qk_norm_rope_f32(agn_ctx *ctx, float *x, const float *w, int64_t T, int32_t n_heads,
                                        int32_t head_dim, float eps, int32_t n_rot, const int32_t *pos,
                                        int32_t pos_start, float theta, float freq_scale, int32_t layout) {
    AGN_CHECK_CTX(ctx);
    return rope_dispatch<float>(ctx, "qk_norm_rope", x, nullptr, w, nullptr, true, T, n_heads, 0, head_dim, eps, n_rot, pos,
                         pos_start, theta, freq_scale, layout);
}

extern "C" int32_t agn_qk_norm_rope_qk_f32(agn_ctx *ctx, float *q, float *k, const float *wq, const float *wk, int64_t T,
                                           int32_t n_q_heads, int32_t n_kv_heads, int32_t head_dim, float eps,
                                           int32_t n_rot, const int32_t *pos, int32_t pos_start, float theta,
                                           float freq_scale, int32_t layout) {
    AGN_CHECK_CTX(ctx);
    return rope_dispatch<float>(ctx, "qk_norm_rope_qk", q, k, wq, wk, true, T, n_q_heads, n_kv_heads, head_dim, eps, n_rot, pos,
                         pos_start, theta, freq_scale, layout);
}

// Per-position QK-norm -> RoPE of Q and K, then the KV-cache write of the rotated K and of V: the
// three steps the reference runs back to back for every layer and token (`launch_qk_norm_rope` on q
// and on k, then `kv_cache_write` / `kv_cache_write_q8_0`; src/model/llama/gpu_resident.rs and
// src/ops/kernels_wgpu.rs:566-698) in one launch: K is packed from the registers that hold its
// rotated values, V is read once and packed.  q and k are still updated in place.  The result is
// byte for byte what agn_qk_norm_rope_qk_f32 (or agn_rope_qk_f32 when wq = wk = NULL) followed by
// agn_kv_write_f32 gives; shapes outside the fused kernel's reach run as exactly those two launches.
extern "C" int32_t agn_qk_norm_rope_kv_write_f32(agn_ctx *ctx, float *q, float *k, const float *v, const float *wq,
                                                 const float *wk, int64_t T, int32_t n_q_heads, int32_t n_kv_heads,
                                                 int32_t head_dim, float eps, int32_t n_rot, const int32_t *pos,
                                                 int32_t pos_start, float theta, float freq_scale, int32_t layout,
                                                 int32_t kv_dtype, void *k_cache, void *v_cache, int64_t max_seq_len) {
    AGN_CHECK_CTX(ctx);
    if (kv_dtype != AGN_F16 && kv_dtype != AGN_Q8_0 && kv_dtype != AGN_KV_Q8_0_WORDS)
        return agn_fail(ctx, AGN_EUNSUPPORTED_DTYPE, "qk_norm_rope_kv_write: cache type %d is neither f16, q8_0 nor q8_0 in words", kv_dtype);
    if (n_kv_heads <= 0 || head_dim <= 0 || max_seq_len <= 0)
        return agn_fail(ctx, AGN_EINVAL, "qk_norm_rope_kv_write: n_kv_heads=%d head_dim=%d max_seq_len=%lld", n_kv_heads, head_dim,
                        (long long)max_seq_len);
    if (T > 0 && (!k || !v || !k_cache || !v_cache)) return agn_fail(ctx, AGN_EINVAL, "qk_norm_rope_kv_write: null pointer");
    const bool norm = wq != nullptr || wk != nullptr;
    const int64_t hd_kv = (int64_t)n_kv_heads * head_dim;
    KvFuse f;
    f.kv = kv_dtype == AGN_F16 ? KV_F16 : KV_Q8_0;
    f.words = kv_dtype == AGN_KV_Q8_0_WORDS ? 1 : 0;
    f.v = v;
    f.k_cache = static_cast<unsigned char *>(k_cache);
    f.v_cache = static_cast<unsigned char *>(v_cache);
    f.max_seq = max_seq_len;
    f.bytes_per_token = (int)agn_kv_bytes_per_token(kv_dtype, hd_kv);
    bool fused = false;
    int32_t rc = rope_dispatch<float>(ctx, "qk_norm_rope_kv_write", q, k, wq, wk, norm, T, n_q_heads, n_kv_heads, head_dim, eps,
                                      n_rot, pos, pos_start, theta, freq_scale, layout, &f, &fused);
    if (rc != AGN_OK || fused) return rc;
    return agn_kv_write_f32(ctx, kv_dtype, k, v, k_cache, v_cache, T, hd_kv, pos, pos_start, max_seq_len);
}

// f16 activation storage (the reference's `Act = f16`; `rope` / `qk_norm_rope`,
// src/ops/kernels_wgpu.rs:225-318): q, k are f16, norm weights f32, arithmetic f32.
// Pass k = NULL, n_kv_heads = 0 for a single buffer; wq = wk = NULL for rope without the norm.
extern "C" int32_t agn_qk_norm_rope_qk_f16(agn_ctx *ctx, void *q, void *k, const float *wq, const float *wk, int64_t T,
                                           int32_t n_q_heads, int32_t n_kv_heads, int32_t head_dim, float eps,
                                           int32_t n_rot, const int32_t *pos, int32_t pos_start, float theta,
                                           float freq_scale, int32_t layout) {
    AGN_CHECK_CTX(ctx);
    const bool norm = wq != nullptr || wk != nullptr;
    return rope_dispatch<__half>(ctx, norm ? "qk_norm_rope_qk_f16" : "rope_qk_f16", static_cast<__half *>(q),
                                 static_cast<__half *>(k), wq, wk, norm, T, n_q_heads, n_kv_heads, head_dim, eps, n_rot, pos,
                                 pos_start, theta, freq_scale, layout);
}

extern "C" int32_t agn_rope_qk_f16(agn_ctx *ctx, void *q, void *k, int64_t T, int32_t n_q_heads, int32_t n_kv_heads,
                                   int32_t head_dim, int32_t n_rot, const int32_t *pos, int32_t pos_start, float theta,
                                   float freq_scale, int32_t layout) {
    return agn_qk_norm_rope_qk_f16(ctx, q, k, nullptr, nullptr, T, n_q_heads, n_kv_heads, head_dim, 0.0f, n_rot, pos,
                                   pos_start, theta, freq_scale, layout);
}
