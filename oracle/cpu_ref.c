/*
 * CPU oracle — TEST INFRASTRUCTURE ONLY (see cpu_ref.h for scope and pinning).
 *
 * Every function restates the cited lines of the reference's Rust CPU path in
 * plain C with the same f32 operation order.  Compile with
 *   gcc -O2 -ffp-contract=off -fno-fast-math -fopenmp
 * so that no multiply-add is contracted and no sum is re-associated.
 */
#include "cpu_ref.h"

#include <math.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* ---------------------------------------------------------------- types -- */

/* src/types.rs:88-123 */
size_t orc_block_size(int dtype) {
    switch (dtype) {
    case ORC_F32: case ORC_F16: case ORC_BF16: return 1;
    case ORC_Q8_0: case ORC_Q5_0: return 32;
    case ORC_Q2_K: case ORC_Q4_K: case ORC_Q5_K: case ORC_Q6_K: return 256;
    default: return 0;
    }
}

/* src/types.rs:126-161 */
size_t orc_block_bytes(int dtype) {
    switch (dtype) {
    case ORC_F32: return 4;
    case ORC_F16: case ORC_BF16: return 2;
    case ORC_Q8_0: return 34;
    case ORC_Q5_0: return 22;
    case ORC_Q5_K: return 176;
    case ORC_Q2_K: return 84; /* q2_k.rs:24 (the codec), not types.rs:137 */
    case ORC_Q4_K: return 144;
    case ORC_Q6_K: return 210;
    default: return 0;
    }
}

/* src/types.rs:164-168 */
size_t orc_type_size(int dtype, size_t n) {
    size_t bs = orc_block_size(dtype);
    if (bs == 0) return 0;
    return ((n + bs - 1) / bs) * orc_block_bytes(dtype);
}

/* half::f16::to_f32 — exact widening incl. subnormals, inf and NaN
 * (call sites src/quant/q8_0.rs:32, q4_k.rs:53-55, q6_k.rs:52-53, mod.rs:153). */
float orc_f16_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else {
            /* subnormal: normalise */
            int e = -1;
            do { man <<= 1; e++; } while ((man & 0x400u) == 0);
            man &= 0x3FFu;
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        /* inf, or NaN with the quiet bit set (what `half` and F16C hardware return) */
        bits = sign | 0x7F800000u | (man ? 0x00400000u : 0u) | (man << 13);
    } else {
        bits = sign | ((exp + (127 - 15)) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

static inline uint16_t rd_u16(const uint8_t *p) { return (uint16_t)(p[0] | (p[1] << 8)); }

/* ------------------------------------------------------------- rms_norm -- */

/* src/model/llama/cpu_path.rs:34-40 */
int orc_rope_freq_scale(const char *type_, int has_factor, float factor, float *scale) {
    if (type_ == NULL || type_[0] == '\0' || strcmp(type_, "none") == 0) {
        *scale = 1.0f;
        return 1;
    }
    if (strcmp(type_, "linear") == 0) {
        float f = has_factor ? factor : 1.0f;
        if (!(f > 1e-6f)) f = 1e-6f; /* f32::max(1e-6) */
        *scale = 1.0f / f;
        return 1;
    }
    return 0;
}

/* src/model/llama/cpu_path.rs:67-74 */
void orc_rms_norm(const float *x, const float *w, float *out, size_t n, float eps) {
    float sum_sq = 0.0f;
    for (size_t i = 0; i < n; i++) sum_sq += x[i] * x[i];
    float rms = sqrtf(sum_sq / (float)n + eps);
    for (size_t i = 0; i < n; i++) out[i] = w[i] * x[i] / rms;
}

void orc_rms_norm_rows(const float *x, const float *w, float *out, size_t T, size_t H,
                       float eps, int threads) {
#pragma omp parallel for schedule(static) num_threads(threads) if (threads > 1)
    for (long t = 0; t < (long)T; t++) orc_rms_norm(x + t * H, w, out + t * H, H, eps);
}

/* residual add src/model/llama/cpu_path.rs:785-787, then rms_norm :790 */
void orc_add_residual_rms_norm_rows(const float *x, const float *delta, const float *w,
                                    float *new_x, float *normed, size_t T, size_t H,
                                    float eps, int threads) {
#pragma omp parallel for schedule(static) num_threads(threads) if (threads > 1)
    for (long t = 0; t < (long)T; t++) {
        const float *xr = x + t * H, *dr = delta + t * H;
        float *nr = new_x + t * H;
        for (size_t i = 0; i < H; i++) nr[i] = xr[i] + dr[i];
        orc_rms_norm(nr, w, normed + t * H, H, eps);
    }
}

/* src/model/llama/cpu_path.rs:78-93 */
void orc_qk_norm(float *x, const float *w, size_t n_heads, size_t head_dim, float eps) {
    for (size_t h = 0; h < n_heads; h++) {
        float *head = x + h * head_dim;
        float sum_sq = 0.0f;
        for (size_t d = 0; d < head_dim; d++) sum_sq += head[d] * head[d];
        float rms = sqrtf(sum_sq / (float)head_dim + eps);
        for (size_t d = 0; d < head_dim; d++) head[d] = w[d] * head[d] / rms;
    }
}

/* ----------------------------------------------------------------- rope -- */

/* theta.powf(2.0 * d as f32 / n_rot as f32), cpu_path.rs:109 / :476 */
void orc_rope_denominators(float theta, size_t n_rot, float *denom) {
    size_t half = n_rot / 2;
    for (size_t d = 0; d < half; d++)
        denom[d] = powf(theta, 2.0f * (float)d / (float)n_rot);
}

/* src/model/llama/cpu_path.rs:99-133 (full) and :461-496 (partial n_rot).
 * NeoX pairs (d, d+half) as the reference does; "normal" pairs (2d, 2d+1)
 * with the same angle (not in the reference). */
void orc_rope(float *x, size_t n_heads, size_t head_dim, size_t n_rot, int64_t pos,
              float theta, float freq_scale, int layout) {
    size_t half = n_rot / 2;
    if (half == 0) return;
    float sin_t[half], cos_t[half];
    for (size_t d = 0; d < half; d++) {
        float freq = (float)pos * freq_scale / powf(theta, 2.0f * (float)d / (float)n_rot);
        sin_t[d] = sinf(freq);
        cos_t[d] = cosf(freq);
    }
    for (size_t h = 0; h < n_heads; h++) {
        float *head = x + h * head_dim;
        for (size_t d = 0; d < half; d++) {
            size_t i0 = layout == ORC_ROPE_NEOX ? d : 2 * d;
            size_t i1 = layout == ORC_ROPE_NEOX ? d + half : 2 * d + 1;
            float x0 = head[i0], x1 = head[i1];
            head[i0] = x0 * cos_t[d] - x1 * sin_t[d];
            head[i1] = x0 * sin_t[d] + x1 * cos_t[d];
        }
    }
}

void orc_rope_rows(float *x, size_t T, size_t n_heads, size_t head_dim, size_t n_rot,
                   const int32_t *pos, float theta, float freq_scale, int layout,
                   int threads) {
    size_t w = n_heads * head_dim;
#pragma omp parallel for schedule(static) num_threads(threads) if (threads > 1)
    for (long t = 0; t < (long)T; t++)
        orc_rope(x + t * w, n_heads, head_dim, n_rot, pos[t], theta, freq_scale, layout);
}

/* per-position QK-norm -> RoPE of run_batch, cpu_path.rs:896-906 */
void orc_qk_norm_rope_rows(float *x, const float *w, size_t T, size_t n_heads,
                           size_t head_dim, float eps, size_t n_rot, const int32_t *pos,
                           float theta, float freq_scale, int layout, int threads) {
    size_t wd = n_heads * head_dim;
#pragma omp parallel for schedule(static) num_threads(threads) if (threads > 1)
    for (long t = 0; t < (long)T; t++) {
        if (w) orc_qk_norm(x + t * wd, w, n_heads, head_dim, eps);
        orc_rope(x + t * wd, n_heads, head_dim, n_rot, pos[t], theta, freq_scale, layout);
    }
}

/* -------------------------------------------------------------- softmax -- */

/* src/model/llama/cpu_path.rs:175-183.  f32::max ignores a NaN operand. */
void orc_softmax(float *s, size_t n) {
    float max = -INFINITY;
    for (size_t i = 0; i < n; i++) max = fmaxf(max, s[i]);
    for (size_t i = 0; i < n; i++) s[i] = expf(s[i] - max);
    float sum = 0.0f;
    for (size_t i = 0; i < n; i++) sum += s[i];
    for (size_t i = 0; i < n; i++) s[i] /= sum;
}

void orc_softmax_rows(const float *in, float *out, size_t n_rows, size_t row_len,
                      size_t row_stride, const int32_t *n_valid, int threads) {
#pragma omp parallel for schedule(static) num_threads(threads) if (threads > 1)
    for (long r = 0; r < (long)n_rows; r++) {
        size_t nv = n_valid ? (size_t)n_valid[r] : row_len;
        if (nv > row_len) nv = row_len;
        float *o = out + r * row_stride;
        const float *i = in + r * row_stride;
        if (o != i) memcpy(o, i, nv * sizeof(float));
        orc_softmax(o, nv);
        for (size_t j = nv; j < row_len; j++) o[j] = 0.0f;
    }
}

/* ------------------------------------------------------------- silu*mul -- */

/* src/model/llama/cpu_path.rs:228-229, :975-978 */
void orc_silu_mul(const float *gate, const float *up, float *out, size_t n, int threads) {
#pragma omp parallel for schedule(static) num_threads(threads) if (threads > 1)
    for (long i = 0; i < (long)n; i++) {
        float g = gate[i];
        float silu = g / (1.0f + expf(-g));
        out[i] = silu * up[i];
    }
}

/* --------------------------------------------------------- quant codecs -- */

/* src/quant/q8_0.rs:14-51 */
int orc_dequant_q8_0(const uint8_t *data, size_t data_len, size_t n, float *out) {
    size_t n_blocks = (n + 31) / 32;
    if (data_len < n_blocks * 34) return ORC_ESHORT;
    size_t o = 0;
    for (size_t b = 0; b < n_blocks; b++) {
        const uint8_t *blk = data + b * 34;
        float scale = orc_f16_to_f32(rd_u16(blk));
        size_t cnt = (b == n_blocks - 1) ? n - b * 32 : 32;
        for (size_t i = 0; i < cnt; i++) out[o++] = scale * (float)(int8_t)blk[2 + i];
    }
    return ORC_OK;
}

/* src/quant/q4_k.rs:26-35 */
void orc_get_scale_min_k4(size_t j, const uint8_t *scales, uint8_t *sc, uint8_t *m) {
    if (j < 4) {
        *sc = scales[j] & 63;
        *m = scales[j + 4] & 63;
    } else {
        *sc = (uint8_t)((scales[j + 4] & 0xF) | ((scales[j - 4] >> 6) << 4));
        *m = (uint8_t)((scales[j + 4] >> 4) | ((scales[j] >> 6) << 4));
    }
}

/* src/quant/q4_k.rs:37-91 */
int orc_dequant_q4_k(const uint8_t *data, size_t data_len, size_t n, float *out) {
    size_t n_blocks = (n + 255) / 256;
    if (data_len < n_blocks * 144) return ORC_ESHORT;
    for (size_t b = 0; b < n_blocks; b++) {
        const uint8_t *blk = data + b * 144;
        float d = orc_f16_to_f32(rd_u16(blk));
        float dmin = orc_f16_to_f32(rd_u16(blk + 2));
        const uint8_t *scales = blk + 4;
        const uint8_t *qs = blk + 16;
        float tmp[256];
        size_t is = 0;
        for (size_t j = 0; j < 256; j += 64) {
            const uint8_t *q = qs + j / 2;
            uint8_t sc, m;
            orc_get_scale_min_k4(is, scales, &sc, &m);
            float d1 = d * (float)sc;
            float m1 = dmin * (float)m;
            orc_get_scale_min_k4(is + 1, scales, &sc, &m);
            float d2 = d * (float)sc;
            float m2 = dmin * (float)m;
            for (size_t l = 0; l < 32; l++) tmp[j + l] = d1 * (float)(q[l] & 0x0F) - m1;
            for (size_t l = 0; l < 32; l++) tmp[j + 32 + l] = d2 * (float)(q[l] >> 4) - m2;
            is += 2;
        }
        size_t base = b * 256;
        size_t cnt = n - base < 256 ? n - base : 256; /* out.truncate(n) */
        memcpy(out + base, tmp, cnt * sizeof(float));
    }
    return ORC_OK;
}

/* src/quant/q5_k.rs:43-103 */
int orc_dequant_q5_k(const uint8_t *data, size_t data_len, size_t n, float *out) {
    size_t n_blocks = (n + 255) / 256;
    if (data_len < n_blocks * 176) return ORC_ESHORT;
    for (size_t b = 0; b < n_blocks; b++) {
        const uint8_t *blk = data + b * 176;
        float d = orc_f16_to_f32(rd_u16(blk));
        float dmin = orc_f16_to_f32(rd_u16(blk + 2));
        const uint8_t *scales = blk + 4, *qh = blk + 16, *qs = blk + 48;
        float tmp[256];
        size_t is = 0;
        uint8_t u1 = 1, u2 = 2;
        for (size_t j = 0; j < 256; j += 64) {
            const uint8_t *q = qs + j / 2;
            uint8_t sc, m;
            orc_get_scale_min_k4(is, scales, &sc, &m);
            float d1 = d * (float)sc;
            float m1 = dmin * (float)m;
            orc_get_scale_min_k4(is + 1, scales, &sc, &m);
            float d2 = d * (float)sc;
            float m2 = dmin * (float)m;
            for (size_t l = 0; l < 32; l++)
                tmp[j + l] = d1 * (float)((q[l] & 0x0F) + ((qh[l] & u1) ? 16 : 0)) - m1;
            for (size_t l = 0; l < 32; l++)
                tmp[j + 32 + l] = d2 * (float)((q[l] >> 4) + ((qh[l] & u2) ? 16 : 0)) - m2;
            is += 2;
            u1 <<= 2;
            u2 <<= 2;
        }
        size_t base = b * 256;
        size_t cnt = n - base < 256 ? n - base : 256;
        memcpy(out + base, tmp, cnt * sizeof(float));
    }
    return ORC_OK;
}

/* src/quant/q2_k.rs:30-98 */
int orc_dequant_q2_k(const uint8_t *data, size_t data_len, size_t n, float *out) {
    if (n % 256 != 0) return ORC_ELEN;
    size_t n_blocks = n / 256;
    if (data_len < n_blocks * 84) return ORC_ESHORT;
    for (size_t b = 0; b < n_blocks; b++) {
        const uint8_t *blk = data + b * 84;
        const uint8_t *scales = blk, *qs = blk + 16;
        float d = orc_f16_to_f32(rd_u16(blk + 80));
        float dmin = orc_f16_to_f32(rd_u16(blk + 82));
        float *o = out + b * 256;
        size_t is = 0, q_off = 0;
        for (int group = 0; group < 2; group++) {
            unsigned shift = 0;
            for (int j = 0; j < 4; j++) {
                for (int half = 0; half < 2; half++) {
                    uint8_t sc = scales[is++];
                    float dl = d * (float)(sc & 0xF);
                    float ml = dmin * (float)(sc >> 4);
                    for (size_t l = 0; l < 16; l++) {
                        int8_t quant = (int8_t)((qs[q_off + 16 * half + l] >> shift) & 3);
                        *o++ = dl * (float)quant - ml;
                    }
                }
                shift += 2;
            }
            q_off += 32;
        }
    }
    return ORC_OK;
}

/* src/quant/q5_0.rs:20-62 */
int orc_dequant_q5_0(const uint8_t *data, size_t data_len, size_t n, float *out) {
    size_t n_blocks = (n + 31) / 32;
    if (data_len < n_blocks * 22) return ORC_ESHORT;
    for (size_t b = 0; b < n_blocks; b++) {
        const uint8_t *blk = data + b * 22;
        float d = orc_f16_to_f32(rd_u16(blk));
        uint32_t qh = (uint32_t)blk[2] | ((uint32_t)blk[3] << 8) | ((uint32_t)blk[4] << 16) | ((uint32_t)blk[5] << 24);
        const uint8_t *qs = blk + 6;
        float tmp[32];
        for (size_t j = 0; j < 16; j++) {
            uint8_t xh0 = (uint8_t)((qh >> j) & 1), xh1 = (uint8_t)((qh >> (j + 16)) & 1);
            int x0 = (int)((qs[j] & 0x0F) | (xh0 << 4)) - 16;
            int x1 = (int)((qs[j] >> 4) | (xh1 << 4)) - 16;
            tmp[j] = (float)x0 * d;
            tmp[j + 16] = (float)x1 * d;
        }
        size_t base = b * 32;
        size_t cnt = n - base < 32 ? n - base : 32;
        memcpy(out + base, tmp, cnt * sizeof(float));
    }
    return ORC_OK;
}

/* src/quant/q6_k.rs:25-77 */
int orc_dequant_q6_k(const uint8_t *data, size_t data_len, size_t n, float *out) {
    size_t n_blocks = (n + 255) / 256;
    if (data_len < n_blocks * 210) return ORC_ESHORT;
    for (size_t b = 0; b < n_blocks; b++) {
        const uint8_t *blk = data + b * 210;
        const uint8_t *ql = blk, *qh = blk + 128;
        const int8_t *scales = (const int8_t *)(blk + 192);
        float d = orc_f16_to_f32(rd_u16(blk + 208));
        float tmp[256];
        for (size_t h = 0; h < 2; h++) {
            const uint8_t *ql_h = ql + h * 64, *qh_h = qh + h * 32;
            const int8_t *sc = scales + h * 8;
            float *y = tmp + h * 128;
            for (size_t l = 0; l < 32; l++) {
                size_t is = l / 16;
                uint8_t qhl = qh_h[l];
                int q1 = (int)((ql_h[l] & 0x0F) | (((qhl >> 0) & 3) << 4)) - 32;
                int q2 = (int)((ql_h[l + 32] & 0x0F) | (((qhl >> 2) & 3) << 4)) - 32;
                int q3 = (int)((ql_h[l] >> 4) | (((qhl >> 4) & 3) << 4)) - 32;
                int q4 = (int)((ql_h[l + 32] >> 4) | (((qhl >> 6) & 3) << 4)) - 32;
                y[l] = d * (float)sc[is] * (float)q1;
                y[l + 32] = d * (float)sc[is + 2] * (float)q2;
                y[l + 64] = d * (float)sc[is + 4] * (float)q3;
                y[l + 96] = d * (float)sc[is + 6] * (float)q4;
            }
        }
        size_t base = b * 256;
        size_t cnt = n - base < 256 ? n - base : 256;
        memcpy(out + base, tmp, cnt * sizeof(float));
    }
    return ORC_OK;
}

/* src/quant/mod.rs:137-144 */
int orc_dequant_f32(const uint8_t *data, size_t data_len, size_t n, float *out) {
    if (data_len < n * 4) return ORC_ESHORT;
    memcpy(out, data, n * 4);
    return ORC_OK;
}

/* src/quant/mod.rs:147-157 */
int orc_dequant_f16(const uint8_t *data, size_t data_len, size_t n, float *out) {
    if (data_len < n * 2) return ORC_ESHORT;
    for (size_t i = 0; i < n; i++) out[i] = orc_f16_to_f32(rd_u16(data + 2 * i));
    return ORC_OK;
}

/* src/quant/mod.rs:160-170 */
int orc_dequant_bf16(const uint8_t *data, size_t data_len, size_t n, float *out) {
    if (data_len < n * 2) return ORC_ESHORT;
    for (size_t i = 0; i < n; i++) {
        uint32_t bits = (uint32_t)rd_u16(data + 2 * i) << 16;
        memcpy(out + i, &bits, 4);
    }
    return ORC_OK;
}

/* src/quant/mod.rs:30-47 (dispatch) + :97-135 (row_view) for a 2-D tensor */
int orc_dequant_row(int dtype, const uint8_t *data, size_t data_len, size_t byte_offset,
                    size_t row_len, size_t n_rows, size_t row, float *out) {
    size_t row_bytes = orc_type_size(dtype, row_len);
    if (row_bytes == 0) return ORC_EDTYPE;
    if (row >= n_rows) return ORC_EROW;
    size_t off = byte_offset + row * row_bytes;
    if (off + row_bytes > data_len) return ORC_ESHORT;
    const uint8_t *p = data + off;
    size_t avail = data_len - off;
    switch (dtype) {
    case ORC_F32: return orc_dequant_f32(p, avail, row_len, out);
    case ORC_F16: return orc_dequant_f16(p, avail, row_len, out);
    case ORC_BF16: return orc_dequant_bf16(p, avail, row_len, out);
    case ORC_Q8_0: return orc_dequant_q8_0(p, avail, row_len, out);
    case ORC_Q4_K: return orc_dequant_q4_k(p, avail, row_len, out);
    case ORC_Q5_K: return orc_dequant_q5_k(p, avail, row_len, out);
    case ORC_Q2_K: return orc_dequant_q2_k(p, avail, row_len, out);
    case ORC_Q5_0: return orc_dequant_q5_0(p, avail, row_len, out);
    case ORC_Q6_K: return orc_dequant_q6_k(p, avail, row_len, out);
    default: return ORC_EDTYPE;
    }
}

/* embedding loop, src/model/llama/cpu_path.rs:865-868 (and :706 for T=1) */
int orc_get_rows(int dtype, const uint8_t *table, size_t table_len, size_t n_vocab,
                 size_t row_len, const uint32_t *ids, size_t T, float *out, int threads) {
    int bad = 0;
    if (orc_type_size(dtype, row_len) == 0) return ORC_EDTYPE;
#pragma omp parallel for schedule(static) num_threads(threads) if (threads > 1) reduction(| : bad)
    for (long t = 0; t < (long)T; t++) {
        int rc = orc_dequant_row(dtype, table, table_len, 0, row_len, n_vocab, ids[t],
                                 out + (size_t)t * row_len);
        if (rc != ORC_OK) {
            memset(out + (size_t)t * row_len, 0, row_len * sizeof(float));
            bad |= rc;
        }
    }
    return bad ? ORC_EROW : ORC_OK;
}

/* ------------------------------------------------------------- KV cache -- */

static uint16_t f32_to_f16_bits(float f) { /* half::f16::from_f32: round to nearest even */
    uint32_t x;
    memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t exp = (x >> 23) & 0xFFu;
    uint32_t man = x & 0x7FFFFFu;
    if (exp == 0xFF) return (uint16_t)(sign | 0x7C00u | (man ? (0x200u | (man >> 13)) : 0));
    int32_t e = (int32_t)exp - 127 + 15;
    if (e >= 31) return (uint16_t)(sign | 0x7C00u);
    if (e <= 0) {
        if (e < -10) return (uint16_t)sign;
        man |= 0x800000u;
        uint32_t shift = (uint32_t)(14 - e);
        uint32_t half_man = man >> shift;
        uint32_t rem = man & ((1u << shift) - 1), halfway = 1u << (shift - 1);
        if (rem > halfway || (rem == halfway && (half_man & 1))) half_man++;
        return (uint16_t)(sign | half_man);
    }
    uint32_t half = ((uint32_t)e << 10) | (man >> 13);
    uint32_t rem = man & 0x1FFFu;
    if (rem > 0x1000u || (rem == 0x1000u && (half & 1))) half++;
    return (uint16_t)(sign | half);
}

size_t orc_kv_bytes_per_token(int dtype, size_t hd) { /* src/model/mod.rs:550-556 */
    if (dtype == ORC_F16) return hd * 2;
    if (dtype == ORC_Q8_0) return ((hd + 31) / 32) * 34;
    if (dtype == ORC_KV_Q8_0_WORDS) return ((hd + 31) / 32) * 36; /* words_per_token * 4, gpu_resident.rs:276-277 */
    return 0;
}

/* The GPU path's Q8_0 cache block (kv_cache_write_q8_0, src/ops/kernels_wgpu.rs:583-698): nine 32-bit words per
 * 32 values — word 0 the scale as f32 bits, words 1..8 four bytes each, offset-binary (byte = q + 128), the low
 * byte first.  Values past n in the last block are 0 (byte 128) and are written.  amax, scale and q as in the
 * CPU packing; the kernel's `round` is taken as f32::round (half away from zero) and a NaN quotient as q = 0,
 * like KvDtype::pack: the two layouts hold the same numbers. */
static void kv_pack_q8_0_words(const float *x, size_t n, uint8_t *out) {
    for (size_t b = 0; b * 32 < n; b++) {
        const float *blk = x + b * 32;
        size_t cnt = n - b * 32 < 32 ? n - b * 32 : 32;
        uint8_t *o = out + b * 36;
        float amax = 0.0f;
        for (size_t i = 0; i < cnt; i++) amax = fmaxf(amax, fabsf(blk[i]));
        float scale = amax > 0.0f ? amax / 127.0f : 1.0f;
        uint32_t sb;
        memcpy(&sb, &scale, 4);
        o[0] = (uint8_t)sb; o[1] = (uint8_t)(sb >> 8); o[2] = (uint8_t)(sb >> 16); o[3] = (uint8_t)(sb >> 24);
        for (size_t i = 0; i < 32; i++) {
            float q = i < cnt ? roundf(blk[i] / scale) : 0.0f;
            q = q < -127.0f ? -127.0f : (q > 127.0f ? 127.0f : q);
            if (q != q) q = 0.0f;
            o[4 + i] = (uint8_t)((int)q + 128);
        }
    }
}

/* KvDtype::pack, src/model/mod.rs:567-585 */
void orc_kv_pack(int dtype, const float *x, size_t n, uint8_t *out) {
    if (dtype == ORC_F16) {
        for (size_t i = 0; i < n; i++) {
            uint16_t h = f32_to_f16_bits(x[i]);
            out[2 * i] = (uint8_t)(h & 0xFF);
            out[2 * i + 1] = (uint8_t)(h >> 8);
        }
        return;
    }
    if (dtype == ORC_KV_Q8_0_WORDS) {
        kv_pack_q8_0_words(x, n, out);
        return;
    }
    for (size_t b = 0; b * 32 < n; b++) {
        const float *blk = x + b * 32;
        size_t cnt = n - b * 32 < 32 ? n - b * 32 : 32;
        uint8_t *o = out + b * 34;
        float amax = 0.0f;
        for (size_t i = 0; i < cnt; i++) amax = fmaxf(amax, fabsf(blk[i])); /* f32::max: a NaN operand is ignored */
        float scale = amax > 0.0f ? amax / 127.0f : 1.0f;
        uint16_t h = f32_to_f16_bits(scale);
        o[0] = (uint8_t)(h & 0xFF);
        o[1] = (uint8_t)(h >> 8);
        for (size_t i = 0; i < cnt; i++) {
            float q = roundf(blk[i] / scale);
            q = q < -127.0f ? -127.0f : (q > 127.0f ? 127.0f : q);
            if (q != q) q = 0.0f; /* `NaN as i8` is 0 in Rust (a NaN value, or inf / inf in a block that holds an inf) */
            o[2 + i] = (uint8_t)(int8_t)q;
        }
    }
}

/* KvDtype::unpack, src/model/mod.rs:587-604 */
void orc_kv_unpack(int dtype, const uint8_t *bytes, size_t n, float *out) {
    if (dtype == ORC_F16) {
        for (size_t i = 0; i < n; i++) out[i] = orc_f16_to_f32(rd_u16(bytes + 2 * i));
        return;
    }
    if (dtype == ORC_KV_Q8_0_WORDS) { /* dequant_kv_q8_0, src/ops/kernels_wgpu.rs:705-718 */
        for (size_t i = 0; i < n; i++) {
            const uint8_t *blk = bytes + (i / 32) * 36;
            float scale;
            memcpy(&scale, blk, 4);
            out[i] = ((float)blk[4 + i % 32] - 128.0f) * scale;
        }
        return;
    }
    for (size_t i = 0; i < n; i++) {
        const uint8_t *blk = bytes + (i / 32) * 34;
        out[i] = (float)(int8_t)blk[2 + i % 32] * orc_f16_to_f32(rd_u16(blk));
    }
}

/* KvCache::write_range, src/model/mod.rs:660-672: token t -> slot pos[t] */
void orc_kv_write_rows(int dtype, const float *x, size_t T, size_t hd, const int32_t *pos, uint8_t *cache) {
    size_t bpt = orc_kv_bytes_per_token(dtype, hd);
    for (size_t t = 0; t < T; t++) orc_kv_pack(dtype, x + t * hd, hd, cache + (size_t)pos[t] * bpt);
}

/* KvCache::read_up_to, src/model/mod.rs:678-697 */
void orc_kv_read(int dtype, const uint8_t *cache, size_t n_pos, size_t hd, float *out) {
    size_t bpt = orc_kv_bytes_per_token(dtype, hd);
    for (size_t p = 0; p < n_pos; p++) orc_kv_unpack(dtype, cache + p * bpt, hd, out + p * hd);
}

/* ------------------------------------------------------------------ MoE -- */

void orc_router_top2(const float *logits, size_t T, size_t n_experts, int32_t *idx,
                     float *w) {
    float p[n_experts];
    for (size_t t = 0; t < T; t++) {
        memcpy(p, logits + t * n_experts, n_experts * sizeof(float));
        orc_softmax(p, n_experts);
        /* softmax is monotonic: rank by logit so that exp rounding cannot reorder picks */
        const float *l = logits + t * n_experts;
        int b0 = 0;
        for (size_t e = 1; e < n_experts; e++)
            if (l[e] > l[b0]) b0 = (int)e;
        int b1 = -1;
        for (size_t e = 0; e < n_experts; e++) {
            if ((int)e == b0) continue;
            if (b1 < 0 || l[e] > l[b1]) b1 = (int)e;
        }
        idx[2 * t] = b0;
        idx[2 * t + 1] = b1;
        w[2 * t] = p[b0];
        w[2 * t + 1] = b1 >= 0 ? p[b1] : 0.0f;
    }
}

void orc_gather_rows_by_expert(const float *x, size_t T, size_t H, const int32_t *idx,
                               size_t n_experts, float *out, int32_t *offsets,
                               int32_t *src_token, int32_t *src_slot) {
    int32_t cursor[n_experts + 1];
    memset(offsets, 0, (n_experts + 1) * sizeof(int32_t));
    for (size_t i = 0; i < 2 * T; i++) offsets[idx[i] + 1]++;
    for (size_t e = 0; e < n_experts; e++) offsets[e + 1] += offsets[e];
    memcpy(cursor, offsets, (n_experts + 1) * sizeof(int32_t));
    /* stable: ascending token, slot 0 before slot 1 */
    for (size_t i = 0; i < 2 * T; i++) {
        int32_t dst = cursor[idx[i]]++;
        src_token[dst] = (int32_t)(i / 2);
        src_slot[dst] = (int32_t)(i % 2);
        memcpy(out + (size_t)dst * H, x + (i / 2) * H, H * sizeof(float));
    }
}

/* ------------------------------------------------ Q8_K activation rows -- */

/* Rust's `f32 as i32`: saturating, NaN -> 0 */
static int32_t f32_as_i32(float v) {
    if (v != v) return 0;
    if (v >= 2147483648.0f) return INT32_MAX;
    if (v <= -2147483648.0f) return INT32_MIN;
    return (int32_t)v;
}

/* src/quant/q8_k.rs:49-92 */
void orc_quantize_row_q8_k(const float *x, size_t n, float *d, int8_t *qs, int16_t *bsums) {
    size_t n_blocks = (n + 255) / 256;
    for (size_t block = 0; block < n_blocks; block++) {
        size_t start = block * 256;
        size_t end = start + 256 < n ? start + 256 : n;
        float amax = 0.0f, max = 0.0f;
        for (size_t i = start; i < end; i++) {
            float av = fabsf(x[i]);
            if (av > amax) {
                amax = av;
                max = x[i];
            }
        }
        int8_t *q = qs + block * 256;
        memset(q, 0, 256);
        d[block] = 0.0f;
        if (amax > 0.0f) {
            float iscale = -127.0f / max;
            for (size_t i = start; i < end; i++) {
                int32_t rounded = f32_as_i32(roundf(iscale * x[i])); /* f32::round: half away from zero */
                if (rounded > 127) rounded = 127;
                q[i - start] = (int8_t)(uint8_t)((uint32_t)rounded & 0xffu); /* `as i8` truncates */
            }
            d[block] = 1.0f / iscale;
        }
        for (size_t g = 0; g < 16; g++) {
            int16_t s = 0;
            for (size_t j = 0; j < 16; j++) s = (int16_t)(s + q[g * 16 + j]);
            bsums[block * 16 + g] = s;
        }
    }
}

void orc_quantize_rows_q8_k(const float *x, size_t T, size_t n, float *d, int8_t *qs, int16_t *bsums,
                            int threads) {
    size_t nb = (n + 255) / 256;
#pragma omp parallel for schedule(static) num_threads(threads) if (threads > 1)
    for (long t = 0; t < (long)T; t++)
        orc_quantize_row_q8_k(x + (size_t)t * n, n, d + (size_t)t * nb, qs + (size_t)t * nb * 256,
                              bsums + (size_t)t * nb * 16);
}

int orc_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
