/*
 * CPU oracle for the layer-op hot path of the gguf-rs engine (agention-infer).
 *
 * TEST INFRASTRUCTURE ONLY.  This is a plain-C restatement of the reference's
 * CPU code, used as the checker for the CUDA library and as the timed CPU
 * baseline.  Nothing in the shipped CUDA path may call it.
 *
 * Parity pinning:
 *   - quant codecs (Q8_0 / Q4_K / Q6_K / Q5_K / Q5_0 / Q2_K / F16 / BF16 / F32
 *     rows) are pinned by the reference's own unit-test vectors
 *     (src/quant/q8_0.rs:110-148, src/quant/q4_k.rs:229-241,
 *     src/quant/q5_0.rs:89-125, src/quant/q5_k.rs:348-392,
 *     src/quant/q2_k.rs:113-177, src/quant/mod.rs:176-205) re-created in the
 *     test-suite, and compute_rope_freq_scale by
 *     src/model/llama/cpu_path.rs:1034-1060.
 *   - KV-cache packing (KvDtype::pack / unpack, src/model/mod.rs:567-604): the
 *     reference has no test for it -> "parity unpinned"; restated line by line.
 *   - rms_norm, qk_norm, rope rotation, softmax, silu*mul: the reference has
 *     no op-level test or golden vector -> "parity unpinned" at op level; the
 *     restatement follows the cited lines statement by statement and is
 *     cross-checked against float64 numpy in the tests.
 *   - "normal" (interleaved) RoPE layout, router top-2 and gather-by-expert
 *     do not exist in the reference -> parity unpinned; defined here.
 *
 * The reference is Rust and cannot be compiled in this environment (no Rust
 * toolchain), so there is no oracle/_ref binary.
 *
 * Build: gcc -O2 -ffp-contract=off -fno-fast-math -fopenmp -shared -fPIC
 * (no FMA contraction, strictly sequential f32 accumulation, glibc libm —
 * the same libm Rust's std calls on Linux).
 */
#ifndef AGN_ORACLE_CPU_REF_H
#define AGN_ORACLE_CPU_REF_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* GgmlType discriminants, src/types.rs:9-46 */
enum {
    ORC_F32 = 0,
    ORC_F16 = 1,
    ORC_Q5_0 = 6,
    ORC_Q8_0 = 8,
    ORC_Q2_K = 10,
    ORC_Q4_K = 12,
    ORC_Q5_K = 13,
    ORC_Q6_K = 14,
    ORC_BF16 = 30,
    /* not a GgmlType: the GPU path's Q8_0 cache layout, 36-byte blocks of nine 32-bit words
     * (src/ops/kernels_wgpu.rs:583-698) */
    ORC_KV_Q8_0_WORDS = 1008
};

enum { ORC_OK = 0, ORC_ESHORT = 1, ORC_EROW = 2, ORC_EDTYPE = 3, ORC_ELEN = 4 };

/* layout of the rotated pairs */
enum { ORC_ROPE_NEOX = 0, ORC_ROPE_NORMAL = 1 };

/* src/types.rs:88-168 */
size_t orc_block_size(int dtype);
size_t orc_block_bytes(int dtype);
size_t orc_type_size(int dtype, size_t n);

/* half::f16::to_f32 (exact IEEE binary16 -> binary32) */
float orc_f16_to_f32(uint16_t bits);

/* src/model/llama/cpu_path.rs:34-40.  type_ may be NULL (None).
 * Returns 1 and writes *scale when the reference returns Some, else 0. */
int orc_rope_freq_scale(const char *type_, int has_factor, float factor, float *scale);

/* src/model/llama/cpu_path.rs:67-74, one row */
void orc_rms_norm(const float *x, const float *w, float *out, size_t n, float eps);
/* per-token loop of run_batch, src/model/llama/cpu_path.rs:873-879.
 * threads<=1: the reference's single-threaded loop; >1: OpenMP over rows. */
void orc_rms_norm_rows(const float *x, const float *w, float *out, size_t T, size_t H,
                       float eps, int threads);
/* residual add (cpu_path.rs:785-787) followed by rms_norm (:790) */
void orc_add_residual_rms_norm_rows(const float *x, const float *delta, const float *w,
                                    float *new_x, float *normed, size_t T, size_t H,
                                    float eps, int threads);

/* src/model/llama/cpu_path.rs:78-93, in place, one token */
void orc_qk_norm(float *x, const float *w, size_t n_heads, size_t head_dim, float eps);

/* denominators theta.powf(2d/n_rot) for d < n_rot/2, cpu_path.rs:107-112 / :474-479 */
void orc_rope_denominators(float theta, size_t n_rot, float *denom);

/* src/model/llama/cpu_path.rs:99-133 (n_rot == head_dim) and :461-496 (partial),
 * one token, in place on one buffer of n_heads heads. */
void orc_rope(float *x, size_t n_heads, size_t head_dim, size_t n_rot, int64_t pos,
              float theta, float freq_scale, int layout);
/* rows: token t uses pos[t]; x is [T, n_heads*head_dim] */
void orc_rope_rows(float *x, size_t T, size_t n_heads, size_t head_dim, size_t n_rot,
                   const int32_t *pos, float theta, float freq_scale, int layout,
                   int threads);
/* qk_norm then rope per token (cpu_path.rs:896-906); w may be NULL (no norm) */
void orc_qk_norm_rope_rows(float *x, const float *w, size_t T, size_t n_heads,
                           size_t head_dim, float eps, size_t n_rot, const int32_t *pos,
                           float theta, float freq_scale, int layout, int threads);

/* src/model/llama/cpu_path.rs:175-183, in place over n entries */
void orc_softmax(float *s, size_t n);
/* rows: row r normalises its first n_valid[r] entries (n_valid NULL -> row_len);
 * entries >= n_valid are written as 0 in out. */
void orc_softmax_rows(const float *in, float *out, size_t n_rows, size_t row_len,
                      size_t row_stride, const int32_t *n_valid, int threads);

/* src/model/llama/cpu_path.rs:228-229 and :975-978 */
void orc_silu_mul(const float *gate, const float *up, float *out, size_t n, int threads);

/* src/quant/q4_k.rs:26-35 */
void orc_get_scale_min_k4(size_t j, const uint8_t *scales, uint8_t *sc, uint8_t *m);

/* src/quant/q8_0.rs:14-51, q4_k.rs:37-91, q6_k.rs:34-77, quant/mod.rs:137-170.
 * data_len is the number of readable bytes; returns ORC_ESHORT as the
 * reference returns Err on short data. */
int orc_dequant_q8_0(const uint8_t *data, size_t data_len, size_t n, float *out);
int orc_dequant_q4_k(const uint8_t *data, size_t data_len, size_t n, float *out);
int orc_dequant_q6_k(const uint8_t *data, size_t data_len, size_t n, float *out);
/* src/quant/q5_k.rs:43-103, src/quant/q5_0.rs:20-62 */
int orc_dequant_q5_k(const uint8_t *data, size_t data_len, size_t n, float *out);
int orc_dequant_q5_0(const uint8_t *data, size_t data_len, size_t n, float *out);
/* src/quant/q2_k.rs:30-98: 84-byte super-blocks (the codec's BLOCK_BYTES, :24; the row
 * stride used here is 84 bytes per 256 values, the GGUF file layout, although
 * GgmlType::block_bytes lists 256 for this type, src/types.rs:137).  ORC_ELEN when n is not
 * a multiple of 256, as the reference returns Err (:31-35). */
int orc_dequant_q2_k(const uint8_t *data, size_t data_len, size_t n, float *out);
int orc_dequant_f32(const uint8_t *data, size_t data_len, size_t n, float *out);
int orc_dequant_f16(const uint8_t *data, size_t data_len, size_t n, float *out);
int orc_dequant_bf16(const uint8_t *data, size_t data_len, size_t n, float *out);

/* quant::dequant_row + row_view, src/quant/mod.rs:30-47,97-135, for a 2-D
 * tensor [row_len (dims[0]), n_rows (dims[1])] starting at byte_offset. */
int orc_dequant_row(int dtype, const uint8_t *data, size_t data_len, size_t byte_offset,
                    size_t row_len, size_t n_rows, size_t row, float *out);

/* embedding loop of run_batch, cpu_path.rs:865-868.  Out-of-range ids leave a
 * zero row and make the call return ORC_EROW (after finishing the others). */
int orc_get_rows(int dtype, const uint8_t *table, size_t table_len, size_t n_vocab,
                 size_t row_len, const uint32_t *ids, size_t T, float *out, int threads);

/* KV cache: KvDtype::bytes_per_token / pack / unpack (src/model/mod.rs:550-604),
 * KvCache::write_range (:660-672), read_up_to (:678-697); dtype ORC_F16 or ORC_Q8_0, or
 * ORC_KV_Q8_0_WORDS for the GPU path's 36-byte blocks (kv_cache_write_q8_0 / dequant_kv_q8_0,
 * src/ops/kernels_wgpu.rs:583-718).
 * Parity unpinned: the reference has no test for them. */
size_t orc_kv_bytes_per_token(int dtype, size_t hd);
void orc_kv_pack(int dtype, const float *x, size_t n, uint8_t *out);
void orc_kv_unpack(int dtype, const uint8_t *bytes, size_t n, float *out);
void orc_kv_write_rows(int dtype, const float *x, size_t T, size_t hd, const int32_t *pos, uint8_t *cache);
void orc_kv_read(int dtype, const uint8_t *cache, size_t n_pos, size_t hd, float *out);

/* MoE router (docs/08-moe-routing.md:27-33; not implemented by the reference):
 * probs = softmax(logits row); pick the 2 largest (ties -> lower index);
 * weights are the probabilities, not renormalised. */
void orc_router_top2(const float *logits, size_t T, size_t n_experts, int32_t *idx,
                     float *w);
/* stable counting sort of the 2T (token, expert) pairs by expert, then gather
 * rows of x [T,H] into out [2T,H].  offsets has n_experts+1 entries;
 * src_token[2T] is the token each output row was copied from, src_slot[2T]
 * which of its two picks. */
void orc_gather_rows_by_expert(const float *x, size_t T, size_t H, const int32_t *idx,
                               size_t n_experts, float *out, int32_t *offsets,
                               int32_t *src_token, int32_t *src_slot);

/* Q8_K activation quantisation, quantize_row_q8_k (src/quant/q8_k.rs:49-92): what the matmul of a
 * Q5_K tensor turns its activation vector into before the int8 dot products
 * (WeightMap::matmul_into, src/model/mod.rs:381-386).  Per block of 256 values (the last one
 * zero-padded): the signed value of largest magnitude (first one on ties) -> iscale = -127 / max;
 * q = min(round_half_away(iscale * v) as i32 (saturating, NaN -> 0), 127) as i8 (wrapping);
 * d = 1 / iscale (0 for an all-zero block); bsums[g] = sum of q over group g of 16.
 * Outputs as the parallel arrays of `Q8KRow` (:27-37): d [nb], qs [nb * 256], bsums [nb * 16],
 * nb = ceil(n / 256).  Pinned by the reference's four unit tests (:97-139). */
void orc_quantize_row_q8_k(const float *x, size_t n, float *d, int8_t *qs, int16_t *bsums);
/* rows of length n, row r at x + r * n; outputs row after row */
void orc_quantize_rows_q8_k(const float *x, size_t T, size_t n, float *d, int8_t *qs, int16_t *bsums,
                            int threads);

int orc_max_threads(void);

#ifdef __cplusplus
}
#endif
#endif
