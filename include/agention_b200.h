/*
 * agention_b200 — C ABI of the CUDA (sm_100a) layer-op backend for the gguf-rs
 * engine (LaurentZuijdwijk/agention-infer).
 *
 * This is the boundary a Rust `CudaBackend` binds with `extern "C"`: plain
 * pointers and sizes, int32 status codes, no exceptions, no C++ or torch types.
 * Every op works on T token rows at once (row-major, token-major f32, the
 * layout `run_batch` uses, src/model/llama/cpu_path.rs:854-862); T = 1 with a
 * scalar position reproduces the reference's per-token call.
 *
 * All device pointers are plain CUDA device addresses owned by the caller.
 * Ops are asynchronous on the context's stream and never allocate; only
 * agn_sync / agn_memcpy_d2h(+sync) block.  Calls on one context must be
 * serialised by the caller (the reference's `forward` is not re-entrant either,
 * src/model/llama/mod.rs:340-343); contexts on different GPUs are independent.
 *
 * There is no CPU fallback anywhere behind this ABI: a call either runs the
 * CUDA kernel or returns an error status.
 */
#ifndef AGENTION_B200_H
#define AGENTION_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(_WIN32)
#define AGN_API
#else
#define AGN_API __attribute__((visibility("default")))
#endif

/* ------------------------------------------------------------------ status */

/* Replaces `Result<T, GgufError>` / `GgufError::BackendError(String)`
 * (src/error.rs:3-42); the message is read with agn_last_error. */
typedef enum agn_status {
    AGN_OK = 0,
    AGN_EINVAL = 1,            /* bad argument (null, size, alignment, n_rot > head_dim ...) */
    AGN_EUNSUPPORTED_DTYPE = 2,/* quant type without a kernel ("dequantization not yet
                                  implemented for ..", src/quant/mod.rs:43-45) */
    AGN_ECUDA = 3,             /* a CUDA runtime call failed */
    AGN_EOOB_ID = 4,           /* get_rows met a row index >= n_rows ("row index .. out of
                                  range", src/quant/mod.rs:116-120); that output row is zero */
    AGN_ENOMEM = 5,            /* device or pinned allocation failed */
    AGN_ETIMEOUT = 6,          /* a bounded device-side wait gave up (staging barrier) */
    AGN_EFORMAT = 7,           /* malformed GGUF data (`GgufError::InvalidMagic`, `UnsupportedVersion`,
                                  `UnexpectedEof`, `UnknownMetadataType`, src/error.rs:3-42) */
    AGN_ENOTFOUND = 8,         /* no such metadata key / tensor, or a value of another type */
    AGN_EIO = 9                /* the file cannot be opened or mapped */
} agn_status;

/* GgmlType discriminants accepted by agn_get_rows_f32 (src/types.rs:9-46). */
typedef enum agn_dtype {
    AGN_F32 = 0,
    AGN_F16 = 1,
    AGN_Q5_0 = 6,
    AGN_Q8_0 = 8,
    AGN_Q2_K = 10,
    AGN_Q4_K = 12,
    AGN_Q5_K = 13,
    AGN_Q6_K = 14,
    AGN_BF16 = 30,
    /* not a GgmlType: a KV-cache layout, Q8_0 values in the GPU path's blocks of nine 32-bit words
     * (see agn_kv_write_f32) */
    AGN_KV_Q8_0_WORDS = 1008
} agn_dtype;

/* Pairing of rotated dims: NeoX (d, d + n_rot/2) is what the reference does
 * (src/model/llama/cpu_path.rs:114-132); NORMAL pairs (2d, 2d+1). */
typedef enum agn_rope_layout { AGN_ROPE_NEOX = 0, AGN_ROPE_NORMAL = 1 } agn_rope_layout;

typedef struct agn_ctx agn_ctx;     /* one device + one stream; replaces WgpuBackend's
                                       ComputeClient (src/ops/wgpu_backend/mod.rs) */
typedef struct agn_event agn_event; /* device timestamp on the context's stream */
typedef struct agn_graph agn_graph; /* a recorded chain of ops, replayed with one launch */

/* ----------------------------------------------------------- context, memory */

/* Replaces `create_backend(BackendPreference::Cuda)` whose Cuda arm falls back to
 * CPU today (src/ops/backend_select.rs:84-95).  Fails with AGN_ECUDA when the
 * device is absent; never falls back. */
AGN_API int32_t agn_ctx_create(int32_t device, agn_ctx **out);
AGN_API int32_t agn_ctx_destroy(agn_ctx *ctx);
/* `Backend::name` (src/ops/mod.rs:99): "cuda-sm100a". */
AGN_API const char *agn_backend_name(void);
AGN_API const char *agn_last_error(agn_ctx *ctx);
AGN_API const char *agn_status_string(int32_t status);
/* Use an existing cudaStream_t (e.g. the host framework's) instead of the
 * context's own; pass NULL to return to the own stream.  (NULL therefore does not
 * mean CUDA's legacy default stream; pass cudaStreamLegacy / cudaStreamPerThread
 * explicitly for those.) */
AGN_API int32_t agn_ctx_set_stream(agn_ctx *ctx, void *cuda_stream);
AGN_API int32_t agn_ctx_get_stream(agn_ctx *ctx, void **cuda_stream);
/* Options.  "pdl" (default 1): launch kernels with programmatic stream serialization, so
 * that a kernel's launch latency overlaps the tail of the previous kernel of the stream
 * (every kernel still waits for the previous one to complete before its first access).
 * Tuning knobs, all with measured defaults: "rms_vpt" (1, 2, 4, 8 vectors per thread; 0 = automatic),
 * "rms_recip" (1: one reciprocal per row, 0: IEEE division per element), "silu_unroll" (2, 4, 8),
 * "silu_threads" (128, 256, 512), "silu_small" (1: decode-sized inputs run one vector pair per thread in
 * 128-thread CTAs), "softmax_vpt" (2, 4; 0 = 8), "softmax_cluster" (rows of more than 16384 entries:
 * 1 = one thread-block cluster per row, 2 = the same with smaller CTAs, 0 = one CTA per row),
 * "softmax_causal_pair" (1: square causal matrices of more than 1024 columns run rows i and L-1-i in one
 * CTA), "softmax_warp16" (1: rows of 1025-2048 entries run one warp per row; default 0), "get_rows_tma"
 * (1: bulk-copy staging, 0: cp.async), "get_rows_threads" (32..256; 0 = automatic), "moe_small_sort"
 * (1: up to 4096 (token, slot) pairs are sorted by one CTA in one launch, 0: always the three-kernel
 * counting sort), "host_slots" (2..16 staging slots of the host-slice ops, read when their ring is created;
 * 0 = 8), "host_chunk_bytes" (bytes of one staging chunk; 0 = a whole 24 MiB slot), "rms_q8k_bpw" (blocks
 * of 256 values a warp owns in the fused norm -> Q8_K kernels: 1, 2, 4; 0 = by row length).
 * Persistent kernels that stage rows through a shared-memory ring with bulk asynchronous copies (off by
 * default: the CTA-per-row kernels measured faster on B200): "rms_ring", "rope_ring", "get_rows_ring",
 * "softmax_ring" = 0 (never), 1 (a ring of the default depth for batches large enough to keep it busy) or
 * 2..8 / 2..16 slots; "<op>_ring_ctas" = resident CTAs per SM (0 = as many as fit); "ring_force" = 1 takes the
 * persistent form however small the batch (tests).
 * "mbar_spin_limit" (default 4194304): polls of a staging barrier before a kernel gives up and the next
 * agn_sync returns AGN_ETIMEOUT; "test_idle_barrier_wait" = 1 is a test hook that makes get_rows wait on a
 * barrier nothing signals, so that this path can be exercised without a fault.
 * An unknown name or a value outside the option's range is AGN_EINVAL. */
AGN_API int32_t agn_ctx_set_option(agn_ctx *ctx, const char *name, int64_t value);
/* Launches one empty kernel: the per-launch floor for launch-bound (decode-shaped) timings,
 * the counterpart of the reference's "dispatch floor" probe
 * (docs/PERFORMANCE_RECOMMENDATIONS.md:829). */
AGN_API int32_t agn_launch_noop(agn_ctx *ctx);
/* Number of kernels this context has launched so far. */
AGN_API uint64_t agn_ctx_launch_count(agn_ctx *ctx);
/* Which kernel family the most recent launch of this context took, e.g. "rms_norm" (one CTA per
 * row) or "rms_norm_ring" (persistent CTAs with a staged row ring): a diagnostic for tests and
 * profiling, the counterpart of the kernel names the reference's per-kernel
 * tracing prints (GGUF_TRACE_KERNEL, src/ops/trace.rs).  Never NULL; "" before the first launch. */
AGN_API const char *agn_ctx_last_kernel(agn_ctx *ctx);

/* `client.empty(bytes)` / `client.create_from_slice` / `read_one_unchecked`
 * (src/ops/wgpu_backend/resident.rs:195,673-700). Copies are stream-ordered;
 * host memory from agn_host_alloc is pinned so they are truly asynchronous. */
AGN_API int32_t agn_malloc(agn_ctx *ctx, size_t bytes, void **dptr);
AGN_API int32_t agn_free(agn_ctx *ctx, void *dptr);
AGN_API int32_t agn_host_alloc(agn_ctx *ctx, size_t bytes, void **hptr);
AGN_API int32_t agn_host_free(agn_ctx *ctx, void *hptr);
AGN_API int32_t agn_memcpy_h2d(agn_ctx *ctx, void *dst, const void *src, size_t bytes);
AGN_API int32_t agn_memcpy_d2h(agn_ctx *ctx, void *dst, const void *src, size_t bytes);
AGN_API int32_t agn_memset(agn_ctx *ctx, void *dst, int value, size_t bytes);
/* Blocks until the stream is idle; also reports (once) AGN_EOOB_ID / AGN_ETIMEOUT
 * raised by kernels since the last sync.  Replaces the sync implied by
 * `read_handle` (src/ops/wgpu_backend/resident.rs:696-699). */
AGN_API int32_t agn_sync(agn_ctx *ctx);

/* GPU-time tracing; replaces the host-side `trace::Timer` around each launch_*
 * (src/ops/trace.rs:148-219), which times only the enqueue. */
AGN_API int32_t agn_event_create(agn_ctx *ctx, agn_event **ev);
AGN_API int32_t agn_event_record(agn_ctx *ctx, agn_event *ev);
AGN_API int32_t agn_event_elapsed_ms(agn_ctx *ctx, agn_event *start, agn_event *stop, float *ms);
AGN_API int32_t agn_event_destroy(agn_ctx *ctx, agn_event *ev);

/* CUDA graphs for launch-bound chains (the decode loop: a fixed sequence of small kernels
 * per token).  Ops enqueued between begin and end are recorded, not run; agn_graph_launch
 * replays them on the context's stream for a fraction of a microsecond per kernel.  The
 * reference's counterpart is its queue of asynchronous launches with one final readback
 * (src/model/llama/gpu_resident.rs:427-697).  Run the chain once before capturing it (the
 * RoPE table of a (theta, n_rot) pair is built on first use); agn_sync, allocation and the
 * host-slice entry points are not allowed inside a capture. */
AGN_API int32_t agn_graph_begin(agn_ctx *ctx);
AGN_API int32_t agn_graph_end(agn_ctx *ctx, agn_graph **out);
AGN_API int32_t agn_graph_launch(agn_ctx *ctx, agn_graph *graph);
AGN_API int32_t agn_graph_destroy(agn_ctx *ctx, agn_graph *graph);

/* ---------------------------------------------------------------- layer ops */

/* `LlamaModel::rms_norm_into` (src/model/llama/cpu_path.rs:67-74) over T rows;
 * GPU twin `WgpuBackend::launch_rms_norm` (src/ops/wgpu_backend/resident.rs:213-235).
 * out[t,i] = (w[i] * x[t,i]) / sqrt(sum_i x[t,i]^2 / H + eps).  out may alias x. */
AGN_API int32_t agn_rms_norm_f32(agn_ctx *ctx, const float *x, const float *w, float *out,
                                 int64_t T, int64_t H, float eps);

/* `launch_add_residual_rms_norm` (src/ops/wgpu_backend/resident.rs:240-266); CPU
 * equivalent = residual loop cpu_path.rs:785-787 followed by rms_norm_into :790.
 * new_x = x + delta; normed = rms_norm(new_x, w).  new_x may alias x. */
AGN_API int32_t agn_add_residual_rms_norm_f32(agn_ctx *ctx, const float *x, const float *delta,
                                              const float *w, float *new_x, float *normed,
                                              int64_t T, int64_t H, float eps);

/* `compute_rope_freq_scale` (src/model/llama/cpu_path.rs:34-40), the freq_scale argument of the
 * rope entry points from the model's `rope.scaling.type` / `rope.scaling.factor` metadata:
 * NULL, "" or "none" -> 1; "linear" -> 1 / max(factor, 1e-6) (has_factor = 0: factor 1).
 * AGN_OK with *scale set; AGN_ENOTFOUND for any other scheme (e.g. "yarn": the reference's `None`,
 * "not applied yet" — its caller warns and uses 1.0).  Host arithmetic only; no context. */
AGN_API int32_t agn_rope_freq_scale(const char *scaling_type, int32_t has_factor, float factor, float *scale);

/* `LlamaModel::rope` / `rope_partial` (src/model/llama/cpu_path.rs:99-133,461-496),
 * GPU twin `launch_rope` (src/ops/wgpu_backend/resident.rs:326-353), in place on
 * x [T, n_heads*head_dim].  Token t rotates with position pos[t] (device int32
 * array) or, when pos is NULL, pos_start + t (cpu_path.rs:897).
 * angle(d) = (pos * freq_scale) / powf(theta, 2d/n_rot); the powf table is built
 * once per (theta, n_rot) on the host with libm and cached in the context, so the
 * angle is bit-identical to the CPU path's. */
AGN_API int32_t agn_rope_f32(agn_ctx *ctx, float *x, int64_t T, int32_t n_heads,
                             int32_t head_dim, int32_t n_rot, const int32_t *pos,
                             int32_t pos_start, float theta, float freq_scale,
                             int32_t layout);
/* Same, Q and K in one launch as the CPU `rope(q, k, pos)` does. */
AGN_API int32_t agn_rope_qk_f32(agn_ctx *ctx, float *q, float *k, int64_t T, int32_t n_q_heads,
                                int32_t n_kv_heads, int32_t head_dim, int32_t n_rot,
                                const int32_t *pos, int32_t pos_start, float theta,
                                float freq_scale, int32_t layout);

/* Fused norm->rope: `launch_qk_norm_rope` (src/ops/wgpu_backend/resident.rs:414-443);
 * CPU = `qk_norm` (cpu_path.rs:78-93) then `rope` (:99-133) per token (:896-906).
 * w is [head_dim], shared by all heads.  In place. */
AGN_API int32_t agn_qk_norm_rope_f32(agn_ctx *ctx, float *x, const float *w, int64_t T,
                                     int32_t n_heads, int32_t head_dim, float eps,
                                     int32_t n_rot, const int32_t *pos, int32_t pos_start,
                                     float theta, float freq_scale, int32_t layout);
/* Q (weights wq) and K (weights wk) in one launch. */
AGN_API int32_t agn_qk_norm_rope_qk_f32(agn_ctx *ctx, float *q, float *k, const float *wq,
                                        const float *wk, int64_t T, int32_t n_q_heads,
                                        int32_t n_kv_heads, int32_t head_dim, float eps,
                                        int32_t n_rot, const int32_t *pos, int32_t pos_start,
                                        float theta, float freq_scale, int32_t layout);

/* Fused gate·up -> SiLU·mul: `launch_silu_mul` (src/ops/wgpu_backend/resident.rs:187-209);
 * CPU cpu_path.rs:228-229 and :975-978.  out[i] = gate[i] / (1 + exp(-gate[i])) * up[i].
 * out may alias gate (the CPU batch path writes into gate). */
AGN_API int32_t agn_silu_mul_f32(agn_ctx *ctx, const float *gate, const float *up, float *out,
                                 int64_t n);

/* Row softmax: the softmax step of `attention_into` (src/model/llama/cpu_path.rs:175-183),
 * GPU twin `attention_softmax` (src/ops/kernels_wgpu.rs:795-864).  Row r of
 * in/out [n_rows, row_stride] is normalised over its first nv(r) entries and the
 * entries nv(r)..row_len-1 of out are set to 0:
 *   n_valid != NULL        : nv(r) = n_valid[r]            (device int32 array)
 *   else causal_period > 0 : nv(r) = causal_offset + (r % causal_period) + 1
 *   else                   : nv(r) = row_len
 * (causality is a row length in the reference, never a -inf mask).  out may alias in. */
AGN_API int32_t agn_softmax_rows_f32(agn_ctx *ctx, const float *in, float *out, int64_t n_rows,
                                     int64_t row_len, int64_t row_stride,
                                     const int32_t *n_valid, int32_t causal_period,
                                     int32_t causal_offset);

/* The same step in the form the reference's GPU kernel leaves it (`attention_softmax`,
 * src/ops/kernels_wgpu.rs:795-864; called from `launch_attention`, resident.rs:551-565):
 * weights = exp(s - max) WITHOUT the division, sums[r] = their sum over the valid entries
 * (`attention_output` divides by it, kernels_wgpu.rs:866-898).  Entries past the valid
 * length are written as 0; sums of a row with no valid entry is 0. */
AGN_API int32_t agn_softmax_rows_unnorm_f32(agn_ctx *ctx, const float *in, float *weights, float *sums,
                                            int64_t n_rows, int64_t row_len, int64_t row_stride,
                                            const int32_t *n_valid, int32_t causal_period,
                                            int32_t causal_offset);

/* Softmax of scale * scores in one pass.  The reference's GPU attention stores `dot * scale`,
 * scale = 1 / sqrt(head_dim), from a kernel of its own (`attention_scores`,
 * src/ops/kernels_wgpu.rs:773-782; the CPU path divides by sqrt(head_dim),
 * src/model/llama/cpu_path.rs:172) and runs the softmax over that buffer; with the scale taken
 * here the caller hands over raw dot products.  scale must be positive and finite (AGN_EINVAL
 * otherwise).  sums == NULL: out = normalised probabilities (agn_softmax_rows_f32 of the scaled
 * scores); sums != NULL: out = exp(scale * (s - max)) and sums[r], as
 * agn_softmax_rows_unnorm_f32.  Other arguments as agn_softmax_rows_f32. */
AGN_API int32_t agn_softmax_rows_scaled_f32(agn_ctx *ctx, const float *in, float *out, float *sums,
                                            int64_t n_rows, int64_t row_len, int64_t row_stride,
                                            const int32_t *n_valid, int32_t causal_period,
                                            int32_t causal_offset, float scale);

/* The same with the probabilities stored as f16 (out_dtype = AGN_F16) or bf16 (AGN_BF16), the f32
 * value rounded to nearest even: the operand of a half-precision weights x V product (two thirds
 * of a causal softmax's traffic is the output row).  Scores and sums stay f32; row_stride counts
 * elements of either buffer; out must not alias in (AGN_EINVAL).  No counterpart in the reference,
 * whose attention weights are f32 (src/ops/kernels_wgpu.rs:795-864).  Any other out_dtype:
 * AGN_EUNSUPPORTED_DTYPE. */
AGN_API int32_t agn_softmax_rows_scaled_f32_out16(agn_ctx *ctx, const float *in, void *out, float *sums,
                                                  int64_t n_rows, int64_t row_len, int64_t row_stride,
                                                  const int32_t *n_valid, int32_t causal_period,
                                                  int32_t causal_offset, float scale, int32_t out_dtype);

/* The softmax exactly as the reference's CPU loop leaves its buffer (src/model/llama/cpu_path.rs:168-183:
 * it runs over `scores[..seq_len]` and never touches `scores[seq_len..]`): entries nv(r)..row_len-1
 * of out are NOT written and keep whatever the buffer held, so a causal softmax stores half as much.
 * Everything else as agn_softmax_rows_scaled_f32 (scale 1 for the plain form, sums optional) and,
 * with out_dtype = AGN_F16 / AGN_BF16 instead of AGN_F32, as agn_softmax_rows_scaled_f32_out16. */
AGN_API int32_t agn_softmax_rows_valid_f32(agn_ctx *ctx, const float *in, void *out, float *sums,
                                           int64_t n_rows, int64_t row_len, int64_t row_stride,
                                           const int32_t *n_valid, int32_t causal_period,
                                           int32_t causal_offset, float scale, int32_t out_dtype);

/* Embedding get_rows with inline dequant: `WeightMap::dequant_row`
 * (src/model/mod.rs:343-348) -> `quant::dequant_row` (src/quant/mod.rs:30-47,97-135)
 * -> dequant_q8_0 / dequant_q4_k / dequant_q6_k (src/quant/q8_0.rs:14-51,
 * q4_k.rs:37-91, q6_k.rs:34-77), also dequant_q5_k (q5_k.rs:43-103) and dequant_q5_0
 * (q5_0.rs:20-62), and dequant_q2_k (q2_k.rs:30-98; 84-byte super-blocks as that codec reads
 * them, rows 84 * row_len / 256 bytes apart as in a GGUF file, although GgmlType::block_bytes,
 * src/types.rs:137, lists 256 for the type; row_len must be a multiple of 256, else AGN_EINVAL
 * as q2_k.rs:31-35 returns Err), looped over tokens as cpu_path.rs:865-868 does.
 * table: n_rows rows of type_size(dtype, row_len) bytes each, 16-byte aligned;
 * table_bytes = readable bytes at table; ids: device u32 [T]; out: [T, row_len] f32.
 * Bit-exact with the CPU codecs.  An id >= n_rows zero-fills its row and makes the
 * next agn_sync return AGN_EOOB_ID. */
AGN_API int32_t agn_get_rows_f32(agn_ctx *ctx, int32_t dtype, const void *table,
                                 size_t table_bytes, int64_t n_rows, int64_t row_len,
                                 const uint32_t *ids, int64_t T, float *out);

/* KV-cache write: `KvCache::write` / `write_range` (src/model/mod.rs:648-672) with
 * `KvDtype::pack` (:567-585); GPU twins `kv_cache_write` / `kv_cache_write_q8_0`
 * (src/ops/kernels_wgpu.rs:566-698).  kv_dtype is AGN_F16 or AGN_Q8_0 (`KvDtype`, :536-539: the
 * CPU path's tight 34-byte blocks, f16 scale + 32 int8), or AGN_KV_Q8_0_WORDS for the block the
 * reference's GPU path stores (`kv_cache_write_q8_0`, kernels_wgpu.rs:583-698; `words_per_token`,
 * src/model/llama/gpu_resident.rs:276): nine 32-bit words per 32 values — the scale as f32 bits,
 * then four bytes per word, offset-binary (byte = q + 128) — with the same amax, scale and q as
 * the 34-byte form, values past head_dim_kv in the last block stored as 0 (byte 128), caches
 * 4-byte aligned.
 * k, v: [T, head_dim_kv] f32 (head_dim_kv = n_kv_heads * head_dim); k_cache, v_cache: one
 * layer's [max_seq_len, agn_kv_bytes_per_token] bytes.  Token t goes to slot pos[t] (device
 * int32) or pos_start + t.  Bit-exact with the CPU pack.  A slot outside [0, max_seq_len)
 * is skipped and makes the next agn_sync return AGN_EOOB_ID. */
AGN_API int32_t agn_kv_write_f32(agn_ctx *ctx, int32_t kv_dtype, const float *k, const float *v,
                                 void *k_cache, void *v_cache, int64_t T, int64_t head_dim_kv,
                                 const int32_t *pos, int32_t pos_start, int64_t max_seq_len);
/* `KvCache::read_up_to` (src/model/mod.rs:678-697) with `KvDtype::unpack` (:587-604):
 * dequantises slots [0, n_pos) into k_out, v_out [n_pos, head_dim_kv] f32. */
/* QK-norm -> RoPE of Q and K (in place) and the cache write of the rotated K and of V in one launch:
 * the per-layer sequence `launch_qk_norm_rope` (q), `launch_qk_norm_rope` (k), `kv_cache_write`
 * of the reference's resident path (src/ops/wgpu_backend/resident.rs:414-443,
 * src/ops/kernels_wgpu.rs:566-698).  wq = wk = NULL: rope without the norm.  Arguments as in
 * agn_qk_norm_rope_qk_f32 and agn_kv_write_f32 (head_dim_kv = n_kv_heads * head_dim; token t goes
 * to slot pos[t] or pos_start + t).  Byte for byte the result of those two calls; head sizes the
 * fused kernel does not cover (anything but head_dim 64 / 128 with full or normal-layout rotation)
 * run as those two launches. */
AGN_API int32_t agn_qk_norm_rope_kv_write_f32(agn_ctx *ctx, float *q, float *k, const float *v,
                                              const float *wq, const float *wk, int64_t T,
                                              int32_t n_q_heads, int32_t n_kv_heads, int32_t head_dim,
                                              float eps, int32_t n_rot, const int32_t *pos,
                                              int32_t pos_start, float theta, float freq_scale,
                                              int32_t layout, int32_t kv_dtype, void *k_cache,
                                              void *v_cache, int64_t max_seq_len);
AGN_API int32_t agn_kv_read_f32(agn_ctx *ctx, int32_t kv_dtype, const void *k_cache,
                                const void *v_cache, int64_t n_pos, int64_t head_dim_kv,
                                float *k_out, float *v_out);
/* `KvDtype::bytes_per_token` (src/model/mod.rs:550-556); 0 for an unknown dtype. */
AGN_API int64_t agn_kv_bytes_per_token(int32_t kv_dtype, int64_t head_dim_kv);

/* MoE router: softmax over the n_experts logits of each token and top-2 selection.  The
 * reference has no MoE forward pass; the semantics follow its design notes
 * (docs/08-moe-routing.md:27-33): weights are the softmax probabilities of the two picks,
 * not renormalised; ties go to the lower expert index.  logits [T, n_experts] f32;
 * idx [T, 2] int32; w [T, 2] f32. */
AGN_API int32_t agn_router_top2_f32(agn_ctx *ctx, const float *logits, int64_t T, int32_t n_experts,
                                    int32_t *idx, float *w);

/* Gather of the hidden rows by expert, the step that feeds the per-expert SwiGLU
 * (docs/05-inference-pipeline.md:271-317; not implemented by the reference).  Stable
 * counting sort of the 2T (token, slot) pairs of idx [T, 2] by expert — inside an expert:
 * ascending token, slot 0 before slot 1 — then out[r, :] = x[src_token[r], :].
 * x [T, H]; out [2T, H]; offsets int32 [n_experts + 1] (rows of expert e are
 * offsets[e] .. offsets[e+1]); src_token, src_slot int32 [2T].  All device pointers.
 * Uses the context's workspace; n_experts <= 64.  An expert index outside
 * [0, n_experts) drops that pair and makes the next agn_sync return AGN_EOOB_ID. */
AGN_API int32_t agn_gather_rows_by_expert_f32(agn_ctx *ctx, const float *x, const int32_t *idx,
                                              int64_t T, int64_t H, int32_t n_experts, float *out,
                                              int32_t *offsets, int32_t *src_token,
                                              int32_t *src_slot);

/* ------------------------------------------------- f16 activation storage (`Act = f16`)
 * The reference's GPU path stores activations as f16 by default and computes in f32
 * (`Act`, src/ops/mod.rs:36-45; kernels src/ops/kernels_wgpu.rs:22-31, 79-163, 225-318).
 * These entry points take and return f16 buffers (IEEE binary16, converted with round to
 * nearest even on store); norm weights stay f32; arguments otherwise as in the _f32 forms.
 * For rope: k = NULL with n_kv_heads = 0 for one buffer; wq = wk = NULL skips the norm.
 * Like the reference's f16 kernels, the fused ops round the intermediate (new_x, the
 * normalised head) to f16 before it is used again. */
AGN_API int32_t agn_silu_mul_f16(agn_ctx *ctx, const void *gate, const void *up, void *out, int64_t n);
AGN_API int32_t agn_rms_norm_f16(agn_ctx *ctx, const void *x, const float *w, void *out, int64_t T,
                                 int64_t H, float eps);
AGN_API int32_t agn_add_residual_rms_norm_f16(agn_ctx *ctx, const void *x, const void *delta,
                                              const float *w, void *new_x, void *normed, int64_t T,
                                              int64_t H, float eps);
/* f32 in, 16-bit out.  agn_silu_mul_f32_out16: the f32 result of agn_silu_mul_f32 rounded to
 * nearest even and stored as f16 / bf16, the operand of a half-precision down projection (10
 * instead of 12 bytes per element); no counterpart in the reference, whose `silu_mul` keeps the
 * `Act` type (src/ops/kernels_wgpu.rs:22-31).
 * The norms: f32 rows in, the NORMED row out as f16 (out_dtype = AGN_F16) or bf16 (AGN_BF16): the f32
 * result of agn_rms_norm_f32 / agn_add_residual_rms_norm_f32 rounded to nearest even on store,
 * i.e. the operand a half-precision matmul takes, without an f32 row and a cast pass in
 * between (6 instead of 8 bytes per element, 14 instead of 16 for the residual form).  new_x,
 * the residual stream, stays f32.  No counterpart in the reference, whose norm kernels read and
 * write the same `Act` type (src/ops/kernels_wgpu.rs:79-163).  Any other out_dtype:
 * AGN_EUNSUPPORTED_DTYPE. */
AGN_API int32_t agn_silu_mul_f32_out16(agn_ctx *ctx, const float *gate, const float *up, void *out,
                                       int64_t n, int32_t out_dtype);
AGN_API int32_t agn_rms_norm_f32_out16(agn_ctx *ctx, const float *x, const float *w, void *out,
                                       int64_t T, int64_t H, float eps, int32_t out_dtype);
AGN_API int32_t agn_add_residual_rms_norm_f32_out16(agn_ctx *ctx, const float *x, const float *delta,
                                                    const float *w, float *new_x, void *normed,
                                                    int64_t T, int64_t H, float eps, int32_t out_dtype);

/* ---- Q8_K activation rows: the input of the int8 dot products -------------------------------
 * quantize_row_q8_k (src/quant/q8_k.rs:49-92), which WeightMap::matmul_into applies to the
 * activation vector in front of a Q5_K tensor (src/model/mod.rs:381-386), over T rows of n values.
 * Per block of 256 values (the last block of a row zero-padded): max = the value of largest
 * magnitude (the first one on ties, NaN never), iscale = -127 / max, d = 1 / iscale,
 * q = min(round_half_away(iscale * v) as i32, 127) as i8, bsums[g] = the sum of q over group g of
 * 16; a block without a magnitude above 0 is d = 0, q = 0.  Outputs are the parallel arrays of
 * `Q8KRow` (:27-37), row after row, with nb = agn_q8_k_blocks(n) = ceil(n / 256):
 *   d [T, nb] f32 ; qs [T, nb * 256] int8 ; bsums [T, nb * 16] int16
 * (d and qs 4-byte aligned, bsums 2-byte aligned, else AGN_EINVAL).  Bit-exact against the
 * reference's arithmetic for every input, NaN and infinities included. */
AGN_API int64_t agn_q8_k_blocks(int64_t n);
AGN_API int32_t agn_quantize_rows_q8_k_f32(agn_ctx *ctx, const float *x, int64_t T, int64_t n, float *d,
                                           int8_t *qs, int16_t *bsums);
/* The producers of a matmul's input with the quantiser fused on, so that the f32 row is never
 * written: RMSNorm (agn_rms_norm_f32's arguments), residual add + RMSNorm (new_x, the residual
 * stream, is still written as f32) and SiLU·mul over [T, I] rows.  agn_silu_mul_q8_k_f32 equals
 * agn_quantize_rows_q8_k_f32 applied to agn_silu_mul_f32's result byte for byte; the two norms sum
 * the squares in another order than agn_rms_norm_f32, so their scale factor can differ from its
 * in the last bit, d by as much, and a q by one step in about one position in a thousand.  H and I
 * must be multiples of 256 — a Q5_K weight row is a whole
 * number of 256-value blocks — and H <= 32768; x, delta, new_x, w, gate, up 16-byte aligned;
 * otherwise AGN_EINVAL.  No counterpart in the reference, which normalises into an f32 vector
 * and quantises it inside matmul_into. */
AGN_API int32_t agn_rms_norm_q8_k_f32(agn_ctx *ctx, const float *x, const float *w, int64_t T, int64_t H,
                                      float eps, float *d, int8_t *qs, int16_t *bsums);
AGN_API int32_t agn_add_residual_rms_norm_q8_k_f32(agn_ctx *ctx, const float *x, const float *delta,
                                                   const float *w, float *new_x, int64_t T, int64_t H,
                                                   float eps, float *d, int8_t *qs, int16_t *bsums);
AGN_API int32_t agn_silu_mul_q8_k_f32(agn_ctx *ctx, const float *gate, const float *up, int64_t T,
                                      int64_t I, float *d, int8_t *qs, int16_t *bsums);
AGN_API int32_t agn_rope_qk_f16(agn_ctx *ctx, void *q, void *k, int64_t T, int32_t n_q_heads,
                                int32_t n_kv_heads, int32_t head_dim, int32_t n_rot,
                                const int32_t *pos, int32_t pos_start, float theta, float freq_scale,
                                int32_t layout);
AGN_API int32_t agn_qk_norm_rope_qk_f16(agn_ctx *ctx, void *q, void *k, const float *wq,
                                        const float *wk, int64_t T, int32_t n_q_heads,
                                        int32_t n_kv_heads, int32_t head_dim, float eps, int32_t n_rot,
                                        const int32_t *pos, int32_t pos_start, float theta,
                                        float freq_scale, int32_t layout);
/* get_rows with the output stored as f16 (`act_encode` of the dequantised row,
 * src/ops/mod.rs:47-60): out is [T, row_len] f16. */
AGN_API int32_t agn_get_rows_f16(agn_ctx *ctx, int32_t dtype, const void *table, size_t table_bytes,
                                 int64_t n_rows, int64_t row_len, const uint32_t *ids, int64_t T,
                                 void *out);

/* ------------------------------------------------------- host-slice entry points
 * The same ops for callers whose activations live in HOST memory, as the reference's CPU
 * path does (`rms_norm_into(x: &[f32], w, out: &mut [f32])`, src/model/llama/cpu_path.rs:67;
 * `rope(q, k, pos)` :99; silu·mul :975-978; embedding loop :865-868).  `*_host` arguments are
 * host pointers (pinned memory from agn_host_alloc makes the copies asynchronous), `*_dev`
 * arguments are device pointers to weights / the embedding table, uploaded once.  Rows are
 * streamed through a ring of device staging slots on three streams (upload, kernel,
 * download) so both directions of the PCIe link stay busy.  The ring (96 MiB of device
 * memory) is created by the first host-slice call on a context.  Calls return after
 * enqueueing; host outputs are valid after agn_sync, and host inputs must not be modified
 * before it.  Arguments otherwise as in the device-pointer entry points. */
AGN_API int32_t agn_host_rms_norm_f32(agn_ctx *ctx, const float *x_host, const float *w_dev,
                                      float *out_host, int64_t T, int64_t H, float eps);
/* x_host += delta_host in place (the residual loop, cpu_path.rs:785-787), then the norm of the
 * sum into normed_host (:790). */
AGN_API int32_t agn_host_add_residual_rms_norm_f32(agn_ctx *ctx, float *x_host, const float *delta_host,
                                                   const float *w_dev, float *normed_host, int64_t T,
                                                   int64_t H, float eps);
AGN_API int32_t agn_host_silu_mul_f32(agn_ctx *ctx, const float *gate_host, const float *up_host,
                                      float *out_host, int64_t n);
/* In place on q_host / k_host; pos_host may be NULL (positions pos_start + t). */
AGN_API int32_t agn_host_rope_qk_f32(agn_ctx *ctx, float *q_host, float *k_host, int64_t T,
                                     int32_t n_q_heads, int32_t n_kv_heads, int32_t head_dim,
                                     int32_t n_rot, const int32_t *pos_host, int32_t pos_start,
                                     float theta, float freq_scale, int32_t layout);
AGN_API int32_t agn_host_qk_norm_rope_qk_f32(agn_ctx *ctx, float *q_host, float *k_host,
                                             const float *wq_dev, const float *wk_dev, int64_t T,
                                             int32_t n_q_heads, int32_t n_kv_heads, int32_t head_dim,
                                             float eps, int32_t n_rot, const int32_t *pos_host,
                                             int32_t pos_start, float theta, float freq_scale,
                                             int32_t layout);
/* Dense rows (row_stride == row_len). */
AGN_API int32_t agn_host_softmax_rows_f32(agn_ctx *ctx, const float *in_host, float *out_host,
                                          int64_t n_rows, int64_t row_len,
                                          const int32_t *n_valid_host, int32_t causal_period,
                                          int32_t causal_offset);
AGN_API int32_t agn_host_get_rows_f32(agn_ctx *ctx, int32_t dtype, const void *table_dev,
                                      size_t table_bytes, int64_t n_rows, int64_t row_len,
                                      const uint32_t *ids_host, int64_t T, float *out_host);
/* `quantize_row_q8_k` (src/quant/q8_k.rs:49-92) on host rows: T rows of n values in, the `Q8KRow` arrays
 * out (see agn_quantize_rows_q8_k_f32), bit-exact. */
AGN_API int32_t agn_host_quantize_rows_q8_k_f32(agn_ctx *ctx, const float *x_host, int64_t T, int64_t n,
                                                float *d_host, int8_t *qs_host, int16_t *bsums_host);

/* Allocation-free variant of agn_gather_rows_by_expert_f32.  It has no counterpart in the
 * reference.  It exists for hosts that cannot allocate device memory: one that has given the
 * whole GPU to its own arena (nothing is left for cudaMalloc), or one that must not allocate
 * in its serving loop because cudaMalloc / cudaFree stall all streams of the device.  Such a
 * host cannot create an agn_ctx either (that allocates), so this call takes no context: it
 * works on the CURRENT device, on `cuda_stream` (a cudaStream_t; NULL = the legacy default
 * stream), and its scratch is a 256 KiB array built into the library and resident on every
 * GPU that loads it until the process exits.  It calls no cudaMalloc, cudaFree or allocating
 * library routine.
 *   - Limit: 256 + ceil(2T / 1024) * n_experts * 4 bytes must fit in 256 KiB (8 experts:
 *     T <= 4,190,208); larger problems are rejected with AGN_EINVAL and a message in `err`.
 *   - `cuda_stream` must be a stream of the CURRENT device (the array's address is looked up for
 *     the current device; with a stream of another device the launches fail with AGN_ECUDA).
 *   - The first call on each device looks up the array's device address (cudaGetSymbolAddress)
 *     and keeps it.  With CUDA's lazy module loading that first call is also what loads the
 *     library's device code and gives the array its memory on that device, so make one warm-up
 *     call per device at start-up, before the host's own arena takes the remaining memory and
 *     outside any stream capture: T = 0 is enough (the look-up runs before the T == 0 return).
 *     After it the array stays resident on that device until the process exits.
 *   - All calls share the array and it keeps the previous call's contents; the call itself
 *     clears what has to start at zero.  Two calls whose kernels can overlap on the GPU
 *     (different streams without an event between them) race on it: serialise them.
 *   - An expert index outside [0, n_experts) drops that pair: offsets[n_experts] is then
 *     smaller than 2T and the unused tail of src_token is -1 (no status is raised, because
 *     reading a flag back would need a synchronisation).
 * Arguments and results are otherwise those of agn_gather_rows_by_expert_f32.  `err` (may be
 * NULL) receives a message of at most err_len bytes when the status is not AGN_OK. */
AGN_API int32_t agn_gather_rows_by_expert_noalloc_f32(void *cuda_stream, const float *x,
                                                      const int32_t *idx, int64_t T, int64_t H,
                                                      int32_t n_experts, float *out, int32_t *offsets,
                                                      int32_t *src_token, int32_t *src_slot,
                                                      char *err, size_t err_len);

/* ----------------------------------------------------------------- GGUF files
 * The container side of get_rows: `parser::parse` (src/parser.rs:9-66), `loader::load`
 * (src/loader.rs:14-19, memory-mapped), `GgufFile::get_*` / `MetadataValue::as_*`
 * (src/types.rs), and the upload of a tensor's bytes (`pre_upload_gpu`,
 * src/model/llama/gpu_resident.rs:112-152).  Versions 2 and 3; the data section starts at
 * the next multiple of 32 after the tensor directory.  Array metadata is indexed (element
 * type and count), its elements are not kept.  `err` (may be NULL) receives a message. */
typedef struct agn_gguf agn_gguf;
typedef struct agn_tensor_info {  /* `TensorInfo` (src/types.rs:373-403) plus derived sizes */
    const char *name;      /* lives as long as the agn_gguf */
    int32_t ggml_type;     /* GgmlType id */
    uint32_t n_dims;
    uint64_t dims[4];      /* dims[0] is the contiguous dimension (row length) */
    uint64_t byte_offset;  /* inside the data section */
    uint64_t file_offset;  /* data_offset + byte_offset */
    uint64_t n_rows;       /* product of dims[1..], 1 for a 1-D tensor (src/quant/mod.rs:107-111) */
    uint64_t row_len;      /* dims[0] */
    uint64_t row_bytes;    /* type_size(row_len); 0 when the type has no codec here */
    uint64_t n_bytes;      /* row_bytes * n_rows */
} agn_tensor_info;
AGN_API int32_t agn_gguf_parse(const void *data, size_t len, agn_gguf **out, char *err, size_t err_len);
/* agn_gguf_open on file 1 of a split model ("name-00001-of-0000N.gguf") also maps files 2..N,
 * which hold only tensor data at offsets that run on from the previous file (`MultiFileMmap`,
 * src/loader.rs:40-103); a tensor must lie inside one file to be uploaded. */
AGN_API int32_t agn_gguf_open(const char *path, agn_gguf **out, char *err, size_t err_len);
/* `parse_split_index` (src/loader.rs:25-38): "name-00003-of-00005.gguf" -> index 3, total 5
 * (1-based); AGN_ENOTFOUND when the name does not follow the pattern. */
AGN_API int32_t agn_gguf_split_index(const char *name, uint64_t *index, uint64_t *total);
AGN_API int32_t agn_gguf_close(agn_gguf *g);
AGN_API uint32_t agn_gguf_version(const agn_gguf *g);
AGN_API uint64_t agn_gguf_tensor_count(const agn_gguf *g);
AGN_API uint64_t agn_gguf_metadata_count(const agn_gguf *g);
AGN_API uint64_t agn_gguf_data_offset(const agn_gguf *g);
AGN_API int32_t agn_gguf_get_u64(const agn_gguf *g, const char *key, uint64_t *out);
AGN_API int32_t agn_gguf_get_f32(const agn_gguf *g, const char *key, float *out);
AGN_API int32_t agn_gguf_get_string(const agn_gguf *g, const char *key, const char **out);
/* `GgufFile::get_i64_array` (src/types.rs:451-454): an integer array of any element width as
 * int64 (token types, a per-layer head_count_kv).  *count = array length; at most cap values are
 * written to out (NULL: length only).  AGN_ENOTFOUND if the key is absent or not an integer array. */
AGN_API int32_t agn_gguf_get_array_i64(const agn_gguf *g, const char *key, int64_t *out, uint64_t cap,
                                       uint64_t *count);
AGN_API int32_t agn_gguf_get_array_info(const agn_gguf *g, const char *key, uint32_t *elem_type, uint64_t *count);
AGN_API int32_t agn_gguf_tensor_at(const agn_gguf *g, uint64_t index, agn_tensor_info *out);
AGN_API int32_t agn_gguf_find_tensor(const agn_gguf *g, const char *name, agn_tensor_info *out);
/* Copies the tensor's bytes into a new device allocation (free with agn_free); complete on
 * return.  The result is what agn_get_rows_* takes as `table` (n_rows, row_len from info). */
AGN_API int32_t agn_gguf_upload_tensor(agn_ctx *ctx, const agn_gguf *g, const char *name, void **dptr,
                                       agn_tensor_info *info);
/* The tensor's bytes in host memory, where the mapping (or the caller's buffer) holds them: the slice
 * the reference passes to its codecs (src/quant/mod.rs:97-135).  Valid until agn_gguf_close.
 * AGN_ENOTFOUND, AGN_EUNSUPPORTED_DTYPE (no codec here, size unknown), AGN_EFORMAT (outside the file). */
AGN_API int32_t agn_gguf_tensor_data(const agn_gguf *g, const char *name, const void **data, uint64_t *n_bytes);
/* The upload loop of `pre_upload_gpu` (src/model/llama/gpu_resident.rs:112-152): the n named tensors
 * are copied in ascending file-offset order, whatever order they are named in, and with
 * release_pages != 0 the part of the memory mapping below each uploaded tensor is dropped from
 * the page cache as the loop goes (`release_mmap_prefix`, gpu_resident.rs:29-49: whole pages only,
 * madvise(MADV_DONTNEED); a later access re-reads the page from the file), so a file of about the
 * size of host memory never sits in the page cache next to its copy on the device.  dptrs[i] /
 * infos[i] (infos may be NULL) belong to names[i]; on an error nothing stays allocated.
 * *released_bytes (may be NULL): bytes of page cache given back (0 for an agn_gguf_parse object,
 * whose memory belongs to the caller). */
AGN_API int32_t agn_gguf_upload_tensors(agn_ctx *ctx, const agn_gguf *g, const char *const *names, uint64_t n,
                                        void **dptrs, agn_tensor_info *infos, int32_t release_pages,
                                        uint64_t *released_bytes);
/* The release step alone, for a caller with its own upload loop: whole pages inside the file bytes
 * [from, to) of a mapped file (or of the files of a split model, in their concatenated offsets). */
AGN_API int32_t agn_gguf_release_pages(const agn_gguf *g, uint64_t from, uint64_t to, uint64_t *released_bytes);

/* `GgmlType::type_size` (src/types.rs:164-168); 0 for a dtype without a kernel. */
AGN_API size_t agn_type_size(int32_t dtype, size_t n);

#ifdef __cplusplus
}
#endif
#endif /* AGENTION_B200_H */
