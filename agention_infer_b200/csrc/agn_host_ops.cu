// Host-slice entry points: the layer ops for callers whose activations live in host memory,
// as the reference's CPU path does (`rms_norm_into(x: &[f32], w, out: &mut [f32])`,
// src/model/llama/cpu_path.rs:67; `rope(q, k, pos)` :99; the silu·mul loop :975-978; the
// embedding loop :865-868).  Weights and the embedding table stay on the device (uploaded
// once, like `pre_upload_gpu`, src/model/llama/gpu_resident.rs:69-152).
//
// PCIe, not HBM, bounds this path, so every op is cut into row chunks that flow through
// three streams — host->device copy, kernel, device->host copy — over a ring of staging
// slots, so that the upload of chunk c+1, the kernel of chunk c and the download of chunk
// c-1 run at the same time and both directions of the link stay busy.  Host buffers should
// be pinned (agn_host_alloc) for the copies to be asynchronous; pageable memory works but
// serialises.  Calls return after enqueueing; results are valid after agn_sync.
#include <utility>
#include <vector>

#include "agn_common.cuh"

namespace {

constexpr int PIPE_MAX_SLOTS = 16;
constexpr size_t PIPE_SLOT_BYTES = 24u << 20;  // capacity of one slot
constexpr int MAX_BUFS = 6;

struct HostBuf {
    const void *h_in;   // host source, or nullptr when the buffer is output-only
    void *h_out;        // host destination, or nullptr when the buffer is input-only
    size_t row_bytes;   // bytes per row unit
};

}  // namespace

struct agn_host_pipe {
    cudaStream_t h2d = nullptr, d2h = nullptr;
    unsigned char *stage = nullptr;
    int slots = 0;                  // slots of the ring (option "host_slots" when the ring is created)
    uint64_t next_chunk = 0;        // chunks enqueued so far over all ops: chunk c uses slot c % slots
    cudaEvent_t h2d_done[PIPE_MAX_SLOTS] = {}, k_done[PIPE_MAX_SLOTS] = {}, d2h_done[PIPE_MAX_SLOTS] = {};
    bool slot_used[PIPE_MAX_SLOTS] = {};
    cudaEvent_t op_done = nullptr;  // last device->host copy of the previous host op
    bool join_pending = false;      // the context's stream has not been made to wait for op_done yet
    bool have_prev = false;
    std::vector<std::pair<uintptr_t, uintptr_t>> prev_out;  // host ranges the previous op writes
};

// Makes the context's stream wait for the downloads of the host-slice ops enqueued so far.  Done
// lazily — by agn_sync and agn_event_record, not at the end of every host-slice op — so that the
// kernels of the next host-slice op do not wait for the previous op's last downloads.
int32_t agn_host_pipe_join(agn_ctx *ctx) {
    agn_host_pipe *p = ctx->host_pipe;
    if (!p || !p->join_pending) return AGN_OK;
    AGN_CUDA(ctx, cudaStreamWaitEvent(ctx->stream, p->op_done, 0));
    p->join_pending = false;
    return AGN_OK;
}

void agn_host_pipe_destroy(agn_ctx *ctx) {
    agn_host_pipe *p = ctx->host_pipe;
    if (!p) return;
    if (p->h2d) { cudaStreamSynchronize(p->h2d); cudaStreamDestroy(p->h2d); }
    if (p->d2h) { cudaStreamSynchronize(p->d2h); cudaStreamDestroy(p->d2h); }
    for (int s = 0; s < PIPE_MAX_SLOTS; s++) {
        if (p->h2d_done[s]) cudaEventDestroy(p->h2d_done[s]);
        if (p->k_done[s]) cudaEventDestroy(p->k_done[s]);
        if (p->d2h_done[s]) cudaEventDestroy(p->d2h_done[s]);
    }
    if (p->op_done) cudaEventDestroy(p->op_done);
    if (p->stage) cudaFree(p->stage);
    (void)cudaGetLastError();
    delete p;
    ctx->host_pipe = nullptr;
}

namespace {

// The staging ring (8 slots of 24 MiB of device memory, two streams, events) is created by the first
// host-slice call on a context, not by agn_ctx_create: device-pointer users never pay for it.
int32_t get_pipe(agn_ctx *ctx, agn_host_pipe **out) {
    if (ctx->host_pipe) {
        *out = ctx->host_pipe;
        return AGN_OK;
    }
    agn_host_pipe *p = new agn_host_pipe();
    ctx->host_pipe = p;
    p->slots = ctx->tune_host_slots >= 2 && ctx->tune_host_slots <= PIPE_MAX_SLOTS ? ctx->tune_host_slots : 8;
    bool ok = cudaStreamCreateWithFlags(&p->h2d, cudaStreamNonBlocking) == cudaSuccess &&
              cudaStreamCreateWithFlags(&p->d2h, cudaStreamNonBlocking) == cudaSuccess &&
              cudaEventCreateWithFlags(&p->op_done, cudaEventDisableTiming) == cudaSuccess &&
              cudaMalloc(&p->stage, (size_t)p->slots * PIPE_SLOT_BYTES) == cudaSuccess;
    for (int s = 0; ok && s < p->slots; s++)
        ok = cudaEventCreateWithFlags(&p->h2d_done[s], cudaEventDisableTiming) == cudaSuccess &&
             cudaEventCreateWithFlags(&p->k_done[s], cudaEventDisableTiming) == cudaSuccess &&
             cudaEventCreateWithFlags(&p->d2h_done[s], cudaEventDisableTiming) == cudaSuccess;
    if (!ok) {
        (void)cudaGetLastError();
        agn_host_pipe_destroy(ctx);
        return agn_fail(ctx, AGN_ENOMEM, "host-slice ops: cannot create the staging ring (%zu bytes of device memory)",
                        (size_t)p->slots * PIPE_SLOT_BYTES);
    }
    *out = p;
    return AGN_OK;
}

inline size_t align256(size_t v) { return (v + 255) & ~(size_t)255; }

// Runs `launch(rows, dptr[], row0)` over [0, n_rows) in chunks.  dptr[b] is the device
// staging address of buffer b for the chunk.
template <class F>
int32_t run_pipelined(agn_ctx *ctx, const char *name, int64_t n_rows, const HostBuf *bufs, int nb, F launch,
                      int64_t chunk_multiple = 1) {
    if (n_rows == 0) return AGN_OK;
    if (ctx->capturing) return agn_fail(ctx, AGN_EINVAL, "%s: host-slice ops cannot be recorded into a graph", name);
    agn_host_pipe *p = nullptr;
    int32_t rc = get_pipe(ctx, &p);
    if (rc != AGN_OK) return rc;
    AGN_CUDA(ctx, cudaSetDevice(ctx->device));
    size_t per_row = 0;
    for (int b = 0; b < nb; b++) per_row += bufs[b].row_bytes;
    if (per_row + 256 * (size_t)nb > PIPE_SLOT_BYTES)
        return agn_fail(ctx, AGN_EINVAL, "%s: one row (%zu bytes over all buffers) exceeds a staging slot", name, per_row);
    size_t slot_budget = PIPE_SLOT_BYTES;
    if (ctx->tune_host_chunk_bytes >= (1 << 20) && (size_t)ctx->tune_host_chunk_bytes < slot_budget) slot_budget = (size_t)ctx->tune_host_chunk_bytes;
    if (slot_budget < per_row + 256 * (size_t)nb) slot_budget = per_row + 256 * (size_t)nb;
    int64_t chunk = (int64_t)((slot_budget - 256 * (size_t)nb) / per_row);
    // at least ~8 chunks per op so that the ring actually overlaps the three stages
    const int64_t want = (n_rows + 7) / 8;
    if (chunk > want) {
        // ... but not below ~1 MB per chunk, where launch and copy set-up costs would dominate
        const int64_t floor_rows = (int64_t)(((size_t)1 << 20) / per_row) + 1;
        const int64_t pick = want > floor_rows ? want : floor_rows;
        if (chunk > pick) chunk = pick;
    }
    if (chunk_multiple > 1) {
        // chunks must start on a multiple (a causal softmax period)
        if (chunk < chunk_multiple)
            return agn_fail(ctx, AGN_EINVAL, "%s: %lld rows of %zu bytes do not fit a staging slot", name,
                            (long long)chunk_multiple, per_row);
        chunk -= chunk % chunk_multiple;
    }
    if (chunk < 1) chunk = 1;

    // An input produced by the previous host op's download must not be uploaded before that
    // download has finished.
    if (p->have_prev) {
        bool overlap = false;
        for (int b = 0; b < nb && !overlap; b++) {
            if (!bufs[b].h_in) continue;
            const uintptr_t lo = (uintptr_t)bufs[b].h_in, hi = lo + (size_t)n_rows * bufs[b].row_bytes;
            for (const auto &r : p->prev_out)
                if (lo < r.second && r.first < hi) overlap = true;
        }
        if (overlap) {
            AGN_CUDA(ctx, cudaStreamWaitEvent(p->h2d, p->op_done, 0));
            // A copy from pageable memory reads the host buffer when it is issued, not in
            // stream order, so the wait above does not protect it: block the host instead.
            bool pageable = false;
            for (int b = 0; b < nb; b++) {
                if (!bufs[b].h_in) continue;
                cudaPointerAttributes attr;
                if (cudaPointerGetAttributes(&attr, bufs[b].h_in) != cudaSuccess) {
                    (void)cudaGetLastError();
                    pageable = true;
                } else if (attr.type != cudaMemoryTypeHost) {
                    pageable = true;
                }
            }
            if (pageable) AGN_CUDA(ctx, cudaEventSynchronize(p->op_done));
        }
    }

    int c = 0;
    for (int64_t row0 = 0; row0 < n_rows; row0 += chunk, c++) {
        const int64_t rows = n_rows - row0 < chunk ? n_rows - row0 : chunk;
        // the ring position runs on from op to op: the next chunk takes the slot whose previous
        // contents are the oldest, so an upload runs ahead of the downloads by a whole ring of chunks
        const int s = (int)(p->next_chunk++ % (uint64_t)p->slots);
        unsigned char *slot = p->stage + (size_t)s * PIPE_SLOT_BYTES;
        void *dptr[MAX_BUFS];
        size_t off = 0;
        for (int b = 0; b < nb; b++) {
            dptr[b] = slot + off;
            off += align256((size_t)chunk * bufs[b].row_bytes);
        }
        // the slot is free once its previous outputs have been copied out
        if (p->slot_used[s]) AGN_CUDA(ctx, cudaStreamWaitEvent(p->h2d, p->d2h_done[s], 0));
        for (int b = 0; b < nb; b++)
            if (bufs[b].h_in)
                AGN_CUDA(ctx, cudaMemcpyAsync(dptr[b], (const unsigned char *)bufs[b].h_in + (size_t)row0 * bufs[b].row_bytes,
                                              (size_t)rows * bufs[b].row_bytes, cudaMemcpyHostToDevice, p->h2d));
        AGN_CUDA(ctx, cudaEventRecord(p->h2d_done[s], p->h2d));
        AGN_CUDA(ctx, cudaStreamWaitEvent(ctx->stream, p->h2d_done[s], 0));
        rc = launch(rows, dptr, row0);
        if (rc != AGN_OK) return rc;
        AGN_CUDA(ctx, cudaEventRecord(p->k_done[s], ctx->stream));
        AGN_CUDA(ctx, cudaStreamWaitEvent(p->d2h, p->k_done[s], 0));
        for (int b = 0; b < nb; b++)
            if (bufs[b].h_out)
                AGN_CUDA(ctx, cudaMemcpyAsync((unsigned char *)bufs[b].h_out + (size_t)row0 * bufs[b].row_bytes, dptr[b],
                                              (size_t)rows * bufs[b].row_bytes, cudaMemcpyDeviceToHost, p->d2h));
        AGN_CUDA(ctx, cudaEventRecord(p->d2h_done[s], p->d2h));
        p->slot_used[s] = true;
    }
    // agn_sync / agn_event_record make the context's stream wait for this (agn_host_pipe_join)
    AGN_CUDA(ctx, cudaEventRecord(p->op_done, p->d2h));
    p->join_pending = true;
    p->prev_out.clear();
    for (int b = 0; b < nb; b++)
        if (bufs[b].h_out)
            p->prev_out.emplace_back((uintptr_t)bufs[b].h_out, (uintptr_t)bufs[b].h_out + (size_t)n_rows * bufs[b].row_bytes);
    p->have_prev = true;
    return AGN_OK;
}

}  // namespace

extern "C" {

int32_t agn_host_rms_norm_f32(agn_ctx *ctx, const float *x_host, const float *w_dev, float *out_host, int64_t T, int64_t H,
                              float eps) {
    AGN_CHECK_CTX(ctx);
    if (T < 0 || H <= 0) return agn_fail(ctx, AGN_EINVAL, "host_rms_norm: T=%lld H=%lld", (long long)T, (long long)H);
    if (T > 0 && (!x_host || !w_dev || !out_host)) return agn_fail(ctx, AGN_EINVAL, "host_rms_norm: null pointer");
    const HostBuf bufs[2] = {{x_host, nullptr, sizeof(float) * (size_t)H}, {nullptr, out_host, sizeof(float) * (size_t)H}};
    return run_pipelined(ctx, "host_rms_norm", T, bufs, 2, [&](int64_t rows, void **d, int64_t) {
        return agn_rms_norm_f32(ctx, (const float *)d[0], w_dev, (float *)d[1], rows, H, eps);
    });
}

// The residual loop `x[i] += delta[i]` (src/model/llama/cpu_path.rs:785-787) followed by
// `rms_norm_into(x, w, normed)` (:790): x_host is updated in place, like the CPU path's x.
int32_t agn_host_add_residual_rms_norm_f32(agn_ctx *ctx, float *x_host, const float *delta_host, const float *w_dev,
                                           float *normed_host, int64_t T, int64_t H, float eps) {
    AGN_CHECK_CTX(ctx);
    if (T < 0 || H <= 0) return agn_fail(ctx, AGN_EINVAL, "host_add_residual_rms_norm: T=%lld H=%lld", (long long)T, (long long)H);
    if (T > 0 && (!x_host || !delta_host || !w_dev || !normed_host))
        return agn_fail(ctx, AGN_EINVAL, "host_add_residual_rms_norm: null pointer");
    const HostBuf bufs[3] = {{x_host, x_host, sizeof(float) * (size_t)H}, {delta_host, nullptr, sizeof(float) * (size_t)H},
                             {nullptr, normed_host, sizeof(float) * (size_t)H}};
    return run_pipelined(ctx, "host_add_residual_rms_norm", T, bufs, 3, [&](int64_t rows, void **d, int64_t) {
        return agn_add_residual_rms_norm_f32(ctx, (const float *)d[0], (const float *)d[1], w_dev, (float *)d[0], (float *)d[2],
                                             rows, H, eps);
    });
}

int32_t agn_host_silu_mul_f32(agn_ctx *ctx, const float *gate_host, const float *up_host, float *out_host, int64_t n) {
    AGN_CHECK_CTX(ctx);
    if (n < 0) return agn_fail(ctx, AGN_EINVAL, "host_silu_mul: n=%lld", (long long)n);
    if (n > 0 && (!gate_host || !up_host || !out_host)) return agn_fail(ctx, AGN_EINVAL, "host_silu_mul: null pointer");
    // elementwise: a "row" is a run of 4096 elements; the tail goes in a last short call
    const int64_t RUN = 4096;
    const int64_t full = n / RUN;
    const HostBuf bufs[3] = {{gate_host, nullptr, sizeof(float) * RUN}, {up_host, nullptr, sizeof(float) * RUN},
                             {nullptr, out_host, sizeof(float) * RUN}};
    int32_t rc = run_pipelined(ctx, "host_silu_mul", full, bufs, 3, [&](int64_t rows, void **d, int64_t) {
        return agn_silu_mul_f32(ctx, (const float *)d[0], (const float *)d[1], (float *)d[2], rows * RUN);
    });
    if (rc != AGN_OK) return rc;
    const int64_t rest = n - full * RUN;
    if (rest > 0) {
        const size_t o = (size_t)full * RUN;
        const HostBuf tail[3] = {{gate_host + o, nullptr, sizeof(float) * (size_t)rest},
                                 {up_host + o, nullptr, sizeof(float) * (size_t)rest},
                                 {nullptr, out_host + o, sizeof(float) * (size_t)rest}};
        rc = run_pipelined(ctx, "host_silu_mul", 1, tail, 3, [&](int64_t, void **d, int64_t) {
            return agn_silu_mul_f32(ctx, (const float *)d[0], (const float *)d[1], (float *)d[2], rest);
        });
    }
    return rc;
}

int32_t agn_host_qk_norm_rope_qk_f32(agn_ctx *ctx, float *q_host, float *k_host, const float *wq_dev, const float *wk_dev,
                                     int64_t T, int32_t n_q_heads, int32_t n_kv_heads, int32_t head_dim, float eps,
                                     int32_t n_rot, const int32_t *pos_host, int32_t pos_start, float theta,
                                     float freq_scale, int32_t layout) {
    AGN_CHECK_CTX(ctx);
    if (T < 0 || n_q_heads < 0 || n_kv_heads < 0 || n_q_heads + n_kv_heads <= 0 || head_dim <= 0)
        return agn_fail(ctx, AGN_EINVAL, "host rope: T=%lld heads=%d+%d head_dim=%d", (long long)T, n_q_heads, n_kv_heads, head_dim);
    if (T > 0 && ((n_q_heads > 0 && !q_host) || (n_kv_heads > 0 && !k_host)))
        return agn_fail(ctx, AGN_EINVAL, "host rope: null activation pointer");
    const bool norm = wq_dev != nullptr || wk_dev != nullptr;
    HostBuf bufs[3];
    int nb = 0, iq = -1, ik = -1, ip = -1;
    if (n_q_heads > 0) { iq = nb; bufs[nb++] = {q_host, q_host, sizeof(float) * (size_t)n_q_heads * head_dim}; }
    if (n_kv_heads > 0) { ik = nb; bufs[nb++] = {k_host, k_host, sizeof(float) * (size_t)n_kv_heads * head_dim}; }
    if (pos_host) { ip = nb; bufs[nb++] = {pos_host, nullptr, sizeof(int32_t)}; }
    return run_pipelined(ctx, "host rope", T, bufs, nb, [&](int64_t rows, void **d, int64_t row0) {
        float *dq = iq >= 0 ? (float *)d[iq] : nullptr;
        float *dk = ik >= 0 ? (float *)d[ik] : nullptr;
        const int32_t *dp = ip >= 0 ? (const int32_t *)d[ip] : nullptr;
        const int32_t ps = pos_start + (int32_t)row0;
        if (norm)
            return agn_qk_norm_rope_qk_f32(ctx, dq, dk, wq_dev, wk_dev, rows, n_q_heads, n_kv_heads, head_dim, eps, n_rot, dp,
                                           ps, theta, freq_scale, layout);
        return agn_rope_qk_f32(ctx, dq, dk, rows, n_q_heads, n_kv_heads, head_dim, n_rot, dp, ps, theta, freq_scale, layout);
    });
}

int32_t agn_host_rope_qk_f32(agn_ctx *ctx, float *q_host, float *k_host, int64_t T, int32_t n_q_heads, int32_t n_kv_heads,
                             int32_t head_dim, int32_t n_rot, const int32_t *pos_host, int32_t pos_start, float theta,
                             float freq_scale, int32_t layout) {
    return agn_host_qk_norm_rope_qk_f32(ctx, q_host, k_host, nullptr, nullptr, T, n_q_heads, n_kv_heads, head_dim, 0.0f, n_rot,
                                        pos_host, pos_start, theta, freq_scale, layout);
}

int32_t agn_host_softmax_rows_f32(agn_ctx *ctx, const float *in_host, float *out_host, int64_t n_rows, int64_t row_len,
                                  const int32_t *n_valid_host, int32_t causal_period, int32_t causal_offset) {
    AGN_CHECK_CTX(ctx);
    if (n_rows < 0 || row_len <= 0) return agn_fail(ctx, AGN_EINVAL, "host_softmax_rows: n_rows=%lld row_len=%lld", (long long)n_rows, (long long)row_len);
    if (n_rows > 0 && (!in_host || !out_host)) return agn_fail(ctx, AGN_EINVAL, "host_softmax_rows: null pointer");
    HostBuf bufs[3] = {{in_host, nullptr, sizeof(float) * (size_t)row_len}, {nullptr, out_host, sizeof(float) * (size_t)row_len}, {}};
    int nb = 2;
    if (n_valid_host) bufs[nb++] = {n_valid_host, nullptr, sizeof(int32_t)};
    // the valid length of a row follows its index modulo the causal period, so chunks start
    // on multiples of the period
    const int64_t multiple = (!n_valid_host && causal_period > 0) ? causal_period : 1;
    return run_pipelined(ctx, "host_softmax_rows", n_rows, bufs, nb, [&](int64_t rows, void **d, int64_t) {
        return agn_softmax_rows_f32(ctx, (const float *)d[0], (float *)d[1], rows, row_len, row_len,
                                    n_valid_host ? (const int32_t *)d[2] : nullptr, causal_period, causal_offset);
    }, multiple);
}

int32_t agn_host_get_rows_f32(agn_ctx *ctx, int32_t dtype, const void *table_dev, size_t table_bytes, int64_t n_rows,
                              int64_t row_len, const uint32_t *ids_host, int64_t T, float *out_host) {
    AGN_CHECK_CTX(ctx);
    if (T < 0 || row_len <= 0) return agn_fail(ctx, AGN_EINVAL, "host_get_rows: T=%lld row_len=%lld", (long long)T, (long long)row_len);
    if (T > 0 && (!ids_host || !out_host)) return agn_fail(ctx, AGN_EINVAL, "host_get_rows: null pointer");
    const HostBuf bufs[2] = {{ids_host, nullptr, sizeof(uint32_t)}, {nullptr, out_host, sizeof(float) * (size_t)row_len}};
    return run_pipelined(ctx, "host_get_rows", T, bufs, 2, [&](int64_t rows, void **d, int64_t) {
        return agn_get_rows_f32(ctx, dtype, table_dev, table_bytes, n_rows, row_len, (const uint32_t *)d[0], rows, (float *)d[1]);
    });
}

// `quantize_row_q8_k(x)` at the top of `WeightMap::matmul_into` (src/model/mod.rs:381-386) for a
// caller whose activations live in host memory: T host rows of n values in, the three `Q8KRow`
// arrays (src/quant/q8_k.rs:27-37) out, row after row.
int32_t agn_host_quantize_rows_q8_k_f32(agn_ctx *ctx, const float *x_host, int64_t T, int64_t n, float *d_host, int8_t *qs_host,
                                        int16_t *bsums_host) {
    AGN_CHECK_CTX(ctx);
    if (T < 0 || n <= 0) return agn_fail(ctx, AGN_EINVAL, "host_quantize_rows_q8_k: T=%lld n=%lld", (long long)T, (long long)n);
    if (T > 0 && (!x_host || !d_host || !qs_host || !bsums_host)) return agn_fail(ctx, AGN_EINVAL, "host_quantize_rows_q8_k: null pointer");
    const size_t nb = (size_t)agn_q8_k_blocks(n);
    const HostBuf bufs[4] = {{x_host, nullptr, sizeof(float) * (size_t)n}, {nullptr, d_host, sizeof(float) * nb},
                             {nullptr, qs_host, 256 * nb}, {nullptr, bsums_host, sizeof(int16_t) * 16 * nb}};
    return run_pipelined(ctx, "host_quantize_rows_q8_k", T, bufs, 4, [&](int64_t rows, void **d, int64_t) {
        return agn_quantize_rows_q8_k_f32(ctx, (const float *)d[0], rows, n, (float *)d[1], (int8_t *)d[2], (int16_t *)d[3]);
    });
}

}  // extern "C"
