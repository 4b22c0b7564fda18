// C++ host-side mirror of the reference's GPU operator surface over the C ABI.
//
// `agn::CudaBackend` has the method names and argument meaning of the reference's
// `WgpuBackend::launch_*` family (src/ops/wgpu_backend/resident.rs:187-443), extended from
// one token vector per call to T token rows per call, plus `dequant_row`
// (`WeightMap::dequant_row`, src/model/mod.rs:343-348).  Header-only; link libagention_b200.so.
// Errors (the reference's `GgufError::BackendError`, src/error.rs:37-38) are thrown as
// `agn::BackendError`.  There is no CPU fallback: construction throws without a CUDA device.
#pragma once

#include <cstdint>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "agention_b200.h"

namespace agn {

class BackendError : public std::runtime_error {
  public:
    BackendError(int32_t status, const std::string &msg) : std::runtime_error(msg), status(status) {}
    int32_t status;
};

class CudaBackend;

// A device allocation owned by a backend (the role of a cubecl `Handle`).
class DeviceBuffer {
  public:
    DeviceBuffer() = default;
    DeviceBuffer(agn_ctx *ctx, void *p, size_t n) : ctx_(ctx), ptr_(p), bytes_(n) {}
    DeviceBuffer(const DeviceBuffer &) = delete;
    DeviceBuffer &operator=(const DeviceBuffer &) = delete;
    DeviceBuffer(DeviceBuffer &&o) noexcept { *this = std::move(o); }
    DeviceBuffer &operator=(DeviceBuffer &&o) noexcept {
        if (this != &o) {
            release();
            ctx_ = o.ctx_; ptr_ = o.ptr_; bytes_ = o.bytes_;
            o.ptr_ = nullptr; o.bytes_ = 0;
        }
        return *this;
    }
    ~DeviceBuffer() { release(); }
    template <typename T> T *as() const { return static_cast<T *>(ptr_); }
    void *ptr() const { return ptr_; }
    size_t bytes() const { return bytes_; }

  private:
    void release() {
        if (ptr_) agn_free(ctx_, ptr_);
        ptr_ = nullptr;
    }
    agn_ctx *ctx_ = nullptr;
    void *ptr_ = nullptr;
    size_t bytes_ = 0;
};

class CudaBackend {
  public:
    // `create_backend(BackendPreference::Cuda)` (src/ops/backend_select.rs:60-108), without the CPU fallback.
    explicit CudaBackend(int device = 0) {
        const int32_t st = agn_ctx_create(device, &ctx_);
        if (st != AGN_OK) throw BackendError(st, std::string("no usable CUDA device: ") + agn_status_string(st));
    }
    CudaBackend(const CudaBackend &) = delete;
    CudaBackend &operator=(const CudaBackend &) = delete;
    ~CudaBackend() { if (ctx_) agn_ctx_destroy(ctx_); }

    const char *name() const { return agn_backend_name(); }  // Backend::name, src/ops/mod.rs:99
    agn_ctx *ctx() const { return ctx_; }
    uint64_t launch_count() const { return agn_ctx_launch_count(ctx_); }
    // kernel family of the most recent launch (a diagnostic; see agn_ctx_last_kernel)
    std::string last_kernel() const { return agn_ctx_last_kernel(ctx_); }
    void sync() { check(agn_sync(ctx_)); }

    DeviceBuffer empty(size_t bytes) {  // client.empty, resident.rs:195
        void *p = nullptr;
        check(agn_malloc(ctx_, bytes ? bytes : 1, &p));
        return DeviceBuffer(ctx_, p, bytes);
    }
    template <typename T> DeviceBuffer upload(const std::vector<T> &host) {  // upload_act, resident.rs:673-690
        DeviceBuffer b = empty(host.size() * sizeof(T));
        check(agn_memcpy_h2d(ctx_, b.ptr(), host.data(), host.size() * sizeof(T)));
        sync();
        return b;
    }
    template <typename T> std::vector<T> read(const DeviceBuffer &b, size_t count) {  // read_handle, resident.rs:696-699
        std::vector<T> host(count);
        check(agn_memcpy_d2h(ctx_, host.data(), b.ptr(), count * sizeof(T)));
        sync();
        return host;
    }

    // launch_rms_norm(x, weight, len, eps) -> Handle   (resident.rs:213-235), T rows
    DeviceBuffer launch_rms_norm(const float *x, const float *w, int64_t T, int64_t H, float eps) {
        DeviceBuffer out = empty(sizeof(float) * T * H);
        check(agn_rms_norm_f32(ctx_, x, w, out.as<float>(), T, H, eps));
        return out;
    }
    // launch_add_residual_rms_norm(..) -> (new_x, normed)   (resident.rs:240-266)
    std::pair<DeviceBuffer, DeviceBuffer> launch_add_residual_rms_norm(const float *x, const float *delta, const float *w,
                                                                        int64_t T, int64_t H, float eps) {
        DeviceBuffer nx = empty(sizeof(float) * T * H), nm = empty(sizeof(float) * T * H);
        check(agn_add_residual_rms_norm_f32(ctx_, x, delta, w, nx.as<float>(), nm.as<float>(), T, H, eps));
        return {std::move(nx), std::move(nm)};
    }
    // launch_rope(handle, n_heads, head_dim, n_rot, pos, theta) in place   (resident.rs:326-353)
    void launch_rope(float *x, int64_t T, int n_heads, int head_dim, int n_rot, const int32_t *pos, int pos_start,
                     float theta, float freq_scale = 1.0f, int layout = AGN_ROPE_NEOX) {
        check(agn_rope_f32(ctx_, x, T, n_heads, head_dim, n_rot, pos, pos_start, theta, freq_scale, layout));
    }
    // CPU rope(q, k, pos)   (src/model/llama/cpu_path.rs:99-133): both buffers, one launch
    void launch_rope_qk(float *q, float *k, int64_t T, int n_q, int n_kv, int head_dim, int n_rot, const int32_t *pos,
                        int pos_start, float theta, float freq_scale = 1.0f, int layout = AGN_ROPE_NEOX) {
        check(agn_rope_qk_f32(ctx_, q, k, T, n_q, n_kv, head_dim, n_rot, pos, pos_start, theta, freq_scale, layout));
    }
    // launch_qk_norm_rope(handle, weight, n_heads, head_dim, eps, n_rot, pos, theta)   (resident.rs:414-443)
    void launch_qk_norm_rope(float *x, const float *w, int64_t T, int n_heads, int head_dim, float eps, int n_rot,
                             const int32_t *pos, int pos_start, float theta, float freq_scale = 1.0f,
                             int layout = AGN_ROPE_NEOX) {
        check(agn_qk_norm_rope_f32(ctx_, x, w, T, n_heads, head_dim, eps, n_rot, pos, pos_start, theta, freq_scale, layout));
    }
    void launch_qk_norm_rope_qk(float *q, float *k, const float *wq, const float *wk, int64_t T, int n_q, int n_kv,
                                int head_dim, float eps, int n_rot, const int32_t *pos, int pos_start, float theta,
                                float freq_scale = 1.0f, int layout = AGN_ROPE_NEOX) {
        check(agn_qk_norm_rope_qk_f32(ctx_, q, k, wq, wk, T, n_q, n_kv, head_dim, eps, n_rot, pos, pos_start, theta,
                                      freq_scale, layout));
    }
    // launch_silu_mul(gate, up, len) -> Handle   (resident.rs:187-209)
    DeviceBuffer launch_silu_mul(const float *gate, const float *up, int64_t n) {
        DeviceBuffer out = empty(sizeof(float) * n);
        check(agn_silu_mul_f32(ctx_, gate, up, out.as<float>(), n));
        return out;
    }
    // softmax step of launch_attention   (resident.rs:551-565; cpu_path.rs:175-183), normalised
    DeviceBuffer launch_softmax_rows(const float *scores, int64_t n_rows, int64_t row_len, const int32_t *n_valid,
                                     int causal_period = 0, int causal_offset = 0) {
        DeviceBuffer out = empty(sizeof(float) * n_rows * row_len);
        check(agn_softmax_rows_f32(ctx_, scores, out.as<float>(), n_rows, row_len, row_len, n_valid, causal_period,
                                   causal_offset));
        return out;
    }
    // embedding loop of run_batch   (cpu_path.rs:865-868)
    DeviceBuffer get_rows(int dtype, const void *table, size_t table_bytes, int64_t n_rows, int64_t row_len,
                          const uint32_t *ids, int64_t T) {
        DeviceBuffer out = empty(sizeof(float) * T * row_len);
        check(agn_get_rows_f32(ctx_, dtype, table, table_bytes, n_rows, row_len, ids, T, out.as<float>()));
        return out;
    }
    // WeightMap::dequant_row(name, row) -> Result<Vec<f32>>   (src/model/mod.rs:343-348)
    std::vector<float> dequant_row(int dtype, const void *table, size_t table_bytes, int64_t n_rows, int64_t row_len,
                                   uint32_t row) {
        DeviceBuffer id = upload(std::vector<uint32_t>{row});
        DeviceBuffer out = get_rows(dtype, table, table_bytes, n_rows, row_len, id.as<uint32_t>(), 1);
        return read<float>(out, (size_t)row_len);  // sync inside throws on an out-of-range row
    }

    // ---- f16 activation storage (`Act = f16`, src/ops/mod.rs:36-45): buffers are IEEE binary16
    DeviceBuffer launch_silu_mul_f16(const void *gate, const void *up, int64_t n) {
        DeviceBuffer out = empty(2 * (size_t)n);
        check(agn_silu_mul_f16(ctx_, gate, up, out.ptr(), n));
        return out;
    }
    DeviceBuffer launch_rms_norm_f16(const void *x, const float *w, int64_t T, int64_t H, float eps) {
        DeviceBuffer out = empty(2 * (size_t)(T * H));
        check(agn_rms_norm_f16(ctx_, x, w, out.ptr(), T, H, eps));
        return out;
    }
    DeviceBuffer launch_silu_mul_out16(const float *gate, const float *up, int64_t n, int out_dtype) {
        DeviceBuffer out = empty(2 * (size_t)n);
        check(agn_silu_mul_f32_out16(ctx_, gate, up, out.ptr(), n, out_dtype));
        return out;
    }
    // f32 rows in, normed rows out as f16 / bf16 (out_dtype = AGN_F16 | AGN_BF16)
    DeviceBuffer launch_rms_norm_out16(const float *x, const float *w, int64_t T, int64_t H, float eps, int out_dtype) {
        DeviceBuffer out = empty(2 * (size_t)(T * H));
        check(agn_rms_norm_f32_out16(ctx_, x, w, out.ptr(), T, H, eps, out_dtype));
        return out;
    }
    std::pair<DeviceBuffer, DeviceBuffer> launch_add_residual_rms_norm_out16(const float *x, const float *delta, const float *w,
                                                                             int64_t T, int64_t H, float eps, int out_dtype) {
        DeviceBuffer new_x = empty(4 * (size_t)(T * H)), normed = empty(2 * (size_t)(T * H));
        check(agn_add_residual_rms_norm_f32_out16(ctx_, x, delta, w, static_cast<float *>(new_x.ptr()), normed.ptr(), T, H, eps,
                                                  out_dtype));
        return {std::move(new_x), std::move(normed)};
    }
    // ---- Q8_K activation rows (quantize_row_q8_k, src/quant/q8_k.rs:49-92): d f32, qs i8, bsums i16 per row
    struct Q8KRows {
        DeviceBuffer d, qs, bsums;
    };
    Q8KRows launch_quantize_rows_q8_k(const float *x, int64_t T, int64_t n) {
        Q8KRows r = q8k_rows(T, n);
        check(agn_quantize_rows_q8_k_f32(ctx_, x, T, n, static_cast<float *>(r.d.ptr()), static_cast<int8_t *>(r.qs.ptr()),
                                         static_cast<int16_t *>(r.bsums.ptr())));
        return r;
    }
    // the producers of a Q5_K matmul's input with the quantiser fused on (no f32 row in between)
    Q8KRows launch_rms_norm_q8_k(const float *x, const float *w, int64_t T, int64_t H, float eps) {
        Q8KRows r = q8k_rows(T, H);
        check(agn_rms_norm_q8_k_f32(ctx_, x, w, T, H, eps, static_cast<float *>(r.d.ptr()), static_cast<int8_t *>(r.qs.ptr()),
                                    static_cast<int16_t *>(r.bsums.ptr())));
        return r;
    }
    std::pair<DeviceBuffer, Q8KRows> launch_add_residual_rms_norm_q8_k(const float *x, const float *delta, const float *w,
                                                                       int64_t T, int64_t H, float eps) {
        DeviceBuffer new_x = empty(4 * (size_t)(T * H));
        Q8KRows r = q8k_rows(T, H);
        check(agn_add_residual_rms_norm_q8_k_f32(ctx_, x, delta, w, static_cast<float *>(new_x.ptr()), T, H, eps,
                                                 static_cast<float *>(r.d.ptr()), static_cast<int8_t *>(r.qs.ptr()),
                                                 static_cast<int16_t *>(r.bsums.ptr())));
        return {std::move(new_x), std::move(r)};
    }
    Q8KRows launch_silu_mul_q8_k(const float *gate, const float *up, int64_t T, int64_t I) {
        Q8KRows r = q8k_rows(T, I);
        check(agn_silu_mul_q8_k_f32(ctx_, gate, up, T, I, static_cast<float *>(r.d.ptr()), static_cast<int8_t *>(r.qs.ptr()),
                                    static_cast<int16_t *>(r.bsums.ptr())));
        return r;
    }
    // softmax of scale * scores; sums != nullptr: unnormalised weights + row sums
    void launch_softmax_rows_scaled(const float *in, float *out, float *sums, int64_t n_rows, int64_t row_len, int64_t row_stride,
                                    const int32_t *n_valid, int causal_period, int causal_offset, float scale) {
        check(agn_softmax_rows_scaled_f32(ctx_, in, out, sums, n_rows, row_len, row_stride, n_valid, causal_period, causal_offset,
                                          scale));
    }
    void launch_softmax_rows_scaled_out16(const float *in, void *out, float *sums, int64_t n_rows, int64_t row_len,
                                          int64_t row_stride, const int32_t *n_valid, int causal_period, int causal_offset,
                                          float scale, int out_dtype) {
        check(agn_softmax_rows_scaled_f32_out16(ctx_, in, out, sums, n_rows, row_len, row_stride, n_valid, causal_period,
                                                causal_offset, scale, out_dtype));
    }
    // the softmax as the CPU loop leaves its buffer: entries past the valid length are not written
    void launch_softmax_rows_valid(const float *in, void *out, float *sums, int64_t n_rows, int64_t row_len, int64_t row_stride,
                                   const int32_t *n_valid, int32_t causal_period, int32_t causal_offset, float scale,
                                   int32_t out_dtype) {
        check(agn_softmax_rows_valid_f32(ctx_, in, out, sums, n_rows, row_len, row_stride, n_valid, causal_period, causal_offset,
                                         scale, out_dtype));
    }
    void launch_qk_norm_rope_qk_f16(void *q, void *k, const float *wq, const float *wk, int64_t T, int n_q, int n_kv,
                                    int head_dim, float eps, int n_rot, const int32_t *pos, int pos_start, float theta,
                                    float freq_scale = 1.0f, int layout = AGN_ROPE_NEOX) {
        check(agn_qk_norm_rope_qk_f16(ctx_, q, k, wq, wk, T, n_q, n_kv, head_dim, eps, n_rot, pos, pos_start, theta,
                                      freq_scale, layout));
    }

    // ---- KV cache: KvCache::write_range / read_up_to (src/model/mod.rs:660-697)
    // norm -> rope of q and k in place and the cache write of the rotated k and of v, one launch
    void launch_qk_norm_rope_kv_write(float *q, float *k, const float *v, const float *wq, const float *wk, int64_t T, int n_q,
                                      int n_kv, int head_dim, float eps, int n_rot, const int32_t *pos, int pos_start, float theta,
                                      int kv_dtype, void *k_cache, void *v_cache, int64_t max_seq_len, float freq_scale = 1.0f,
                                      int layout = AGN_ROPE_NEOX) {
        check(agn_qk_norm_rope_kv_write_f32(ctx_, q, k, v, wq, wk, T, n_q, n_kv, head_dim, eps, n_rot, pos, pos_start, theta,
                                            freq_scale, layout, kv_dtype, k_cache, v_cache, max_seq_len));
    }
    void kv_write(int kv_dtype, const float *k, const float *v, void *k_cache, void *v_cache, int64_t T,
                  int64_t head_dim_kv, const int32_t *pos, int pos_start, int64_t max_seq_len) {
        check(agn_kv_write_f32(ctx_, kv_dtype, k, v, k_cache, v_cache, T, head_dim_kv, pos, pos_start, max_seq_len));
    }
    void kv_read(int kv_dtype, const void *k_cache, const void *v_cache, int64_t n_pos, int64_t head_dim_kv, float *k_out,
                 float *v_out) {
        check(agn_kv_read_f32(ctx_, kv_dtype, k_cache, v_cache, n_pos, head_dim_kv, k_out, v_out));
    }

    // ---- host slices, as the CPU path takes them (src/model/llama/cpu_path.rs:67,975-978)
    void rms_norm_into(const float *x_host, const float *w_dev, float *out_host, int64_t T, int64_t H, float eps) {
        check(agn_host_rms_norm_f32(ctx_, x_host, w_dev, out_host, T, H, eps));
    }
    void add_residual_rms_norm_into(float *x_host, const float *delta_host, const float *w_dev, float *normed_host, int64_t T,
                                    int64_t H, float eps) {  // x += delta (cpu_path.rs:785-787), then the norm (:790)
        check(agn_host_add_residual_rms_norm_f32(ctx_, x_host, delta_host, w_dev, normed_host, T, H, eps));
    }
    void silu_mul_into(const float *gate_host, const float *up_host, float *out_host, int64_t n) {
        check(agn_host_silu_mul_f32(ctx_, gate_host, up_host, out_host, n));
    }

    // ---- a recorded chain of ops (the decode loop), replayed with one launch
    void graph_begin() { check(agn_graph_begin(ctx_)); }
    agn_graph *graph_end() {
        agn_graph *g = nullptr;
        check(agn_graph_end(ctx_, &g));
        return g;
    }
    void graph_launch(agn_graph *g) { check(agn_graph_launch(ctx_, g)); }
    void graph_destroy(agn_graph *g) { check(agn_graph_destroy(ctx_, g)); }

    void check(int32_t st) const {
        if (st != AGN_OK) throw BackendError(st, agn_last_error(ctx_));
    }

  private:
    Q8KRows q8k_rows(int64_t T, int64_t n) {
        const size_t nb = (size_t)agn_q8_k_blocks(n) * (size_t)T;
        return Q8KRows{empty(4 * nb), empty(256 * nb), empty(32 * nb)};
    }
    agn_ctx *ctx_ = nullptr;
};

// A parsed GGUF container (`loader::load` + `parser::parse`, src/loader.rs:14-19, src/parser.rs:9-66):
// metadata accessors like `GgufFile::get_*` (src/types.rs) and tensor upload for get_rows.
class GgufFile {
  public:
    explicit GgufFile(const std::string &path) {  // memory-maps the file (and the siblings of a split model)
        char err[256];
        const int32_t st = agn_gguf_open(path.c_str(), &g_, err, sizeof err);
        if (st != AGN_OK) throw BackendError(st, err);
    }
    GgufFile(const void *data, size_t len) {  // parses caller-owned memory, which must outlive this object
        char err[256];
        const int32_t st = agn_gguf_parse(data, len, &g_, err, sizeof err);
        if (st != AGN_OK) throw BackendError(st, err);
    }
    GgufFile(const GgufFile &) = delete;
    GgufFile &operator=(const GgufFile &) = delete;
    ~GgufFile() { agn_gguf_close(g_); }

    uint32_t version() const { return agn_gguf_version(g_); }
    uint64_t tensor_count() const { return agn_gguf_tensor_count(g_); }
    bool get_u64(const char *key, uint64_t *out) const { return agn_gguf_get_u64(g_, key, out) == AGN_OK; }
    bool get_f32(const char *key, float *out) const { return agn_gguf_get_f32(g_, key, out) == AGN_OK; }
    const char *get_string(const char *key) const {  // nullptr when absent or not a string
        const char *s = nullptr;
        return agn_gguf_get_string(g_, key, &s) == AGN_OK ? s : nullptr;
    }
    bool find(const char *name, agn_tensor_info *out) const { return agn_gguf_find_tensor(g_, name, out) == AGN_OK; }
    // the tensor's bytes in a new device allocation: the `table` argument of get_rows
    DeviceBuffer upload(CudaBackend &be, const char *name, agn_tensor_info *info = nullptr) const {
        void *d = nullptr;
        agn_tensor_info ti;
        be.check(agn_gguf_upload_tensor(be.ctx(), g_, name, &d, &ti));
        if (info) *info = ti;
        return DeviceBuffer(be.ctx(), d, (size_t)ti.n_bytes);
    }
    // `pre_upload_gpu` (src/model/llama/gpu_resident.rs:112-152): all named tensors, uploaded in ascending
    // file-offset order, the consumed part of the mapping dropped from the page cache on the way
    std::vector<DeviceBuffer> upload_all(CudaBackend &be, const std::vector<const char *> &names, bool release_pages = true,
                                         std::vector<agn_tensor_info> *infos = nullptr, uint64_t *released_bytes = nullptr) const {
        std::vector<void *> d(names.size(), nullptr);
        std::vector<agn_tensor_info> ti(names.size());
        be.check(agn_gguf_upload_tensors(be.ctx(), g_, names.data(), names.size(), d.data(), ti.data(), release_pages ? 1 : 0,
                                         released_bytes));
        std::vector<DeviceBuffer> out;
        out.reserve(names.size());
        for (size_t i = 0; i < names.size(); i++) out.emplace_back(be.ctx(), d[i], (size_t)ti[i].n_bytes);
        if (infos) *infos = ti;
        return out;
    }

  private:
    agn_gguf *g_ = nullptr;
};

}  // namespace agn
