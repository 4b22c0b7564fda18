//! `CudaBackend`: the reference-side binding of libagention_b200.so, to be added to the engine as
//! `src/ops/cuda_backend.rs` (with `ffi.rs` beside it as `src/ops/cuda_ffi.rs`) behind a cargo
//! feature `cuda`.  It carries the `launch_*` names and argument meaning of `WgpuBackend`
//! (src/ops/wgpu_backend/resident.rs:187-443), extended from one token vector to `t` token rows
//! per call; `t = 1` with a scalar position reproduces today's per-token call.
//!
//! build.rs of the engine:
//!     println!("cargo:rustc-link-search=native={}", env!("AGENTION_B200_LIB_DIR"));
//!     println!("cargo:rustc-link-lib=dylib=agention_b200");
//!
//! This file has not been compiled: the build environment of the CUDA library holds no Rust
//! toolchain.  `ffi.rs` is generated from the C header, so names, argument order and types of the
//! extern block follow the header by construction.
use std::ffi::{c_void, CStr, CString};

use crate::error::{GgufError, Result};
use crate::ops::cuda_ffi::*;
use crate::types::GgmlType;

/// A device allocation: the role `cubecl::server::Handle` plays for `WgpuBackend`.
pub struct DevBuf {
    ctx: *mut AgnCtx,
    pub ptr: *mut c_void,
    pub bytes: usize,
}
impl Drop for DevBuf {
    fn drop(&mut self) {
        unsafe { agn_free(self.ctx, self.ptr) };
    }
}

/// Device-resident `Q8KRow`s (src/quant/q8_k.rs:27-37) of `t` rows: per row `ceil(n / 256)` scales, 256 times as
/// many quantised values (zero past `n`) and 16 times as many group sums.
pub struct Q8KRows {
    pub d: DevBuf,
    pub qs: DevBuf,
    pub bsums: DevBuf,
    pub n: usize,
}

/// A recorded chain of ops (`agn_graph_begin` .. `agn_graph_end`), replayed with one launch.
pub struct OpGraph {
    ctx: *mut AgnCtx,
    graph: *mut AgnGraph,
}
impl Drop for OpGraph {
    fn drop(&mut self) {
        unsafe { agn_graph_destroy(self.ctx, self.graph) };
    }
}

pub struct CudaBackend {
    ctx: *mut AgnCtx,
}
// One context = one GPU + one stream; `forward` already serialises calls
// (src/model/llama/mod.rs:340-343), which is what the C library asks of its caller.
unsafe impl Send for CudaBackend {}
unsafe impl Sync for CudaBackend {}

impl Drop for CudaBackend {
    fn drop(&mut self) {
        unsafe { agn_ctx_destroy(self.ctx) };
    }
}

/// RoPE pairing; the reference rotates NeoX pairs (src/model/llama/cpu_path.rs:114-132).
#[derive(Clone, Copy)]
pub enum RopeLayout {
    Neox = AGN_ROPE_NEOX as isize,
    Normal = AGN_ROPE_NORMAL as isize,
}

impl CudaBackend {
    /// `BackendPreference::Cuda` arm of `create_backend` (src/ops/backend_select.rs:84-95): an
    /// error instead of the CPU fallback when there is no device.
    pub fn new(device: i32) -> Result<Self> {
        let mut ctx = std::ptr::null_mut();
        let st = unsafe { agn_ctx_create(device, &mut ctx) };
        if st != AGN_OK {
            let why = unsafe { CStr::from_ptr(agn_status_string(st)) }.to_string_lossy().into_owned();
            return Err(GgufError::BackendError(format!("CUDA backend unavailable: {why}")));
        }
        Ok(Self { ctx })
    }

    fn check(&self, st: i32) -> Result<()> {
        if st == AGN_OK {
            return Ok(());
        }
        let msg = unsafe { CStr::from_ptr(agn_last_error(self.ctx)) }.to_string_lossy().into_owned();
        Err(GgufError::BackendError(msg))
    }

    /// `Backend::name` (src/ops/mod.rs:99).
    pub fn name(&self) -> &str {
        "cuda-sm100a"
    }

    /// `Backend::matmul_dequant` (src/ops/mod.rs:101-105): not part of this library.
    pub fn matmul_dequant(&self, _dtype: GgmlType, _w: &[u8], _x: &[f32], _out: &mut [f32]) -> Result<()> {
        Err(GgufError::BackendError("unsupported: the CUDA layer-op backend has no matmul".into()))
    }

    // ---- memory: `client.empty` / `upload_act` / `read_handle` (resident.rs:673-700) ----------

    pub fn empty(&self, bytes: usize) -> Result<DevBuf> {
        let mut p = std::ptr::null_mut();
        self.check(unsafe { agn_malloc(self.ctx, bytes, &mut p) })?;
        Ok(DevBuf { ctx: self.ctx, ptr: p, bytes })
    }

    pub fn upload<T: Copy>(&self, host: &[T]) -> Result<DevBuf> {
        let bytes = std::mem::size_of_val(host);
        let buf = self.empty(bytes)?;
        self.check(unsafe { agn_memcpy_h2d(self.ctx, buf.ptr, host.as_ptr() as *const c_void, bytes) })?;
        Ok(buf)
    }

    /// Blocks until the stream has drained; an out-of-range token id of an earlier `get_rows`
    /// surfaces here as `Err` (the reference returns it from `row_view`, src/quant/mod.rs:116-120).
    pub fn read<T: Copy + Default>(&self, buf: &DevBuf, n: usize) -> Result<Vec<T>> {
        let mut out = vec![T::default(); n];
        let bytes = n * std::mem::size_of::<T>();
        self.check(unsafe { agn_memcpy_d2h(self.ctx, out.as_mut_ptr() as *mut c_void, buf.ptr, bytes) })?;
        self.check(unsafe { agn_sync(self.ctx) })?;
        Ok(out)
    }

    pub fn sync(&self) -> Result<()> {
        self.check(unsafe { agn_sync(self.ctx) })
    }

    pub fn set_option(&self, name: &str, value: i64) -> Result<()> {
        let c = CString::new(name).map_err(|e| GgufError::BackendError(e.to_string()))?;
        self.check(unsafe { agn_ctx_set_option(self.ctx, c.as_ptr(), value) })
    }

    // ---- the launch_* family ------------------------------------------------------------------

    /// `launch_rms_norm(x, weight, len, eps) -> Handle` (resident.rs:213-235), `t` rows of `h`.
    pub fn launch_rms_norm(&self, x: &DevBuf, w: &DevBuf, t: usize, h: usize, eps: f32) -> Result<DevBuf> {
        let out = self.empty(4 * t * h)?;
        self.check(unsafe {
            agn_rms_norm_f32(self.ctx, x.ptr as *const f32, w.ptr as *const f32, out.ptr as *mut f32, t as i64, h as i64, eps)
        })?;
        Ok(out)
    }

    /// The same into a buffer the caller allocated (the form to use inside `record`, where
    /// allocation is refused).
    pub fn launch_rms_norm_into(&self, x: &DevBuf, w: &DevBuf, out: &DevBuf, t: usize, h: usize, eps: f32) -> Result<()> {
        self.check(unsafe {
            agn_rms_norm_f32(self.ctx, x.ptr as *const f32, w.ptr as *const f32, out.ptr as *mut f32, t as i64, h as i64, eps)
        })
    }

    /// `launch_add_residual_rms_norm(x, delta, weight, len, eps) -> (new_x, normed)` (resident.rs:240-266).
    pub fn launch_add_residual_rms_norm(&self, x: &DevBuf, delta: &DevBuf, w: &DevBuf, t: usize, h: usize,
                                        eps: f32) -> Result<(DevBuf, DevBuf)> {
        let new_x = self.empty(4 * t * h)?;
        let normed = self.empty(4 * t * h)?;
        self.check(unsafe {
            agn_add_residual_rms_norm_f32(self.ctx, x.ptr as *const f32, delta.ptr as *const f32, w.ptr as *const f32,
                                          new_x.ptr as *mut f32, normed.ptr as *mut f32, t as i64, h as i64, eps)
        })?;
        Ok((new_x, normed))
    }

    /// The same with the normed row stored as f16 (`out_dtype = AGN_F16`) or bf16 (`AGN_BF16`)
    /// for a half-precision matmul; the residual stream stays f32.
    pub fn launch_add_residual_rms_norm_out16(&self, x: &DevBuf, delta: &DevBuf, w: &DevBuf, t: usize, h: usize,
                                              eps: f32, out_dtype: i32) -> Result<(DevBuf, DevBuf)> {
        let new_x = self.empty(4 * t * h)?;
        let normed = self.empty(2 * t * h)?;
        self.check(unsafe {
            agn_add_residual_rms_norm_f32_out16(self.ctx, x.ptr as *const f32, delta.ptr as *const f32,
                                                w.ptr as *const f32, new_x.ptr as *mut f32, normed.ptr, t as i64,
                                                h as i64, eps, out_dtype)
        })?;
        Ok((new_x, normed))
    }

    /// `quantize_row_q8_k` (src/quant/q8_k.rs:49-92) over `t` rows of `n` values already on the device:
    /// the `Q8KRow` arrays (`d` f32, `qs` i8, `bsums` i16) for `ceil(n / 256)` blocks per row.
    pub fn launch_quantize_rows_q8_k(&self, x: &DevBuf, t: usize, n: usize) -> Result<Q8KRows> {
        let out = self.q8k_rows(t, n)?;
        self.check(unsafe {
            agn_quantize_rows_q8_k_f32(self.ctx, x.ptr as *const f32, t as i64, n as i64, out.d.ptr as *mut f32,
                                       out.qs.ptr as *mut i8, out.bsums.ptr as *mut i16)
        })?;
        Ok(out)
    }

    /// `launch_rms_norm` with the quantiser of `matmul_into` (src/model/mod.rs:381-386) fused on: the input of a
    /// Q5_K projection without the f32 row in between.
    pub fn launch_rms_norm_q8_k(&self, x: &DevBuf, w: &DevBuf, t: usize, h: usize, eps: f32) -> Result<Q8KRows> {
        let out = self.q8k_rows(t, h)?;
        self.check(unsafe {
            agn_rms_norm_q8_k_f32(self.ctx, x.ptr as *const f32, w.ptr as *const f32, t as i64, h as i64, eps,
                                  out.d.ptr as *mut f32, out.qs.ptr as *mut i8, out.bsums.ptr as *mut i16)
        })?;
        Ok(out)
    }

    /// `launch_add_residual_rms_norm` whose normed row leaves as Q8_K blocks; `new_x` stays f32.
    pub fn launch_add_residual_rms_norm_q8_k(&self, x: &DevBuf, delta: &DevBuf, w: &DevBuf, t: usize, h: usize,
                                             eps: f32) -> Result<(DevBuf, Q8KRows)> {
        let new_x = self.empty(4 * t * h)?;
        let out = self.q8k_rows(t, h)?;
        self.check(unsafe {
            agn_add_residual_rms_norm_q8_k_f32(self.ctx, x.ptr as *const f32, delta.ptr as *const f32, w.ptr as *const f32,
                                               new_x.ptr as *mut f32, t as i64, h as i64, eps, out.d.ptr as *mut f32,
                                               out.qs.ptr as *mut i8, out.bsums.ptr as *mut i16)
        })?;
        Ok((new_x, out))
    }

    /// `launch_silu_mul` over `[t, i]` rows whose product leaves as Q8_K blocks (input of a Q5_K down projection).
    pub fn launch_silu_mul_q8_k(&self, gate: &DevBuf, up: &DevBuf, t: usize, i: usize) -> Result<Q8KRows> {
        let out = self.q8k_rows(t, i)?;
        self.check(unsafe {
            agn_silu_mul_q8_k_f32(self.ctx, gate.ptr as *const f32, up.ptr as *const f32, t as i64, i as i64,
                                  out.d.ptr as *mut f32, out.qs.ptr as *mut i8, out.bsums.ptr as *mut i16)
        })?;
        Ok(out)
    }

    /// `quantize_row_q8_k(x)` at the top of `WeightMap::matmul_into` (src/model/mod.rs:386) for a host vector: the
    /// reference's own `Q8KRow`, filled by the GPU through the host-slice staging ring.
    pub fn quantize_row_q8_k(&self, x: &[f32]) -> Result<crate::quant::q8_k::Q8KRow> {
        let n = x.len();
        let nb = unsafe { agn_q8_k_blocks(n as i64) } as usize;
        let (mut d, mut qs, mut bsums) = (vec![0f32; nb], vec![0i8; nb * 256], vec![0i16; nb * 16]);
        self.check(unsafe {
            agn_host_quantize_rows_q8_k_f32(self.ctx, x.as_ptr(), 1, n as i64, d.as_mut_ptr(), qs.as_mut_ptr(), bsums.as_mut_ptr())
        })?;
        self.sync()?;
        Ok(crate::quant::q8_k::Q8KRow { d, qs, bsums, n })
    }

    fn q8k_rows(&self, t: usize, n: usize) -> Result<Q8KRows> {
        let nb = unsafe { agn_q8_k_blocks(n as i64) } as usize;
        Ok(Q8KRows { d: self.empty(4 * t * nb)?, qs: self.empty(256 * t * nb)?, bsums: self.empty(32 * t * nb)?, n })
    }

    /// `launch_rope(handle, n_heads, head_dim, n_rot, pos, theta)` in place (resident.rs:326-353)
    /// on Q and K of `t` tokens at positions `pos_start + row`.
    #[allow(clippy::too_many_arguments)]
    pub fn launch_rope_qk(&self, q: &DevBuf, k: &DevBuf, t: usize, n_q_heads: usize, n_kv_heads: usize, head_dim: usize,
                          n_rot: usize, pos_start: usize, theta: f32, freq_scale: f32, layout: RopeLayout) -> Result<()> {
        self.check(unsafe {
            agn_rope_qk_f32(self.ctx, q.ptr as *mut f32, k.ptr as *mut f32, t as i64, n_q_heads as i32, n_kv_heads as i32,
                            head_dim as i32, n_rot as i32, std::ptr::null(), pos_start as i32, theta, freq_scale,
                            layout as i32)
        })
    }

    /// `launch_qk_norm_rope(handle, weight, n_heads, head_dim, eps, n_rot, pos, theta)` in place
    /// (resident.rs:414-443) on Q and K in one launch.
    #[allow(clippy::too_many_arguments)]
    pub fn launch_qk_norm_rope_qk(&self, q: &DevBuf, k: &DevBuf, wq: &DevBuf, wk: &DevBuf, t: usize, n_q_heads: usize,
                                  n_kv_heads: usize, head_dim: usize, eps: f32, n_rot: usize, pos_start: usize,
                                  theta: f32, freq_scale: f32, layout: RopeLayout) -> Result<()> {
        self.check(unsafe {
            agn_qk_norm_rope_qk_f32(self.ctx, q.ptr as *mut f32, k.ptr as *mut f32, wq.ptr as *const f32,
                                    wk.ptr as *const f32, t as i64, n_q_heads as i32, n_kv_heads as i32, head_dim as i32,
                                    eps, n_rot as i32, std::ptr::null(), pos_start as i32, theta, freq_scale,
                                    layout as i32)
        })
    }

    /// `launch_silu_mul(gate, up, len) -> Handle` (resident.rs:187-209).
    pub fn launch_silu_mul(&self, gate: &DevBuf, up: &DevBuf, len: usize) -> Result<DevBuf> {
        let out = self.empty(4 * len)?;
        self.check(unsafe {
            agn_silu_mul_f32(self.ctx, gate.ptr as *const f32, up.ptr as *const f32, out.ptr as *mut f32, len as i64)
        })?;
        Ok(out)
    }

    pub fn launch_silu_mul_into(&self, gate: &DevBuf, up: &DevBuf, out: &DevBuf, len: usize) -> Result<()> {
        self.check(unsafe {
            agn_silu_mul_f32(self.ctx, gate.ptr as *const f32, up.ptr as *const f32, out.ptr as *mut f32, len as i64)
        })
    }

    /// The softmax step of `launch_attention(.., pos, n_heads, max_seq)` (resident.rs:551-565) in
    /// the form the reference's kernel leaves it: unnormalised weights and `sums[h]` over the
    /// entries `0..=pos`; `scale` multiplies the raw dot products (1/sqrt(head_dim)).
    pub fn launch_attention_softmax(&self, scores: &DevBuf, n_heads: usize, max_seq: usize, pos: usize,
                                    scale: f32) -> Result<(DevBuf, DevBuf)> {
        let weights = self.empty(4 * n_heads * max_seq)?;
        let sums = self.empty(4 * n_heads)?;
        self.check(unsafe {
            agn_softmax_rows_scaled_f32(self.ctx, scores.ptr as *const f32, weights.ptr as *mut f32, sums.ptr as *mut f32,
                                        n_heads as i64, max_seq as i64, max_seq as i64, std::ptr::null(), 1, pos as i32,
                                        scale)
        })?;
        Ok((weights, sums))
    }

    /// Causal prefill softmax over `[n_heads, seq, seq]` scores: row `i` of a head has `i + 1`
    /// valid entries (cpu_path.rs:175-183 applied per query position), normalised.
    pub fn launch_softmax_causal(&self, scores: &DevBuf, n_heads: usize, seq: usize, scale: f32) -> Result<DevBuf> {
        let out = self.empty(4 * n_heads * seq * seq)?;
        self.check(unsafe {
            agn_softmax_rows_scaled_f32(self.ctx, scores.ptr as *const f32, out.ptr as *mut f32, std::ptr::null_mut(),
                                        (n_heads * seq) as i64, seq as i64, seq as i64, std::ptr::null(), seq as i32, 0,
                                        scale)
        })?;
        Ok(out)
    }

    /// The causal prefill softmax exactly as the CPU loop leaves its buffer (cpu_path.rs:168-183 runs over
    /// `scores[..seq_len]` only): entries past a row's valid length keep what `out` held.  `out_dtype` is
    /// `AGN_F32`, `AGN_F16` or `AGN_BF16`.
    pub fn launch_softmax_causal_valid(&self, scores: &DevBuf, out: &DevBuf, n_heads: usize, seq: usize, scale: f32,
                                       out_dtype: i32) -> Result<()> {
        self.check(unsafe {
            agn_softmax_rows_valid_f32(self.ctx, scores.ptr as *const f32, out.ptr, std::ptr::null_mut(),
                                       (n_heads * seq) as i64, seq as i64, seq as i64, std::ptr::null(), seq as i32, 0,
                                       scale, out_dtype)
        })
    }

    /// Kernel family of the most recent launch (the per-kernel name `GGUF_TRACE_KERNEL` would print).
    pub fn last_kernel(&self) -> String {
        unsafe { CStr::from_ptr(agn_ctx_last_kernel(self.ctx)) }.to_string_lossy().into_owned()
    }

    /// Embedding rows for a batch of tokens: replaces the per-token CPU `dequant_row` + upload of
    /// `run_gpu_resident` (src/model/llama/gpu_resident.rs:436-437).  `table` holds the tensor's
    /// bytes as they are in the GGUF file, uploaded once.
    pub fn get_rows(&self, ty: GgmlType, table: &DevBuf, vocab: usize, h: usize, ids: &DevBuf, t: usize) -> Result<DevBuf> {
        let out = self.empty(4 * t * h)?;
        self.check(unsafe {
            agn_get_rows_f32(self.ctx, ty as i32, table.ptr as *const c_void, table.bytes, vocab as i64, h as i64,
                             ids.ptr as *const u32, t as i64, out.ptr as *mut f32)
        })?;
        Ok(out)
    }

    /// `KvCache::write_range` (src/model/mod.rs:660-672) for one layer: `kv_dtype` is `AGN_F16`
    /// or `AGN_Q8_0` (`KvDtype`, :536-539); token `i` goes to slot `pos_start + i`.
    #[allow(clippy::too_many_arguments)]
    pub fn kv_write(&self, kv_dtype: i32, k: &DevBuf, v: &DevBuf, k_cache: &DevBuf, v_cache: &DevBuf, t: usize,
                    head_dim_kv: usize, pos_start: usize, max_seq_len: usize) -> Result<()> {
        self.check(unsafe {
            agn_kv_write_f32(self.ctx, kv_dtype, k.ptr as *const f32, v.ptr as *const f32, k_cache.ptr, v_cache.ptr,
                             t as i64, head_dim_kv as i64, std::ptr::null(), pos_start as i32, max_seq_len as i64)
        })
    }

    /// `launch_qk_norm_rope` on q and on k followed by `kv_cache_write` (the per-layer, per-token
    /// sequence of the resident path) as one launch; `wq`/`wk` = `None`: rope without the norm.
    #[allow(clippy::too_many_arguments)]
    pub fn launch_qk_norm_rope_kv_write(&self, q: &DevBuf, k: &DevBuf, v: &DevBuf, wq: Option<&DevBuf>, wk: Option<&DevBuf>,
                                        t: usize, n_q_heads: usize, n_kv_heads: usize, head_dim: usize, eps: f32,
                                        n_rot: usize, pos_start: usize, theta: f32, freq_scale: f32, layout: RopeLayout,
                                        kv_dtype: i32, k_cache: &DevBuf, v_cache: &DevBuf, max_seq_len: usize) -> Result<()> {
        let wq_ptr = wq.map_or(std::ptr::null(), |b| b.ptr as *const f32);
        let wk_ptr = wk.map_or(std::ptr::null(), |b| b.ptr as *const f32);
        self.check(unsafe {
            agn_qk_norm_rope_kv_write_f32(self.ctx, q.ptr as *mut f32, k.ptr as *mut f32, v.ptr as *const f32, wq_ptr, wk_ptr,
                                          t as i64, n_q_heads as i32, n_kv_heads as i32, head_dim as i32, eps, n_rot as i32,
                                          std::ptr::null(), pos_start as i32, theta, freq_scale, layout as i32, kv_dtype,
                                          k_cache.ptr, v_cache.ptr, max_seq_len as i64)
        })
    }

    /// Router logits `[t, n_experts]` -> the two largest per token (ties to the lower index) and
    /// their softmax probabilities, not renormalised (docs/08-moe-routing.md:27-33).
    pub fn router_top2(&self, logits: &DevBuf, t: usize, n_experts: usize) -> Result<(DevBuf, DevBuf)> {
        let idx = self.empty(4 * 2 * t)?;
        let w = self.empty(4 * 2 * t)?;
        self.check(unsafe {
            agn_router_top2_f32(self.ctx, logits.ptr as *const f32, t as i64, n_experts as i32, idx.ptr as *mut i32,
                                w.ptr as *mut f32)
        })?;
        Ok((idx, w))
    }

    // ---- recorded chains: the per-token queue of launches (gpu_resident.rs:427-697) -----------

    /// Records the ops issued by `body` into a graph instead of running them.  Inside `body` only
    /// the in-place ops and the `_into` forms may be used: allocation, upload, read and sync are
    /// refused while recording.
    pub fn record<F: FnOnce(&Self) -> Result<()>>(&self, body: F) -> Result<OpGraph> {
        self.check(unsafe { agn_graph_begin(self.ctx) })?;
        let r = body(self);
        let mut g = std::ptr::null_mut();
        let st = unsafe { agn_graph_end(self.ctx, &mut g) };
        r?;
        self.check(st)?;
        Ok(OpGraph { ctx: self.ctx, graph: g })
    }

    pub fn replay(&self, graph: &OpGraph) -> Result<()> {
        self.check(unsafe { agn_graph_launch(self.ctx, graph.graph) })
    }
}
