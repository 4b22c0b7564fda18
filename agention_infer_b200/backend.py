"""Host-side mirror of the reference's GPU operator surface over the C ABI.

`CudaBackend` carries the same operator names and argument meaning as the
reference's `WgpuBackend::launch_*` family (src/ops/wgpu_backend/resident.rs:187-443)
and `WeightMap::dequant_row` (src/model/mod.rs:343-348), extended from one token
vector per call to T token rows per call.  It is a thin ctypes layer: every method
is one call into libagention_b200.so; nothing is computed in Python.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Tuple

import numpy as np

from . import _abi
from ._abi import (AGN_BF16, AGN_F16, AGN_F32, AGN_Q4_K, AGN_Q6_K, AGN_Q8_0,  # noqa: F401
                   AGN_ROPE_NEOX, AGN_ROPE_NORMAL)


class BackendError(RuntimeError):
    """`GgufError::BackendError` (src/error.rs:37-38) plus the ABI status code."""

    def __init__(self, status: int, message: str):
        super().__init__(f"[agn status {status}] {message}")
        self.status = status


class DeviceBuffer:
    """A device allocation owned by a backend (the role of a cubecl `Handle`)."""

    def __init__(self, backend: "CudaBackend", ptr: int, nbytes: int):
        self.backend, self.ptr, self.nbytes = backend, ptr, nbytes

    def data_ptr(self) -> int:
        return self.ptr

    def free(self) -> None:
        if self.ptr:
            self.backend._free(self.ptr)
            self.ptr = 0

    def __del__(self):  # best effort
        try:
            self.free()
        except Exception:
            pass


def _ptr(obj) -> Optional[int]:
    if obj is None:
        return None
    if isinstance(obj, int):
        return obj
    return int(obj.data_ptr())  # DeviceBuffer or torch CUDA tensor


class CudaBackend:
    """One GPU, one stream.  Replaces `create_backend(BackendPreference::Cuda)`
    (src/ops/backend_select.rs:60-108), whose Cuda arm silently falls back to CPU."""

    def __init__(self, device: int = 0):
        self._lib = _abi.load()
        ctx = C.c_void_p()
        st = self._lib.agn_ctx_create(device, C.byref(ctx))
        if st != _abi.AGN_OK:
            raise BackendError(st, f"no usable CUDA device {device} (this backend has no CPU fallback)")
        self._ctx = ctx
        self.device = device

    # ------------------------------------------------------------ plumbing
    def close(self) -> None:
        if getattr(self, "_ctx", None):
            self._lib.agn_ctx_destroy(self._ctx)
            self._ctx = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, st: int) -> None:
        if st != _abi.AGN_OK:
            raise BackendError(st, self._lib.agn_last_error(self._ctx).decode())

    def name(self) -> str:
        """`Backend::name` (src/ops/mod.rs:99)."""
        return self._lib.agn_backend_name().decode()

    @property
    def launch_count(self) -> int:
        return int(self._lib.agn_ctx_launch_count(self._ctx))

    @property
    def last_kernel(self) -> str:
        """Kernel family of the most recent launch (e.g. "rms_norm" or "rms_norm_ring")."""
        return self._lib.agn_ctx_last_kernel(self._ctx).decode()

    def graph_begin(self) -> None:
        """Start recording the ops enqueued on this backend into a CUDA graph."""
        self._check(self._lib.agn_graph_begin(self._ctx))

    def graph_end(self) -> int:
        g = C.c_void_p()
        self._check(self._lib.agn_graph_end(self._ctx, C.byref(g)))
        return g.value

    def graph_launch(self, graph: int) -> None:
        self._check(self._lib.agn_graph_launch(self._ctx, graph))

    def graph_destroy(self, graph: int) -> None:
        self._check(self._lib.agn_graph_destroy(self._ctx, graph))

    def launch_noop(self) -> None:
        """One empty kernel (the launch-latency floor)."""
        self._check(self._lib.agn_launch_noop(self._ctx))

    def set_option(self, name: str, value: int) -> None:
        self._check(self._lib.agn_ctx_set_option(self._ctx, name.encode(), value))

    def set_stream(self, cuda_stream: Optional[int]) -> None:
        self._check(self._lib.agn_ctx_set_stream(self._ctx, cuda_stream))

    def stream(self) -> int:
        p = C.c_void_p()
        self._check(self._lib.agn_ctx_get_stream(self._ctx, C.byref(p)))
        return p.value or 0

    def sync(self) -> None:
        self._check(self._lib.agn_sync(self._ctx))

    def empty(self, nbytes: int) -> DeviceBuffer:
        """`client.empty(bytes)` (src/ops/wgpu_backend/resident.rs:195)."""
        p = C.c_void_p()
        self._check(self._lib.agn_malloc(self._ctx, nbytes, C.byref(p)))
        return DeviceBuffer(self, p.value or 0, nbytes)

    def _free(self, ptr: int) -> None:
        if getattr(self, "_ctx", None):
            self._lib.agn_free(self._ctx, ptr)

    def upload(self, arr: np.ndarray) -> DeviceBuffer:
        """`upload_act` / `create_from_slice` (src/ops/wgpu_backend/resident.rs:673-690)."""
        arr = np.ascontiguousarray(arr)
        buf = self.empty(max(arr.nbytes, 1))
        self.copy_h2d(buf, arr)
        self.sync()  # pageable source: make the copy complete before `arr` can change
        return buf

    def copy_h2d(self, dst, src: np.ndarray, nbytes: Optional[int] = None) -> None:
        n = src.nbytes if nbytes is None else nbytes
        self._check(self._lib.agn_memcpy_h2d(self._ctx, _ptr(dst), src.ctypes.data, n))

    def copy_d2h(self, dst: np.ndarray, src, nbytes: Optional[int] = None) -> None:
        n = dst.nbytes if nbytes is None else nbytes
        self._check(self._lib.agn_memcpy_d2h(self._ctx, dst.ctypes.data, _ptr(src), n))

    def read(self, buf, dtype, shape) -> np.ndarray:
        """`read_handle` (src/ops/wgpu_backend/resident.rs:696-699): copy back and sync."""
        out = np.empty(shape, dtype=dtype)
        self.copy_d2h(out, buf)
        self.sync()
        return out

    def pinned(self, shape, dtype) -> np.ndarray:
        """A page-locked host array (freed with `free_pinned`)."""
        nbytes = int(np.prod(shape)) * np.dtype(dtype).itemsize
        p = C.c_void_p()
        self._check(self._lib.agn_host_alloc(self._ctx, max(nbytes, 1), C.byref(p)))
        raw = (C.c_uint8 * max(nbytes, 1)).from_address(p.value)
        arr = np.frombuffer(raw, dtype=dtype, count=int(np.prod(shape))).reshape(shape)
        self._pinned = getattr(self, "_pinned", {})
        self._pinned[arr.ctypes.data] = p.value
        return arr

    def free_pinned(self, arr: np.ndarray) -> None:
        p = getattr(self, "_pinned", {}).pop(arr.ctypes.data, None)
        if p:
            self._check(self._lib.agn_host_free(self._ctx, p))

    # ---------------------------------------------------------- GPU timing
    def event(self) -> int:
        e = C.c_void_p()
        self._check(self._lib.agn_event_create(self._ctx, C.byref(e)))
        return e.value

    def record(self, ev: int) -> None:
        self._check(self._lib.agn_event_record(self._ctx, ev))

    def elapsed_ms(self, start: int, stop: int) -> float:
        ms = C.c_float()
        self._check(self._lib.agn_event_elapsed_ms(self._ctx, start, stop, C.byref(ms)))
        return float(ms.value)

    def destroy_event(self, ev: int) -> None:
        self._check(self._lib.agn_event_destroy(self._ctx, ev))

    # ------------------------------------------------------------ layer ops
    def launch_rms_norm(self, x, w, T: int, H: int, eps: float, out=None):
        """`launch_rms_norm(x, weight, len, eps) -> Handle` (resident.rs:213-235) over T rows."""
        if out is None:
            out = self.empty(4 * T * H)
        self._check(self._lib.agn_rms_norm_f32(self._ctx, _ptr(x), _ptr(w), _ptr(out), T, H, eps))
        return out

    def launch_add_residual_rms_norm(self, x, delta, w, T: int, H: int, eps: float, new_x=None, normed=None) -> Tuple:
        """`launch_add_residual_rms_norm(..) -> (new_x, normed)` (resident.rs:240-266)."""
        if new_x is None:
            new_x = self.empty(4 * T * H)
        if normed is None:
            normed = self.empty(4 * T * H)
        self._check(self._lib.agn_add_residual_rms_norm_f32(self._ctx, _ptr(x), _ptr(delta), _ptr(w), _ptr(new_x),
                                                            _ptr(normed), T, H, eps))
        return new_x, normed

    def launch_rope(self, x, T: int, n_heads: int, head_dim: int, n_rot: int, pos, theta: float,
                    freq_scale: float = 1.0, layout: int = AGN_ROPE_NEOX, pos_start: int = 0) -> None:
        """`launch_rope(handle, n_heads, head_dim, n_rot, pos, theta)` in place (resident.rs:326-353).
        `pos` is a device int32 array [T], or None for positions pos_start + t."""
        self._check(self._lib.agn_rope_f32(self._ctx, _ptr(x), T, n_heads, head_dim, n_rot, _ptr(pos), pos_start,
                                           theta, freq_scale, layout))

    def launch_rope_qk(self, q, k, T: int, n_q_heads: int, n_kv_heads: int, head_dim: int, n_rot: int, pos,
                       theta: float, freq_scale: float = 1.0, layout: int = AGN_ROPE_NEOX, pos_start: int = 0) -> None:
        """CPU `rope(q, k, pos)` (src/model/llama/cpu_path.rs:99-133): both buffers, one launch."""
        self._check(self._lib.agn_rope_qk_f32(self._ctx, _ptr(q), _ptr(k), T, n_q_heads, n_kv_heads, head_dim, n_rot,
                                              _ptr(pos), pos_start, theta, freq_scale, layout))

    def launch_qk_norm_rope(self, x, w, T: int, n_heads: int, head_dim: int, eps: float, n_rot: int, pos,
                            theta: float, freq_scale: float = 1.0, layout: int = AGN_ROPE_NEOX,
                            pos_start: int = 0) -> None:
        """`launch_qk_norm_rope(handle, weight, n_heads, head_dim, eps, n_rot, pos, theta)` (resident.rs:414-443)."""
        self._check(self._lib.agn_qk_norm_rope_f32(self._ctx, _ptr(x), _ptr(w), T, n_heads, head_dim, eps, n_rot,
                                                   _ptr(pos), pos_start, theta, freq_scale, layout))

    def launch_qk_norm_rope_qk(self, q, k, wq, wk, T: int, n_q_heads: int, n_kv_heads: int, head_dim: int, eps: float,
                               n_rot: int, pos, theta: float, freq_scale: float = 1.0, layout: int = AGN_ROPE_NEOX,
                               pos_start: int = 0) -> None:
        """Per-position QK-norm -> RoPE of both Q and K (cpu_path.rs:896-906), one launch."""
        self._check(self._lib.agn_qk_norm_rope_qk_f32(self._ctx, _ptr(q), _ptr(k), _ptr(wq), _ptr(wk), T, n_q_heads,
                                                      n_kv_heads, head_dim, eps, n_rot, _ptr(pos), pos_start, theta,
                                                      freq_scale, layout))

    def launch_silu_mul(self, gate, up, n: int, out=None):
        """`launch_silu_mul(gate, up, len) -> Handle` (resident.rs:187-209)."""
        if out is None:
            out = self.empty(4 * n)
        self._check(self._lib.agn_silu_mul_f32(self._ctx, _ptr(gate), _ptr(up), _ptr(out), n))
        return out

    def launch_softmax_rows(self, scores, n_rows: int, row_len: int, out=None, row_stride: Optional[int] = None,
                            n_valid=None, causal_period: int = 0, causal_offset: int = 0):
        """Softmax step of `launch_attention` (resident.rs:551-565) / cpu_path.rs:175-183, normalised."""
        if row_stride is None:
            row_stride = row_len
        if out is None:
            out = self.empty(4 * n_rows * row_stride)
        self._check(self._lib.agn_softmax_rows_f32(self._ctx, _ptr(scores), _ptr(out), n_rows, row_len, row_stride,
                                                   _ptr(n_valid), causal_period, causal_offset))
        return out

    def launch_softmax_rows_scaled(self, scores, n_rows: int, row_len: int, scale: float, out=None, sums=None,
                                   row_stride: Optional[int] = None, n_valid=None, causal_period: int = 0,
                                   causal_offset: int = 0):
        """Softmax of scale * scores (`attention_scores` writes dot * scale, kernels_wgpu.rs:773-782, then the
        softmax runs); sums given: unnormalised weights + row sums."""
        if row_stride is None:
            row_stride = row_len
        if out is None:
            out = self.empty(4 * n_rows * row_stride)
        self._check(self._lib.agn_softmax_rows_scaled_f32(self._ctx, _ptr(scores), _ptr(out), _ptr(sums), n_rows, row_len,
                                                          row_stride, _ptr(n_valid), causal_period, causal_offset, scale))
        return out

    def launch_softmax_rows_scaled_out16(self, scores, n_rows: int, row_len: int, scale: float, out_dtype: int, out=None,
                                         sums=None, row_stride: Optional[int] = None, n_valid=None, causal_period: int = 0,
                                         causal_offset: int = 0):
        """The scaled softmax with the probabilities stored as f16 / bf16 (operand of a half-precision P x V)."""
        if row_stride is None:
            row_stride = row_len
        if out is None:
            out = self.empty(2 * n_rows * row_stride)
        self._check(self._lib.agn_softmax_rows_scaled_f32_out16(self._ctx, _ptr(scores), _ptr(out), _ptr(sums), n_rows,
                                                                row_len, row_stride, _ptr(n_valid), causal_period,
                                                                causal_offset, scale, out_dtype))
        return out

    def launch_softmax_rows_valid(self, scores, n_rows: int, row_len: int, out, scale: float = 1.0, out_dtype: int = AGN_F32,
                                  sums=None, row_stride: Optional[int] = None, n_valid=None, causal_period: int = 0,
                                  causal_offset: int = 0):
        """The softmax as the CPU loop leaves its buffer (cpu_path.rs:168-183): entries past a row's valid
        length are not written.  `out` is required (its tail keeps what it held); f32, f16 or bf16 rows."""
        if row_stride is None:
            row_stride = row_len
        self._check(self._lib.agn_softmax_rows_valid_f32(self._ctx, _ptr(scores), _ptr(out), _ptr(sums), n_rows, row_len,
                                                         row_stride, _ptr(n_valid), causal_period, causal_offset, scale,
                                                         out_dtype))
        return out

    def launch_attention_softmax(self, scores, n_heads: int, max_seq: int, pos: int, weights=None, sums=None):
        """The softmax step of `launch_attention(.., pos, n_heads, max_seq)` (resident.rs:551-565) as the reference's
        kernel leaves it: unnormalised weights [n_heads, max_seq] and sums [n_heads] over entries 0..=pos."""
        if weights is None:
            weights = self.empty(4 * n_heads * max_seq)
        if sums is None:
            sums = self.empty(4 * n_heads)
        self._check(self._lib.agn_softmax_rows_unnorm_f32(self._ctx, _ptr(scores), _ptr(weights), _ptr(sums), n_heads,
                                                          max_seq, max_seq, None, 1, pos))
        return weights, sums

    def get_rows(self, dtype: int, table, table_bytes: int, n_rows: int, row_len: int, ids, T: int, out=None):
        """Embedding loop `dequant_row(token_embd, token)` for T tokens (cpu_path.rs:865-868)."""
        if out is None:
            out = self.empty(4 * T * row_len)
        self._check(self._lib.agn_get_rows_f32(self._ctx, dtype, _ptr(table), table_bytes, n_rows, row_len, _ptr(ids),
                                               T, _ptr(out)))
        return out

    def kv_bytes_per_token(self, kv_dtype: int, head_dim_kv: int) -> int:
        """`KvDtype::bytes_per_token` (src/model/mod.rs:550-556)."""
        return int(self._lib.agn_kv_bytes_per_token(kv_dtype, head_dim_kv))

    def kv_write(self, kv_dtype: int, k, v, k_cache, v_cache, T: int, head_dim_kv: int, pos, max_seq_len: int,
                 pos_start: int = 0) -> None:
        """`KvCache::write_range(layer, pos_start, k, v)` (src/model/mod.rs:660-672): pack T tokens into the cache."""
        self._check(self._lib.agn_kv_write_f32(self._ctx, kv_dtype, _ptr(k), _ptr(v), _ptr(k_cache), _ptr(v_cache), T,
                                               head_dim_kv, _ptr(pos), pos_start, max_seq_len))

    def launch_qk_norm_rope_kv_write(self, q, k, v, wq, wk, T: int, n_q_heads: int, n_kv_heads: int, head_dim: int, eps: float,
                                     n_rot: int, pos, theta: float, kv_dtype: int, k_cache, v_cache, max_seq_len: int,
                                     freq_scale: float = 1.0, layout: int = AGN_ROPE_NEOX, pos_start: int = 0) -> None:
        """QK-norm -> RoPE of q and k in place (wq = wk = None: rope only) and the cache write of the rotated k and of v,
        one launch: `launch_qk_norm_rope` x 2 + `kv_cache_write` of the reference's per-layer sequence."""
        self._check(self._lib.agn_qk_norm_rope_kv_write_f32(self._ctx, _ptr(q), _ptr(k), _ptr(v), _ptr(wq), _ptr(wk), T,
                                                            n_q_heads, n_kv_heads, head_dim, eps, n_rot, _ptr(pos), pos_start,
                                                            theta, freq_scale, layout, kv_dtype, _ptr(k_cache), _ptr(v_cache),
                                                            max_seq_len))

    def kv_read(self, kv_dtype: int, k_cache, v_cache, n_pos: int, head_dim_kv: int, k_out=None, v_out=None):
        """`KvCache::read_up_to(layer, pos)` (src/model/mod.rs:678-697) with n_pos = pos + 1."""
        if k_out is None:
            k_out = self.empty(4 * n_pos * head_dim_kv)
        if v_out is None:
            v_out = self.empty(4 * n_pos * head_dim_kv)
        self._check(self._lib.agn_kv_read_f32(self._ctx, kv_dtype, _ptr(k_cache), _ptr(v_cache), n_pos, head_dim_kv,
                                              _ptr(k_out), _ptr(v_out)))
        return k_out, v_out

    def router_top2(self, logits, T: int, n_experts: int, idx=None, w=None):
        """MoE router: softmax + top-2 per token (docs/08-moe-routing.md:27-33). Returns (idx [T,2] i32, w [T,2] f32)."""
        if idx is None:
            idx = self.empty(8 * max(T, 1))
        if w is None:
            w = self.empty(8 * max(T, 1))
        self._check(self._lib.agn_router_top2_f32(self._ctx, _ptr(logits), T, n_experts, _ptr(idx), _ptr(w)))
        return idx, w

    def gather_rows_by_expert(self, x, idx, T: int, H: int, n_experts: int, out=None, offsets=None, src_token=None,
                              src_slot=None):
        """Expert-sorted copy of the hidden rows: returns (out [2T,H], offsets [E+1], src_token [2T], src_slot [2T])."""
        if out is None:
            out = self.empty(8 * max(T, 1) * H)
        if offsets is None:
            offsets = self.empty(4 * (n_experts + 1))
        if src_token is None:
            src_token = self.empty(8 * max(T, 1))
        if src_slot is None:
            src_slot = self.empty(8 * max(T, 1))
        self._check(self._lib.agn_gather_rows_by_expert_f32(self._ctx, _ptr(x), _ptr(idx), T, H, n_experts, _ptr(out),
                                                            _ptr(offsets), _ptr(src_token), _ptr(src_slot)))
        return out, offsets, src_token, src_slot

    def dequant_row(self, dtype: int, table, table_bytes: int, n_rows: int, row_len: int, row: int) -> np.ndarray:
        """`WeightMap::dequant_row(name, row) -> Vec<f32>` (src/model/mod.rs:343-348) on the GPU.
        An out-of-range row raises, as the reference returns Err (src/quant/mod.rs:116-120)."""
        ids = self.upload(np.array([row], dtype=np.uint32))
        out = self.get_rows(dtype, table, table_bytes, n_rows, row_len, ids, 1)
        return self.read(out, np.float32, (row_len,))

    # ------------------------------------------------- f16 activation storage (the reference's `Act = f16`)
    def launch_silu_mul_f16(self, gate, up, n: int, out=None):
        if out is None:
            out = self.empty(2 * n)
        self._check(self._lib.agn_silu_mul_f16(self._ctx, _ptr(gate), _ptr(up), _ptr(out), n))
        return out

    def launch_rms_norm_f16(self, x, w, T: int, H: int, eps: float, out=None):
        if out is None:
            out = self.empty(2 * T * H)
        self._check(self._lib.agn_rms_norm_f16(self._ctx, _ptr(x), _ptr(w), _ptr(out), T, H, eps))
        return out

    def launch_silu_mul_out16(self, gate, up, n: int, out_dtype: int, out=None):
        """f32 gate / up in, silu(gate) * up stored as f16 / bf16 (operand of a half-precision down projection)."""
        if out is None:
            out = self.empty(2 * n)
        self._check(self._lib.agn_silu_mul_f32_out16(self._ctx, _ptr(gate), _ptr(up), _ptr(out), n, out_dtype))
        return out

    def launch_rms_norm_out16(self, x, w, T: int, H: int, eps: float, out_dtype: int, out=None):
        """f32 rows in, normed rows out as f16 / bf16 (the operand of a half-precision matmul)."""
        if out is None:
            out = self.empty(2 * T * H)
        self._check(self._lib.agn_rms_norm_f32_out16(self._ctx, _ptr(x), _ptr(w), _ptr(out), T, H, eps, out_dtype))
        return out

    def launch_add_residual_rms_norm_out16(self, x, delta, w, T: int, H: int, eps: float, out_dtype: int, new_x=None,
                                           normed=None):
        """new_x = x + delta stays f32; normed is stored as f16 / bf16."""
        if new_x is None:
            new_x = self.empty(4 * T * H)
        if normed is None:
            normed = self.empty(2 * T * H)
        self._check(self._lib.agn_add_residual_rms_norm_f32_out16(self._ctx, _ptr(x), _ptr(delta), _ptr(w), _ptr(new_x),
                                                                  _ptr(normed), T, H, eps, out_dtype))
        return new_x, normed

    # -- Q8_K activation rows (quantize_row_q8_k, src/quant/q8_k.rs:49-92): (d, qs, bsums) device buffers -----
    def _q8k_outputs(self, T: int, n: int, out):
        nb = int(self._lib.agn_q8_k_blocks(n))
        return out if out is not None else (self.empty(4 * T * nb), self.empty(256 * T * nb), self.empty(32 * T * nb))

    def launch_quantize_rows_q8_k(self, x, T: int, n: int, out=None):
        """T rows of n f32 values -> d [T, nb] f32, qs [T, nb*256] i8, bsums [T, nb*16] i16, nb = ceil(n / 256)."""
        d, qs, bs = self._q8k_outputs(T, n, out)
        self._check(self._lib.agn_quantize_rows_q8_k_f32(self._ctx, _ptr(x), T, n, _ptr(d), _ptr(qs), _ptr(bs)))
        return d, qs, bs

    def launch_rms_norm_q8_k(self, x, w, T: int, H: int, eps: float, out=None):
        """RMSNorm with the Q8_K quantiser fused on: the normed f32 row is never written."""
        d, qs, bs = self._q8k_outputs(T, H, out)
        self._check(self._lib.agn_rms_norm_q8_k_f32(self._ctx, _ptr(x), _ptr(w), T, H, eps, _ptr(d), _ptr(qs), _ptr(bs)))
        return d, qs, bs

    def launch_add_residual_rms_norm_q8_k(self, x, delta, w, T: int, H: int, eps: float, new_x=None, out=None):
        """new_x = x + delta stays f32; the normed row leaves as Q8_K blocks."""
        if new_x is None:
            new_x = self.empty(4 * T * H)
        d, qs, bs = self._q8k_outputs(T, H, out)
        self._check(self._lib.agn_add_residual_rms_norm_q8_k_f32(self._ctx, _ptr(x), _ptr(delta), _ptr(w), _ptr(new_x), T, H,
                                                                 eps, _ptr(d), _ptr(qs), _ptr(bs)))
        return new_x, (d, qs, bs)

    def launch_silu_mul_q8_k(self, gate, up, T: int, I: int, out=None):
        """silu(gate) * up over [T, I] rows, stored as Q8_K blocks (the input of a Q5_K down projection)."""
        d, qs, bs = self._q8k_outputs(T, I, out)
        self._check(self._lib.agn_silu_mul_q8_k_f32(self._ctx, _ptr(gate), _ptr(up), T, I, _ptr(d), _ptr(qs), _ptr(bs)))
        return d, qs, bs

    def launch_add_residual_rms_norm_f16(self, x, delta, w, T: int, H: int, eps: float, new_x=None, normed=None):
        if new_x is None:
            new_x = self.empty(2 * T * H)
        if normed is None:
            normed = self.empty(2 * T * H)
        self._check(self._lib.agn_add_residual_rms_norm_f16(self._ctx, _ptr(x), _ptr(delta), _ptr(w), _ptr(new_x),
                                                            _ptr(normed), T, H, eps))
        return new_x, normed

    def launch_qk_norm_rope_qk_f16(self, q, k, wq, wk, T: int, n_q_heads: int, n_kv_heads: int, head_dim: int, eps: float,
                                   n_rot: int, pos, theta: float, freq_scale: float = 1.0, layout: int = AGN_ROPE_NEOX,
                                   pos_start: int = 0) -> None:
        """f16 q/k in place; wq = wk = None is rope without the norm; k = None with n_kv_heads = 0 is one buffer."""
        self._check(self._lib.agn_qk_norm_rope_qk_f16(self._ctx, _ptr(q), _ptr(k), _ptr(wq), _ptr(wk), T, n_q_heads,
                                                      n_kv_heads, head_dim, eps, n_rot, _ptr(pos), pos_start, theta,
                                                      freq_scale, layout))

    def get_rows_f16(self, dtype: int, table, table_bytes: int, n_rows: int, row_len: int, ids, T: int, out=None):
        if out is None:
            out = self.empty(2 * T * row_len)
        self._check(self._lib.agn_get_rows_f16(self._ctx, dtype, _ptr(table), table_bytes, n_rows, row_len, _ptr(ids), T,
                                               _ptr(out)))
        return out

    # ------------------------------------------------- host-slice ops (activations in host memory)
    # The arrays must stay alive and unmodified until sync(); pinned arrays (pinned()) make the
    # transfers asynchronous.  Weights / tables are device buffers.
    @staticmethod
    def _h(a: np.ndarray, dtype) -> int:
        if a.dtype != dtype or not a.flags["C_CONTIGUOUS"]:
            raise ValueError(f"host array must be C-contiguous {np.dtype(dtype).name}")
        return a.ctypes.data

    def rms_norm_into(self, x: np.ndarray, w_dev, out: np.ndarray, eps: float) -> None:
        """`rms_norm_into(x, weight, out)` (src/model/llama/cpu_path.rs:67-74) over the rows of host x [T, H]."""
        T, H = x.shape
        self._check(self._lib.agn_host_rms_norm_f32(self._ctx, self._h(x, np.float32), _ptr(w_dev),
                                                    self._h(out, np.float32), T, H, eps))

    def add_residual_rms_norm_into(self, x: np.ndarray, delta: np.ndarray, w_dev, normed: np.ndarray, eps: float) -> None:
        """`x += delta` (cpu_path.rs:785-787) then `rms_norm_into(x, weight, normed)` (:790); host x is updated in place."""
        T, H = x.shape
        self._check(self._lib.agn_host_add_residual_rms_norm_f32(self._ctx, self._h(x, np.float32), self._h(delta, np.float32),
                                                                 _ptr(w_dev), self._h(normed, np.float32), T, H, eps))

    def silu_mul_into(self, gate: np.ndarray, up: np.ndarray, out: np.ndarray) -> None:
        """The batched silu-combine loop (cpu_path.rs:975-978) on host arrays; out may be gate."""
        self._check(self._lib.agn_host_silu_mul_f32(self._ctx, self._h(gate, np.float32), self._h(up, np.float32),
                                                    self._h(out, np.float32), gate.size))

    def rope_host(self, q: np.ndarray, k: np.ndarray, n_q_heads: int, n_kv_heads: int, head_dim: int, n_rot: int,
                  pos: Optional[np.ndarray], theta: float, freq_scale: float = 1.0, layout: int = AGN_ROPE_NEOX,
                  pos_start: int = 0, wq_dev=None, wk_dev=None, eps: float = 0.0) -> None:
        """`rope(q, k, pos)` per token (cpu_path.rs:896-906), in place on host q [T, nq*hd], k [T, nkv*hd];
        with wq_dev / wk_dev the per-head QK-norm runs first (fused)."""
        T = q.shape[0]
        pp = None if pos is None else self._h(pos, np.int32)
        if wq_dev is None and wk_dev is None:
            st = self._lib.agn_host_rope_qk_f32(self._ctx, self._h(q, np.float32), self._h(k, np.float32), T, n_q_heads,
                                                n_kv_heads, head_dim, n_rot, pp, pos_start, theta, freq_scale, layout)
        else:
            st = self._lib.agn_host_qk_norm_rope_qk_f32(self._ctx, self._h(q, np.float32), self._h(k, np.float32),
                                                        _ptr(wq_dev), _ptr(wk_dev), T, n_q_heads, n_kv_heads, head_dim,
                                                        eps, n_rot, pp, pos_start, theta, freq_scale, layout)
        self._check(st)

    def softmax_rows_into(self, scores: np.ndarray, out: np.ndarray, n_valid: Optional[np.ndarray] = None,
                          causal_period: int = 0, causal_offset: int = 0) -> None:
        """Row softmax (cpu_path.rs:175-183) on host rows [n_rows, row_len]."""
        rows = scores.reshape(-1, scores.shape[-1])
        nv = None if n_valid is None else self._h(n_valid, np.int32)
        self._check(self._lib.agn_host_softmax_rows_f32(self._ctx, self._h(scores, np.float32), self._h(out, np.float32),
                                                        rows.shape[0], rows.shape[1], nv, causal_period, causal_offset))

    def get_rows_into(self, dtype: int, table_dev, table_bytes: int, n_rows: int, row_len: int, ids: np.ndarray,
                      out: np.ndarray) -> None:
        """The embedding loop (cpu_path.rs:865-868): host ids [T] -> host out [T, row_len]."""
        self._check(self._lib.agn_host_get_rows_f32(self._ctx, dtype, _ptr(table_dev), table_bytes, n_rows, row_len,
                                                    self._h(ids, np.uint32), ids.size, self._h(out, np.float32)))

    def quantize_rows_q8_k_into(self, x: np.ndarray, d: np.ndarray, qs: np.ndarray, bsums: np.ndarray) -> None:
        """`quantize_row_q8_k` (src/quant/q8_k.rs:49-92) on host rows x [T, n] -> d [T, nb] f32, qs [T, nb*256] i8,
        bsums [T, nb*16] i16."""
        rows = x.reshape(-1, x.shape[-1])
        self._check(self._lib.agn_host_quantize_rows_q8_k_f32(self._ctx, self._h(x, np.float32), rows.shape[0], rows.shape[1],
                                                              self._h(d, np.float32), self._h(qs, np.int8), self._h(bsums, np.int16)))

    @staticmethod
    def type_size(dtype: int, n: int) -> int:
        """`GgmlType::type_size` (src/types.rs:164-168)."""
        return int(_abi.load().agn_type_size(dtype, n))
