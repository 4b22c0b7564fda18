"""ctypes binding of the CPU oracle (oracle/cpu_ref.c).

TEST INFRASTRUCTURE ONLY: imported by tests/, by __graft_entry__.smoke() and by the
CPU-baseline legs of bench.py — never by the agention_infer_b200 package.
"""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
LIB = HERE / "liboracle.so"

F32, F16, Q8_0, Q4_K, Q6_K, BF16 = 0, 1, 8, 12, 14, 30
KV_Q8_0_WORDS = 1008  # the GPU path's Q8_0 cache layout (36-byte blocks), not a GgmlType
Q5_0, Q5_K, Q2_K = 6, 13, 10
NEOX, NORMAL = 0, 1
OK, ESHORT, EROW, EDTYPE, ELEN = 0, 1, 2, 3, 4


def build(force: bool = False) -> Path:
    src = [HERE / "cpu_ref.c", HERE / "cpu_ref.h", HERE / "Makefile"]
    if force or not LIB.exists() or any(s.stat().st_mtime > LIB.stat().st_mtime for s in src):
        subprocess.run(["make", "-C", str(HERE), "-B", "liboracle.so"], check=True, capture_output=True)
    return LIB


_lib = None
_vp, _sz, _f, _i = C.c_void_p, C.c_size_t, C.c_float, C.c_int


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        l = C.CDLL(str(LIB))
        sig = {
            "orc_block_size": (_sz, [_i]), "orc_block_bytes": (_sz, [_i]), "orc_type_size": (_sz, [_i, _sz]),
            "orc_f16_to_f32": (_f, [C.c_uint16]),
            "orc_rope_freq_scale": (_i, [C.c_char_p, _i, _f, C.POINTER(_f)]),
            "orc_rms_norm_rows": (None, [_vp, _vp, _vp, _sz, _sz, _f, _i]),
            "orc_add_residual_rms_norm_rows": (None, [_vp, _vp, _vp, _vp, _vp, _sz, _sz, _f, _i]),
            "orc_qk_norm": (None, [_vp, _vp, _sz, _sz, _f]),
            "orc_rope_denominators": (None, [_f, _sz, _vp]),
            "orc_rope_rows": (None, [_vp, _sz, _sz, _sz, _sz, _vp, _f, _f, _i, _i]),
            "orc_qk_norm_rope_rows": (None, [_vp, _vp, _sz, _sz, _sz, _f, _sz, _vp, _f, _f, _i, _i]),
            "orc_softmax_rows": (None, [_vp, _vp, _sz, _sz, _sz, _vp, _i]),
            "orc_silu_mul": (None, [_vp, _vp, _vp, _sz, _i]),
            "orc_get_scale_min_k4": (None, [_sz, _vp, _vp, _vp]),
            "orc_dequant_q8_0": (_i, [_vp, _sz, _sz, _vp]), "orc_dequant_q4_k": (_i, [_vp, _sz, _sz, _vp]),
            "orc_dequant_q5_k": (_i, [_vp, _sz, _sz, _vp]), "orc_dequant_q5_0": (_i, [_vp, _sz, _sz, _vp]),
            "orc_dequant_q2_k": (_i, [_vp, _sz, _sz, _vp]),
            "orc_dequant_q6_k": (_i, [_vp, _sz, _sz, _vp]), "orc_dequant_f32": (_i, [_vp, _sz, _sz, _vp]),
            "orc_dequant_f16": (_i, [_vp, _sz, _sz, _vp]), "orc_dequant_bf16": (_i, [_vp, _sz, _sz, _vp]),
            "orc_dequant_row": (_i, [_i, _vp, _sz, _sz, _sz, _sz, _sz, _vp]),
            "orc_get_rows": (_i, [_i, _vp, _sz, _sz, _sz, _vp, _sz, _vp, _i]),
            "orc_kv_bytes_per_token": (_sz, [_i, _sz]),
            "orc_kv_write_rows": (None, [_i, _vp, _sz, _sz, _vp, _vp]),
            "orc_kv_read": (None, [_i, _vp, _sz, _sz, _vp]),
            "orc_router_top2": (None, [_vp, _sz, _sz, _vp, _vp]),
            "orc_gather_rows_by_expert": (None, [_vp, _sz, _sz, _vp, _sz, _vp, _vp, _vp, _vp]),
            "orc_quantize_rows_q8_k": (None, [_vp, _sz, _sz, _vp, _vp, _vp, _i]),
            "orc_max_threads": (_i, []),
        }
        for name, (res, args) in sig.items():
            fn = getattr(l, name)
            fn.restype, fn.argtypes = res, args
        _lib = l
    return _lib


def _p(a: np.ndarray):
    return a.ctypes.data


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def max_threads() -> int:
    return int(lib().orc_max_threads())


def type_size(dtype: int, n: int) -> int:
    return int(lib().orc_type_size(dtype, n))


def f16_to_f32(bits: int) -> float:
    return float(lib().orc_f16_to_f32(bits))


def rope_freq_scale(type_, factor):
    out = _f()
    ok = lib().orc_rope_freq_scale(None if type_ is None else type_.encode(), 0 if factor is None else 1,
                                   0.0 if factor is None else factor, C.byref(out))
    return float(out.value) if ok else None


def rms_norm_rows(x, w, eps: float, threads: int = 1) -> np.ndarray:
    x, w = _f32(x), _f32(w)
    T, H = x.shape
    out = np.empty_like(x)
    lib().orc_rms_norm_rows(_p(x), _p(w), _p(out), T, H, eps, threads)
    return out


def add_residual_rms_norm_rows(x, delta, w, eps: float, threads: int = 1):
    x, delta, w = _f32(x), _f32(delta), _f32(w)
    T, H = x.shape
    new_x, normed = np.empty_like(x), np.empty_like(x)
    lib().orc_add_residual_rms_norm_rows(_p(x), _p(delta), _p(w), _p(new_x), _p(normed), T, H, eps, threads)
    return new_x, normed


def rope_denominators(theta: float, n_rot: int) -> np.ndarray:
    out = np.empty(n_rot // 2, dtype=np.float32)
    lib().orc_rope_denominators(theta, n_rot, _p(out))
    return out


def rope_rows(x, n_heads, head_dim, n_rot, pos, theta, freq_scale=1.0, layout=NEOX, threads: int = 1) -> np.ndarray:
    x = _f32(x).copy()
    pos = np.ascontiguousarray(pos, dtype=np.int32)
    T = x.shape[0]
    lib().orc_rope_rows(_p(x), T, n_heads, head_dim, n_rot, _p(pos), theta, freq_scale, layout, threads)
    return x


def qk_norm_rope_rows(x, w, n_heads, head_dim, eps, n_rot, pos, theta, freq_scale=1.0, layout=NEOX,
                      threads: int = 1) -> np.ndarray:
    x = _f32(x).copy()
    w = None if w is None else _f32(w)
    pos = np.ascontiguousarray(pos, dtype=np.int32)
    T = x.shape[0]
    lib().orc_qk_norm_rope_rows(_p(x), None if w is None else _p(w), T, n_heads, head_dim, eps, n_rot, _p(pos),
                                theta, freq_scale, layout, threads)
    return x


def softmax_rows(scores, n_valid=None, threads: int = 1) -> np.ndarray:
    s = _f32(scores)
    rows = s.reshape(-1, s.shape[-1])
    out = np.empty_like(rows)
    nv = None if n_valid is None else np.ascontiguousarray(n_valid, dtype=np.int32)
    lib().orc_softmax_rows(_p(rows), _p(out), rows.shape[0], rows.shape[1], rows.shape[1],
                           None if nv is None else _p(nv), threads)
    return out.reshape(s.shape)


def silu_mul(gate, up, threads: int = 1) -> np.ndarray:
    g, u = _f32(gate), _f32(up)
    out = np.empty_like(g)
    lib().orc_silu_mul(_p(g), _p(u), _p(out), g.size, threads)
    return out


def quantize_rows_q8_k(x, threads: int = 1):
    """Rows of `x` [..., n] -> (d [T, nb] f32, qs [T, nb*256] i8, bsums [T, nb*16] i16), nb = ceil(n / 256)."""
    a = _f32(x)
    rows = a.reshape(-1, a.shape[-1])
    T, n = rows.shape
    nb = (n + 255) // 256
    d = np.empty((T, nb), np.float32); qs = np.empty((T, nb * 256), np.int8); bs = np.empty((T, nb * 16), np.int16)
    lib().orc_quantize_rows_q8_k(_p(rows), T, n, _p(d), _p(qs), _p(bs), threads)
    return d, qs, bs


def get_scale_min_k4(j: int, scales) -> tuple:
    s = np.ascontiguousarray(scales, dtype=np.uint8)
    sc, m = C.c_uint8(), C.c_uint8()
    lib().orc_get_scale_min_k4(j, _p(s), C.byref(sc), C.byref(m))
    return int(sc.value), int(m.value)


_DEQ = {Q2_K: "orc_dequant_q2_k", Q5_0: "orc_dequant_q5_0", Q5_K: "orc_dequant_q5_k", Q8_0: "orc_dequant_q8_0", Q4_K: "orc_dequant_q4_k", Q6_K: "orc_dequant_q6_k", F32: "orc_dequant_f32",
        F16: "orc_dequant_f16", BF16: "orc_dequant_bf16"}


def dequant(dtype: int, data, n: int):
    """Returns (status, values) like the reference's Result<Vec<f32>>."""
    d = np.ascontiguousarray(data, dtype=np.uint8)
    out = np.zeros(n, dtype=np.float32)
    st = getattr(lib(), _DEQ[dtype])(_p(d), d.size, n, _p(out))
    return int(st), out


def dequant_row(dtype: int, data, byte_offset: int, row_len: int, n_rows: int, row: int):
    d = np.ascontiguousarray(data, dtype=np.uint8).reshape(-1)
    out = np.zeros(row_len, dtype=np.float32)
    st = lib().orc_dequant_row(dtype, _p(d), d.size, byte_offset, row_len, n_rows, row, _p(out))
    return int(st), out


def get_rows(dtype: int, table, n_vocab: int, row_len: int, ids, threads: int = 1):
    t = np.ascontiguousarray(table, dtype=np.uint8).reshape(-1)
    ids = np.ascontiguousarray(ids, dtype=np.uint32)
    out = np.empty((ids.size, row_len), dtype=np.float32)
    st = lib().orc_get_rows(dtype, _p(t), t.size, n_vocab, row_len, _p(ids), ids.size, _p(out), threads)
    return int(st), out


def kv_bytes_per_token(dtype: int, hd: int) -> int:
    return int(lib().orc_kv_bytes_per_token(dtype, hd))


def kv_write_rows(dtype: int, x, pos, cache: np.ndarray) -> None:
    """Packs the rows of x [T, hd] into the slots pos[t] of cache [max_seq, bytes_per_token] (uint8, in place)."""
    x = _f32(x)
    pos = np.ascontiguousarray(pos, dtype=np.int32)
    T, hd = x.shape
    lib().orc_kv_write_rows(dtype, _p(x), T, hd, _p(pos), _p(cache))


def kv_read(dtype: int, cache: np.ndarray, n_pos: int, hd: int) -> np.ndarray:
    out = np.empty((n_pos, hd), dtype=np.float32)
    lib().orc_kv_read(dtype, _p(cache), n_pos, hd, _p(out))
    return out


def router_top2(logits):
    l = _f32(logits)
    T, E = l.shape
    idx = np.empty((T, 2), dtype=np.int32)
    w = np.empty((T, 2), dtype=np.float32)
    lib().orc_router_top2(_p(l), T, E, _p(idx), _p(w))
    return idx, w


def gather_rows_by_expert(x, idx, n_experts: int):
    x = _f32(x)
    idx = np.ascontiguousarray(idx, dtype=np.int32)
    T, H = x.shape
    out = np.empty((2 * T, H), dtype=np.float32)
    offsets = np.empty(n_experts + 1, dtype=np.int32)
    src_token = np.empty(2 * T, dtype=np.int32)
    src_slot = np.empty(2 * T, dtype=np.int32)
    lib().orc_gather_rows_by_expert(_p(x), T, H, _p(idx), n_experts, _p(out), _p(offsets), _p(src_token), _p(src_slot))
    return out, offsets, src_token, src_slot
