"""Independent numpy statements of the quant codecs and float ops, used to cross-check the
C oracle (a second restatement written from the block-layout descriptions in
src/quant/q8_0.rs:1-7, q4_k.rs:1-16, q6_k.rs:1-15 and from the GPU kernels' second statement
of the same layouts, src/ops/kernels_wgpu.rs:1380-1410, :1655-1701)."""
import numpy as np


def f16(bits_u8_pairs: np.ndarray) -> np.ndarray:
    """[..., 2] uint8 little-endian -> f32 (exact widening)."""
    return np.ascontiguousarray(bits_u8_pairs).view(np.float16)[..., 0].astype(np.float32)


def dequant_q8_0(data: np.ndarray, n: int) -> np.ndarray:
    nb = (n + 31) // 32
    blk = np.ascontiguousarray(data[: nb * 34]).reshape(nb, 34)
    d = f16(blk[:, 0:2])
    q = blk[:, 2:].view(np.int8).astype(np.float32)
    return (d[:, None] * q).reshape(-1)[:n]


def scale_min_k4(scales: np.ndarray):
    """[nb, 12] uint8 -> (sc [nb, 8], m [nb, 8]) uint8."""
    s = scales.astype(np.uint8)
    sc = np.empty(s.shape[:-1] + (8,), dtype=np.uint8)
    m = np.empty_like(sc)
    sc[..., :4] = s[..., 0:4] & 63
    m[..., :4] = s[..., 4:8] & 63
    sc[..., 4:] = (s[..., 8:12] & 0xF) | ((s[..., 0:4] >> 6) << 4)
    m[..., 4:] = (s[..., 8:12] >> 4) | ((s[..., 4:8] >> 6) << 4)
    return sc, m


def dequant_q4_k(data: np.ndarray, n: int) -> np.ndarray:
    nb = (n + 255) // 256
    blk = np.ascontiguousarray(data[: nb * 144]).reshape(nb, 144)
    d, dmin = f16(blk[:, 0:2]), f16(blk[:, 2:4])
    sc, m = scale_min_k4(blk[:, 4:16])
    qs = blk[:, 16:].reshape(nb, 4, 32)
    lo = (qs & 0xF).astype(np.float32)
    hi = (qs >> 4).astype(np.float32)
    q = np.stack([lo, hi], axis=2).reshape(nb, 8, 32)  # group g: low run then high run
    dd = (d[:, None] * sc.astype(np.float32)).astype(np.float32)
    mm = (dmin[:, None] * m.astype(np.float32)).astype(np.float32)
    out = (dd[:, :, None] * q).astype(np.float32) - mm[:, :, None]
    return out.astype(np.float32).reshape(-1)[:n]


def dequant_q5_k(data: np.ndarray, n: int) -> np.ndarray:
    nb = (n + 255) // 256
    blk = np.ascontiguousarray(data[: nb * 176]).reshape(nb, 176)
    d, dmin = f16(blk[:, 0:2]), f16(blk[:, 2:4])
    sc, m = scale_min_k4(blk[:, 4:16])
    qh = blk[:, 16:48]                                   # [nb, 32]
    qs = blk[:, 48:].reshape(nb, 4, 32)
    sub = np.arange(8)
    hbit = ((qh[:, None, :] >> sub[None, :, None]) & 1).astype(np.uint8) * 16   # sub-block s uses bit s
    lo = (qs & 0xF)
    hi = (qs >> 4)
    q = np.stack([lo, hi], axis=2).reshape(nb, 8, 32) + hbit
    dd = (d[:, None] * sc.astype(np.float32)).astype(np.float32)
    mm = (dmin[:, None] * m.astype(np.float32)).astype(np.float32)
    out = (dd[:, :, None] * q.astype(np.float32)).astype(np.float32) - mm[:, :, None]
    return out.astype(np.float32).reshape(-1)[:n]


def dequant_q5_0(data: np.ndarray, n: int) -> np.ndarray:
    nb = (n + 31) // 32
    blk = np.ascontiguousarray(data[: nb * 22]).reshape(nb, 22)
    d = f16(blk[:, 0:2])
    qh = np.ascontiguousarray(blk[:, 2:6]).view("<u4")[:, 0]
    qs = blk[:, 6:]
    j = np.arange(16)
    b0 = ((qh[:, None] >> j[None, :]) & 1).astype(np.int32)
    b1 = ((qh[:, None] >> (j[None, :] + 16)) & 1).astype(np.int32)
    x0 = ((qs & 0xF).astype(np.int32) | (b0 << 4)) - 16
    x1 = ((qs >> 4).astype(np.int32) | (b1 << 4)) - 16
    x = np.concatenate([x0, x1], axis=1).astype(np.float32)
    return (x * d[:, None]).astype(np.float32).reshape(-1)[:n]


def dequant_q2_k(data: np.ndarray, n: int) -> np.ndarray:
    nb = n // 256
    blk = np.ascontiguousarray(data[: nb * 84]).reshape(nb, 84)
    sc = blk[:, 0:16]
    qs = blk[:, 16:80].reshape(nb, 2, 32)                 # [group][byte]
    d, dmin = f16(blk[:, 80:82]), f16(blk[:, 82:84])
    shifts = np.arange(4, dtype=np.uint8) * 2
    q = ((qs[:, :, None, :] >> shifts[None, None, :, None]) & 3).astype(np.float32)   # [nb, group, shift, 32]
    q = q.reshape(nb, 16, 16)                             # 16 runs of 16 values, one scale byte each
    dl = (d[:, None] * (sc & 0xF).astype(np.float32)).astype(np.float32)
    ml = (dmin[:, None] * (sc >> 4).astype(np.float32)).astype(np.float32)
    out = (dl[:, :, None] * q).astype(np.float32) - ml[:, :, None]
    return out.astype(np.float32).reshape(-1)[:n]


def dequant_q6_k(data: np.ndarray, n: int) -> np.ndarray:
    nb = (n + 255) // 256
    blk = np.ascontiguousarray(data[: nb * 210]).reshape(nb, 210)
    ql = blk[:, 0:128].reshape(nb, 2, 2, 32)      # [half][first/second 32][l]
    qh = blk[:, 128:192].reshape(nb, 2, 32)
    sc = blk[:, 192:208].view(np.int8).astype(np.float32).reshape(nb, 2, 8)
    d = f16(blk[:, 208:210])
    q = np.empty((nb, 2, 4, 32), dtype=np.int32)
    q[:, :, 0] = (ql[:, :, 0] & 0xF) | (((qh >> 0) & 3) << 4)
    q[:, :, 1] = (ql[:, :, 1] & 0xF) | (((qh >> 2) & 3) << 4)
    q[:, :, 2] = (ql[:, :, 0] >> 4) | (((qh >> 4) & 3) << 4)
    q[:, :, 3] = (ql[:, :, 1] >> 4) | (((qh >> 6) & 3) << 4)
    q -= 32
    l = np.arange(32)
    c = np.arange(4)
    sidx = (l[None, :] // 16) + 2 * c[:, None]           # [4, 32] scale index inside the half
    s = sc[:, :, sidx]                                    # [nb, 2, 4, 32]
    ds = (d[:, None, None, None] * s).astype(np.float32)
    return (ds * q.astype(np.float32)).astype(np.float32).reshape(-1)[:n]


def quantize_rows_q8_k(x: np.ndarray):
    """Second statement of quantize_row_q8_k (src/quant/q8_k.rs:49-92), vectorised over rows and blocks:
    x [T, n] f32 -> (d [T, nb], qs [T, nb*256] i8, bsums [T, nb*16] i16)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    T, n = x.shape
    nb = (n + 255) // 256
    xp = np.zeros((T, nb * 256), np.float32); xp[:, :n] = x
    valid = np.zeros((T, nb * 256), bool); valid[:, :n] = True
    xb, vb = xp.reshape(T, nb, 256), valid.reshape(T, nb, 256)
    av = np.where(vb & ~np.isnan(xb), np.abs(xb), np.float32(0.0))  # NaN never passes `av > amax`
    first = np.argmax(av, axis=2)  # first index of the largest magnitude, like the strict `>` scan
    amax = np.take_along_axis(av, first[..., None], 2)[..., 0]
    mx = np.take_along_axis(xb, first[..., None], 2)[..., 0]
    with np.errstate(all="ignore"):
        iscale = np.where(amax > 0, np.float32(-127.0) / np.where(amax > 0, mx, np.float32(1.0)), np.float32(0.0)).astype(np.float32)
        prod = (iscale[..., None] * xb).astype(np.float32)
        r = np.where(prod >= 0, np.floor(prod + np.float32(0.5)), np.ceil(prod - np.float32(0.5)))  # f64 intermediate is exact here
        # exact round-half-away on the f32 value: |prod| < 2^23 has an exact f64 sum with 0.5
        r = np.where(np.isnan(prod), 0.0, np.clip(r, -2147483648.0, 2147483647.0)).astype(np.int64)
        d = np.where(amax > 0, np.float32(1.0) / np.where(amax > 0, iscale, np.float32(1.0)), np.float32(0.0)).astype(np.float32)
    q = (np.minimum(r, 127) & 0xFF).astype(np.uint8).view(np.int8)
    q = np.where((amax > 0)[..., None] & vb, q, np.int8(0)).astype(np.int8)
    bs = q.reshape(T, nb, 16, 16).astype(np.int16).sum(axis=3, dtype=np.int16)
    return d, q.reshape(T, nb * 256), bs.reshape(T, nb * 16)


def rms_norm64(x, w, eps):
    x64 = x.astype(np.float64)
    rms = np.sqrt((x64 * x64).mean(axis=-1, keepdims=True) + eps)
    return w.astype(np.float64) * x64 / rms


def rope64(x, n_heads, head_dim, n_rot, pos, theta, freq_scale=1.0, layout=0):
    T = x.shape[0]
    xr = x.astype(np.float64).reshape(T, n_heads, head_dim).copy()
    half = n_rot // 2
    d = np.arange(half, dtype=np.float64)
    ang = (pos.astype(np.float64)[:, None] * freq_scale) / np.power(float(theta), 2.0 * d / n_rot)
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    if layout == 0:
        x0, x1 = xr[:, :, :half].copy(), xr[:, :, half:n_rot].copy()
        xr[:, :, :half] = x0 * c - x1 * s
        xr[:, :, half:n_rot] = x0 * s + x1 * c
    else:
        x0, x1 = xr[:, :, 0:n_rot:2].copy(), xr[:, :, 1:n_rot:2].copy()
        xr[:, :, 0:n_rot:2] = x0 * c - x1 * s
        xr[:, :, 1:n_rot:2] = x0 * s + x1 * c
    return xr.reshape(T, n_heads * head_dim)


def softmax64(s, n_valid=None):
    s64 = s.astype(np.float64)
    rows = s64.reshape(-1, s64.shape[-1])
    out = np.zeros_like(rows)
    for r in range(rows.shape[0]):
        nv = rows.shape[1] if n_valid is None else int(n_valid[r])
        if nv > 0:
            e = np.exp(rows[r, :nv] - rows[r, :nv].max())
            out[r, :nv] = e / e.sum()
    return out.reshape(s.shape)


def silu_mul64(g, u):
    g64 = g.astype(np.float64)
    return g64 / (1.0 + np.exp(-g64)) * u.astype(np.float64)
