"""Non-finite and extreme inputs: the kernels must answer like the reference's CPU loops do —
NaN where they give NaN, the same infinities and zeros, and the usual tolerance on what stays
finite.  (No kernel traps or stalls on such data; these are ordinary values to the hardware.)"""
import numpy as np
import pytest

from agention_infer_b200 import AGN_ROPE_NEOX, AGN_ROPE_NORMAL, synth
from oracle import oracle as orc

pytestmark = pytest.mark.gpu
TOL = 1e-5
NAN, INF = np.float32(np.nan), np.float32(np.inf)


def same(got, ref, scale_rows=True):
    got, ref = np.asarray(got, np.float32), np.asarray(ref, np.float32)
    assert np.array_equal(np.isnan(got), np.isnan(ref)), (np.argwhere(np.isnan(got) != np.isnan(ref))[:5])
    inf = np.isinf(ref)
    assert np.array_equal(got[inf], ref[inf])
    fin = np.isfinite(ref)
    if scale_rows:
        scale = np.where(fin, np.abs(ref), 0).max(axis=-1, keepdims=True)
        scale = np.broadcast_to(np.maximum(scale, 1e-30), ref.shape)
    else:
        scale = np.maximum(np.abs(ref), 1.0)
    with np.errstate(invalid="ignore"):
        assert np.all(np.abs(got[fin].astype(np.float64) - ref[fin]) <= TOL * scale[fin])


def test_silu_mul_extremes(backend):
    g = np.array([0.0, -0.0, 1e-40, -1e-40, 88.0, -88.0, 100.0, -100.0, 1e30, -1e30, INF, -INF, NAN, 1.0, -1.0, 20.0] * 9, np.float32)
    u = np.array([1.0, -2.0, 3.0, 1e30, INF, 0.0, NAN, -0.0, 1e-40] * 16, np.float32)
    ref = orc.silu_mul(g, u)
    out = backend.launch_silu_mul(backend.upload(g), backend.upload(u), g.size)
    with np.errstate(all="ignore"):
        same(backend.read(out, np.float32, (g.size,)), ref, scale_rows=False)


@pytest.mark.parametrize("H", [256, 3584, 250])
def test_rms_norm_rows_with_nonfinite_values(backend, H):
    x = synth.activations(2, "x", (8, H))
    x[1, 5] = INF; x[2, 7] = NAN; x[3, :] = 0.0; x[4, :] = np.float32(1e-30); x[5, 3] = -INF; x[6, :] *= np.float32(1e15)
    w = synth.norm_weight(2, "w", H)
    with np.errstate(all="ignore"):
        ref = orc.rms_norm_rows(x, w, 1e-6)
        same(backend.read(backend.launch_rms_norm(backend.upload(x), backend.upload(w), 8, H, 1e-6), np.float32, (8, H)), ref)
        d = synth.activations(2, "delta", (8, H))
        rx, rn = orc.add_residual_rms_norm_rows(x, d, w, 1e-6)
        nx, nm = backend.launch_add_residual_rms_norm(backend.upload(x), backend.upload(d), backend.upload(w), 8, H, 1e-6)
        same(backend.read(nx, np.float32, (8, H)), rx)
        same(backend.read(nm, np.float32, (8, H)), rn)


@pytest.mark.parametrize("L", [8, 100, 512, 4096, 9999, 20000])
def test_softmax_rows_with_nonfinite_values(backend, L):
    """L covers the thread-, warp- and CTA-per-row kernels, the scalar fallback (9999) and the
    cluster kernel (20000)."""
    R = 8
    s = synth.activations(1, "scores", (R, L), std=2.0)
    nv = np.array([L, L - 1, L, max(1, L - 2), L, L // 2 + 1, L, 3], dtype=np.int32)
    s[0, 1] = -INF; s[0, L - 1] = -INF        # masked entries: probability 0
    s[1, 2] = NAN                             # one NaN poisons the row, but not the zero tail
    s[2, 0] = INF                             # inf - inf
    s[3, : L - 2] = -INF if L > 2 else s[3, : L - 2]   # every valid entry masked
    s[5, L // 2 + 1:] = NAN                   # garbage past the valid length is never read
    s[6, :] = np.float32(-1e30)               # constant huge negative row: uniform
    with np.errstate(all="ignore"):
        ref = orc.softmax_rows(s, nv)
        got = backend.read(backend.launch_softmax_rows(backend.upload(s), R, L, n_valid=backend.upload(nv)), np.float32, (R, L))
        same(got, ref)
    assert np.all(got[np.arange(L)[None, :] >= nv[:, None]] == 0.0)


@pytest.mark.parametrize("layout", [AGN_ROPE_NEOX, AGN_ROPE_NORMAL])
def test_rope_with_nonfinite_values(backend, layout):
    T, nq, nkv, hd = 6, 4, 2, 128
    q, k = synth.activations(2, "q", (T, nq * hd)), synth.activations(2, "k", (T, nkv * hd))
    q[0, 3] = INF; q[1, 70] = NAN; k[2, 5] = -INF; q[3, :] = 0.0; k[4, 64] = np.float32(1e38)
    pos = np.array([0, 1, 5, 7, 31000, 2], np.int32)
    with np.errstate(all="ignore"):
        rq = orc.rope_rows(q.copy(), nq, hd, hd, pos, 1e6, 1.0, layout)
        rk = orc.rope_rows(k.copy(), nkv, hd, hd, pos, 1e6, 1.0, layout)
        dq, dk = backend.upload(q), backend.upload(k)
        backend.launch_rope_qk(dq, dk, T, nq, nkv, hd, hd, backend.upload(pos), 1e6, 1.0, layout)
        same(backend.read(dq, np.float32, (T, nq, hd)), rq.reshape(T, nq, hd))
        same(backend.read(dk, np.float32, (T, nkv, hd)), rk.reshape(T, nkv, hd))
