"""The float ops of the oracle have no op-level test in the reference ("parity unpinned");
they are checked here against float64 numpy and through properties of the maths."""
import numpy as np
import pytest

import tests.ref_numpy as rn
from agention_infer_b200 import synth
from oracle import oracle as orc


def test_rms_norm_vs_float64():
    x = synth.activations(1, "x", (37, 2048))
    w = synth.norm_weight(1, "w", 2048)
    got = orc.rms_norm_rows(x, w, 1e-5)
    assert synth.max_rel_to_row_scale(got, rn.rms_norm64(x, w, 1e-5).astype(np.float32)) < 2e-6


def test_rms_norm_constant_row():
    x = np.full((1, 64), 3.0, dtype=np.float32)
    got = orc.rms_norm_rows(x, np.ones(64, dtype=np.float32), 0.0)
    assert np.allclose(got, 1.0, atol=1e-6)


def test_add_residual_rms_norm_is_add_then_norm():
    x = synth.activations(1, "x", (5, 256)); d = synth.activations(1, "delta", (5, 256))
    w = synth.norm_weight(1, "w", 256)
    nx, nm = orc.add_residual_rms_norm_rows(x, d, w, 1e-5)
    assert np.array_equal(nx, x + d)
    assert np.array_equal(nm, orc.rms_norm_rows(x + d, w, 1e-5))


@pytest.mark.parametrize("layout", [orc.NEOX, orc.NORMAL])
@pytest.mark.parametrize("hd,n_rot", [(64, 64), (128, 128), (128, 64), (96, 96)])
def test_rope_vs_float64(layout, hd, n_rot):
    T, nh = 33, 6
    x = synth.activations(1, "q", (T, nh * hd))
    pos = np.arange(T, dtype=np.int32) * 7
    got = orc.rope_rows(x, nh, hd, n_rot, pos, 500000.0, 1.0, layout)
    want = rn.rope64(x, nh, hd, n_rot, pos, 500000.0, 1.0, layout)
    # f32 angle at pos ~ 230 carries ~1e-5 absolute error, so the bound is loose; the GPU is
    # compared with the oracle, not with float64
    assert np.max(np.abs(got - want)) < 2e-4
    if n_rot < hd:
        xr = x.reshape(T, nh, hd)
        assert np.array_equal(got.reshape(T, nh, hd)[:, :, n_rot:], xr[:, :, n_rot:])


def test_rope_position_zero_is_identity_and_norm_preserved():
    x = synth.activations(2, "q", (4, 4 * 128))
    assert np.array_equal(orc.rope_rows(x, 4, 128, 128, np.zeros(4, np.int32), 1e6), x)
    y = orc.rope_rows(x, 4, 128, 128, np.array([1, 100, 5000, 32767], np.int32), 1e6)
    n0 = np.linalg.norm(x.reshape(4, 4, 128), axis=-1)
    n1 = np.linalg.norm(y.reshape(4, 4, 128), axis=-1)
    assert np.allclose(n0, n1, rtol=1e-5)


def test_rope_denominators_are_libm_powf():
    d = orc.rope_denominators(1e6, 128)
    want = np.power(np.float64(1e6), 2.0 * np.arange(64) / 128.0)
    assert d[0] == 1.0 and np.allclose(d, want, rtol=2e-7)


def test_qk_norm_rope_is_norm_then_rope():
    T, nh, hd = 9, 3, 128
    x = synth.activations(2, "q", (T, nh * hd)); w = synth.norm_weight(2, "wq", hd)
    pos = np.arange(T, dtype=np.int32) + 3
    fused = orc.qk_norm_rope_rows(x, w, nh, hd, 1e-6, hd, pos, 1e6)
    normed = orc.rms_norm_rows(x.reshape(T * nh, hd), w, 1e-6).reshape(T, nh * hd)
    assert np.array_equal(fused, orc.rope_rows(normed, nh, hd, hd, pos, 1e6))


def test_softmax_vs_float64_and_rows_sum_to_one():
    s = synth.causal_scores(1, 2, 64)
    nv = np.tile(np.arange(1, 65, dtype=np.int32), 2)
    got = orc.softmax_rows(s, nv)
    want = rn.softmax64(s.reshape(-1, 64), nv).reshape(s.shape)
    assert np.max(np.abs(got - want)) < 1e-6
    assert np.allclose(got.reshape(-1, 64).sum(axis=1), 1.0, atol=1e-5)
    tri = np.triu(np.ones((64, 64), dtype=bool), k=1)
    assert not got[:, tri].any()


def test_silu_mul_vs_float64():
    g = synth.activations(1, "gate", (3, 8192)); u = synth.activations(1, "up", (3, 8192))
    got = orc.silu_mul(g, u)
    assert synth.max_rel_to_row_scale(got, rn.silu_mul64(g, u).astype(np.float32)) < 1e-6
    assert np.array_equal(got, orc.silu_mul(g, u, threads=4))


def test_router_top2_and_gather():
    logits = synth.activations(5, "logits", (50, 8))
    idx, w = orc.router_top2(logits)
    p = rn.softmax64(logits)
    order = np.argsort(-p, axis=1, kind="stable")[:, :2]
    assert np.array_equal(idx, order.astype(np.int32))
    assert np.allclose(w, np.take_along_axis(p, order, axis=1), atol=1e-6)
    x = synth.activations(5, "x", (50, 16))
    out, offs, tok, slot = orc.gather_rows_by_expert(x, idx, 8)
    assert offs[0] == 0 and offs[-1] == 100
    assert np.array_equal(out, x[tok])
    for e in range(8):
        seg = slice(offs[e], offs[e + 1])
        assert np.all(idx[tok[seg], slot[seg]] == e)
        assert np.all(np.diff(tok[seg]) >= 0)  # stable: ascending token order
