"""CUDA-graph entry points: a recorded decode-shaped chain (fused norm->rope, silu*mul, rms_norm)
replays with new input contents and matches the oracle; nothing runs while recording."""
import numpy as np
import pytest

from agention_infer_b200 import BackendError, synth
from oracle import oracle as orc

pytestmark = pytest.mark.gpu
TOL = 1e-5


def test_graph_capture_and_replay(backend):
    be = backend
    T, nq, nkv, hd, I, H = 8, 28, 4, 128, 18944, 3584
    wq = synth.norm_weight(3, "wq", hd); wk = synth.norm_weight(3, "wk", hd); w = synth.norm_weight(3, "w", H)
    pos = synth.positions(3, T, True)
    dq, dk = be.empty(4 * T * nq * hd), be.empty(4 * T * nkv * hd)
    dg, du, da = be.empty(4 * T * I), be.empty(4 * T * I), be.empty(4 * T * I)
    dx, dxn = be.empty(4 * T * H), be.empty(4 * T * H)
    dwq, dwk, dw, dpos = be.upload(wq), be.upload(wk), be.upload(w), be.upload(pos)

    def chain():
        be.launch_qk_norm_rope_qk(dq, dk, dwq, dwk, T, nq, nkv, hd, 1e-6, hd, dpos, 1e6)
        be.launch_silu_mul(dg, du, T * I, out=da)
        be.launch_rms_norm(dx, dw, T, H, 1e-6, out=dxn)

    def load(salt):
        a = {n: synth.activations(3, n, s, salt=salt) for n, s in
             (("q", (T, nq * hd)), ("k", (T, nkv * hd)), ("gate", (T, I)), ("up", (T, I)), ("x", (T, H)))}
        for buf, n in ((dq, "q"), (dk, "k"), (dg, "gate"), (du, "up"), (dx, "x")):
            be.copy_h2d(buf, a[n])
        be.sync()
        return a

    load(0)
    chain(); be.sync()  # first run outside a capture builds the RoPE table
    n0 = be.launch_count
    marker = np.full((T, I), 7.0, np.float32)
    be.copy_h2d(da, marker); be.sync()
    be.graph_begin()
    chain()
    with pytest.raises(BackendError):
        be.sync()  # not allowed while recording
    g = be.graph_end()
    assert be.launch_count == n0  # recording launched nothing ...
    assert np.array_equal(be.read(da, np.float32, (T, I)), marker)  # ... and wrote nothing
    for salt in (1, 2):
        a = load(salt)
        be.graph_launch(g)
        got_q = be.read(dq, np.float32, a["q"].shape)
        assert synth.max_rel_to_row_scale(got_q, orc.qk_norm_rope_rows(a["q"], wq, nq, hd, 1e-6, hd, pos, 1e6)) <= TOL
        assert synth.max_rel_to_row_scale(be.read(dk, np.float32, a["k"].shape),
                                          orc.qk_norm_rope_rows(a["k"], wk, nkv, hd, 1e-6, hd, pos, 1e6)) <= TOL
        assert synth.max_rel_to_row_scale(be.read(da, np.float32, (T, I)), orc.silu_mul(a["gate"], a["up"])) <= TOL
        assert synth.max_rel_to_row_scale(be.read(dxn, np.float32, (T, H)), orc.rms_norm_rows(a["x"], w, 1e-6)) <= TOL
    assert be.launch_count == n0 + 2 * 3
    be.graph_destroy(g)


def test_graph_misuse_is_reported(backend):
    with pytest.raises(BackendError):
        backend.graph_end()
    w = backend.empty(256)
    backend.graph_begin()
    with pytest.raises(BackendError):
        backend.graph_begin()
    with pytest.raises(BackendError):
        backend.empty(1024)  # allocation would invalidate the capture: refused, the capture survives
    x = np.zeros((4, 64), np.float32)
    with pytest.raises(BackendError):
        backend.rms_norm_into(x, w, x.copy(), 1e-5)
    g = backend.graph_end()
    backend.graph_destroy(g)
    backend.sync()


def test_rope_with_a_cold_table_cannot_be_recorded(backend):
    """The (theta, n_rot) table is built on the host and copied from a staging slot: recording that copy would make
    every replay re-copy whatever the slot holds later.  A rope op whose table does not exist yet is refused inside a
    capture (the capture survives); after one run outside, the same op records and replays."""
    be = backend
    T, nh, hd, theta = 4, 2, 64, 12345.0 + 0.25  # a theta no other test uses: its table is certainly cold
    x = synth.activations(3, "q", (T, nh * hd)); pos = synth.positions(3, T, True)
    dx, dp = be.upload(x), be.upload(pos)
    be.graph_begin()
    with pytest.raises(BackendError) as e:
        be.launch_rope(dx, T, nh, hd, hd, dp, theta)
    assert "before" in str(e.value) and "graph" in str(e.value)
    g = be.graph_end()  # an empty graph: the refused op recorded nothing
    be.graph_destroy(g)
    assert np.array_equal(be.read(dx, np.float32, x.shape), x)
    be.launch_rope(dx, T, nh, hd, hd, dp, theta); be.sync()  # builds the table
    be.copy_h2d(dx, x); be.sync()
    be.graph_begin()
    be.launch_rope(dx, T, nh, hd, hd, dp, theta)
    g = be.graph_end()
    be.graph_launch(g)
    assert synth.max_rel_to_row_scale(be.read(dx, np.float32, x.shape), orc.rope_rows(x, nh, hd, hd, pos, theta)) <= TOL
    be.graph_destroy(g)


def test_rope_tables_used_by_a_graph_are_not_evicted(backend):
    """More (theta, n_rot) pairs than the table cache holds: a pair that a recorded graph uses keeps its slot, so the
    graph still computes with its own theta afterwards."""
    be = backend
    T, nh, hd, theta = 3, 2, 64, 777.5
    x = synth.activations(3, "q", (T, nh * hd)); pos = synth.positions(3, T, True)
    dx, dp, scratch = be.upload(x), be.upload(pos), be.upload(x)
    be.launch_rope(dx, T, nh, hd, hd, dp, theta); be.sync()
    be.copy_h2d(dx, x); be.sync()
    be.graph_begin()
    be.launch_rope(dx, T, nh, hd, hd, dp, theta)
    g = be.graph_end()
    for k in range(24):  # cycle through more pairs than there are slots
        be.launch_rope(scratch, T, nh, hd, hd, dp, 1000.0 + 17.0 * k)
    be.sync()
    be.graph_launch(g)
    assert synth.max_rel_to_row_scale(be.read(dx, np.float32, x.shape), orc.rope_rows(x, nh, hd, hd, pos, theta)) <= TOL
    be.graph_destroy(g)
