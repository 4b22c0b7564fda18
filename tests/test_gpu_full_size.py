"""Full benchmark sizes (T = 65536 Llama-3-8B-shaped rows, the large prefill configuration):
the oracle would take minutes there, so the CUDA path is checked through properties that do
not depend on size, plus an oracle comparison on a strided sample of rows."""
import numpy as np
import pytest

from agention_infer_b200 import AGN_Q6_K, synth
from oracle import oracle as orc

pytestmark = pytest.mark.gpu
TOL = 1e-5
T, H, hd, nq, nkv, I = 65536, 4096, 128, 32, 8, 14336
THREADS = max(1, orc.max_threads())


def test_rms_norm_full_size_sample_and_scale_invariance(backend):
    x = synth.activations(4, "x", (T, H)); w = synth.norm_weight(4, "w", H)
    dx, dw = backend.upload(x), backend.upload(w)
    out = backend.launch_rms_norm(dx, dw, T, H, 0.0)
    got = backend.read(out, np.float32, (T, H))
    rows = np.arange(0, T, 257)
    assert synth.max_rel_to_row_scale(got[rows], orc.rms_norm_rows(x[rows], w, 0.0, THREADS)) <= TOL
    # with eps = 0 the op is invariant to a power-of-two scaling of x (exact in f32)
    backend.copy_h2d(dx, x * np.float32(4.0)); backend.sync()
    out2 = backend.launch_rms_norm(dx, dw, T, H, 0.0)
    assert np.array_equal(backend.read(out2, np.float32, (T, H)), got)
    # every normalised row (divided by w) has unit mean square
    ms = np.mean((got[rows] / w).astype(np.float64) ** 2, axis=1)
    assert np.allclose(ms, 1.0, rtol=1e-5)


def test_rope_full_size_inverse_rotation_and_sample(backend):
    q = synth.activations(4, "q", (T, nq * hd))
    pos = np.arange(T, dtype=np.int32)
    dq, dp = backend.upload(q), backend.upload(pos)
    backend.launch_rope(dq, T, nq, hd, hd, dp, 500000.0)
    got = backend.read(dq, np.float32, q.shape)
    rows = np.arange(0, T, 509)
    assert synth.max_rel_to_row_scale(got[rows], orc.rope_rows(q[rows], nq, hd, hd, pos[rows], 500000.0, threads=THREADS)) <= TOL
    # rotation preserves the norm of every (d, d+half) pair ...
    g3, q3 = got.reshape(T, nq, 2, hd // 2), q.reshape(T, nq, 2, hd // 2)
    n_got = g3[:, :, 0] ** 2 + g3[:, :, 1] ** 2
    n_ref = q3[:, :, 0] ** 2 + q3[:, :, 1] ** 2
    assert np.allclose(n_got, n_ref, rtol=2e-5, atol=1e-6)
    # ... and rotating back with negated positions restores the input
    backend.launch_rope(dq, T, nq, hd, hd, backend.upload(-pos), 500000.0)
    back = backend.read(dq, np.float32, q.shape)
    assert synth.max_rel_to_row_scale(back, q) <= 5e-6


def test_silu_mul_full_size_linearity_in_up(backend):
    n = 16384 * I  # 2.8 GB over the three arrays
    g = synth.activations(4, "gate", (n,)); u = synth.activations(4, "up", (n,))
    dg, du = backend.upload(g), backend.upload(u)
    out = backend.launch_silu_mul(dg, du, n)
    got = backend.read(out, np.float32, (n,))
    sl = slice(0, n, 4099)
    ref = orc.silu_mul(g[sl], u[sl])
    assert np.max(np.abs(got[sl] - ref) / np.maximum(np.abs(ref), 1.0)) <= TOL
    # out is linear in `up`: scaling up by 2 scales out by exactly 2; up = 0 gives 0
    backend.copy_h2d(du, u * np.float32(2.0)); backend.sync()
    out2 = backend.launch_silu_mul(dg, du, n)
    assert np.array_equal(backend.read(out2, np.float32, (n,)), got * np.float32(2.0))


def test_get_rows_full_size_q6k_equal_ids_equal_rows(backend):
    vocab = 128256
    table = synth.quant_table(AGN_Q6_K, vocab, H, cfg_index=4)
    ids = synth.token_ids(4, T, vocab)
    ids[1::2] = ids[0::2]  # every id appears at least twice
    dt = backend.upload(table)
    out = backend.get_rows(AGN_Q6_K, dt, table.nbytes, vocab, H, backend.upload(ids), T)
    got = backend.read(out, np.float32, (T, H))
    assert np.array_equal(got[0::2].view(np.uint32), got[1::2].view(np.uint32))
    rows = np.arange(0, T, 331)
    st, ref = orc.get_rows(AGN_Q6_K, table, vocab, H, ids[rows], THREADS)
    assert st == orc.OK and np.array_equal(got[rows].view(np.uint32), ref.view(np.uint32))
    # gathering the gathered order again from an identity id list reproduces the table rows
    ident = np.arange(4096, dtype=np.uint32)
    a = backend.read(backend.get_rows(AGN_Q6_K, dt, table.nbytes, vocab, H, backend.upload(ident), 4096), np.float32, (4096, H))
    b = backend.read(backend.get_rows(AGN_Q6_K, dt, table.nbytes, vocab, H, backend.upload(ident[::-1].copy()), 4096), np.float32, (4096, H))
    assert np.array_equal(a, b[::-1])


def test_softmax_full_rows_sum_to_one(backend):
    R, L = 32 * 2048, 2048  # 64k rows of 2048 scores, causal
    s = synth.activations(4, "scores", (R, L), std=2.0)
    out = backend.launch_softmax_rows(backend.upload(s), R, L, causal_period=L)
    got = backend.read(out, np.float32, (R, L))
    assert np.allclose(got.sum(axis=1, dtype=np.float64), 1.0, atol=2e-5)
    assert got.min() >= 0.0
    r = np.arange(0, R, 997)
    nv = (r % L + 1).astype(np.int32)
    assert synth.max_rel_to_row_scale(got[r], orc.softmax_rows(s[r], nv, THREADS)) <= TOL
    # idempotence of the support: entries past the valid length are exactly zero
    assert not got[0, 1:].any() and not got[L - 2, L - 1:].any()


def test_silu_mul_headline_size_against_the_oracle_in_full(backend):
    """The dominant kernel on the headline shape (Qwen2.5-7B-shaped prefill: 4096 rows x 18944, 77.6 M elements):
    every element against the oracle, not a sample."""
    Tq, Iq = 4096, 18944
    g = synth.activations(2, "gate", (Tq, Iq)); u = synth.activations(2, "up", (Tq, Iq))
    ref = orc.silu_mul(g, u, THREADS)
    out = backend.launch_silu_mul(backend.upload(g), backend.upload(u), Tq * Iq)
    assert backend.last_kernel == "silu_mul_vec4"
    got = backend.read(out, np.float32, (Tq, Iq))
    assert synth.max_rel_to_row_scale(got, ref) <= TOL
    assert np.max(np.abs(got - ref) / np.maximum(np.abs(ref), 1.0)) <= TOL
