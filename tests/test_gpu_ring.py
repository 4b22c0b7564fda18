"""The persistent kernels with a staged row ring (rms_norm, add_residual_rms_norm, rope, fused
norm->rope, get_rows) against the CPU oracle, called through the C ABI.

They are opt-in (options "rms_ring", "rope_ring", "get_rows_ring"; the CTA-per-row kernels are
the measured-faster default); the option "ring_force" makes small and ragged batches take them too, so that the partial last unit, rows that wrap the ring several times, one
row per CTA and the chunked copy of the table's last row are all covered.  get_rows is
bit-exact; float ops are within 1e-5 of the row scale.  The persistent and the CTA-per-row
kernels perform the same operations in the same order, so their outputs are also compared bit
for bit."""
import numpy as np
import pytest

from agention_infer_b200 import _abi
from agention_infer_b200 import (AGN_BF16, AGN_F16, AGN_Q4_K, AGN_Q5_0, AGN_Q5_K, AGN_Q6_K, AGN_Q8_0, AGN_Q2_K, AGN_ROPE_NEOX,
                                 AGN_ROPE_NORMAL, BackendError, synth)
from oracle import oracle as orc

pytestmark = pytest.mark.gpu

TOL = 1e-5
THREADS = max(1, orc.max_threads())


def rel(got, ref):
    return synth.max_rel_to_row_scale(got, ref)


def bits(a):
    return np.ascontiguousarray(a).view(np.uint32)


@pytest.fixture()
def ring(backend):
    """Backend with the persistent kernels forced on; options restored afterwards."""
    for name in ("ring_force", "rms_ring", "rope_ring", "get_rows_ring", "softmax_ring"):
        backend.set_option(name, 1)
    yield backend
    for name in ("ring_force", "rms_ring", "rms_ring_ctas", "rope_ring", "rope_ring_ctas", "get_rows_ring", "get_rows_ring_ctas",
                 "softmax_ring", "softmax_ring_ctas"):
        backend.set_option(name, 0)


@pytest.mark.parametrize("slots,ctas", [(1, 0), (2, 1), (5, 2)])
@pytest.mark.parametrize("T,H", [(1, 3584), (7, 1024), (700, 3584), (333, 4096), (41, 8192), (9, 16384), (1500, 128)])
def test_rms_norm_ring(ring, T, H, slots, ctas):
    ring.set_option("rms_ring", slots); ring.set_option("rms_ring_ctas", ctas)
    x = synth.activations(2, "x", (T, H)); w = synth.norm_weight(2, "w", H)
    ref = orc.rms_norm_rows(x, w, 1e-6, THREADS)
    dx, dw = ring.upload(x), ring.upload(w)
    got = ring.read(ring.launch_rms_norm(dx, dw, T, H, 1e-6), np.float32, (T, H))
    assert ring.last_kernel == "rms_norm_ring"
    assert rel(got, ref) <= TOL
    ring.set_option("rms_ring", 0)
    old = ring.read(ring.launch_rms_norm(dx, dw, T, H, 1e-6), np.float32, (T, H))
    assert ring.last_kernel == "rms_norm"
    assert np.array_equal(bits(got), bits(old))


@pytest.mark.parametrize("T,H", [(5, 3584), (600, 4096), (37, 1024)])
def test_add_residual_rms_norm_ring(ring, T, H):
    x = synth.activations(4, "x", (T, H)); d = synth.activations(4, "delta", (T, H)); w = synth.norm_weight(4, "w", H)
    ref_nx, ref_nm = orc.add_residual_rms_norm_rows(x, d, w, 1e-5)
    nx, nm = ring.launch_add_residual_rms_norm(ring.upload(x), ring.upload(d), ring.upload(w), T, H, 1e-5)
    assert ring.last_kernel == "rms_norm_ring"
    assert np.array_equal(bits(ring.read(nx, np.float32, (T, H))), bits(ref_nx))
    assert rel(ring.read(nm, np.float32, (T, H)), ref_nm) <= TOL


def test_rms_norm_ring_in_place(ring):
    T, H = 900, 2048
    x = synth.activations(2, "x", (T, H)); w = synth.norm_weight(2, "w", H)
    ref = orc.rms_norm_rows(x, w, 1e-5, THREADS)
    dx = ring.upload(x)
    ring.launch_rms_norm(dx, ring.upload(w), T, H, 1e-5, out=dx)  # a row is staged before it is overwritten
    assert ring.last_kernel == "rms_norm_ring"
    assert rel(ring.read(dx, np.float32, (T, H)), ref) <= TOL


@pytest.mark.parametrize("out_dtype", [AGN_F16, AGN_BF16])
def test_rms_norm_out16_ring(ring, out_dtype):
    T, H = 450, 3584
    x = synth.activations(2, "x", (T, H)); w = synth.norm_weight(2, "w", H)
    dx, dw = ring.upload(x), ring.upload(w)
    got = ring.read(ring.launch_rms_norm_out16(dx, dw, T, H, 1e-6, out_dtype), np.uint16, (T, H))
    assert ring.last_kernel == "rms_norm_ring"
    ring.set_option("rms_ring", 0)
    old = ring.read(ring.launch_rms_norm_out16(dx, dw, T, H, 1e-6, out_dtype), np.uint16, (T, H))
    assert np.array_equal(got, old)


def test_rms_norm_natural_ring_size(backend):
    """With "rms_ring" = 1 (automatic depth) 4096 rows engage the persistent kernel; 64 rows do not."""
    T, H = 4096, 3584
    backend.set_option("rms_ring", 1)
    try:
        _rms_natural(backend, T, H)
    finally:
        backend.set_option("rms_ring", 0)


def _rms_natural(backend, T, H):
    x = synth.activations(2, "x", (T, H)); w = synth.norm_weight(2, "w", H)
    ref = orc.rms_norm_rows(x, w, 1e-6, THREADS)
    got = backend.read(backend.launch_rms_norm(backend.upload(x), backend.upload(w), T, H, 1e-6), np.float32, (T, H))
    assert backend.last_kernel == "rms_norm_ring"
    assert rel(got, ref) <= TOL
    backend.launch_rms_norm(backend.upload(x[:64]), backend.upload(w), 64, H, 1e-6)
    assert backend.last_kernel == "rms_norm"


ROPE_RING_CASES = [  # T, n_q, n_kv, head_dim, n_rot, theta
    (700, 28, 4, 128, 128, 1e6), (1, 28, 4, 128, 128, 1e6), (333, 32, 8, 64, 64, 5e5), (77, 8, 2, 128, 64, 1e4),
    (50, 16, 0, 256, 256, 1e7), (91, 2, 1, 32, 32, 1e4), (45, 3, 3, 96, 96, 1e4), (19, 2, 2, 512, 512, 1e4),
]


@pytest.mark.parametrize("norm", [False, True])
@pytest.mark.parametrize("layout", [AGN_ROPE_NEOX, AGN_ROPE_NORMAL])
@pytest.mark.parametrize("T,nq,nkv,hd,n_rot,theta", ROPE_RING_CASES)
def test_rope_ring(ring, norm, layout, T, nq, nkv, hd, n_rot, theta):
    ring.set_option("rope_ring", 2 if T % 2 else 4); ring.set_option("rope_ring_ctas", 1 if T < 100 else 0)
    q = synth.activations(3, "q", (T, nq * hd)); k = synth.activations(3, "k", (T, max(nkv, 1) * hd))
    wq = synth.norm_weight(3, "wq", hd); wk = synth.norm_weight(3, "wk", hd)
    pos = synth.positions(3, T, True)
    if norm:
        rq = orc.qk_norm_rope_rows(q, wq, nq, hd, 1e-6, n_rot, pos, theta, 1.0, layout, THREADS)
        rk = orc.qk_norm_rope_rows(k, wk, max(nkv, 1), hd, 1e-6, n_rot, pos, theta, 1.0, layout, THREADS)
    else:
        rq = orc.rope_rows(q, nq, hd, n_rot, pos, theta, 1.0, layout, THREADS)
        rk = orc.rope_rows(k, max(nkv, 1), hd, n_rot, pos, theta, 1.0, layout, THREADS)
    dp, dwq, dwk = ring.upload(pos), ring.upload(wq), ring.upload(wk)

    def run():
        dq, dk = ring.upload(q), ring.upload(k)
        if norm:
            ring.launch_qk_norm_rope_qk(dq, dk if nkv else None, dwq, dwk if nkv else None, T, nq, nkv, hd, 1e-6, n_rot, dp, theta,
                                        1.0, layout)
        else:
            ring.launch_rope_qk(dq, dk if nkv else None, T, nq, nkv, hd, n_rot, dp, theta, 1.0, layout)
        kernels.append(ring.last_kernel)
        return ring.read(dq, np.float32, q.shape), ring.read(dk, np.float32, k.shape)

    kernels = []
    gq, gk = run()
    assert rel(gq, rq) <= TOL
    if nkv:
        assert rel(gk, rk) <= TOL
    else:
        assert np.array_equal(gk, k)  # untouched
    ring.set_option("rope_ring", 0)
    oq, ok = run()
    assert np.array_equal(bits(gq), bits(oq)) and np.array_equal(bits(gk), bits(ok))
    # (head_dim 96 with NeoX pairing has no register fast path, persistent or not: it runs the generic kernel)
    has_fast_path = not (hd == 96 and layout == AGN_ROPE_NEOX)
    assert kernels[0].endswith("_ring") == has_fast_path and not kernels[1].endswith("_ring")
    if has_fast_path:
        assert kernels[0] == ("qk_norm_rope_ring" if norm else "rope_ring")


def test_rope_natural_ring_size(backend):
    T, nq, nkv, hd = 4096, 28, 4, 128
    q = synth.activations(2, "q", (T, nq * hd)); k = synth.activations(2, "k", (T, nkv * hd))
    pos = synth.positions(2, T, False)
    rq = orc.rope_rows(q, nq, hd, hd, pos, 1e6, 1.0, 0, THREADS); rk = orc.rope_rows(k, nkv, hd, hd, pos, 1e6, 1.0, 0, THREADS)
    dq, dk = backend.upload(q), backend.upload(k)
    backend.set_option("rope_ring", 1)
    try:
        backend.launch_rope_qk(dq, dk, T, nq, nkv, hd, hd, backend.upload(pos), 1e6)
        assert backend.last_kernel == "rope_ring"
    finally:
        backend.set_option("rope_ring", 0)
    assert rel(backend.read(dq, np.float32, q.shape), rq) <= TOL
    assert rel(backend.read(dk, np.float32, k.shape), rk) <= TOL


@pytest.mark.parametrize("slots,ctas", [(1, 0), (2, 1), (7, 3)])
@pytest.mark.parametrize("dtype,vocab,H,T", [(AGN_Q4_K, 3000, 3584, 700), (AGN_Q8_0, 1000, 2048, 333), (AGN_Q6_K, 900, 4096, 41),
                                             (AGN_Q5_K, 500, 1024, 1), (AGN_Q5_0, 400, 96, 1200), (AGN_Q2_K, 300, 512, 65),
                                             (AGN_Q8_0, 50, 33, 77)])
def test_get_rows_ring(ring, dtype, vocab, H, T, slots, ctas):
    ring.set_option("get_rows_ring", slots); ring.set_option("get_rows_ring_ctas", ctas)
    table = synth.quant_table(dtype, vocab, H, cfg_index=2)
    ids = synth.token_ids(2, T, vocab)
    ids[::7] = vocab - 1  # the table's last row: its 16-byte rounded span may reach past the end (chunked copy)
    st, ref = orc.get_rows(dtype, table, vocab, H, ids)
    assert st == orc.OK
    out = ring.get_rows(dtype, ring.upload(table), table.nbytes, vocab, H, ring.upload(ids), T)
    assert ring.last_kernel == "get_rows_ring"
    assert np.array_equal(bits(ring.read(out, np.float32, (T, H))), bits(ref))


def test_get_rows_ring_out_of_range_id(ring):
    dtype, vocab, H, T = AGN_Q4_K, 2000, 1024, 500
    table = synth.quant_table(dtype, vocab, H, cfg_index=2)
    ids = synth.token_ids(2, T, vocab)
    ids[[3, 250, 499]] = [vocab, 2 ** 31, 2 ** 32 - 1]
    _, ref = orc.get_rows(dtype, table, vocab, H, ids)
    out = ring.get_rows(dtype, ring.upload(table), table.nbytes, vocab, H, ring.upload(ids), T)
    assert ring.last_kernel == "get_rows_ring"
    with pytest.raises(BackendError) as e:
        ring.sync()
    assert e.value.status == _abi.AGN_EOOB_ID
    got = ring.read(out, np.float32, (T, H))
    assert np.array_equal(bits(got), bits(ref))  # zero rows for the bad ids, every other row exact
    assert not got[[3, 250, 499]].any()


def test_get_rows_natural_ring_size(backend):
    dtype, vocab, H, T = AGN_Q4_K, 20000, 3584, 8192
    table = synth.quant_table(dtype, vocab, H, cfg_index=2)
    ids = synth.token_ids(2, T, vocab)
    _, ref = orc.get_rows(dtype, table, vocab, H, ids, THREADS)
    backend.set_option("get_rows_ring", 1)
    try:
        out = backend.get_rows(dtype, backend.upload(table), table.nbytes, vocab, H, backend.upload(ids), T)
        assert backend.last_kernel == "get_rows_ring"
    finally:
        backend.set_option("get_rows_ring", 0)
    assert np.array_equal(bits(backend.read(out, np.float32, (T, H))), bits(ref))


@pytest.mark.parametrize("slots,ctas", [(1, 0), (2, 1), (6, 2)])
@pytest.mark.parametrize("R,L", [(300, 2048), (77, 1028), (9, 8192), (5, 16384), (1, 4096)])
def test_softmax_ring_ragged_rows(ring, R, L, slots, ctas):
    """Rows of 1K-32K entries with ragged valid lengths (full, one entry, none, everything in between): the
    persistent kernel against the oracle, and bit for bit against the CTA-per-row kernel (same thread
    mapping, same reduction order).  Zero-filled and valid-only forms, f32 and bf16 rows, sums."""
    ring.set_option("softmax_ring", slots); ring.set_option("softmax_ring_ctas", ctas)
    s = synth.activations(5, "logits", (R, L), std=2.0)
    nv = synth.rng_for(5, "pos").integers(0, L + 1, size=R, dtype=np.int32)
    nv[:3] = [L, 1, 0][:min(3, R)]
    ref = orc.softmax_rows(s, nv, THREADS)
    ds, dnv = ring.upload(s), ring.upload(nv)
    got = ring.read(ring.launch_softmax_rows(ds, R, L, n_valid=dnv), np.float32, (R, L))
    assert ring.last_kernel == "softmax_ring"
    drift = 0.0
    assert rel(got, ref) <= TOL + drift
    valid = np.arange(L)[None, :] < nv[:, None]
    assert not got[~valid].any()
    sentinel = ring.upload(np.full((R, L), -7.25, np.float32))
    ring.launch_softmax_rows_valid(ds, R, L, sentinel, n_valid=dnv)
    assert ring.last_kernel == "softmax_ring"
    g2 = ring.read(sentinel, np.float32, (R, L))
    assert np.array_equal(bits(g2[valid]), bits(got[valid])) and np.all(g2[~valid] == -7.25)
    sums = ring.empty(4 * R)
    w16 = ring.read(ring.launch_softmax_rows_scaled_out16(ds, R, L, 0.5, AGN_BF16, sums=sums, n_valid=dnv), np.uint16, (R, L))
    sm = ring.read(sums, np.float32, (R,))
    ring.set_option("softmax_ring", 0)
    old = ring.read(ring.launch_softmax_rows(ds, R, L, n_valid=dnv), np.float32, (R, L))
    assert not ring.last_kernel.endswith("_ring")
    assert np.array_equal(bits(got), bits(old))
    sums2 = ring.empty(4 * R)
    w16_old = ring.read(ring.launch_softmax_rows_scaled_out16(ds, R, L, 0.5, AGN_BF16, sums=sums2, n_valid=dnv), np.uint16, (R, L))
    assert np.array_equal(w16, w16_old) and np.array_equal(bits(sm), bits(ring.read(sums2, np.float32, (R,))))


def test_softmax_ring_square_causal(ring):
    heads, L = 3, 2048
    s = synth.causal_scores(1, heads, L)
    nv = np.tile(np.arange(1, L + 1, dtype=np.int32), heads)
    ref = orc.softmax_rows(s, nv, THREADS)
    got = ring.read(ring.launch_softmax_rows(ring.upload(s), heads * L, L, causal_period=L), np.float32, s.shape)
    assert ring.last_kernel == "softmax_ring"
    assert rel(got, ref) <= TOL
    assert not got[:, np.triu(np.ones((L, L), dtype=bool), k=1)].any()
