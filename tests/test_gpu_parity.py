"""GPU parity: every CUDA entry point, called through the C ABI, against the CPU oracle on the
same seeded inputs.  get_rows is bit-exact; the float ops are within 1e-5 of the row scale
(max |gpu - cpu| / max |cpu row|), the tolerance the benchmark contract states."""
import numpy as np
import pytest

from agention_infer_b200 import (AGN_BF16, AGN_F16, AGN_F32, AGN_Q2_K, AGN_Q4_K, AGN_Q5_0, AGN_Q5_K, AGN_Q6_K, AGN_Q8_0, AGN_ROPE_NEOX,
                                 AGN_ROPE_NORMAL, BackendError, synth)
from oracle import oracle as orc

pytestmark = pytest.mark.gpu

TOL = 1e-5  # relative to row scale, f32
THREADS = max(1, orc.max_threads())


def rel(got, ref):
    return synth.max_rel_to_row_scale(got, ref)


def bits(a):
    return np.ascontiguousarray(a).view(np.uint32)


# ------------------------------------------------------------------ rms_norm

@pytest.mark.parametrize("T,H,eps", [(1, 3584, 1e-6), (512, 2048, 1e-5), (4096, 3584, 1e-6), (33, 4096, 1e-5),
                                     (7, 1024, 1e-5), (3, 128, 1e-6), (5, 8192, 1e-5), (2, 16384, 1e-5),
                                     (3, 2050, 1e-5), (4, 77, 1e-6), (2, 40000, 1e-5)])
def test_rms_norm(backend, T, H, eps):
    x = synth.activations(2, "x", (T, H)); w = synth.norm_weight(2, "w", H)
    ref = orc.rms_norm_rows(x, w, eps, THREADS)
    dx, dw = backend.upload(x), backend.upload(w)
    out = backend.launch_rms_norm(dx, dw, T, H, eps)
    got = backend.read(out, np.float32, (T, H))
    assert rel(got, ref) <= TOL


def test_rms_norm_in_place_and_unaligned(backend):
    T, H = 6, 1000
    x = synth.activations(2, "x", (T, H)); w = synth.norm_weight(2, "w", H)
    ref = orc.rms_norm_rows(x, w, 1e-5)
    dx, dw = backend.upload(x), backend.upload(w)
    backend.launch_rms_norm(dx, dw, T, H, 1e-5, out=dx)  # out aliases x
    assert rel(backend.read(dx, np.float32, (T, H)), ref) <= TOL
    # x at a 4-byte (not 16-byte) aligned address
    buf = backend.empty(4 * (T * H + 1))
    backend.copy_h2d(buf.ptr + 4, x); backend.sync()
    out = backend.launch_rms_norm(buf.ptr + 4, dw, T, H, 1e-5)
    assert rel(backend.read(out, np.float32, (T, H)), ref) <= TOL


def test_rms_norm_large_dynamic_range(backend):
    # adversarial for the reduction order: a few huge entries among tiny ones
    T, H = 16, 4096
    x = synth.activations(4, "x", (T, H)) * np.float32(1e-3)
    x[:, ::512] *= np.float32(1e5)
    w = synth.norm_weight(4, "w", H)
    ref = orc.rms_norm_rows(x, w, 1e-5)
    out = backend.launch_rms_norm(backend.upload(x), backend.upload(w), T, H, 1e-5)
    assert rel(backend.read(out, np.float32, (T, H)), ref) <= TOL


@pytest.mark.parametrize("T,H", [(64, 4096), (5, 3584), (3, 250)])
def test_add_residual_rms_norm(backend, T, H):
    x = synth.activations(4, "x", (T, H)); d = synth.activations(4, "delta", (T, H)); w = synth.norm_weight(4, "w", H)
    ref_nx, ref_nm = orc.add_residual_rms_norm_rows(x, d, w, 1e-5)
    nx, nm = backend.launch_add_residual_rms_norm(backend.upload(x), backend.upload(d), backend.upload(w), T, H, 1e-5)
    assert np.array_equal(bits(backend.read(nx, np.float32, (T, H))), bits(ref_nx))  # one f32 add: exact
    assert rel(backend.read(nm, np.float32, (T, H)), ref_nm) <= TOL


# ---------------------------------------------------------------------- rope

ROPE_CASES = [  # T, n_heads, head_dim, n_rot, theta, random positions
    (512, 32, 64, 64, 500000.0, False), (512, 8, 64, 64, 500000.0, False),
    (4096, 28, 128, 128, 1e6, False), (4096, 4, 128, 128, 1e6, False),
    (64, 28, 128, 128, 1e6, True), (1, 28, 128, 128, 1e6, True), (8, 4, 128, 128, 1e6, True),
    (17, 16, 256, 256, 1e7, True), (17, 16, 256, 64, 1e7, True), (9, 5, 128, 64, 10000.0, True),
    (9, 3, 96, 96, 10000.0, True), (9, 3, 80, 40, 10000.0, True), (5, 2, 32, 32, 10000.0, True),
    (5, 2, 512, 512, 10000.0, True), (5, 7, 64, 32, 10000.0, True), (3, 2, 6, 6, 10000.0, True),
]


@pytest.mark.parametrize("layout", [AGN_ROPE_NEOX, AGN_ROPE_NORMAL])
@pytest.mark.parametrize("T,nh,hd,n_rot,theta,rand", ROPE_CASES)
def test_rope(backend, layout, T, nh, hd, n_rot, theta, rand):
    x = synth.activations(3, "q", (T, nh * hd)); pos = synth.positions(3, T, rand)
    ref = orc.rope_rows(x, nh, hd, n_rot, pos, theta, 1.0, layout, THREADS)
    dx, dp = backend.upload(x), backend.upload(pos)
    backend.launch_rope(dx, T, nh, hd, n_rot, dp, theta, 1.0, layout)
    assert rel(backend.read(dx, np.float32, (T, nh * hd)), ref) <= TOL


def test_rope_pos_start_and_freq_scale(backend):
    T, nh, hd = 40, 8, 128
    x = synth.activations(3, "q", (T, nh * hd))
    pos = (np.arange(T) + 1000).astype(np.int32)
    ref = orc.rope_rows(x, nh, hd, hd, pos, 1e6, 0.25)
    dx = backend.upload(x)
    backend.launch_rope(dx, T, nh, hd, hd, None, 1e6, freq_scale=0.25, pos_start=1000)
    assert rel(backend.read(dx, np.float32, (T, nh * hd)), ref) <= TOL


def test_rope_qk_one_launch(backend):
    T, nq, nkv, hd = 300, 28, 4, 128
    q = synth.activations(2, "q", (T, nq * hd)); k = synth.activations(2, "k", (T, nkv * hd))
    pos = synth.positions(3, T, True)
    rq = orc.rope_rows(q, nq, hd, hd, pos, 1e6); rk = orc.rope_rows(k, nkv, hd, hd, pos, 1e6)
    dq, dk, dp = backend.upload(q), backend.upload(k), backend.upload(pos)
    n0 = backend.launch_count
    backend.launch_rope_qk(dq, dk, T, nq, nkv, hd, hd, dp, 1e6)
    assert backend.launch_count == n0 + 1
    assert rel(backend.read(dq, np.float32, q.shape), rq) <= TOL
    assert rel(backend.read(dk, np.float32, k.shape), rk) <= TOL


def test_rope_identity_at_position_zero_and_norm_preserving(backend):
    T, nh, hd = 1024, 32, 128
    x = synth.activations(4, "q", (T, nh * hd))
    dx = backend.upload(x)
    backend.launch_rope(dx, T, nh, hd, hd, backend.upload(np.zeros(T, np.int32)), 500000.0)
    assert np.array_equal(backend.read(dx, np.float32, x.shape), x)
    backend.launch_rope(dx, T, nh, hd, hd, None, 500000.0, pos_start=7)
    y = backend.read(dx, np.float32, x.shape).reshape(T, nh, hd)
    assert np.allclose(np.linalg.norm(y, axis=-1), np.linalg.norm(x.reshape(T, nh, hd), axis=-1), rtol=1e-5)


@pytest.mark.parametrize("layout", [AGN_ROPE_NEOX, AGN_ROPE_NORMAL])
@pytest.mark.parametrize("T,nh,hd,n_rot,theta,rand", ROPE_CASES)
def test_qk_norm_rope(backend, layout, T, nh, hd, n_rot, theta, rand):
    x = synth.activations(3, "q", (T, nh * hd)); w = synth.norm_weight(3, "wq", hd); pos = synth.positions(3, T, rand)
    ref = orc.qk_norm_rope_rows(x, w, nh, hd, 1e-6, n_rot, pos, theta, 1.0, layout, THREADS)
    dx = backend.upload(x)
    backend.launch_qk_norm_rope(dx, backend.upload(w), T, nh, hd, 1e-6, n_rot, backend.upload(pos), theta, 1.0, layout)
    assert rel(backend.read(dx, np.float32, (T, nh * hd)), ref) <= TOL


def test_qk_norm_rope_qk_one_launch(backend):
    T, nq, nkv, hd = 257, 32, 8, 128
    q = synth.activations(4, "q", (T, nq * hd)); k = synth.activations(4, "k", (T, nkv * hd))
    wq = synth.norm_weight(4, "wq", hd); wk = synth.norm_weight(4, "wk", hd); pos = synth.positions(3, T, True)
    rq = orc.qk_norm_rope_rows(q, wq, nq, hd, 1e-5, hd, pos, 500000.0)
    rk = orc.qk_norm_rope_rows(k, wk, nkv, hd, 1e-5, hd, pos, 500000.0)
    dq, dk = backend.upload(q), backend.upload(k)
    backend.launch_qk_norm_rope_qk(dq, dk, backend.upload(wq), backend.upload(wk), T, nq, nkv, hd, 1e-5, hd,
                                   backend.upload(pos), 500000.0)
    assert rel(backend.read(dq, np.float32, q.shape), rq) <= TOL
    assert rel(backend.read(dk, np.float32, k.shape), rk) <= TOL


def test_qk_norm_alone_is_the_fused_op_without_rotation(backend):
    # `qk_norm` (src/model/llama/cpu_path.rs:78-93) without rope: n_rot = 0
    T, nh, hd = 50, 8, 128
    x = synth.activations(3, "q", (T, nh * hd)); w = synth.norm_weight(3, "wq", hd)
    ref = orc.rms_norm_rows(x.reshape(T * nh, hd), w, 1e-6).reshape(T, nh * hd)
    dx = backend.upload(x)
    backend.launch_qk_norm_rope(dx, backend.upload(w), T, nh, hd, 1e-6, 0, None, 1e6)
    assert rel(backend.read(dx, np.float32, x.shape), ref) <= TOL


def test_rope_rejects_bad_arguments(backend):
    dx = backend.empty(4 * 128)
    for n_rot in (130, 63, -2):
        with pytest.raises(BackendError) as e:
            backend.launch_rope(dx, 1, 1, 128, n_rot, None, 1e4)
        assert e.value.status == 1
    with pytest.raises(BackendError):
        backend.launch_rope(dx, 1, 1, 128, 128, None, 1e4, layout=7)


# ------------------------------------------------------------------ silu_mul

@pytest.mark.parametrize("n", [1, 3, 4, 1023, 4096, 512 * 8192, 18944 * 64 + 5])
def test_silu_mul(backend, n):
    g = synth.activations(1, "gate", (n,)); u = synth.activations(1, "up", (n,))
    ref = orc.silu_mul(g, u, THREADS)
    out = backend.launch_silu_mul(backend.upload(g), backend.upload(u), n)
    got = backend.read(out, np.float32, (n,))
    # elementwise op: scale of the "row" is the element's own reference magnitude floor-ed at 1
    assert np.max(np.abs(got - ref) / np.maximum(np.abs(ref), 1.0)) <= TOL


def test_silu_mul_c2_rows_in_place_and_extremes(backend):
    T, I = 256, 18944
    g = synth.activations(2, "gate", (T, I)); u = synth.activations(2, "up", (T, I))
    g[0, :8] = [-100.0, -88.0, -20.0, 0.0, 20.0, 88.0, 100.0, -0.0]
    ref = orc.silu_mul(g, u, THREADS)
    dg = backend.upload(g)
    backend.launch_silu_mul(dg, backend.upload(u), T * I, out=dg)  # the CPU batch path writes into gate
    assert rel(backend.read(dg, np.float32, (T, I)), ref) <= TOL


def test_silu_mul_unaligned(backend):
    n = 1001
    g = synth.activations(1, "gate", (n,)); u = synth.activations(1, "up", (n,))
    buf = backend.empty(4 * (n + 1))
    backend.copy_h2d(buf.ptr + 4, g); backend.sync()
    out = backend.launch_silu_mul(buf.ptr + 4, backend.upload(u), n)
    ref = orc.silu_mul(g, u)
    assert np.max(np.abs(backend.read(out, np.float32, (n,)) - ref) / np.maximum(np.abs(ref), 1.0)) <= TOL


# ------------------------------------------------------------------- softmax

def test_softmax_causal_c1(backend):
    nh, L = 32, 512
    s = synth.causal_scores(1, nh, L)
    nv = np.tile(np.arange(1, L + 1, dtype=np.int32), nh)
    ref = orc.softmax_rows(s, nv, THREADS)
    out = backend.launch_softmax_rows(backend.upload(s), nh * L, L, causal_period=L)
    got = backend.read(out, np.float32, s.shape)
    assert rel(got, ref) <= TOL
    assert not got[:, np.triu(np.ones((L, L), dtype=bool), k=1)].any()
    # same through an explicit n_valid array
    out2 = backend.launch_softmax_rows(backend.upload(s), nh * L, L, n_valid=backend.upload(nv))
    assert np.array_equal(bits(backend.read(out2, np.float32, s.shape)), bits(got))


@pytest.mark.parametrize("R,L", [(64, 8), (8192, 8), (5, 4), (33, 128), (9, 1024), (7, 2048), (3, 8192), (2, 32768),
                                 (2, 65536), (5, 1000), (4, 7), (3, 1)])
def test_softmax_dense_and_ragged(backend, R, L):
    s = synth.activations(5, "logits", (R, L), std=2.0)
    ref = orc.softmax_rows(s, None, THREADS)
    out = backend.launch_softmax_rows(backend.upload(s), R, L)
    got = backend.read(out, np.float32, (R, L))
    assert rel(got, ref) <= TOL
    assert np.allclose(got.sum(axis=1, dtype=np.float64), 1.0, atol=1e-5)
    nv = synth.rng_for(5, "pos").integers(0, L + 1, size=R, dtype=np.int32)
    ref = orc.softmax_rows(s, nv, THREADS)
    ds = backend.upload(s)
    backend.launch_softmax_rows(ds, R, L, out=ds, n_valid=backend.upload(nv))  # in place
    assert rel(backend.read(ds, np.float32, (R, L)), ref) <= TOL


def test_softmax_decode_shape_with_offset_and_stride(backend):
    # one token at position 700 against a cache of max_seq 1024: n_heads rows, nv = pos+1
    nh, max_seq, pos = 28, 1024, 700
    s = synth.activations(3, "scores", (nh, max_seq), std=2.0)
    ref = orc.softmax_rows(s, np.full(nh, pos + 1, np.int32))
    out = backend.launch_softmax_rows(backend.upload(s), nh, max_seq, causal_period=1, causal_offset=pos)
    assert rel(backend.read(out, np.float32, s.shape), ref) <= TOL
    # row_stride > row_len: the padding columns are not written
    ds = backend.upload(s)
    backend.launch_softmax_rows(ds, nh, 512, out=ds, row_stride=max_seq)
    got = backend.read(ds, np.float32, s.shape)
    assert rel(got[:, :512], orc.softmax_rows(np.ascontiguousarray(s[:, :512]))) <= TOL
    assert np.array_equal(got[:, 512:], s[:, 512:])


def test_attention_softmax_unnormalised_form(backend):
    # the GPU twin's contract: weights = exp(s - max), sums[h] = sum of them, over entries 0..=pos
    nh, max_seq, pos = 28, 2048, 1500
    s = synth.activations(3, "scores", (nh, max_seq), std=2.0)
    w, sums = backend.launch_attention_softmax(backend.upload(s), nh, max_seq, pos)
    gw = backend.read(w, np.float32, (nh, max_seq)); gs = backend.read(sums, np.float32, (nh,))
    v = s[:, :pos + 1].astype(np.float64)
    e = np.exp(v - v.max(axis=1, keepdims=True))
    assert np.max(np.abs(gw[:, :pos + 1] - e)) <= 2e-6 and not gw[:, pos + 1:].any()
    assert np.allclose(gs, e.sum(axis=1), rtol=1e-5)
    # dividing by the sums gives the normalised softmax of the CPU path
    ref = orc.softmax_rows(s, np.full(nh, pos + 1, np.int32))
    assert rel(gw / gs[:, None], ref) <= TOL


# ------------------------------------------------------------------ get_rows

@pytest.mark.parametrize("dtype,vocab,row_len,T", [
    (AGN_Q8_0, 128256, 2048, 512), (AGN_Q4_K, 152064, 3584, 4096), (AGN_Q6_K, 16384, 4096, 2048),
    (AGN_Q4_K, 32000, 4096, 512), (AGN_Q8_0, 100, 96, 33), (AGN_Q8_0, 64, 33, 17), (AGN_Q6_K, 50, 768, 50),
    (AGN_Q6_K, 20, 300, 9), (AGN_Q4_K, 20, 300, 9), (AGN_Q4_K, 7, 256, 1), (AGN_Q8_0, 1, 32, 5),
    (AGN_Q5_K, 32000, 4096, 2048), (AGN_Q5_K, 20, 300, 9), (AGN_Q5_0, 4096, 2048, 1024), (AGN_Q5_0, 64, 33, 17),
    (AGN_Q5_0, 10, 96, 33), (AGN_Q2_K, 32000, 4096, 2048), (AGN_Q2_K, 33, 256, 40), (AGN_Q2_K, 5, 768, 9),
])
def test_get_rows_bit_exact(backend, dtype, vocab, row_len, T):
    table = synth.quant_table(dtype, vocab, row_len, cfg_index=2)
    ids = synth.token_ids(2, T, vocab)
    ids[0], ids[-1] = vocab - 1, 0  # last row touches the end of the table
    st, ref = orc.get_rows(dtype, table, vocab, row_len, ids, THREADS)
    assert st == orc.OK
    dt = backend.upload(table)
    out = backend.get_rows(dtype, dt, table.nbytes, vocab, row_len, backend.upload(ids), T)
    got = backend.read(out, np.float32, (T, row_len))
    assert np.array_equal(bits(got), bits(ref))


@pytest.mark.parametrize("dtype,vocab,row_len,T", [(AGN_Q4_K, 4096, 3584, 2048), (AGN_Q8_0, 300, 96, 300),
                                                   (AGN_Q6_K, 128, 768, 128), (AGN_Q5_0, 64, 33, 64), (AGN_Q6_K, 50, 4096, 50), (AGN_Q2_K, 77, 512, 77)])
def test_get_rows_both_staging_paths_bit_exact(backend, dtype, vocab, row_len, T):
    # default staging is one bulk asynchronous copy (TMA, cp.async.bulk + mbarrier) per row, with
    # rows that start off a 16-byte boundary and the last row of the table (which falls back to
    # cp.async); with the option off every row is staged by 16-byte cp.async copies
    table = synth.quant_table(dtype, vocab, row_len, cfg_index=3)
    ids = synth.token_ids(3, T, vocab); ids[0], ids[-1] = vocab - 1, 0
    st, ref = orc.get_rows(dtype, table, vocab, row_len, ids, THREADS)
    dt, di = backend.upload(table), backend.upload(ids)
    got_tma = backend.read(backend.get_rows(dtype, dt, table.nbytes, vocab, row_len, di, T), np.float32, (T, row_len))
    backend.set_option("get_rows_tma", 0)
    try:
        got_cp = backend.read(backend.get_rows(dtype, dt, table.nbytes, vocab, row_len, di, T), np.float32, (T, row_len))
    finally:
        backend.set_option("get_rows_tma", 1)
    assert st == orc.OK and np.array_equal(bits(got_tma), bits(ref)) and np.array_equal(bits(got_cp), bits(ref))


@pytest.mark.parametrize("dtype,np_dtype", [(AGN_F32, np.float32), (AGN_F16, np.float16), (AGN_BF16, None)])
def test_get_rows_plain_types(backend, dtype, np_dtype):
    vocab, row_len, T = 40, 72, 25
    if np_dtype is None:
        raw = synth.rng_for(0, "table").integers(0, 65536, size=(vocab, row_len), dtype=np.uint16)
        raw &= np.uint16(0xFF7F)  # keep away from NaN payload differences
        table = raw.view(np.uint8)
    else:
        table = synth.activations(0, "x", (vocab, row_len)).astype(np_dtype).view(np.uint8)
    table = np.ascontiguousarray(table).reshape(vocab, -1)
    ids = synth.token_ids(0, T, vocab)
    st, ref = orc.get_rows(dtype, table, vocab, row_len, ids)
    assert st == orc.OK
    out = backend.get_rows(dtype, backend.upload(table), table.nbytes, vocab, row_len, backend.upload(ids), T)
    assert np.array_equal(bits(backend.read(out, np.float32, (T, row_len))), bits(ref))


def test_get_rows_out_of_range_id_zero_row_and_status(backend):
    vocab, row_len = 16, 256
    table = synth.quant_table(AGN_Q4_K, vocab, row_len)
    ids = np.array([3, 16, 5, 4000000000], dtype=np.uint32)
    st, ref = orc.get_rows(AGN_Q4_K, table, vocab, row_len, ids)
    assert st == orc.EROW
    out = backend.get_rows(AGN_Q4_K, backend.upload(table), table.nbytes, vocab, row_len, backend.upload(ids), 4)
    host = np.empty((4, row_len), np.float32)
    backend.copy_d2h(host, out)
    with pytest.raises(BackendError) as e:
        backend.sync()
    assert e.value.status == 4  # AGN_EOOB_ID
    backend.sync()  # reported once; the context stays usable
    assert np.array_equal(bits(host), bits(ref))
    assert not host[1].any() and not host[3].any()


def test_get_rows_argument_errors(backend):
    t = backend.empty(4096)
    ids = backend.upload(np.zeros(1, np.uint32))
    o = backend.empty(4 * 256)
    with pytest.raises(BackendError) as e:  # Q3_K has no codec: "dequantization not yet implemented" in the reference too
        backend.get_rows(11, t, 4096, 1, 256, ids, 1, out=o)
    assert e.value.status == 2
    with pytest.raises(BackendError) as e:  # rows extend beyond the data section
        backend.get_rows(AGN_Q4_K, t, 100, 1, 256, ids, 1, out=o)
    assert e.value.status == 1
    with pytest.raises(BackendError) as e:  # "Q2_K row length .. is not a multiple of 256", src/quant/q2_k.rs:31-35
        backend.get_rows(AGN_Q2_K, t, 4096, 1, 300, ids, 1, out=backend.empty(4 * 300))
    assert e.value.status == 1


def test_dequant_row_single(backend):
    vocab, row_len = 10, 2048
    table = synth.quant_table(AGN_Q8_0, vocab, row_len)
    dt = backend.upload(table)
    row = backend.dequant_row(AGN_Q8_0, dt, table.nbytes, vocab, row_len, 7)
    st, ref = orc.dequant_row(AGN_Q8_0, table, 0, row_len, vocab, 7)
    assert st == orc.OK and np.array_equal(bits(row), bits(ref))
    with pytest.raises(BackendError):
        backend.dequant_row(AGN_Q8_0, dt, table.nbytes, vocab, row_len, 10)


# --------------------------------------------------------------- empty input

def test_empty_inputs_are_no_ops(backend):
    n0 = backend.launch_count
    backend.launch_rms_norm(0, 0, 0, 128, 1e-5, out=0)
    backend.launch_silu_mul(0, 0, 0, out=0)
    backend.launch_rope(0, 0, 4, 64, 64, None, 1e4)
    backend.launch_softmax_rows(0, 0, 16, out=0)
    backend.get_rows(AGN_Q8_0, 0, 0, 0, 32, 0, 0, out=0)
    backend.sync()
    assert backend.launch_count == n0
