"""Host-slice entry points (activations in host memory, pipelined through the staging ring)
against the CPU oracle: same tolerances as the device-pointer ops, sizes chosen so that
every op runs over several chunks and the ring wraps around."""
import numpy as np
import pytest

from agention_infer_b200 import AGN_Q4_K, AGN_Q6_K, AGN_Q8_0, synth
from oracle import oracle as orc

pytestmark = pytest.mark.gpu
TOL = 1e-5
THREADS = max(1, orc.max_threads())


def test_host_rms_norm_pageable_and_pinned(backend):
    T, H = 5000, 3584  # 143 MB in+out: about 8 chunks
    x = synth.activations(2, "x", (T, H)); w = synth.norm_weight(2, "w", H)
    ref = orc.rms_norm_rows(x, w, 1e-6, THREADS)
    dw = backend.upload(w)
    out = np.empty_like(x)
    backend.rms_norm_into(x, dw, out, 1e-6); backend.sync()
    assert synth.max_rel_to_row_scale(out, ref) <= TOL
    px = backend.pinned((T, H), np.float32); po = backend.pinned((T, H), np.float32)
    px[:] = x
    backend.rms_norm_into(px, dw, po, 1e-6); backend.sync()
    assert np.array_equal(po, out)
    backend.free_pinned(px); backend.free_pinned(po)


def test_host_add_residual_rms_norm_updates_x_in_place(backend):
    T, H = 3000, 4096  # 147 MB over the three buffers
    x = synth.activations(4, "x", (T, H)); d = synth.activations(4, "delta", (T, H)); w = synth.norm_weight(4, "w", H)
    ref_x, ref_n = orc.add_residual_rms_norm_rows(x, d, w, 1e-5, THREADS)
    hx = x.copy(); normed = np.empty_like(x)
    backend.add_residual_rms_norm_into(hx, d, backend.upload(w), normed, 1e-5); backend.sync()
    assert np.array_equal(hx.view(np.uint32), ref_x.view(np.uint32))  # the sum is exact
    assert synth.max_rel_to_row_scale(normed, ref_n) <= TOL


def test_host_silu_mul_with_tail_and_in_place(backend):
    n = 4096 * 3000 + 123
    g = synth.activations(2, "gate", (n,)); u = synth.activations(2, "up", (n,))
    ref = orc.silu_mul(g, u, THREADS)
    backend.silu_mul_into(g, u, g); backend.sync()  # the CPU batch path writes into gate
    assert np.max(np.abs(g - ref) / np.maximum(np.abs(ref), 1.0)) <= TOL


@pytest.mark.parametrize("norm", [False, True])
def test_host_rope_qk_chunks_keep_positions(backend, norm):
    T, nq, nkv, hd = 6000, 28, 4, 128
    q = synth.activations(2, "q", (T, nq * hd)); k = synth.activations(2, "k", (T, nkv * hd))
    wq = synth.norm_weight(2, "wq", hd); wk = synth.norm_weight(2, "wk", hd)
    for pos in (synth.positions(3, T, True), None):
        p = np.arange(T, dtype=np.int32) + 5 if pos is None else pos
        if norm:
            rq = orc.qk_norm_rope_rows(q, wq, nq, hd, 1e-6, hd, p, 1e6, threads=THREADS)
            rk = orc.qk_norm_rope_rows(k, wk, nkv, hd, 1e-6, hd, p, 1e6, threads=THREADS)
        else:
            rq = orc.rope_rows(q, nq, hd, hd, p, 1e6, threads=THREADS)
            rk = orc.rope_rows(k, nkv, hd, hd, p, 1e6, threads=THREADS)
        hq, hk = q.copy(), k.copy()
        backend.rope_host(hq, hk, nq, nkv, hd, hd, pos, 1e6, pos_start=5, eps=1e-6,
                          wq_dev=backend.upload(wq) if norm else None, wk_dev=backend.upload(wk) if norm else None)
        backend.sync()
        assert synth.max_rel_to_row_scale(hq, rq) <= TOL
        assert synth.max_rel_to_row_scale(hk, rk) <= TOL


def test_host_softmax_causal_period_survives_chunking(backend):
    nh, L = 40, 512  # 20480 rows x 2 KB in+out = 84 MB: several chunks, each a multiple of L rows
    s = synth.causal_scores(1, nh, L)
    nv = np.tile(np.arange(1, L + 1, dtype=np.int32), nh)
    ref = orc.softmax_rows(s, nv, THREADS)
    out = np.empty_like(s)
    backend.softmax_rows_into(s, out, causal_period=L); backend.sync()
    assert synth.max_rel_to_row_scale(out, ref) <= TOL
    out2 = np.empty_like(s)
    backend.softmax_rows_into(s, out2, n_valid=nv); backend.sync()
    assert np.array_equal(out2, out)


@pytest.mark.parametrize("dtype,vocab,H", [(AGN_Q4_K, 4096, 3584), (AGN_Q8_0, 2048, 2048), (AGN_Q6_K, 1024, 4096)])
def test_host_get_rows_bit_exact(backend, dtype, vocab, H):
    T = 3000
    table = synth.quant_table(dtype, vocab, H, cfg_index=2)
    ids = synth.token_ids(2, T, vocab)
    st, ref = orc.get_rows(dtype, table, vocab, H, ids, THREADS)
    out = np.empty((T, H), np.float32)
    backend.get_rows_into(dtype, backend.upload(table), table.nbytes, vocab, H, ids, out); backend.sync()
    assert st == orc.OK and np.array_equal(out.view(np.uint32), ref.view(np.uint32))


def test_host_ops_chain_output_feeds_next_input(backend):
    # the second op uploads what the first op downloads: the ring must order them
    T, H = 3000, 2048
    x = synth.activations(1, "x", (T, H)); w = synth.norm_weight(1, "w", H)
    dw = backend.upload(w)
    mid = np.zeros_like(x); out = np.zeros_like(x)
    backend.rms_norm_into(x, dw, mid, 1e-5)
    backend.rms_norm_into(mid, dw, out, 1e-5)
    backend.sync()
    ref = orc.rms_norm_rows(orc.rms_norm_rows(x, w, 1e-5, THREADS), w, 1e-5, THREADS)
    assert synth.max_rel_to_row_scale(out, ref) <= 2 * TOL


def test_hostlink_probe_one_gpu():
    """The pinned-copy probe that bounds the host-slice path: runs, and reports plausible figures."""
    from agention_infer_b200 import hostlink
    r = hostlink.probe(1, mb=32, reps=3)
    row = r["active_gpus"]["1"]
    assert set(row) == {"h2d", "d2h", "both_per_direction"}
    assert all(1.0 < row[c]["mean_gbs_per_gpu"] < 1000.0 for c in row)


def test_host_quantize_rows_q8_k_bit_exact(backend):
    """Host rows in, the three Q8KRow arrays out, through the staging ring (several chunks), ragged rows included."""
    for T, n in ((6000, 3584), (300, 1000), (3, 100)):
        x = synth.activations(3, "x", (T, n)) * np.float32(2.5)
        x[0, : min(n, 256)] = 0.0
        nb = (n + 255) // 256
        d, qs, bs = np.empty((T, nb), np.float32), np.empty((T, nb * 256), np.int8), np.empty((T, nb * 16), np.int16)
        backend.quantize_rows_q8_k_into(x, d, qs, bs); backend.sync()
        rd, rq, rb = orc.quantize_rows_q8_k(x, THREADS)
        assert np.array_equal(d.view(np.uint32), rd.view(np.uint32)) and np.array_equal(qs, rq) and np.array_equal(bs, rb), (T, n)
