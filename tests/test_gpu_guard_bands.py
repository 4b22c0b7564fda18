"""Out-of-bounds writes: every output buffer sits between two 4 KiB guard bands filled with a
known byte; after the op the bands must be untouched and the payload must still match the oracle.
Shapes are the awkward ones (odd row lengths, tails, one row, sizes that select every kernel
variant).  This is the stand-in for a memory checker, which cannot be run on the GPUs used here."""
import numpy as np
import pytest

from agention_infer_b200 import (AGN_BF16, AGN_F16, AGN_Q2_K, AGN_Q4_K, AGN_Q5_0, AGN_Q5_K, AGN_Q6_K, AGN_Q8_0,
                                 AGN_ROPE_NEOX, AGN_ROPE_NORMAL, synth)
from oracle import oracle as orc

pytestmark = pytest.mark.gpu
GUARD = 4096
FILL = 0xA5


class Guarded:
    """nbytes of device memory at .ptr (an int address, 256-byte aligned plus `skew`), guard bands on both sides."""

    def __init__(self, backend, nbytes: int, skew: int = 0):
        self.be, self.nbytes, self.skew = backend, int(nbytes), skew
        self.total = self.nbytes + skew + 2 * GUARD
        self.buf = backend.empty(self.total)
        backend.copy_h2d(self.buf, np.full(self.total, FILL, np.uint8))
        backend.sync()
        self.ptr = self.buf.data_ptr() + GUARD + skew

    def put(self, arr):
        a = np.ascontiguousarray(arr)
        assert a.nbytes <= self.nbytes
        self.be.copy_h2d(self.ptr, a)
        self.be.sync()
        return self

    def get(self, dtype, shape):
        return self.be.read(self.ptr, dtype, shape)

    def check(self, what=""):
        raw = self.be.read(self.buf, np.uint8, (self.total,))
        lo, hi = raw[: GUARD + self.skew], raw[GUARD + self.skew + self.nbytes:]
        assert np.all(lo == FILL), f"{what}: wrote before the buffer at offset {int(np.argmax(lo != FILL)) - GUARD - self.skew}"
        assert np.all(hi == FILL), f"{what}: wrote past the buffer at offset {self.nbytes + int(np.argmax(hi != FILL))}"


def guarded_like(backend, arr, skew=0):
    return Guarded(backend, arr.nbytes, skew).put(arr)


@pytest.mark.parametrize("T,H", [(1, 4), (3, 250), (5, 3584), (2, 40000), (7, 36)])
def test_rms_norm_and_residual_stay_inside(backend, T, H):
    x, d, w = synth.activations(2, "x", (T, H)), synth.activations(2, "delta", (T, H)), synth.norm_weight(2, "w", H)
    gx, gd, gw = guarded_like(backend, x), guarded_like(backend, d), guarded_like(backend, w)
    out, nx, nm = Guarded(backend, x.nbytes), Guarded(backend, x.nbytes), Guarded(backend, x.nbytes)
    backend.launch_rms_norm(gx.ptr, gw.ptr, T, H, 1e-6, out=out.ptr)
    backend.launch_add_residual_rms_norm(gx.ptr, gd.ptr, gw.ptr, T, H, 1e-6, new_x=nx.ptr, normed=nm.ptr)
    o16, n16 = Guarded(backend, x.nbytes // 2), Guarded(backend, x.nbytes // 2)
    backend.launch_rms_norm_out16(gx.ptr, gw.ptr, T, H, 1e-6, AGN_BF16, out=o16.ptr)
    backend.launch_add_residual_rms_norm_out16(gx.ptr, gd.ptr, gw.ptr, T, H, 1e-6, AGN_F16, new_x=nx.ptr, normed=n16.ptr)
    for g, name in ((out, "rms_norm"), (nx, "new_x"), (nm, "normed"), (o16, "rms_norm bf16"), (n16, "normed f16"), (gx, "x"), (gd, "delta")):
        g.check(name)
    assert synth.max_rel_to_row_scale(out.get(np.float32, (T, H)), orc.rms_norm_rows(x, w, 1e-6)) <= 1e-5


@pytest.mark.parametrize("layout", [AGN_ROPE_NEOX, AGN_ROPE_NORMAL])
@pytest.mark.parametrize("T,nq,nkv,hd,n_rot", [(3, 28, 4, 128, 128), (1, 32, 8, 64, 64), (5, 3, 1, 80, 40), (2, 2, 2, 256, 128), (9, 5, 0, 96, 96)])
def test_rope_and_fused_norm_rope_stay_inside(backend, T, nq, nkv, hd, n_rot, layout):
    q = synth.activations(2, "q", (T, nq * hd)); k = synth.activations(2, "k", (T, max(nkv, 1) * hd))
    wq, wk = synth.norm_weight(2, "wq", hd), synth.norm_weight(2, "wk", hd)
    pos = synth.positions(3, T, True)
    gp, gwq, gwk = guarded_like(backend, pos), guarded_like(backend, wq), guarded_like(backend, wk)
    for fused in (False, True):
        gq, gk = guarded_like(backend, q), guarded_like(backend, k)
        kp = gk.ptr if nkv else None
        if fused:
            backend.launch_qk_norm_rope_qk(gq.ptr, kp, gwq.ptr, gwk.ptr if nkv else None, T, nq, nkv, hd, 1e-6, n_rot, gp.ptr, 1e6, 1.0, layout)
            ref = orc.qk_norm_rope_rows(q, wq, nq, hd, 1e-6, n_rot, pos, 1e6, 1.0, layout)
        else:
            backend.launch_rope_qk(gq.ptr, kp, T, nq, nkv, hd, n_rot, gp.ptr, 1e6, 1.0, layout)
            ref = orc.rope_rows(q, nq, hd, n_rot, pos, 1e6, 1.0, layout)
        gq.check("q"); gk.check("k")
        assert synth.max_rel_to_row_scale(gq.get(np.float32, (T * nq, hd)), ref.reshape(T * nq, hd)) <= 1e-5
        if not nkv:  # an absent K buffer must not be touched at all
            assert np.array_equal(gk.get(np.float32, k.shape), k)


@pytest.mark.parametrize("n", [1, 7, 4097, 256 * 4 * 4 + 3, 18944 * 3])
def test_silu_mul_stays_inside(backend, n):
    g, u = synth.activations(2, "gate", (n,)), synth.activations(2, "up", (n,))
    gg, gu = guarded_like(backend, g), guarded_like(backend, u)
    out, o16 = Guarded(backend, 4 * n), Guarded(backend, 2 * n)
    backend.launch_silu_mul(gg.ptr, gu.ptr, n, out=out.ptr)
    backend.launch_silu_mul_out16(gg.ptr, gu.ptr, n, AGN_BF16, out=o16.ptr)
    out.check("silu_mul"); o16.check("silu_mul bf16")
    ref = orc.silu_mul(g, u)
    assert np.max(np.abs(out.get(np.float32, (n,)) - ref) / np.maximum(np.abs(ref), 1.0)) <= 1e-5
    # 4-byte aligned but not 16-byte aligned buffers take the scalar kernel
    sg, su, so = guarded_like(backend, g, skew=4), guarded_like(backend, u, skew=4), Guarded(backend, 4 * n, skew=4)
    backend.launch_silu_mul(sg.ptr, su.ptr, n, out=so.ptr)
    so.check("silu_mul unaligned")
    assert np.array_equal(so.get(np.float32, (n,)).view(np.uint32), out.get(np.float32, (n,)).view(np.uint32))


@pytest.mark.parametrize("R,L", [(5, 8), (3, 30), (7, 100), (4, 516), (3, 4100), (2, 9999), (2, 16388), (1, 40004), (1, 152064)])
def test_softmax_stays_inside(backend, R, L):
    s = synth.activations(1, "scores", (R, L), std=2.0)
    nv = np.array([L, 1, L // 2 + 1, L - 1, 0, 3, L][:R], dtype=np.int32)
    gs, gnv = guarded_like(backend, s), guarded_like(backend, nv)
    out, o16, wts, sums = Guarded(backend, s.nbytes), Guarded(backend, s.nbytes // 2), Guarded(backend, s.nbytes), Guarded(backend, 4 * R)
    backend.launch_softmax_rows(gs.ptr, R, L, out=out.ptr, n_valid=gnv.ptr)
    backend.launch_softmax_rows_scaled_out16(gs.ptr, R, L, 0.5, AGN_F16, out=o16.ptr, n_valid=gnv.ptr)
    backend.launch_softmax_rows_scaled(gs.ptr, R, L, 1.0, out=wts.ptr, sums=sums.ptr, n_valid=gnv.ptr)
    for g, name in ((out, "softmax"), (o16, "softmax f16"), (wts, "weights"), (sums, "sums"), (gs, "scores")):
        g.check(name)
    got = out.get(np.float32, (R, L))
    assert np.all(got[np.arange(L)[None, :] >= nv[:, None]] == 0.0)
    if L <= 40000:
        assert synth.max_rel_to_row_scale(got, orc.softmax_rows(s, nv)) <= 1e-5


@pytest.mark.parametrize("dtype", [AGN_Q8_0, AGN_Q4_K, AGN_Q6_K, AGN_Q5_K, AGN_Q5_0, AGN_Q2_K])
@pytest.mark.parametrize("row_len,T", [(256, 1), (768, 5), (3584, 3)])
def test_get_rows_stays_inside(backend, dtype, row_len, T):
    lens = [row_len] if dtype == AGN_Q2_K else [row_len, row_len - 3, row_len + 33]
    for rl in lens:
        vocab = 9
        table = synth.quant_table(dtype, vocab, rl, cfg_index=1)
        ids = np.array([vocab - 1, 0, 4, 8, 8][:T], np.uint32)
        gt, gi = guarded_like(backend, table), guarded_like(backend, ids)
        out, o16 = Guarded(backend, 4 * T * rl), Guarded(backend, 2 * T * rl)
        backend.get_rows(dtype, gt.ptr, table.nbytes, vocab, rl, gi.ptr, T, out=out.ptr)
        backend.get_rows_f16(dtype, gt.ptr, table.nbytes, vocab, rl, gi.ptr, T, out=o16.ptr)
        out.check(f"get_rows {dtype} len {rl}"); o16.check(f"get_rows_f16 {dtype} len {rl}")
        st, ref = orc.get_rows(dtype, table, vocab, rl, ids)
        assert st == orc.OK and np.array_equal(out.get(np.float32, (T, rl)).view(np.uint32), ref.view(np.uint32))


@pytest.mark.parametrize("kv_dtype", [AGN_F16, AGN_Q8_0, 1008])
@pytest.mark.parametrize("T,hd", [(1, 512), (5, 100), (3, 33), (4, 1024)])
def test_kv_write_and_read_stay_inside(backend, kv_dtype, T, hd):
    max_seq = 16
    k, v = synth.activations(2, "k", (T, hd)), synth.activations(2, "q", (T, hd))
    pos = np.array([15, 0, 7, 3, 9][:T], np.int32)
    bpt = backend.kv_bytes_per_token(kv_dtype, hd)
    gk, gv, gp = guarded_like(backend, k), guarded_like(backend, v), guarded_like(backend, pos)
    kc, vc = Guarded(backend, max_seq * bpt), Guarded(backend, max_seq * bpt)
    backend.kv_write(kv_dtype, gk.ptr, gv.ptr, kc.ptr, vc.ptr, T, hd, gp.ptr, max_seq)
    kc.check("k_cache"); vc.check("v_cache")
    ko, vo = Guarded(backend, 4 * max_seq * hd), Guarded(backend, 4 * max_seq * hd)
    backend.kv_read(kv_dtype, kc.ptr, vc.ptr, max_seq, hd, k_out=ko.ptr, v_out=vo.ptr)
    ko.check("k_out"); vo.check("v_out")
    cache = np.full((max_seq, bpt), FILL, np.uint8)
    orc.kv_write_rows(kv_dtype, k, pos, cache)
    assert np.array_equal(kc.get(np.uint8, (max_seq, bpt)), cache)


@pytest.mark.parametrize("T,H,E", [(1, 4, 2), (33, 100, 5), (2049, 64, 8), (700, 36, 64)])
def test_router_and_gather_stay_inside(backend, T, H, E):
    logits, x = synth.activations(5, "logits", (T, E)), synth.activations(5, "x", (T, H))
    gl, gx = guarded_like(backend, logits), guarded_like(backend, x)
    idx, w = Guarded(backend, 8 * T), Guarded(backend, 8 * T)
    backend.router_top2(gl.ptr, T, E, idx=idx.ptr, w=w.ptr)
    idx.check("idx"); w.check("w")
    ref_idx, _ = orc.router_top2(logits)
    assert np.array_equal(idx.get(np.int32, (T, 2)), ref_idx)
    out, off, tok, slot = Guarded(backend, 8 * T * H), Guarded(backend, 4 * (E + 1)), Guarded(backend, 8 * T), Guarded(backend, 8 * T)
    backend.gather_rows_by_expert(gx.ptr, idx.ptr, T, H, E, out=out.ptr, offsets=off.ptr, src_token=tok.ptr, src_slot=slot.ptr)
    for g, name in ((out, "gathered rows"), (off, "offsets"), (tok, "src_token"), (slot, "src_slot")):
        g.check(name)
    ref_out, ref_off, ref_tok, _ = orc.gather_rows_by_expert(x, ref_idx, E)
    assert np.array_equal(off.get(np.int32, (E + 1,)), ref_off) and np.array_equal(tok.get(np.int32, (2 * T,)), ref_tok)
    assert np.array_equal(out.get(np.float32, (2 * T, H)).view(np.uint32), ref_out.view(np.uint32))


@pytest.mark.parametrize("heads,L", [(1, 1028), (2, 2048)])
def test_softmax_square_causal_forms_stay_inside(backend, heads, L):
    """The row-pair kernel of square causal matrices, zero-filled, valid entries only and with 16-bit rows."""
    s = synth.causal_scores(1, heads, L)
    nv = np.tile(np.arange(1, L + 1, dtype=np.int32), heads)
    ref = orc.softmax_rows(s, nv, max(1, orc.max_threads()))
    gs = guarded_like(backend, s)
    out, val, o16 = Guarded(backend, s.nbytes), Guarded(backend, s.nbytes).put(np.zeros_like(s)), Guarded(backend, s.nbytes // 2)
    backend.launch_softmax_rows(gs.ptr, heads * L, L, out=out.ptr, causal_period=L)
    assert backend.last_kernel == "softmax_causal_pair"
    backend.launch_softmax_rows_valid(gs.ptr, heads * L, L, val.ptr, causal_period=L)
    backend.launch_softmax_rows_scaled_out16(gs.ptr, heads * L, L, 1.0, AGN_BF16, out=o16.ptr, causal_period=L)
    for g, name in ((out, "probs"), (val, "valid-only probs"), (o16, "bf16 probs"), (gs, "scores")):
        g.check(name)
    assert synth.max_rel_to_row_scale(out.get(np.float32, s.shape), ref) <= 1e-5
    assert synth.max_rel_to_row_scale(val.get(np.float32, s.shape), ref) <= 1e-5


def test_persistent_ring_kernels_stay_inside(backend):
    """The opt-in persistent kernels (rows staged through shared memory by bulk copies): every buffer between guard
    bands, row counts that leave a partial last round and lengths that are not multiples of the copy granularity."""
    opts = ("ring_force", "rms_ring", "rope_ring", "get_rows_ring", "softmax_ring")
    for o in opts:
        backend.set_option(o, 1)
    try:
        T, H = 301, 1000
        x, d, w = synth.activations(2, "x", (T, H)), synth.activations(2, "delta", (T, H)), synth.norm_weight(2, "w", H)
        gx, gd, gw = guarded_like(backend, x), guarded_like(backend, d), guarded_like(backend, w)
        out, nx, nm = Guarded(backend, x.nbytes), Guarded(backend, x.nbytes), Guarded(backend, x.nbytes)
        backend.launch_rms_norm(gx.ptr, gw.ptr, T, H, 1e-6, out=out.ptr)
        assert backend.last_kernel == "rms_norm_ring"
        backend.launch_add_residual_rms_norm(gx.ptr, gd.ptr, gw.ptr, T, H, 1e-6, new_x=nx.ptr, normed=nm.ptr)
        for g, name in ((out, "rms_norm"), (nx, "new_x"), (nm, "normed"), (gx, "x"), (gd, "delta")):
            g.check("ring " + name)
        assert synth.max_rel_to_row_scale(out.get(np.float32, x.shape), orc.rms_norm_rows(x, w, 1e-6)) <= 1e-5
        nq, nkv, hd = 5, 3, 64
        q, k = synth.activations(3, "q", (T, nq * hd)), synth.activations(3, "k", (T, nkv * hd))
        pos = synth.positions(3, T, True)
        gq, gk, gp = guarded_like(backend, q), guarded_like(backend, k), guarded_like(backend, pos)
        backend.launch_rope_qk(gq.ptr, gk.ptr, T, nq, nkv, hd, hd, gp.ptr, 1e4)
        assert backend.last_kernel == "rope_ring"
        gq.check("ring rope q"); gk.check("ring rope k")
        assert synth.max_rel_to_row_scale(gq.get(np.float32, q.shape), orc.rope_rows(q, nq, hd, hd, pos, 1e4)) <= 1e-5
        vocab, Hq = 77, 96
        table = synth.quant_table(AGN_Q8_0, vocab, Hq)
        ids = synth.token_ids(2, T, vocab); ids[::5] = vocab - 1
        gt, gi = guarded_like(backend, table), guarded_like(backend, ids)
        emb = Guarded(backend, 4 * T * Hq)
        backend.get_rows(AGN_Q8_0, gt.ptr, table.nbytes, vocab, Hq, gi.ptr, T, out=emb.ptr)
        assert backend.last_kernel == "get_rows_ring"
        emb.check("ring get_rows")
        _, ref = orc.get_rows(AGN_Q8_0, table, vocab, Hq, ids)
        assert np.array_equal(emb.get(np.float32, (T, Hq)).view(np.uint32), ref.view(np.uint32))
        R, L = 37, 1100
        s = synth.activations(5, "logits", (R, L), std=2.0)
        nv = synth.rng_for(5, "pos").integers(0, L + 1, size=R, dtype=np.int32)
        gs, gn, pr = guarded_like(backend, s), guarded_like(backend, nv), Guarded(backend, s.nbytes)
        backend.launch_softmax_rows(gs.ptr, R, L, out=pr.ptr, n_valid=gn.ptr)
        assert backend.last_kernel == "softmax_ring"
        pr.check("ring softmax")
        assert synth.max_rel_to_row_scale(pr.get(np.float32, s.shape), orc.softmax_rows(s, nv)) <= 1e-5
    finally:
        for o in opts:
            backend.set_option(o, 0)
