"""Seeded random shapes for every op against the oracle: odd sizes, unaligned offsets, partial
blocks, ragged lengths — the cases the fixed parity tests do not enumerate."""
import numpy as np
import pytest

from agention_infer_b200 import (AGN_BF16, AGN_F16, AGN_F32, AGN_Q2_K, AGN_Q4_K, AGN_Q5_0, AGN_Q5_K, AGN_Q6_K, AGN_Q8_0, AGN_ROPE_NEOX,
                                 AGN_ROPE_NORMAL, synth)
from oracle import oracle as orc

pytestmark = pytest.mark.gpu
TOL = 1e-5


def rel(a, b):
    return synth.max_rel_to_row_scale(a, b)


def _offset_upload(be, arr, off_elems):
    """Uploads arr at an element offset inside a larger allocation (to break 16-byte alignment)."""
    buf = be.empty(arr.nbytes + 64)
    ptr = buf.ptr + arr.itemsize * off_elems
    be.copy_h2d(ptr, arr); be.sync()
    return buf, ptr


def test_fuzz_rms_norm_and_residual(backend):
    r = np.random.default_rng(101)
    for it in range(40):
        T = int(r.integers(1, 8)); H = int(r.choice([1, 2, 3, 4, 5, 31, 32, 33, 100, 255, 256, 257, 600, 1028, 4100]))
        off = int(r.integers(0, 4))
        x = r.standard_normal((T, H), dtype=np.float32) * np.float32(10.0 ** r.integers(-3, 3))
        d = r.standard_normal((T, H), dtype=np.float32); w = (1 + 0.1 * r.standard_normal(H)).astype(np.float32)
        eps = float(r.choice([0.0, 1e-6, 1e-5]))
        if eps == 0.0:
            x[:, 0] += 1.0  # avoid the all-zero row
        bx, px = _offset_upload(backend, x, off)
        dw = backend.upload(w)
        out = backend.launch_rms_norm(px, dw, T, H, eps)
        assert rel(backend.read(out, np.float32, (T, H)), orc.rms_norm_rows(x, w, eps)) <= TOL, (T, H, off, eps)
        nx, nm = backend.launch_add_residual_rms_norm(px, backend.upload(d), dw, T, H, eps)
        rnx, rnm = orc.add_residual_rms_norm_rows(x, d, w, eps)
        assert np.array_equal(backend.read(nx, np.float32, (T, H)), rnx)
        assert rel(backend.read(nm, np.float32, (T, H)), rnm) <= TOL, (T, H, off, eps)


def test_fuzz_rope_and_fused(backend):
    r = np.random.default_rng(102)
    for it in range(60):
        hd = int(r.choice([2, 4, 6, 8, 16, 24, 32, 48, 64, 80, 96, 128, 160, 256]))
        n_rot = int(r.choice([n for n in (0, 2, 4, 8, 16, 32, 48, 64, 96, 128, 256, hd) if n <= hd]))
        nq, nkv, T = int(r.integers(1, 10)), int(r.integers(0, 4)), int(r.integers(1, 12))
        layout = int(r.choice([AGN_ROPE_NEOX, AGN_ROPE_NORMAL])); theta = float(r.choice([1e4, 5e5, 1e6]))
        fs = float(r.choice([1.0, 0.5, 0.125]))
        q = r.standard_normal((T, nq * hd), dtype=np.float32); k = r.standard_normal((T, max(nkv, 1) * hd), dtype=np.float32)
        wq = (1 + 0.1 * r.standard_normal(hd)).astype(np.float32); wk = (1 + 0.1 * r.standard_normal(hd)).astype(np.float32)
        pos = r.integers(0, 40000, size=T).astype(np.int32)
        dpos = backend.upload(pos)
        case = (hd, n_rot, nq, nkv, T, layout, theta, fs)
        if n_rot > 0:
            dq, dk = backend.upload(q), backend.upload(k)
            backend.launch_rope_qk(dq, dk if nkv else None, T, nq, nkv, hd, n_rot, dpos, theta, fs, layout)
            assert rel(backend.read(dq, np.float32, q.shape), orc.rope_rows(q, nq, hd, n_rot, pos, theta, fs, layout)) <= TOL, case
            if nkv:
                assert rel(backend.read(dk, np.float32, k.shape), orc.rope_rows(k, nkv, hd, n_rot, pos, theta, fs, layout)) <= TOL, case
        dq, dk = backend.upload(q), backend.upload(k)
        backend.launch_qk_norm_rope_qk(dq, dk if nkv else None, backend.upload(wq), backend.upload(wk) if nkv else None, T, nq,
                                       nkv, hd, 1e-6, n_rot, dpos, theta, fs, layout)
        assert rel(backend.read(dq, np.float32, q.shape),
                   orc.qk_norm_rope_rows(q, wq, nq, hd, 1e-6, n_rot, pos, theta, fs, layout)) <= TOL, case
        if nkv:
            assert rel(backend.read(dk, np.float32, k.shape),
                       orc.qk_norm_rope_rows(k, wk, nkv, hd, 1e-6, n_rot, pos, theta, fs, layout)) <= TOL, case


def test_fuzz_softmax(backend):
    r = np.random.default_rng(103)
    for it in range(40):
        R = int(r.integers(1, 20)); L = int(r.choice([1, 2, 3, 4, 7, 8, 33, 128, 129, 500, 512, 1024, 1028, 3000, 8192]))
        stride = L + int(r.choice([0, 0, 4, 5]))
        s = np.zeros((R, stride), np.float32); s[:, :L] = r.standard_normal((R, L), dtype=np.float32) * np.float32(r.choice([0.1, 2, 30]))
        nv = r.integers(0, L + 1, size=R).astype(np.int32)
        ref = orc.softmax_rows(np.ascontiguousarray(s[:, :L]), nv)
        out = backend.launch_softmax_rows(backend.upload(s), R, L, row_stride=stride, n_valid=backend.upload(nv))
        got = backend.read(out, np.float32, (R, stride))
        assert rel(got[:, :L], ref) <= TOL, (R, L, stride)


def test_fuzz_silu_mul(backend):
    r = np.random.default_rng(104)
    for it in range(30):
        n = int(r.choice([1, 2, 3, 5, 8, 63, 1000, 1023, 1025, 4097, 100003])); off = int(r.integers(0, 4))
        g = r.standard_normal(n, dtype=np.float32) * np.float32(r.choice([0.1, 1, 10, 50])); u = r.standard_normal(n, dtype=np.float32)
        bg, pg = _offset_upload(backend, g, off); bu, pu = _offset_upload(backend, u, off)
        out = backend.launch_silu_mul(pg, pu, n)
        ref = orc.silu_mul(g, u)
        assert np.max(np.abs(backend.read(out, np.float32, (n,)) - ref) / np.maximum(np.abs(ref), 1.0)) <= TOL, (n, off)


@pytest.mark.parametrize("dtype", [AGN_Q8_0, AGN_Q4_K, AGN_Q5_K, AGN_Q5_0, AGN_Q6_K, AGN_Q2_K])
def test_fuzz_get_rows(backend, dtype):
    r = np.random.default_rng(105 + dtype)
    lens = [256, 512, 768, 1024, 2048, 2304] if dtype == AGN_Q2_K else [1, 3, 31, 32, 33, 64, 100, 255, 256, 257, 300, 511, 512, 768, 1000, 2049]
    for it in range(25):
        vocab = int(r.integers(1, 40)); row_len = int(r.choice(lens))
        T = int(r.integers(1, 30))
        table = synth.quant_table(dtype, vocab, row_len, cfg_index=it % 5, salt=it)
        ids = r.integers(0, vocab, size=T).astype(np.uint32)
        st, ref = orc.get_rows(dtype, table, vocab, row_len, ids)
        out = backend.get_rows(dtype, backend.upload(table), table.nbytes, vocab, row_len, backend.upload(ids), T)
        got = backend.read(out, np.float32, (T, row_len))
        assert st == orc.OK and np.array_equal(got.view(np.uint32), ref.view(np.uint32)), (dtype, vocab, row_len, T)


def test_fuzz_plain_rows_and_kv(backend):
    r = np.random.default_rng(106)
    for it in range(20):
        vocab, row_len, T = int(r.integers(1, 20)), int(r.choice([1, 2, 5, 8, 33, 100, 257])), int(r.integers(1, 20))
        for dtype, width in ((AGN_F32, 4), (AGN_F16, 2), (AGN_BF16, 2)):
            raw = r.integers(0, 256, size=(vocab, row_len * width), dtype=np.uint8)
            raw[:, width - 1::width] &= 0x7B if width == 2 else 0x7E  # finite values only
            ids = r.integers(0, vocab, size=T).astype(np.uint32)
            st, ref = orc.get_rows(dtype, raw, vocab, row_len, ids)
            # the table must be 16-byte aligned; row sizes need not be
            out = backend.get_rows(dtype, backend.upload(raw), raw.nbytes, vocab, row_len, backend.upload(ids), T)
            assert st == orc.OK
            assert np.array_equal(backend.read(out, np.float32, (T, row_len)).view(np.uint32), ref.view(np.uint32)), (dtype, row_len)
        hd = int(r.choice([1, 7, 32, 33, 64, 100, 512])); max_seq = T + int(r.integers(0, 5))
        k = r.standard_normal((T, hd), dtype=np.float32) * np.float32(r.choice([1e-3, 1, 100]))
        pos = r.permutation(max_seq)[:T].astype(np.int32)
        for kvd in (AGN_F16, AGN_Q8_0):
            bpt = backend.kv_bytes_per_token(kvd, hd)
            ref_c = np.zeros((max_seq, bpt), np.uint8); orc.kv_write_rows(kvd, k, pos, ref_c)
            dc, dc2 = backend.upload(np.zeros_like(ref_c)), backend.upload(np.zeros_like(ref_c))
            backend.kv_write(kvd, backend.upload(k), backend.upload(k), dc, dc2, T, hd, backend.upload(pos), max_seq)
            got = backend.read(dc, np.uint8, ref_c.shape)
            if kvd == AGN_Q8_0 and hd % 32:
                keep = np.ones(bpt, bool); keep[(bpt // 34 - 1) * 34 + 2 + hd % 32:] = False
                got, ref_c = got[:, keep], ref_c[:, keep]
            assert np.array_equal(got, ref_c), (kvd, hd, T)
