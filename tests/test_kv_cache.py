"""KV-cache pack / unpack (f16 and Q8_0): the oracle against numpy on CPU, the CUDA kernels
against the oracle on the GPU (bytes and floats bit-exact)."""
import numpy as np
import pytest

from agention_infer_b200 import AGN_F16, AGN_Q8_0, BackendError, synth
from oracle import oracle as orc


def np_pack_q8_0(x):
    T, hd = x.shape
    nb = (hd + 31) // 32
    xp = np.zeros((T, nb * 32), np.float32); xp[:, :hd] = x
    blk = xp.reshape(T, nb, 32)
    amax = np.max(np.abs(blk), axis=2)
    scale = np.where(amax > 0, (amax / np.float32(127.0)).astype(np.float32), np.float32(1.0)).astype(np.float32)
    r = (blk / scale[:, :, None]).astype(np.float32)
    q = np.clip(np.sign(r) * np.floor(np.abs(r) + np.float32(0.5)), -127, 127).astype(np.int8)  # round half away
    out = np.zeros((T, nb, 34), np.uint8)
    out[:, :, 0:2] = scale.astype(np.float16).view(np.uint8).reshape(T, nb, 2)
    out[:, :, 2:] = q.view(np.uint8)
    return out.reshape(T, nb * 34)


def test_oracle_f16_pack_matches_numpy_rounding():
    r = synth.rng_for(0, "x")
    vals = np.concatenate([r.standard_normal(20000).astype(np.float32) * np.float32(s) for s in (1, 1e-4, 1e-7, 1e4, 7e4)]
                          + [np.array([0.0, -0.0, 65504.0, 65520.0, 65519.9, 1e-8, 5.96e-8, 2.98e-8, 2.9802322e-8, np.inf,
                                       -np.inf, 6.1035156e-5, 6.0975552e-5], np.float32)])
    x = vals.reshape(1, -1)
    cache = np.zeros((1, 2 * x.shape[1]), np.uint8)
    orc.kv_write_rows(orc.F16, x, [0], cache)
    with np.errstate(over="ignore"):  # values past 65504 become inf on both sides
        want = x[0].astype(np.float16)
    assert np.array_equal(cache.view(np.uint16)[0], want.view(np.uint16))
    back = orc.kv_read(orc.F16, cache, 1, x.shape[1])
    assert np.array_equal(back[0], want.astype(np.float32))


@pytest.mark.parametrize("hd", [32, 512, 100, 33])
def test_oracle_q8_0_pack_matches_numpy(hd):
    T = 9
    x = synth.activations(2, "k", (T, hd)); x[0, :] = 0.0; x[1, :32] *= 1e-3
    bpt = orc.kv_bytes_per_token(orc.Q8_0, hd)
    assert bpt == ((hd + 31) // 32) * 34
    cache = np.zeros((T, bpt), np.uint8)
    orc.kv_write_rows(orc.Q8_0, x, np.arange(T), cache)
    want = np_pack_q8_0(x)
    nb = (hd + 31) // 32
    got = cache.reshape(T, nb, 34); want = want.reshape(T, nb, 34)
    full = hd // 32
    assert np.array_equal(got[:, :full], want[:, :full])
    if hd % 32:
        assert np.array_equal(got[:, full, :2 + hd % 32], want[:, full, :2 + hd % 32])
    back = orc.kv_read(orc.Q8_0, cache, T, hd)
    assert np.max(np.abs(back - x)) <= np.max(np.abs(x)) / 127.0 * 0.51 + 1e-6


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [AGN_F16, AGN_Q8_0])
@pytest.mark.parametrize("T,hd,max_seq", [(4096, 512, 8192), (512, 1024, 512), (1, 512, 64), (33, 100, 50), (17, 33, 40),
                                          (64, 2048, 64)])
def test_kv_write_and_read_bit_exact(backend, dtype, T, hd, max_seq):
    k = synth.activations(2, "k", (T, hd)); v = synth.activations(2, "q", (T, hd)) * np.float32(3.0)
    k[0, :min(hd, 32)] = 0.0  # an all-zero block: scale 1
    n_slots = min(T, max_seq)
    pos = synth.rng_for(2, "pos").permutation(max_seq)[:T].astype(np.int32) if T <= max_seq else None
    if pos is None:
        pytest.skip("more tokens than slots")
    bpt = backend.kv_bytes_per_token(dtype, hd)
    assert bpt == orc.kv_bytes_per_token(dtype, hd)
    ref_k = np.zeros((max_seq, bpt), np.uint8); ref_v = np.zeros((max_seq, bpt), np.uint8)
    orc.kv_write_rows(dtype, k, pos, ref_k); orc.kv_write_rows(dtype, v, pos, ref_v)
    dkc, dvc = backend.upload(np.zeros_like(ref_k)), backend.upload(np.zeros_like(ref_v))
    backend.kv_write(dtype, backend.upload(k), backend.upload(v), dkc, dvc, T, hd, backend.upload(pos), max_seq)
    got_k = backend.read(dkc, np.uint8, ref_k.shape); got_v = backend.read(dvc, np.uint8, ref_v.shape)
    if dtype == AGN_Q8_0 and hd % 32:  # bytes past a partial block's values are never written by either side
        nb = (hd + 31) // 32
        keep = np.ones(bpt, bool); keep[(nb - 1) * 34 + 2 + hd % 32:] = False
        got_k, got_v, ref_k2, ref_v2 = got_k[:, keep], got_v[:, keep], ref_k[:, keep], ref_v[:, keep]
    else:
        ref_k2, ref_v2 = ref_k, ref_v
    assert np.array_equal(got_k, ref_k2) and np.array_equal(got_v, ref_v2)
    ko, vo = backend.kv_read(dtype, backend.upload(ref_k), backend.upload(ref_v), max_seq, hd)
    assert np.array_equal(backend.read(ko, np.float32, (max_seq, hd)).view(np.uint32),
                          orc.kv_read(dtype, ref_k, max_seq, hd).view(np.uint32))
    assert np.array_equal(backend.read(vo, np.float32, (max_seq, hd)).view(np.uint32),
                          orc.kv_read(dtype, ref_v, max_seq, hd).view(np.uint32))


def _nonfinite_rows(hd):
    x = synth.activations(2, "k", (6, hd))
    x[0, 3] = np.nan                     # a NaN value: ignored by the block maximum, packs as 0
    x[1, 5] = np.inf                     # an inf in the block: scale inf, every value of that block packs as 0
    x[2, 1] = -np.inf; x[2, 2] = np.nan
    x[3, :32] = np.nan                   # a block of NaN only: scale 1, all zeros
    x[4, 40 % hd] = np.float32(3e38)     # huge but finite
    return x


def test_oracle_q8_0_pack_of_nonfinite_values_follows_rust_casts():
    """`(v / scale).round().clamp(-127.0, 127.0) as i8` (src/model/mod.rs:580): a NaN casts to 0, and
    `f32::max` skips a NaN operand in the block maximum (:576)."""
    hd = 64
    x = _nonfinite_rows(hd)
    cache = np.zeros((6, orc.kv_bytes_per_token(orc.Q8_0, hd)), np.uint8)
    orc.kv_write_rows(orc.Q8_0, x, np.arange(6), cache)
    blk = cache.reshape(6, 2, 34)
    q = blk[:, :, 2:].view(np.int8)
    scale = blk[:, :, :2].copy().view(np.float16)[..., 0]
    assert q[0, 0, 3] == 0 and np.isfinite(scale[0, 0]) and q[0, 0].any()  # only the NaN entry is 0
    assert np.isinf(scale[1, 0]) and not q[1, 0].any()                     # inf block: all 0 (finite / inf, inf / inf)
    assert np.isinf(scale[2, 0]) and not q[2, 0].any()
    assert scale[3, 0] == 1.0 and not q[3, 0].any()


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [AGN_F16, AGN_Q8_0])
def test_kv_write_of_nonfinite_values_bit_exact(backend, dtype):
    hd, max_seq = 64, 8
    k = _nonfinite_rows(hd); v = _nonfinite_rows(hd)[::-1].copy()
    T = k.shape[0]
    pos = np.arange(T, dtype=np.int32)
    bpt = backend.kv_bytes_per_token(dtype, hd)
    ref_k = np.zeros((max_seq, bpt), np.uint8); ref_v = np.zeros((max_seq, bpt), np.uint8)
    with np.errstate(all="ignore"):
        orc.kv_write_rows(dtype, k, pos, ref_k); orc.kv_write_rows(dtype, v, pos, ref_v)
    dkc, dvc = backend.upload(np.zeros_like(ref_k)), backend.upload(np.zeros_like(ref_v))
    backend.kv_write(dtype, backend.upload(k), backend.upload(v), dkc, dvc, T, hd, backend.upload(pos), max_seq)
    got_k, got_v = backend.read(dkc, np.uint8, ref_k.shape), backend.read(dvc, np.uint8, ref_v.shape)
    if dtype == AGN_F16:  # NaN payloads may differ between converters; compare NaN-ness and everything else exactly
        gk, rk = got_k.view(np.float16), ref_k.view(np.float16)
        assert np.array_equal(np.isnan(gk), np.isnan(rk)) and np.array_equal(gk[~np.isnan(rk)], rk[~np.isnan(rk)])
        gv, rv = got_v.view(np.float16), ref_v.view(np.float16)
        assert np.array_equal(np.isnan(gv), np.isnan(rv)) and np.array_equal(gv[~np.isnan(rv)], rv[~np.isnan(rv)])
    else:
        assert np.array_equal(got_k, ref_k) and np.array_equal(got_v, ref_v)


@pytest.mark.gpu
def test_fused_q8_0_cache_write_of_nonfinite_v_rows(backend):
    """The fused norm -> rope + cache write packs with the same rule (V rows pass through unrotated)."""
    T, nq, nkv, hd, max_seq = 600, 28, 4, 128, 1024
    q = synth.activations(2, "q", (T, nq * hd)); k = synth.activations(2, "k", (T, nkv * hd))
    v = synth.activations(2, "x", (T, nkv * hd))
    v[0, 3] = np.nan; v[1, 5] = np.inf; v[2, :32] = np.nan; v[599, 100] = -np.inf
    bpt = backend.kv_bytes_per_token(AGN_Q8_0, nkv * hd)
    ref_v = np.zeros((max_seq, bpt), np.uint8)
    with np.errstate(all="ignore"):
        orc.kv_write_rows(AGN_Q8_0, v, np.arange(T, dtype=np.int32), ref_v)
    dkc = backend.upload(np.zeros((max_seq, bpt), np.uint8)); dvc = backend.upload(np.zeros((max_seq, bpt), np.uint8))
    backend.launch_qk_norm_rope_kv_write(backend.upload(q), backend.upload(k), backend.upload(v), None, None, T, nq, nkv, hd, 0.0, hd,
                                  None, 1e6, AGN_Q8_0, dkc, dvc, max_seq)
    assert np.array_equal(backend.read(dvc, np.uint8, ref_v.shape), ref_v)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [AGN_F16, AGN_Q8_0])
@pytest.mark.parametrize("T,hd", [(2501, 256), (4096, 1024), (3000, 32)])
def test_kv_write_four_tokens_per_cta(backend, dtype, T, hd):
    """Large batches pack four tokens per CTA: a token count that is not a multiple of four, positions out of
    range in the middle of a group (skipped and reported), bytes identical to the CTA-per-token kernel and the oracle."""
    max_seq = T + 7
    k = synth.activations(2, "k", (T, hd)); v = synth.activations(2, "q", (T, hd)) * np.float32(3.0)
    k[5, :32] = 0.0
    pos = synth.rng_for(2, "pos").permutation(max_seq)[:T].astype(np.int32)
    bad = [1, 1234, T - 1]
    pos_bad = pos.copy(); pos_bad[bad] = [-2, max_seq, 2 ** 30]  # (-2 of all values: no sentinel may swallow it)
    bpt = backend.kv_bytes_per_token(dtype, hd)
    ref_k = np.zeros((max_seq, bpt), np.uint8); ref_v = np.zeros((max_seq, bpt), np.uint8)
    keep = np.ones(T, bool); keep[bad] = False
    orc.kv_write_rows(dtype, k[keep], pos[keep], ref_k); orc.kv_write_rows(dtype, v[keep], pos[keep], ref_v)
    dk, dv, dp = backend.upload(k), backend.upload(v), backend.upload(pos_bad)
    got = {}
    for multi in (1, 0):
        backend.set_option("kv_multi", multi)
        try:
            dkc, dvc = backend.upload(np.zeros_like(ref_k)), backend.upload(np.zeros_like(ref_v))
            backend.kv_write(dtype, dk, dv, dkc, dvc, T, hd, dp, max_seq)
            assert backend.last_kernel == ("kv_write_multi" if multi else "kv_write")
            with pytest.raises(BackendError) as e:
                backend.sync()
            assert e.value.status == 4 and "kv_write" in str(e.value)
            got[multi] = (backend.read(dkc, np.uint8, ref_k.shape), backend.read(dvc, np.uint8, ref_v.shape))
        finally:
            backend.set_option("kv_multi", 1)
    assert np.array_equal(got[1][0], ref_k) and np.array_equal(got[1][1], ref_v)
    assert np.array_equal(got[1][0], got[0][0]) and np.array_equal(got[1][1], got[0][1])
    # a single bad position, and that one is -2: still reported
    one_bad = pos.copy(); one_bad[T // 2] = -2
    backend.kv_write(dtype, dk, dv, backend.upload(np.zeros_like(ref_k)), backend.upload(np.zeros_like(ref_v)), T, hd,
                     backend.upload(one_bad), max_seq)
    assert backend.last_kernel == "kv_write_multi"
    with pytest.raises(BackendError) as e:
        backend.sync()
    assert e.value.status == 4


@pytest.mark.gpu
def test_kv_write_pos_start_and_out_of_range_slot(backend):
    T, hd, max_seq = 8, 64, 10
    k = synth.activations(2, "k", (T, hd))
    bpt = backend.kv_bytes_per_token(AGN_F16, hd)
    dkc = backend.upload(np.zeros((max_seq, bpt), np.uint8)); dvc = backend.upload(np.zeros((max_seq, bpt), np.uint8))
    backend.kv_write(AGN_F16, backend.upload(k), backend.upload(k), dkc, dvc, T, hd, None, max_seq, pos_start=2)
    backend.sync()
    got = backend.read(dkc, np.uint16, (max_seq, hd))
    assert np.array_equal(got[2:10], k.astype(np.float16).view(np.uint16)) and not got[:2].any()
    backend.kv_write(AGN_F16, backend.upload(k), backend.upload(k), dkc, dvc, T, hd, None, max_seq, pos_start=5)
    with pytest.raises(BackendError) as e:
        backend.sync()
    assert e.value.status == 4
    backend.sync()
    with pytest.raises(BackendError) as e:
        backend.kv_write(12, dkc, dkc, dkc, dvc, 1, hd, None, max_seq)
    assert e.value.status == 2


# ---------------------------------------------------------------- norm -> rope + cache write, one launch

@pytest.mark.gpu
@pytest.mark.parametrize("kv_dtype", [1, 8])  # f16, q8_0
@pytest.mark.parametrize("norm", [True, False])
@pytest.mark.parametrize("T,nq,nkv,hd,n_rot,layout", [
    (1, 28, 4, 128, 128, 0), (64, 28, 4, 128, 128, 0), (300, 32, 8, 128, 128, 1), (600, 28, 4, 128, 128, 0), (513, 8, 2, 64, 64, 0), (5, 32, 8, 64, 64, 0), (17, 8, 2, 64, 64, 1),
    (9, 4, 2, 128, 64, 0),    # partial rotation: not covered by the fused kernel, runs as two launches
    (7, 3, 1, 80, 80, 0),     # head_dim 80: two launches
    (4, 2, 2, 256, 256, 0),   # head_dim 256: two launches
])
def test_fused_rope_kv_write_equals_the_two_ops(backend, kv_dtype, norm, T, nq, nkv, hd, n_rot, layout):
    """q, k and both caches must be byte for byte what rope (or norm -> rope) followed by kv_write gives."""
    max_seq = 1024
    q, k, v = synth.activations(2, "q", (T, nq * hd)), synth.activations(2, "k", (T, nkv * hd)), synth.activations(2, "x", (T, nkv * hd))
    k[0, :32] = 0.0  # an all-zero block: scale 1
    wq, wk = synth.norm_weight(2, "wq", hd), synth.norm_weight(2, "wk", hd)
    pos = synth.rng_for(2, "pos").permutation(max_seq)[:T].astype(np.int32)
    bpt = backend.kv_bytes_per_token(kv_dtype, nkv * hd)
    dwq, dwk = (backend.upload(wq), backend.upload(wk)) if norm else (None, None)
    dp, dv = backend.upload(pos), backend.upload(v)

    def caches():
        kc, vc = backend.empty(max_seq * bpt), backend.empty(max_seq * bpt)
        backend.copy_h2d(kc, np.full(max_seq * bpt, 0x5A, np.uint8)); backend.copy_h2d(vc, np.full(max_seq * bpt, 0x5A, np.uint8))
        backend.sync()
        return kc, vc

    # the two ops
    q1, k1 = backend.upload(q), backend.upload(k)
    kc1, vc1 = caches()
    if norm:
        backend.launch_qk_norm_rope_qk(q1, k1, dwq, dwk, T, nq, nkv, hd, 1e-6, n_rot, dp, 1e6, 1.0, layout)
    else:
        backend.launch_rope_qk(q1, k1, T, nq, nkv, hd, n_rot, dp, 1e6, 1.0, layout)
    backend.kv_write(kv_dtype, k1, dv, kc1, vc1, T, nkv * hd, dp, max_seq)
    # one call
    q2, k2 = backend.upload(q), backend.upload(k)
    kc2, vc2 = caches()
    n0 = backend.launch_count
    backend.launch_qk_norm_rope_kv_write(q2, k2, dv, dwq, dwk, T, nq, nkv, hd, 1e-6, n_rot, dp, 1e6, kv_dtype, kc2, vc2, max_seq,
                                         layout=layout)
    launches = backend.launch_count - n0
    covered = hd in (64, 128) and n_rot == hd and (kv_dtype == 1 or T >= 512)  # small batches fuse only the f16 cache
    assert launches == (1 if covered else 2)
    for a, b, dt, shape in ((q1, q2, np.uint32, (T, nq * hd)), (k1, k2, np.uint32, (T, nkv * hd)),
                            (kc1, kc2, np.uint8, (max_seq, bpt)), (vc1, vc2, np.uint8, (max_seq, bpt))):
        assert np.array_equal(backend.read(a, dt, shape), backend.read(b, dt, shape))
    # and the cache is what the oracle packs from the oracle's rotated k
    rk = orc.qk_norm_rope_rows(k, wk, nkv, hd, 1e-6, n_rot, pos, 1e6, 1.0, layout) if norm else orc.rope_rows(k, nkv, hd, n_rot, pos, 1e6, 1.0, layout)
    got_k = backend.read(backend.kv_read(kv_dtype, kc2, vc2, max_seq, nkv * hd)[0], np.float32, (max_seq, nkv * hd))
    tol = 2.0 ** -10 if kv_dtype == 1 else 1.0 / 127
    assert synth.max_rel_to_row_scale(got_k[pos].reshape(T * nkv, hd), rk.reshape(T * nkv, hd)) <= tol + 1e-5


@pytest.mark.gpu
def test_fused_rope_kv_write_reports_a_slot_out_of_range(backend):
    T, nq, nkv, hd, max_seq = 4, 4, 2, 128, 8
    q, k, v = synth.activations(2, "q", (T, nq * hd)), synth.activations(2, "k", (T, nkv * hd)), synth.activations(2, "x", (T, nkv * hd))
    pos = np.array([0, 9, 3, -1], np.int32)
    bpt = backend.kv_bytes_per_token(1, nkv * hd)
    kc, vc = backend.empty(max_seq * bpt), backend.empty(max_seq * bpt)
    backend.copy_h2d(kc, np.zeros(max_seq * bpt, np.uint8)); backend.copy_h2d(vc, np.zeros(max_seq * bpt, np.uint8)); backend.sync()
    backend.launch_qk_norm_rope_kv_write(backend.upload(q), backend.upload(k), backend.upload(v), None, None, T, nq, nkv, hd, 0.0, hd,
                                         backend.upload(pos), 1e6, 1, kc, vc, max_seq)
    from agention_infer_b200 import BackendError
    with pytest.raises(BackendError) as e:
        backend.sync()
    assert e.value.status == 4
    got = backend.read(vc, np.uint8, (max_seq, bpt))
    assert np.all(got[[1, 2, 4, 5, 6, 7]] == 0) and np.any(got[0] != 0) and np.any(got[3] != 0)  # only slots 0 and 3 were written


@pytest.mark.gpu
@pytest.mark.parametrize("amax", [127.0, 100.0, 1.0, 3.3e-3, 6.02e4, 1e-30, 1e-39])
def test_q8_0_quotients_at_the_rounding_boundaries_bit_exact(backend, amax):
    """Values whose quotient by the block scale falls on k + 0.5, or within a few ulps of it, for every k: the
    cases where an approximate quotient and the reference's IEEE division could round to different integers.
    Each block holds `amax` (which fixes the scale), and 31 such values; through the stand-alone kernels (a CTA
    per token, four tokens per CTA) and through the write fused into the norm -> RoPE launch."""
    amax = np.float32(amax)
    scale = amax / np.float32(127.0) if amax > 0 else np.float32(1.0)
    k = np.arange(-127, 127, dtype=np.float32) + np.float32(0.5)
    with np.errstate(all="ignore"):
        base = (k * scale).astype(np.float32)
    vals = [base]
    for steps in (1, 2, 3, 6):
        up, dn = base.copy(), base.copy()
        for _ in range(steps):
            up, dn = np.nextafter(up, np.float32(np.inf)), np.nextafter(dn, np.float32(-np.inf))
        vals += [up, dn]
    vals = np.concatenate(vals)
    vals = vals[np.abs(vals) <= amax]
    n_blocks = -(-vals.size // 31)
    body = np.zeros(n_blocks * 31, np.float32); body[: vals.size] = vals
    x = np.empty((n_blocks, 32), np.float32)
    x[:, 0] = amax
    x[:, 1:] = body.reshape(n_blocks, 31)
    hd = 128
    T = -(-n_blocks // (hd // 32))
    rows = np.zeros((T, hd), np.float32); rows.reshape(-1, 32)[:n_blocks] = x
    rows.reshape(-1, 32)[n_blocks:, 0] = amax
    pos = np.arange(T, dtype=np.int32)
    bpt = backend.kv_bytes_per_token(AGN_Q8_0, hd)
    ref = np.zeros((T, bpt), np.uint8)
    orc.kv_write_rows(AGN_Q8_0, rows, pos, ref)
    for reps in (1, 40):  # 40 copies of the rows: enough tokens for the four-tokens-per-CTA kernel (T >= 16 * SMs)
        big = np.tile(rows, (reps, 1)); Tb = big.shape[0]
        dk, dv = backend.upload(np.zeros((Tb, bpt), np.uint8)), backend.upload(np.zeros((Tb, bpt), np.uint8))
        backend.kv_write(AGN_Q8_0, backend.upload(big), backend.upload(big), dk, dv, Tb, hd, backend.upload(np.arange(Tb, dtype=np.int32)), Tb)
        for buf in (dk, dv):
            got = backend.read(buf, np.uint8, (Tb, bpt))
            assert np.array_equal(got, np.tile(ref, (reps, 1))), (float(amax), reps, backend.last_kernel)
    # fused: V rides along unrotated, so its cache bytes are the pack of the input rows
    nq = nkv = 1
    q = synth.activations(2, "q", (T, nq * hd)); kk = synth.activations(2, "k", (T, nkv * hd))
    dk, dv = backend.upload(np.zeros((T, bpt), np.uint8)), backend.upload(np.zeros((T, bpt), np.uint8))
    backend.launch_qk_norm_rope_kv_write(backend.upload(q), backend.upload(kk), backend.upload(rows), None, None, T, nq, nkv, hd, 1e-6,
                                         hd, backend.upload(pos), 1e6, AGN_Q8_0, dk, dv, T)
    assert np.array_equal(backend.read(dv, np.uint8, (T, bpt)), ref), float(amax)


@pytest.mark.gpu
def test_q8_0_pack_random_blocks_over_the_whole_exponent_range_bit_exact(backend):
    """262,144 blocks whose magnitudes span 1e-44 .. 3e38 (subnormal scales, scales near f16 overflow, blocks made of
    small integers times the scale, i.e. quotients on or next to k and k + 0.5): the bytes of the reference's division."""
    r = np.random.default_rng(2611)
    T, hd = 8192, 1024
    mag = (10.0 ** r.uniform(-44, 38.5, size=(T, hd // 32, 1))).astype(np.float32)
    base = r.standard_normal((T, hd // 32, 32)).astype(np.float32)
    half_steps = r.integers(-254, 255, size=(T, hd // 32, 32)).astype(np.float32) * np.float32(0.5)
    pick = r.random((T, hd // 32, 1)) < 0.5  # half of the blocks: values k/2 * scale with max 127 * scale
    with np.errstate(all="ignore"):
        vals = np.where(pick, half_steps / np.float32(127.0), base / np.float32(4.5))
        vals[..., 0] = np.where(pick[..., 0], 1.0, vals[..., 0])
        x = (vals * mag).astype(np.float32).reshape(T, hd)
    x[~np.isfinite(x)] = 0.0
    pos = np.arange(T, dtype=np.int32)
    bpt = backend.kv_bytes_per_token(AGN_Q8_0, hd)
    ref = np.zeros((T, bpt), np.uint8)
    orc.kv_write_rows(AGN_Q8_0, x, pos, ref)
    dk, dv = backend.upload(np.zeros((T, bpt), np.uint8)), backend.upload(np.zeros((T, bpt), np.uint8))
    dx = backend.upload(x)
    backend.kv_write(AGN_Q8_0, dx, dx, dk, dv, T, hd, backend.upload(pos), T)
    got = backend.read(dk, np.uint8, (T, bpt))
    bad = np.argwhere(got != ref)
    assert bad.size == 0, f"{len(bad)} bytes differ, first at token {bad[0][0]} byte {bad[0][1]}: {got[tuple(bad[0])]} vs {ref[tuple(bad[0])]}"
    assert np.array_equal(backend.read(dv, np.uint8, (T, bpt)), ref)


def test_oracle_q8_0_words_layout_by_hand():
    """kv_cache_write_q8_0 / dequant_kv_q8_0 (src/ops/kernels_wgpu.rs:583-718): nine words per 32 values, the f32 scale
    first, then offset-binary bytes; a ragged last block is padded with zeros (byte 128)."""
    W = orc.KV_Q8_0_WORDS
    x = np.zeros((1, 40), np.float32); x[0, :5] = [1.0, -2.0, 0.5, 127.0, -127.0]; x[0, 33] = 3.0
    assert orc.kv_bytes_per_token(W, 40) == 72 and orc.kv_bytes_per_token(W, 512) == 576
    c = np.zeros((1, 72), np.uint8)
    orc.kv_write_rows(W, x, np.array([0], np.int32), c)
    assert c[0, :4].view(np.float32)[0] == 1.0                       # amax 127 -> scale 1
    assert list(c[0, 4:10]) == [129, 126, 129, 255, 1, 128]           # q + 128, round half away (0.5 -> 1)
    assert c[0, 36:40].view(np.float32)[0] == np.float32(3.0) / np.float32(127.0)
    assert list(c[0, 40:44]) == [128, 255, 128, 128] and np.all(c[0, 48:72] == 128)  # padding is written as q = 0
    back = orc.kv_read(W, c, 1, 40)
    assert list(back[0, :5]) == [1.0, -2.0, 1.0, 127.0, -127.0] and back[0, 33] == np.float32(127.0) * (np.float32(3.0) / np.float32(127.0))
    # the same numbers as the 34-byte form: q equal, scale equal before its rounding to f16
    c34 = np.zeros((1, orc.kv_bytes_per_token(orc.Q8_0, 40)), np.uint8)
    orc.kv_write_rows(orc.Q8_0, x, np.array([0], np.int32), c34)
    assert np.array_equal(c34[0, 2:34].view(np.int8).astype(np.int16) + 128, c[0, 4:36].astype(np.int16))


@pytest.mark.gpu
@pytest.mark.parametrize("T,hd,max_seq", [(4096, 512, 4096), (300, 1024, 512), (1, 512, 64), (33, 100, 50), (17, 33, 40), (2500, 256, 2500)])
def test_kv_write_and_read_q8_0_words_bit_exact(backend, T, hd, max_seq):
    from agention_infer_b200 import AGN_KV_Q8_0_WORDS as W
    k = synth.activations(2, "k", (T, hd)); v = synth.activations(2, "q", (T, hd)) * np.float32(3.0)
    k[0, :min(hd, 32)] = 0.0
    if hd >= 64:
        v[0, 40] = np.nan; v[0, 3] = np.inf
    pos = synth.rng_for(2, "pos").permutation(max_seq)[:T].astype(np.int32)
    bpt = backend.kv_bytes_per_token(W, hd)
    assert bpt == orc.kv_bytes_per_token(orc.KV_Q8_0_WORDS, hd) == ((hd + 31) // 32) * 36
    ref_k = np.zeros((max_seq, bpt), np.uint8); ref_v = np.zeros((max_seq, bpt), np.uint8)
    with np.errstate(all="ignore"):
        orc.kv_write_rows(orc.KV_Q8_0_WORDS, k, pos, ref_k); orc.kv_write_rows(orc.KV_Q8_0_WORDS, v, pos, ref_v)
    dkc, dvc = backend.upload(np.zeros_like(ref_k)), backend.upload(np.zeros_like(ref_v))
    backend.kv_write(W, backend.upload(k), backend.upload(v), dkc, dvc, T, hd, backend.upload(pos), max_seq)
    assert np.array_equal(backend.read(dkc, np.uint8, ref_k.shape), ref_k)
    assert np.array_equal(backend.read(dvc, np.uint8, ref_v.shape), ref_v)
    clean = np.ascontiguousarray(ref_k)
    ko, vo = backend.kv_read(W, backend.upload(clean), backend.upload(clean), max_seq, hd)
    want = orc.kv_read(orc.KV_Q8_0_WORDS, clean, max_seq, hd)
    assert np.array_equal(backend.read(ko, np.float32, (max_seq, hd)).view(np.uint32), want.view(np.uint32))
    assert np.array_equal(backend.read(vo, np.float32, (max_seq, hd)).view(np.uint32), want.view(np.uint32))


@pytest.mark.gpu
@pytest.mark.parametrize("norm", [True, False])
def test_fused_rope_kv_write_q8_0_words_equals_the_two_ops(backend, norm):
    from agention_infer_b200 import AGN_KV_Q8_0_WORDS as W
    T, nq, nkv, hd = 600, 8, 2, 128
    q = synth.activations(2, "q", (T, nq * hd)); k = synth.activations(2, "k", (T, nkv * hd)); v = synth.activations(2, "x", (T, nkv * hd))
    wq, wk = synth.norm_weight(2, "wq", hd), synth.norm_weight(2, "wk", hd)
    pos = synth.positions(2, T, False)
    dpos = backend.upload(pos)
    dwq, dwk = (backend.upload(wq), backend.upload(wk)) if norm else (None, None)
    bpt = backend.kv_bytes_per_token(W, nkv * hd)
    # the two launches
    dq, dk, dv = backend.upload(q), backend.upload(k), backend.upload(v)
    if norm:
        backend.launch_qk_norm_rope_qk(dq, dk, dwq, dwk, T, nq, nkv, hd, 1e-6, hd, dpos, 1e6)
    else:
        backend.launch_rope_qk(dq, dk, T, nq, nkv, hd, hd, dpos, 1e6)
    k1, v1 = backend.upload(np.zeros((T, bpt), np.uint8)), backend.upload(np.zeros((T, bpt), np.uint8))
    backend.kv_write(W, dk, dv, k1, v1, T, nkv * hd, dpos, T)
    # one launch
    dq2, dk2 = backend.upload(q), backend.upload(k)
    k2, v2 = backend.upload(np.zeros((T, bpt), np.uint8)), backend.upload(np.zeros((T, bpt), np.uint8))
    backend.launch_qk_norm_rope_kv_write(dq2, dk2, dv, dwq, dwk, T, nq, nkv, hd, 1e-6, hd, dpos, 1e6, W, k2, v2, T)
    for a_, b_ in ((k1, k2), (v1, v2)):
        assert np.array_equal(backend.read(a_, np.uint8, (T, bpt)), backend.read(b_, np.uint8, (T, bpt)))
    assert np.array_equal(backend.read(dq, np.float32, q.shape).view(np.uint32), backend.read(dq2, np.float32, q.shape).view(np.uint32))
