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
