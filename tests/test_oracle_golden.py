"""Pins the CPU oracle against the reference's own unit-test vectors (quant codecs, f16/bf16
rows, compute_rope_freq_scale) and against an independent numpy statement of the codecs."""
import json
from pathlib import Path

import numpy as np
import pytest

import tests.ref_numpy as rn
from oracle import oracle as orc

KA = json.loads((Path(__file__).parent / "golden" / "reference_known_answers.json").read_text())


def _data(name):
    return np.array(KA[name]["data"], dtype=np.uint8)


def test_q8_0_single_block():  # src/quant/q8_0.rs:110-126
    c = KA["q8_0_single_block"]
    st, out = orc.dequant(orc.Q8_0, _data("q8_0_single_block"), c["n"])
    assert st == orc.OK and out.size == 32
    assert np.max(np.abs(out - np.array(c["expected"], dtype=np.float32))) < c["tol"]


def test_q8_0_partial_block():  # src/quant/q8_0.rs:129-148
    c = KA["q8_0_partial_block"]
    st, out = orc.dequant(orc.Q8_0, _data("q8_0_partial_block"), c["n"])
    assert st == orc.OK and out.size == c["expected_len"]
    assert out[32] == 42.0
    assert np.array_equal(out[:32], np.arange(32, dtype=np.float32))


def test_q8_0_short_data_is_an_error():  # src/quant/q8_0.rs:18-23
    st, _ = orc.dequant(orc.Q8_0, _data("q8_0_partial_block")[:60], 33)
    assert st == orc.ESHORT


def test_get_scale_min_k4_known_answers():  # src/quant/q4_k.rs:229-241
    for case in KA["q4_k_scale_min"]["cases"]:
        for j, exp in case["expect"].items():
            assert orc.get_scale_min_k4(int(j), case["scales"]) == tuple(exp)


def test_q5_0_reference_vectors():  # src/quant/q5_0.rs:89-125
    c = KA["q5_0_roundtrip"]
    st, out = orc.dequant(orc.Q5_0, _data("q5_0_roundtrip"), 32)
    assert st == orc.OK and np.max(np.abs(out - np.array(c["expected"], dtype=np.float32))) < c["tol"]
    st, out = orc.dequant(orc.Q5_0, _data("q5_0_high_bit_extremes"), 32)
    for i, v in KA["q5_0_high_bit_extremes"]["expected_at"].items():
        assert out[int(i)] == v


def test_q5_k_reference_vectors():  # src/quant/q5_k.rs:348-373
    for name in ("q5_k_range", "q5_k_zero_scale"):
        c = KA[name]
        st, out = orc.dequant(orc.Q5_K, _data(name), 256)
        assert st == orc.OK and np.all(np.abs(out - c["expected_all"]) <= c["tol"])


def test_q2_k_reference_vectors():  # src/quant/q2_k.rs:108-177
    assert orc.type_size(orc.Q2_K, 256) == 84 and orc.type_size(orc.Q2_K, 512) == 168
    c = KA["q2_k_zero_block"]
    st, out = orc.dequant(orc.Q2_K, _data("q2_k_zero_block"), 256)
    assert st == orc.OK and np.all(out == c["expected_all"])
    c = KA["q2_k_basic_pattern"]
    st, out = orc.dequant(orc.Q2_K, _data("q2_k_basic_pattern"), 256)
    assert st == orc.OK
    for lo, hi, v in c["expected_ranges"]:
        assert np.all(np.abs(out[lo:hi] - v) < c["tol"])
    # "row length is not a multiple of 256" and "data too short" are errors (q2_k.rs:31-46)
    assert orc.dequant(orc.Q2_K, _data("q2_k_basic_pattern"), 100)[0] == orc.ELEN
    assert orc.dequant(orc.Q2_K, _data("q2_k_basic_pattern")[:80], 256)[0] == orc.ESHORT


@pytest.mark.parametrize("name,dtype,fn", [("q8_0_three_blocks", orc.Q8_0, rn.dequant_q8_0),
                                           ("q2_k_basic_pattern", orc.Q2_K, rn.dequant_q2_k),
                                           ("q5_k_block", orc.Q5_K, rn.dequant_q5_k),
                                           ("q5_0_roundtrip", orc.Q5_0, rn.dequant_q5_0),
                                           ("q4_k_block", orc.Q4_K, rn.dequant_q4_k),
                                           ("q6_k_block", orc.Q6_K, rn.dequant_q6_k)])
def test_reference_test_blocks_match_numpy_statement(name, dtype, fn):
    d, n = _data(name), KA[name]["n"]
    st, out = orc.dequant(dtype, d, n)
    assert st == orc.OK
    assert np.array_equal(out.view(np.uint32), fn(d, n).view(np.uint32))


def test_q4_k_block_spot_values():
    # hand evaluation of src/quant/q4_k.rs:66-82 on the block of q4_k.rs:244-259:
    # d=f16(0.05), dmin=f16(-0.01); sub-block 0: sc=10, m=50; qs[0]=0 -> low nibble 0
    d = np.float32(np.float16(0.05)); dmin = np.float32(np.float16(-0.01))
    _, out = orc.dequant(orc.Q4_K, _data("q4_k_block"), 256)
    assert out[0] == np.float32(np.float32(d * np.float32(10)) * np.float32(0) - np.float32(dmin * np.float32(50)))
    # element 33: high nibble of qs[1]=13 -> 0, sub-block 1: sc=20, m=60
    assert out[33] == np.float32(np.float32(d * np.float32(20)) * np.float32(0) - np.float32(dmin * np.float32(60)))
    # element 1: low nibble of qs[1]=13 -> 13
    assert out[1] == np.float32(np.float32(d * np.float32(10)) * np.float32(13) - np.float32(dmin * np.float32(50)))


def test_q6_k_block_spot_values():
    # src/quant/q6_k.rs:25-32,67-70 on the block of q6_k.rs:148-164
    blk = _data("q6_k_block")
    d = np.float32(np.float16(0.02))
    _, out = orc.dequant(orc.Q6_K, blk, 256)
    ql, qh, sc = blk[:128], blk[128:192], blk[192:208].view(np.int8)
    l = 5
    q1 = int((ql[l] & 0xF) | (((qh[l] >> 0) & 3) << 4)) - 32
    q4 = int((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32
    assert out[l] == np.float32(np.float32(d * np.float32(sc[0])) * np.float32(q1))
    assert out[l + 96] == np.float32(np.float32(d * np.float32(sc[6])) * np.float32(q4))


@pytest.mark.parametrize("name,dtype", [("f32_row", orc.F32), ("f16_row", orc.F16), ("bf16_row", orc.BF16)])
def test_plain_rows(name, dtype):  # src/quant/mod.rs:176-205
    c = KA[name]
    st, out = orc.dequant(dtype, _data(name), c["n"])
    assert st == orc.OK
    assert np.max(np.abs(out - np.array(c["expected"], dtype=np.float32))) <= c["tol"]


def test_rope_freq_scale():  # src/model/llama/cpu_path.rs:1034-1060
    for ty, factor, exp in KA["rope_freq_scale"]["cases"]:
        assert orc.rope_freq_scale(ty, factor) == exp


def test_f16_widening_is_exact_for_every_bit_pattern():
    bits = np.arange(65536, dtype=np.uint16)
    want = bits.view(np.float16).astype(np.float32)
    got = np.array([orc.f16_to_f32(int(b)) for b in bits], dtype=np.float32)
    nan = np.isnan(want)
    assert np.array_equal(np.isnan(got), nan)
    assert np.array_equal(got[~nan].view(np.uint32), want[~nan].view(np.uint32))


@pytest.mark.parametrize("dtype,fn,blk", [(orc.Q8_0, rn.dequant_q8_0, 34 / 32), (orc.Q4_K, rn.dequant_q4_k, 144 / 256),
                                          (orc.Q5_K, rn.dequant_q5_k, 176 / 256), (orc.Q5_0, rn.dequant_q5_0, 22 / 32),
                                          (orc.Q6_K, rn.dequant_q6_k, 210 / 256), (orc.Q2_K, rn.dequant_q2_k, 84 / 256)])
def test_random_blocks_match_numpy_statement_bitwise(dtype, fn, blk):
    from agention_infer_b200 import synth
    row_len, n_rows = 1024, 64
    table = synth.quant_table(dtype, n_rows, row_len, cfg_index=0)
    assert table.shape[1] == orc.type_size(dtype, row_len) == int(row_len * blk)
    ids = np.arange(n_rows, dtype=np.uint32)
    st, out = orc.get_rows(dtype, table, n_rows, row_len, ids)
    assert st == orc.OK
    want = fn(table.reshape(-1), n_rows * row_len).reshape(n_rows, row_len)
    assert np.array_equal(out.view(np.uint32), want.view(np.uint32))


def _bits_f32(bits):
    return np.array(bits, dtype=np.uint32).view(np.float32)


def test_q8_k_reference_tests():  # src/quant/q8_k.rs:97-139
    c = KA["q8_k_roundtrip_error"]
    x = _bits_f32(c["x_bits"])
    d, qs, bs = orc.quantize_rows_q8_k(x[None])
    assert d.shape == (1, c["n_blocks"])
    assert np.abs(d[0, 0] * qs[0].astype(np.float32) - x).max() < c["dequant_abs_err_below"]
    x = _bits_f32(KA["q8_k_bsums"]["x_bits"])
    d, qs, bs = orc.quantize_rows_q8_k(x[None])
    assert np.array_equal(bs[0], qs[0].reshape(16, 16).astype(np.int16).sum(axis=1))
    c = KA["q8_k_all_zero"]
    d, qs, bs = orc.quantize_rows_q8_k(_bits_f32(c["x_bits"])[None])
    assert d[0, 0] == c["d"][0] and np.all(qs == c["qs_all"])
    c = KA["q8_k_partial_block"]
    x = _bits_f32(c["x_bits"])
    assert x.size == c["n"]
    d, qs, bs = orc.quantize_rows_q8_k(x[None])
    assert d.shape[1] == c["n_blocks"] and qs.shape[1] == c["qs_len"] and bs.shape[1] == c["bsums_len"]
    assert np.all(qs[0, c["n"]:] == 0)  # "padded block should still be safe to read": zero past n


def test_q8_k_hand_values():
    """One block worked by hand: max magnitude is the NEGATIVE value -4 at index 2 (first of the ties with +4 at
    index 9) -> iscale = -127 / -4 = 31.75, d = 1 / 31.75; 1.0 -> 31.75 -> 32; 0.5 -> 15.875 -> 16; -4 -> -127;
    +4 -> 127; -1 -> -32.  Then the same with the positive 4 first, and exact .5 products."""
    x = np.zeros(256, np.float32)
    x[0], x[1], x[2], x[9], x[17] = 1.0, 0.5, -4.0, 4.0, -1.0
    d, qs, bs = orc.quantize_rows_q8_k(x[None])
    assert d[0, 0] == np.float32(1.0) / np.float32(31.75)
    assert list(qs[0, [0, 1, 2, 9, 17]]) == [32, 16, -127, 127, -32]
    assert list(bs[0, :2]) == [32 + 16 - 127 + 127, -32]
    y = x.copy(); y[2], y[9] = 4.0, -4.0  # the positive one first: signs flip, d is negative
    d2, q2, _ = orc.quantize_rows_q8_k(y[None])
    assert d2[0, 0] == -d[0, 0] and list(q2[0, [0, 1, 2, 9, 17]]) == [-32, -16, -127, 127, 32]
    # round half away from zero: iscale = -127 / -127 = 1 -> values k + 0.5 round outwards
    z = np.zeros(256, np.float32); z[0], z[1], z[2], z[3], z[4] = -127.0, 0.5, 1.5, -0.5, -2.5
    _, q3, _ = orc.quantize_rows_q8_k(z[None])
    assert list(q3[0, :5]) == [-127, 1, 2, -1, -3]


def test_q8_k_matches_numpy_statement_bitwise():
    rng = np.random.default_rng(815)
    for n in (256, 100, 1000, 3584, 257):
        x = (rng.standard_normal((9, n)) * rng.choice([1e-3, 1.0, 50.0], size=(9, 1))).astype(np.float32)
        x[1, : min(n, 256)] = 0.0  # an all-zero block
        x[2, 3] = np.nan; x[3, 5] = np.inf; x[4, 7] = 1e-41  # NaN skipped by the scan; inf and a subnormal maximum
        x[5, :] = 0.0; x[5, 7] = 1e-41  # subnormal maximum alone: iscale overflows to -inf
        got = orc.quantize_rows_q8_k(x)
        want = rn.quantize_rows_q8_k(x)
        assert np.array_equal(got[0].view(np.uint32), want[0].view(np.uint32)), n
        assert np.array_equal(got[1], want[1]), n
        assert np.array_equal(got[2], want[2]), n


def test_type_sizes():  # src/types.rs:88-168
    assert orc.type_size(orc.Q8_0, 2048) == 2176
    assert orc.type_size(orc.Q4_K, 3584) == 2016
    assert orc.type_size(orc.Q6_K, 4096) == 3360
    assert orc.type_size(orc.Q8_0, 33) == 68
    assert orc.type_size(orc.F16, 7) == 14
    assert orc.type_size(99, 7) == 0


def test_dequant_row_range_and_bounds():  # src/quant/mod.rs:116-131
    from agention_infer_b200 import synth
    table = synth.quant_table(orc.Q8_0, 4, 64)
    st, _ = orc.dequant_row(orc.Q8_0, table, 0, 64, 4, 4)
    assert st == orc.EROW
    st, _ = orc.dequant_row(orc.Q8_0, table.reshape(-1)[:-1], 0, 64, 4, 3)
    assert st == orc.ESHORT
    st, row = orc.dequant_row(orc.Q8_0, table, 0, 64, 4, 3)
    assert st == orc.OK and np.array_equal(row, rn.dequant_q8_0(table[3], 64))


def test_get_rows_bad_id_zero_row_and_status():
    from agention_infer_b200 import synth
    table = synth.quant_table(orc.Q4_K, 8, 256)
    st, out = orc.get_rows(orc.Q4_K, table, 8, 256, np.array([1, 8, 7], dtype=np.uint32))
    assert st == orc.EROW
    assert not out[1].any() and out[0].any() and out[2].any()
