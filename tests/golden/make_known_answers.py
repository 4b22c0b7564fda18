"""Writes tests/golden/reference_known_answers.json: the input/expected pairs of the
reference's own unit tests for the quant codecs and the RoPE scale helper, transcribed from
the cited test bodies (the reference is Rust and cannot be run here, so its tests are read
as data).  Run: python tests/golden/make_known_answers.py
"""
import json
from pathlib import Path

import numpy as np


def f16_bytes(v: float) -> list:
    return list(np.array([v], dtype=np.float16).view(np.uint8))


def q8_block(scale: float, vals) -> list:
    return [int(b) for b in f16_bytes(scale)] + [int(np.uint8(np.int8(v))) for v in vals]


cases = {}

# src/quant/q8_0.rs:110-126  test_dequant_q8_0_single_block
vals = [(i % 5) - 2 for i in range(32)]
cases["q8_0_single_block"] = {
    "cite": "src/quant/q8_0.rs:110-126", "data": q8_block(2.0, vals), "n": 32,
    "expected": [2.0 * v for v in vals], "tol": 1e-6}

# src/quant/q8_0.rs:129-148  test_dequant_q8_0_partial_block
data = q8_block(1.0, list(range(32))) + q8_block(1.0, [42] + [0] * 31)
cases["q8_0_partial_block"] = {
    "cite": "src/quant/q8_0.rs:129-148", "data": data, "n": 33, "expected_len": 33,
    "expected_at": {"32": 42.0}}

# src/quant/q8_0.rs:151-170  test_dot_q8_0_matches_dequant (inputs only; the assertion is dot == dequant.x)
data = []
for b in range(3):
    data += q8_block(0.75, [((i + b) % 7) - 3 for i in range(32)])
cases["q8_0_three_blocks"] = {"cite": "src/quant/q8_0.rs:151-170", "data": data, "n": 70}

# src/quant/q4_k.rs:229-241  test_get_scale_min_k4
cases["q4_k_scale_min"] = {
    "cite": "src/quant/q4_k.rs:229-241",
    "cases": [
        {"scales": [10, 20, 30, 40, 50, 60, 70, 80, 0, 0, 0, 0],
         "expect": {"0": [10, 50], "1": [20, 60], "2": [30, 6], "3": [40, 16]}},
        {"scales": [0xC0, 0x80, 0x40, 0x00, 0x00, 0x00, 0x00, 0x00, 0x3F, 0x2F, 0x1F, 0x0F],
         "expect": {"4": [0x3F, 3], "5": [0x2F, 2]}},
    ]}

# src/quant/q4_k.rs:244-259  test_dot_q4_k_matches_dequant (block inputs)
scales = [10, 20, 30, 40, 50, 60, 70, 80, 0x3F, 0x2F, 0x1F, 0x0F]
quants = [(i * 13) & 0xFF for i in range(128)]
cases["q4_k_block"] = {
    "cite": "src/quant/q4_k.rs:244-259",
    "data": [int(b) for b in f16_bytes(0.05)] + [int(b) for b in f16_bytes(-0.01)] + scales + quants, "n": 256}

# src/quant/q6_k.rs:148-164  test_dot_q6_k_matches_dequant (block inputs)
ql = [(i * 37) & 0xFF for i in range(128)]
qh = [((i * 53) + 1) & 0xFF for i in range(64)]
sc = [int(np.uint8(np.int8(i - 6))) for i in range(16)]
cases["q6_k_block"] = {
    "cite": "src/quant/q6_k.rs:148-164", "data": ql + qh + sc + [int(b) for b in f16_bytes(0.02)], "n": 256}

# src/quant/q5_0.rs:89-125  roundtrip_single_block / high_bit_extremes (packer of q5_0.rs:68-87)
def q5_0_block(scale, values):
    qh = 0
    qs = [0] * 16
    for j in range(16):
        v0, v1 = values[j] + 16, values[j + 16] + 16
        if (v0 >> 4) & 1:
            qh |= 1 << j
        if (v1 >> 4) & 1:
            qh |= 1 << (j + 16)
        qs[j] = (v0 & 0x0F) | ((v1 & 0x0F) << 4)
    return [int(b) for b in f16_bytes(scale)] + [(qh >> (8 * i)) & 0xFF for i in range(4)] + qs


vals = [(i % 32) - 16 for i in range(32)]
cases["q5_0_roundtrip"] = {"cite": "src/quant/q5_0.rs:89-107", "data": q5_0_block(0.5, vals), "n": 32,
                           "expected": [0.5 * v for v in vals], "tol": 1e-4}
vals = [0] * 32
vals[0], vals[16], vals[1] = 15, -16, -1
cases["q5_0_high_bit_extremes"] = {"cite": "src/quant/q5_0.rs:109-125", "data": q5_0_block(1.0, vals), "n": 32,
                                   "expected_at": {"0": 15.0, "16": -16.0, "1": -1.0}}


# src/quant/q5_k.rs:348-392  range / zero-scale / dot-vs-dequant blocks (d, dmin, scales[12], qh[32], qs[128])
def q5_k_block(d, dmin, scales, qh, qs):
    return [int(b) for b in f16_bytes(d)] + [int(b) for b in f16_bytes(dmin)] + list(scales) + list(qh) + list(qs)


cases["q5_k_range"] = {"cite": "src/quant/q5_k.rs:348-363",
                       "data": q5_k_block(1.0, 0.0, [0xFF] * 4 + [0] * 4 + [0x0F] * 4, [0xFF] * 32, [0xFF] * 128),
                       "n": 256, "expected_all": 63.0 * 31.0, "tol": 1.0}
cases["q5_k_zero_scale"] = {"cite": "src/quant/q5_k.rs:365-373",
                            "data": q5_k_block(1.0, 0.0, [0] * 12, [0] * 32, [0] * 128), "n": 256,
                            "expected_all": 0.0, "tol": 0.0}
cases["q5_k_block"] = {"cite": "src/quant/q5_k.rs:375-392",
                       "data": q5_k_block(0.05, -0.01, [10, 20, 30, 40, 50, 60, 70, 80, 0x3F, 0x2F, 0x1F, 0x0F],
                                          [((i * 29) + 3) & 0xFF for i in range(32)],
                                          [(i * 13) & 0xFF for i in range(128)]), "n": 256}

# src/quant/q2_k.rs:113-177  zero block and basic pattern (scales[16] | qs[64] | f16 d | f16 dmin)
def q2_k_block(d, dmin, scales, qs):
    return list(scales) + list(qs) + [int(b) for b in f16_bytes(d)] + [int(b) for b in f16_bytes(dmin)]


cases["q2_k_zero_block"] = {"cite": "src/quant/q2_k.rs:113-127", "data": q2_k_block(1.0, 0.0, [0] * 16, [0] * 64),
                            "n": 256, "expected_all": 0.0, "tol": 0.0}
cases["q2_k_basic_pattern"] = {"cite": "src/quant/q2_k.rs:129-177",
                               "data": q2_k_block(2.0, 0.5, [0x21, 0x43] + [0] * 14, [0xFF] * 32 + [0] * 32), "n": 256,
                               "expected_ranges": [[0, 16, 5.0], [16, 32, 16.0]], "tol": 1e-5}

# src/quant/mod.rs:176-205  f32 / f16 / bf16 rows
cases["f32_row"] = {"cite": "src/quant/mod.rs:176-185",
                    "data": [int(b) for b in np.array([1.0, 2.0, -3.5], dtype="<f4").view(np.uint8)], "n": 3,
                    "expected": [1.0, 2.0, -3.5], "tol": 0.0}
cases["f16_row"] = {"cite": "src/quant/mod.rs:187-196",
                    "data": [int(b) for b in np.array([1.5, -2.25], dtype="<f2").view(np.uint8)], "n": 2,
                    "expected": [1.5, -2.25], "tol": 1e-3}
cases["bf16_row"] = {"cite": "src/quant/mod.rs:198-205", "data": [0x80, 0x3F, 0x00, 0xC0], "n": 2,
                     "expected": [1.0, -2.0], "tol": 1e-3}

# src/quant/q8_k.rs:97-139  quantize_row_q8_k: the four test inputs (as f32 bit patterns) and what each test asserts
def f32_bits(a) -> list:
    return [int(v) for v in np.asarray(a, dtype=np.float32).view(np.uint32)]


cases["q8_k_roundtrip_error"] = {
    "cite": "src/quant/q8_k.rs:97-109", "x_bits": f32_bits((np.arange(256, dtype=np.float32) - np.float32(128.0)) * np.float32(0.1)),
    "n_blocks": 1, "dequant_abs_err_below": 0.15}
cases["q8_k_bsums"] = {
    "cite": "src/quant/q8_k.rs:111-119", "x_bits": f32_bits(((np.arange(256) % 7).astype(np.float32) - np.float32(3.0)) * np.float32(0.3)),
    "bsums_are_group_sums": True}
cases["q8_k_all_zero"] = {"cite": "src/quant/q8_k.rs:121-127", "x_bits": f32_bits(np.zeros(256)), "d": [0.0], "qs_all": 0}
cases["q8_k_partial_block"] = {
    "cite": "src/quant/q8_k.rs:129-139", "x_bits": f32_bits(np.arange(100, dtype=np.float32) * np.float32(0.01)),
    "n": 100, "n_blocks": 1, "qs_len": 256, "bsums_len": 16}

# src/model/llama/cpu_path.rs:1034-1060  compute_rope_freq_scale
cases["rope_freq_scale"] = {
    "cite": "src/model/llama/cpu_path.rs:1034-1060",
    "cases": [[None, None, 1.0], ["none", 8.0, 1.0], ["", 8.0, 1.0], ["linear", 4.0, 0.25], ["linear", 2.0, 0.5],
              ["linear", None, 1.0], ["yarn", 4.0, None]]}

out = Path(__file__).with_name("reference_known_answers.json")
out.write_text(json.dumps(cases, indent=1) + "\n")
print("wrote", out)
