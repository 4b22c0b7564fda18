"""Committed golden fixtures (tests/golden/oracle_small.npz, written by
tests/golden/make_oracle_fixtures.py).  On CPU: the oracle built here must reproduce them
bit for bit (integer codecs) or within 2 ulp-scale (float ops; libm versions may differ in
the last bit of exp/sin/cos).  On the GPU: the CUDA library is compared with the same
committed numbers, independent of the oracle build on that machine."""
from pathlib import Path

import numpy as np
import pytest

from agention_infer_b200 import AGN_Q4_K, AGN_Q6_K, AGN_Q8_0, AGN_ROPE_NEOX, AGN_ROPE_NORMAL, synth
from oracle import oracle as orc

G = np.load(Path(__file__).parent / "golden" / "oracle_small.npz")
T, H, hd, nq, nkv, I = 12, 512, 64, 4, 2, 768
LIBM = 5e-7  # relative to row scale: last-bit differences between libm builds
TOL = 1e-5   # GPU vs committed oracle output


def rel(a, b):
    return synth.max_rel_to_row_scale(a, b)


def test_oracle_reproduces_quant_fixtures_bitwise():
    for name, dt, rl in (("q8_0", orc.Q8_0, 96), ("q4_k", orc.Q4_K, 512), ("q6_k", orc.Q6_K, 512)):
        st, rows = orc.get_rows(dt, G[f"{name}_table"], 24, rl, G[f"{name}_ids"])
        assert st == orc.OK and np.array_equal(rows.view(np.uint32), G[f"{name}_rows"].view(np.uint32))


def test_oracle_reproduces_float_fixtures():
    assert rel(orc.rms_norm_rows(G["rms_x"], G["rms_w"], 1e-5), G["rms_out"]) <= LIBM
    nx, nm = orc.add_residual_rms_norm_rows(G["rms_x"], G["res_delta"], G["rms_w"], 1e-5)
    assert np.array_equal(nx, G["res_new_x"]) and rel(nm, G["res_normed"]) <= LIBM
    q, k, pos = G["rope_q"], G["rope_k"], G["rope_pos"]
    assert rel(orc.rope_rows(q, nq, hd, hd, pos, 500000.0, 1.0, orc.NEOX), G["rope_q_neox"]) <= LIBM
    assert rel(orc.rope_rows(k, nkv, hd, hd, pos, 500000.0, 1.0, orc.NEOX), G["rope_k_neox"]) <= LIBM
    assert rel(orc.rope_rows(q, nq, hd, hd, pos, 500000.0, 1.0, orc.NORMAL), G["rope_q_normal"]) <= LIBM
    assert rel(orc.rope_rows(q, nq, hd, 32, pos, 10000.0, 0.5, orc.NEOX), G["rope_q_partial"]) <= LIBM
    assert rel(orc.qk_norm_rope_rows(q, G["qknorm_w"], nq, hd, 1e-6, hd, pos, 1e6), G["qknorm_rope_q"]) <= LIBM
    assert rel(orc.silu_mul(G["silu_gate"], G["silu_up"]), G["silu_out"]) <= LIBM
    assert rel(orc.softmax_rows(G["softmax_in"], G["softmax_nv"]), G["softmax_out"]) <= LIBM
    idx, w = orc.router_top2(G["router_logits"])
    assert np.array_equal(idx, G["router_idx"]) and rel(w, G["router_w"]) <= LIBM
    go, goff, gtok, gslot = orc.gather_rows_by_expert(G["gather_x"], idx, 8)
    assert np.array_equal(go, G["gather_out"]) and np.array_equal(goff, G["gather_offsets"])
    assert np.array_equal(gtok, G["gather_token"]) and np.array_equal(gslot, G["gather_slot"])


@pytest.mark.gpu
def test_gpu_matches_committed_fixtures(backend):
    be = backend
    up = be.upload
    for name, dt, rl in (("q8_0", AGN_Q8_0, 96), ("q4_k", AGN_Q4_K, 512), ("q6_k", AGN_Q6_K, 512)):
        table = np.ascontiguousarray(G[f"{name}_table"])
        out = be.get_rows(dt, up(table), table.nbytes, 24, rl, up(G[f"{name}_ids"]), 6)
        assert np.array_equal(be.read(out, np.float32, (6, rl)).view(np.uint32), G[f"{name}_rows"].view(np.uint32))
    out = be.launch_rms_norm(up(G["rms_x"]), up(G["rms_w"]), T, H, 1e-5)
    assert rel(be.read(out, np.float32, (T, H)), G["rms_out"]) <= TOL
    nx, nm = be.launch_add_residual_rms_norm(up(G["rms_x"]), up(G["res_delta"]), up(G["rms_w"]), T, H, 1e-5)
    assert np.array_equal(be.read(nx, np.float32, (T, H)), G["res_new_x"])
    assert rel(be.read(nm, np.float32, (T, H)), G["res_normed"]) <= TOL
    dpos = up(G["rope_pos"])
    for key, n_rot, theta, fs, layout in (("rope_q_neox", hd, 500000.0, 1.0, AGN_ROPE_NEOX),
                                          ("rope_q_normal", hd, 500000.0, 1.0, AGN_ROPE_NORMAL),
                                          ("rope_q_partial", 32, 10000.0, 0.5, AGN_ROPE_NEOX)):
        dq = up(G["rope_q"])
        be.launch_rope(dq, T, nq, hd, n_rot, dpos, theta, fs, layout)
        assert rel(be.read(dq, np.float32, (T, nq * hd)), G[key]) <= TOL, key
    dq, dk = up(G["rope_q"]), up(G["rope_k"])
    be.launch_rope_qk(dq, dk, T, nq, nkv, hd, hd, dpos, 500000.0)
    assert rel(be.read(dq, np.float32, (T, nq * hd)), G["rope_q_neox"]) <= TOL
    assert rel(be.read(dk, np.float32, (T, nkv * hd)), G["rope_k_neox"]) <= TOL
    dq = up(G["rope_q"])
    be.launch_qk_norm_rope(dq, up(G["qknorm_w"]), T, nq, hd, 1e-6, hd, dpos, 1e6)
    assert rel(be.read(dq, np.float32, (T, nq * hd)), G["qknorm_rope_q"]) <= TOL
    out = be.launch_silu_mul(up(G["silu_gate"]), up(G["silu_up"]), T * I)
    assert rel(be.read(out, np.float32, (T, I)), G["silu_out"]) <= TOL
    out = be.launch_softmax_rows(up(G["softmax_in"]), 64, 32, n_valid=up(G["softmax_nv"]))
    assert rel(be.read(out, np.float32, (2, 32, 32)), G["softmax_out"]) <= TOL
    idx, w = be.router_top2(up(G["router_logits"]), 16, 8)
    assert np.array_equal(be.read(idx, np.int32, (16, 2)), G["router_idx"])
    assert rel(be.read(w, np.float32, (16, 2)), G["router_w"]) <= TOL
    go, goff, gtok, gslot = be.gather_rows_by_expert(up(G["gather_x"]), idx, 16, 64, 8)
    assert np.array_equal(be.read(go, np.float32, (32, 64)), G["gather_out"])
    assert np.array_equal(be.read(goff, np.int32, (9,)), G["gather_offsets"])
    assert np.array_equal(be.read(gtok, np.int32, (32,)), G["gather_token"])


Q8K = np.load(Path(__file__).parent / "golden" / "q8k_small.npz")


def _same_q8k(got, what):
    assert np.array_equal(got[0].view(np.uint32), Q8K["d"].view(np.uint32)), f"{what}: d"
    assert np.array_equal(got[1], Q8K["qs"]) and np.array_equal(got[2], Q8K["bsums"]), f"{what}: qs / bsums"


def test_oracle_reproduces_q8_k_fixture_bitwise():
    with np.errstate(all="ignore"):
        _same_q8k(orc.quantize_rows_q8_k(Q8K["x"]), "oracle")


@pytest.mark.gpu
def test_gpu_matches_committed_q8_k_fixture(backend):
    x = np.ascontiguousarray(Q8K["x"])
    T, n = x.shape
    nb = (n + 255) // 256
    d, qs, bs = backend.launch_quantize_rows_q8_k(backend.upload(x), T, n)
    _same_q8k((backend.read(d, np.float32, (T, nb)), backend.read(qs, np.int8, (T, nb * 256)),
               backend.read(bs, np.int16, (T, nb * 16))), "gpu")
