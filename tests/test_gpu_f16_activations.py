"""f16 activation storage (the reference's default `Act = f16`): f16 buffers in and out, f32
arithmetic.  The expected value is the f32 oracle applied to the f16-decoded inputs and
rounded to f16 where the reference's f16 kernels store (`Act::cast_from`).  Tolerance: one
f16 ulp of the row scale (2^-10), since the f32 value before the final rounding may differ
from the oracle's by an f32 ulp and land on the other side of an f16 rounding boundary;
get_rows (a pure conversion of bit-exact f32 values) is bit-exact."""
import numpy as np
import pytest

from agention_infer_b200 import AGN_Q4_K, AGN_Q6_K, AGN_Q8_0, AGN_ROPE_NEOX, AGN_ROPE_NORMAL, synth
from oracle import oracle as orc

pytestmark = pytest.mark.gpu
F16_ULP = 2.0 ** -10
THREADS = max(1, orc.max_threads())


def h(a):
    return a.astype(np.float16)


def f(a):
    return a.astype(np.float32)


def close(got16, ref16):
    got, ref = f(got16), f(ref16)
    err = synth.max_rel_to_row_scale(got, ref)
    same = float(np.mean(got16.view(np.uint16) == ref16.view(np.uint16)))
    assert err <= F16_ULP, err
    assert same > 0.995, same  # almost every element is bit-identical


@pytest.mark.parametrize("n", [4096 * 3 + 1, 512 * 8192, 7])
def test_silu_mul_f16(backend, n):
    g, u = h(synth.activations(1, "gate", (n,))), h(synth.activations(1, "up", (n,)))
    ref = h(orc.silu_mul(f(g), f(u), THREADS))
    out = backend.launch_silu_mul_f16(backend.upload(g), backend.upload(u), n)
    got = backend.read(out, np.float16, (n,))
    assert np.max(np.abs(f(got) - f(ref)) / np.maximum(np.abs(f(ref)), 1.0)) <= F16_ULP
    assert np.mean(got.view(np.uint16) == ref.view(np.uint16)) > 0.995


@pytest.mark.parametrize("T,H", [(512, 2048), (64, 3584), (3, 250), (2, 40000)])
def test_rms_norm_f16(backend, T, H):
    x = h(synth.activations(2, "x", (T, H))); w = synth.norm_weight(2, "w", H)
    ref = h(orc.rms_norm_rows(f(x), w, 1e-6, THREADS))
    out = backend.launch_rms_norm_f16(backend.upload(x), backend.upload(w), T, H, 1e-6)
    close(backend.read(out, np.float16, (T, H)), ref)


@pytest.mark.parametrize("T,H", [(64, 4096), (5, 250)])
def test_add_residual_rms_norm_f16(backend, T, H):
    x = h(synth.activations(4, "x", (T, H))); d = h(synth.activations(4, "delta", (T, H))); w = synth.norm_weight(4, "w", H)
    new_x = h(f(x) + f(d))  # stored as f16, and that stored value is what gets normalised
    ref = h(orc.rms_norm_rows(f(new_x), w, 1e-5, THREADS))
    nx, nm = backend.launch_add_residual_rms_norm_f16(backend.upload(x), backend.upload(d), backend.upload(w), T, H, 1e-5)
    assert np.array_equal(backend.read(nx, np.float16, (T, H)).view(np.uint16), new_x.view(np.uint16))
    close(backend.read(nm, np.float16, (T, H)), ref)


@pytest.mark.parametrize("layout", [AGN_ROPE_NEOX, AGN_ROPE_NORMAL])
@pytest.mark.parametrize("T,nq,nkv,hd,n_rot", [(300, 28, 4, 128, 128), (64, 32, 8, 64, 64), (9, 4, 2, 256, 64), (5, 3, 1, 96, 96)])
def test_rope_and_fused_norm_rope_f16(backend, layout, T, nq, nkv, hd, n_rot):
    q = h(synth.activations(3, "q", (T, nq * hd))); k = h(synth.activations(3, "k", (T, nkv * hd)))
    wq = synth.norm_weight(3, "wq", hd); wk = synth.norm_weight(3, "wk", hd); pos = synth.positions(3, T, True)
    dpos = backend.upload(pos)
    # rope alone
    rq = h(orc.rope_rows(f(q), nq, hd, n_rot, pos, 1e6, 1.0, layout, THREADS))
    rk = h(orc.rope_rows(f(k), nkv, hd, n_rot, pos, 1e6, 1.0, layout, THREADS))
    dq, dk = backend.upload(q), backend.upload(k)
    backend.launch_qk_norm_rope_qk_f16(dq, dk, None, None, T, nq, nkv, hd, 0.0, n_rot, dpos, 1e6, 1.0, layout)
    close(backend.read(dq, np.float16, q.shape), rq); close(backend.read(dk, np.float16, k.shape), rk)
    # fused: per-head norm, stored as f16 (the reference's f16 kernel re-reads it), then rope
    def fused(x, w, nh):
        normed = h(orc.rms_norm_rows(f(x).reshape(T * nh, hd), w, 1e-6, THREADS)).reshape(T, nh * hd)
        return h(orc.rope_rows(f(normed), nh, hd, n_rot, pos, 1e6, 1.0, layout, THREADS))
    dq, dk = backend.upload(q), backend.upload(k)
    backend.launch_qk_norm_rope_qk_f16(dq, dk, backend.upload(wq), backend.upload(wk), T, nq, nkv, hd, 1e-6, n_rot, dpos,
                                       1e6, 1.0, layout)
    got_q, got_k = backend.read(dq, np.float16, q.shape), backend.read(dk, np.float16, k.shape)
    # the intermediate f16 rounding can flip on an f32 ulp: allow two f16 ulps of the row scale
    assert synth.max_rel_to_row_scale(f(got_q), f(fused(q, wq, nq))) <= 2 * F16_ULP
    assert synth.max_rel_to_row_scale(f(got_k), f(fused(k, wk, nkv))) <= 2 * F16_ULP


@pytest.mark.parametrize("dtype,vocab,H,T", [(AGN_Q4_K, 4096, 3584, 1024), (AGN_Q8_0, 500, 96, 77), (AGN_Q6_K, 64, 300, 33)])
def test_get_rows_f16_is_the_rounded_f32_row(backend, dtype, vocab, H, T):
    table = synth.quant_table(dtype, vocab, H, cfg_index=2); ids = synth.token_ids(2, T, vocab)
    st, ref = orc.get_rows(dtype, table, vocab, H, ids, THREADS)
    out = backend.get_rows_f16(dtype, backend.upload(table), table.nbytes, vocab, H, backend.upload(ids), T)
    got = backend.read(out, np.float16, (T, H))
    assert st == orc.OK and np.array_equal(got.view(np.uint16), h(ref).view(np.uint16))
