"""Entry points that widen the path toward its callers: normed rows stored as f16 / bf16 from
f32 inputs, and a softmax that takes the score scale.

16-bit outputs: the kernel computes the same f32 value as the f32 entry point and rounds it to
nearest even on store, so (a) it must equal the f32 entry point's own output rounded on the host
bit for bit, and (b) it sits within one ulp of the 16-bit format (2^-10 of the row scale for f16,
2^-7 for bf16) of the oracle's f32 result rounded the same way.
Scaled softmax: the oracle runs the softmax over scale * scores computed in f32 first (what the
reference's `attention_scores` stores, src/ops/kernels_wgpu.rs:773-782); tolerance 1e-5 of the
row scale as for the plain softmax."""
import numpy as np
import pytest

from agention_infer_b200 import AGN_BF16, AGN_F16, AGN_Q8_0, BackendError, synth
from oracle import oracle as orc
from tests.ref_numpy import softmax64

pytestmark = pytest.mark.gpu
THREADS = max(1, orc.max_threads())
TOL = 1e-5
# Rows of more than ~40000 entries: the reference sums exp() sequentially in f32, and that sum alone
# drifts from the exact one (1e-5 at 65536 entries of N(0, 4), 2e-4 over a 128256-entry vocabulary
# where a few terms dominate and every small term is rounded against the large partial sum), while
# the kernels sum in a tree.  Such rows are held to TOL against a float64 softmax, and against the f32
# oracle to TOL plus the oracle's own distance from float64.
def check_softmax(got, s_scaled, nv, ref32):
    L = s_scaled.shape[-1]
    if L <= 40000:
        assert synth.max_rel_to_row_scale(got, ref32) <= TOL
    else:
        ref64 = softmax64(s_scaled, nv).astype(np.float32)
        assert synth.max_rel_to_row_scale(got, ref64) <= TOL
        assert synth.max_rel_to_row_scale(got, ref32) <= TOL + synth.max_rel_to_row_scale(ref32, ref64)


def to_bf16_bits(a: np.ndarray) -> np.ndarray:
    """f32 -> bf16 bit patterns, round to nearest even (finite inputs)."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def from_bf16_bits(b: np.ndarray) -> np.ndarray:
    return (b.astype(np.uint32) << 16).view(np.float32)


def check16(backend, buf, f32_gpu, f32_ref, out_dtype, shape):
    if out_dtype == AGN_F16:
        got = backend.read(buf, np.float16, shape)
        assert np.array_equal(got.view(np.uint16), f32_gpu.astype(np.float16).view(np.uint16))
        assert synth.max_rel_to_row_scale(got.astype(np.float32), f32_ref.astype(np.float16).astype(np.float32)) <= 2.0 ** -10
    else:
        got = backend.read(buf, np.uint16, shape)
        assert np.array_equal(got, to_bf16_bits(f32_gpu))
        assert synth.max_rel_to_row_scale(from_bf16_bits(got), from_bf16_bits(to_bf16_bits(f32_ref))) <= 2.0 ** -7


@pytest.mark.parametrize("out_dtype", [AGN_F16, AGN_BF16])
@pytest.mark.parametrize("T,H", [(512, 2048), (256, 3584), (3, 250), (2, 40000), (1, 4)])
def test_rms_norm_f32_to_16bit_output(backend, T, H, out_dtype):
    x, w = synth.activations(2, "x", (T, H)), synth.norm_weight(2, "w", H)
    ref = orc.rms_norm_rows(x, w, 1e-6, THREADS)
    dx, dw = backend.upload(x), backend.upload(w)
    f32_gpu = backend.read(backend.launch_rms_norm(dx, dw, T, H, 1e-6), np.float32, (T, H))
    out = backend.launch_rms_norm_out16(dx, dw, T, H, 1e-6, out_dtype)
    check16(backend, out, f32_gpu, ref, out_dtype, (T, H))


@pytest.mark.parametrize("out_dtype", [AGN_F16, AGN_BF16])
@pytest.mark.parametrize("T,H", [(128, 4096), (5, 250)])
def test_add_residual_rms_norm_f32_to_16bit_output(backend, T, H, out_dtype):
    x, d, w = synth.activations(4, "x", (T, H)), synth.activations(4, "delta", (T, H)), synth.norm_weight(4, "w", H)
    ref_x, ref_n = orc.add_residual_rms_norm_rows(x, d, w, 1e-5, THREADS)
    dx, dd, dw = backend.upload(x), backend.upload(d), backend.upload(w)
    nx32, nm32 = backend.launch_add_residual_rms_norm(dx, dd, dw, T, H, 1e-5)
    f32_gpu = backend.read(nm32, np.float32, (T, H))
    nx, nm = backend.launch_add_residual_rms_norm_out16(dx, dd, dw, T, H, 1e-5, out_dtype)
    # the residual stream stays f32 and is the exact sum
    assert np.array_equal(backend.read(nx, np.float32, (T, H)).view(np.uint32), ref_x.view(np.uint32))
    check16(backend, nm, f32_gpu, ref_n, out_dtype, (T, H))


def test_16bit_output_rejects_other_types(backend):
    x, w = backend.upload(np.ones((1, 8), np.float32)), backend.upload(np.ones(8, np.float32))
    with pytest.raises(BackendError) as e:
        backend.launch_rms_norm_out16(x, w, 1, 8, 1e-6, AGN_Q8_0)
    assert e.value.status == 2


@pytest.mark.parametrize("nh,L,hd", [(32, 512, 64), (28, 1024, 128), (4, 9999, 128), (2, 20000, 128), (3, 37, 80), (64, 8, 128), (5, 200, 96)])
def test_softmax_scaled_causal(backend, nh, L, hd):
    rows = min(L, 64)  # the last `rows` query positions of each head
    s = synth.activations(1, "scores", (nh, rows, L), std=2.0 * np.sqrt(hd))  # raw dot products: std grows with sqrt(hd)
    scale = np.float32(1.0) / np.sqrt(np.float32(hd))
    nv = np.tile(np.arange(L - rows, L, dtype=np.int32) + 1, nh)
    ref = orc.softmax_rows((s * scale).astype(np.float32).reshape(nh * rows, L), nv, THREADS)
    out = backend.launch_softmax_rows_scaled(backend.upload(s), nh * rows, L, float(scale), causal_period=rows,
                                             causal_offset=L - rows)
    got = backend.read(out, np.float32, (nh * rows, L))
    assert synth.max_rel_to_row_scale(got, ref) <= TOL
    assert np.all(got[np.arange(L)[None, :] >= nv[:, None]] == 0.0)
    # unnormalised form: weights / sums reproduces the probabilities
    sums = backend.empty(4 * nh * rows)
    wts = backend.launch_softmax_rows_scaled(backend.upload(s), nh * rows, L, float(scale), sums=sums, causal_period=rows,
                                             causal_offset=L - rows)
    gw, gs = backend.read(wts, np.float32, (nh * rows, L)), backend.read(sums, np.float32, (nh * rows,))
    assert synth.max_rel_to_row_scale(gw / gs[:, None], ref) <= TOL


def test_softmax_scale_one_is_the_plain_softmax(backend):
    s = synth.activations(1, "scores", (64, 512), std=2.0)
    ds = backend.upload(s)
    a = backend.read(backend.launch_softmax_rows(ds, 64, 512), np.float32, (64, 512))
    b = backend.read(backend.launch_softmax_rows_scaled(ds, 64, 512, 1.0), np.float32, (64, 512))
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))


@pytest.mark.parametrize("scale", [0.0, -1.0, float("inf"), float("nan")])
def test_softmax_scale_must_be_positive_and_finite(backend, scale):
    s = backend.upload(np.zeros((1, 8), np.float32))
    with pytest.raises(BackendError) as e:
        backend.launch_softmax_rows_scaled(s, 1, 8, scale)
    assert e.value.status == 1


@pytest.mark.parametrize("L", [16388, 20000, 32768, 49152, 152064])
@pytest.mark.parametrize("cluster", [1, 2, 0])
def test_softmax_long_rows_cluster_kernel(backend, L, cluster):
    """Rows of more than 16384 entries run as one thread-block cluster per row (partial maxima and
    sums merged through distributed shared memory); every valid length, the unnormalised form and
    the scaled form must agree with the oracle like the one-CTA kernels do."""
    R = 8
    s = synth.activations(1, "scores", (R, L), std=2.0)
    nv = np.array([L, L - 1, 1, 0, L // 2 + 1, 8193, 4, L - 4097], dtype=np.int32)
    ref = orc.softmax_rows(s, nv, THREADS)
    ds, dnv = backend.upload(s), backend.upload(nv)
    backend.set_option("softmax_cluster", cluster)
    try:
        got = backend.read(backend.launch_softmax_rows(ds, R, L, n_valid=dnv), np.float32, (R, L))
        sums = backend.empty(4 * R)
        wts = backend.read(backend.launch_softmax_rows_scaled(ds, R, L, 1.0, sums=sums, n_valid=dnv), np.float32, (R, L))
        gs = backend.read(sums, np.float32, (R,))
        sc = backend.read(backend.launch_softmax_rows_scaled(ds, R, L, 0.5, n_valid=dnv), np.float32, (R, L))
    finally:
        backend.set_option("softmax_cluster", 1)
    check_softmax(got, s, nv, ref)
    assert np.all(got[np.arange(L)[None, :] >= nv[:, None]] == 0.0)
    ok = nv > 0
    check_softmax(wts[ok] / gs[ok, None], s[ok], nv[ok], ref[ok])
    assert np.all(wts[~ok] == 0.0) and np.all(gs[~ok] == 0.0)
    half = (s * np.float32(0.5)).astype(np.float32)
    check_softmax(sc, half, nv, orc.softmax_rows(half, nv, THREADS))


@pytest.mark.parametrize("vocab", [128256, 152064, 262144])
def test_sampler_softmax_with_temperature(backend, vocab):
    """The sampler's softmax over a whole vocabulary, `exp((l - max) * inv_temp) / sum`
    (src/sampler.rs:79-89), for a few sequences at once."""
    rows, temp = 3, 0.7
    logits = synth.activations(3, "logits", (rows, vocab), std=3.0)
    inv_temp = np.float32(1.0) / np.float32(temp)
    scaled = (logits * inv_temp).astype(np.float32)
    got = backend.read(backend.launch_softmax_rows_scaled(backend.upload(logits), rows, vocab, float(inv_temp)),
                       np.float32, (rows, vocab))
    check_softmax(got, scaled, None, orc.softmax_rows(scaled, None, THREADS))
    assert np.all(np.abs(got.sum(axis=1, dtype=np.float64) - 1.0) < 1e-4)
    assert np.array_equal(got.argmax(axis=1), logits.argmax(axis=1))


@pytest.mark.parametrize("out_dtype", [AGN_F16, AGN_BF16])
@pytest.mark.parametrize("R,L,causal", [(64, 8, 0), (96, 200, 1), (512, 512, 1), (64, 4096, 1), (6, 9999, 0), (4, 20000, 1)])
def test_softmax_with_16bit_probabilities(backend, R, L, causal, out_dtype):
    """Every kernel family (thread, warp, CTA, scalar fallback, cluster): the 16-bit row is the f32
    entry point's own output rounded to nearest even."""
    s = synth.activations(1, "scores", (R, L), std=2.0 * 8.0)
    scale = 0.125
    ds = backend.upload(s)
    kw = dict(causal_period=min(R, L) if causal else 0, causal_offset=L - min(R, L) if causal else 0)
    f32_gpu = backend.read(backend.launch_softmax_rows_scaled(ds, R, L, scale, **kw), np.float32, (R, L))
    sums16 = backend.empty(4 * R)
    out = backend.launch_softmax_rows_scaled_out16(ds, R, L, scale, out_dtype, **kw)
    if out_dtype == AGN_F16:
        got = backend.read(out, np.float16, (R, L))
        assert np.array_equal(got.view(np.uint16), f32_gpu.astype(np.float16).view(np.uint16))
    else:
        assert np.array_equal(backend.read(out, np.uint16, (R, L)), to_bf16_bits(f32_gpu))
    # unnormalised weights in 16 bits + f32 sums
    w32 = backend.empty(4 * R * L); s32 = backend.empty(4 * R)
    backend.launch_softmax_rows_scaled(ds, R, L, scale, out=w32, sums=s32, **kw)
    w16 = backend.launch_softmax_rows_scaled_out16(ds, R, L, scale, out_dtype, sums=sums16, **kw)
    assert np.array_equal(backend.read(sums16, np.float32, (R,)).view(np.uint32), backend.read(s32, np.float32, (R,)).view(np.uint32))
    ref_w = backend.read(w32, np.float32, (R, L))
    if out_dtype == AGN_F16:
        assert np.array_equal(backend.read(w16, np.float16, (R, L)).view(np.uint16), ref_w.astype(np.float16).view(np.uint16))
    else:
        assert np.array_equal(backend.read(w16, np.uint16, (R, L)), to_bf16_bits(ref_w))


def test_softmax_16bit_output_argument_errors(backend):
    s = backend.upload(np.zeros((2, 8), np.float32))
    with pytest.raises(BackendError) as e:
        backend.launch_softmax_rows_scaled_out16(s, 2, 8, 1.0, AGN_Q8_0)
    assert e.value.status == 2
    with pytest.raises(BackendError) as e:
        backend.launch_softmax_rows_scaled_out16(s, 2, 8, 1.0, AGN_F16, out=s)
    assert e.value.status == 1


@pytest.mark.parametrize("out_dtype", [AGN_F16, AGN_BF16])
@pytest.mark.parametrize("n", [4096 * 18944 // 8, 4096 * 3 + 1, 7, 1])
def test_silu_mul_f32_to_16bit_output(backend, n, out_dtype):
    g, u = synth.activations(2, "gate", (n,)), synth.activations(2, "up", (n,))
    ref = orc.silu_mul(g, u, THREADS)
    dg, du = backend.upload(g), backend.upload(u)
    f32_gpu = backend.read(backend.launch_silu_mul(dg, du, n), np.float32, (n,))
    out = backend.launch_silu_mul_out16(dg, du, n, out_dtype)
    if out_dtype == AGN_F16:
        got = backend.read(out, np.float16, (n,))
        assert np.array_equal(got.view(np.uint16), f32_gpu.astype(np.float16).view(np.uint16))
        assert np.max(np.abs(got.astype(np.float32) - ref) / np.maximum(np.abs(ref), 1.0)) <= 2.0 ** -10
    else:
        got = backend.read(out, np.uint16, (n,))
        assert np.array_equal(got, to_bf16_bits(f32_gpu))
        assert np.max(np.abs(from_bf16_bits(got) - ref) / np.maximum(np.abs(ref), 1.0)) <= 2.0 ** -7


@pytest.mark.parametrize("R,L", [(6, 8), (5, 30), (7, 100), (4, 516), (6, 4100), (3, 9999), (3, 16388), (2, 152064)])
def test_softmax_leave_tail_untouched(backend, R, L):
    """agn_softmax_rows_valid_f32: the entries past a row's valid length keep what the buffer held (the
    reference never touches them, src/model/llama/cpu_path.rs:168-183); the valid entries are the same
    bits as the zero-filling entry points give.  Every kernel family, f32 and 16-bit rows, in place too."""
    s = synth.activations(1, "scores", (R, L), std=2.0)
    nv = np.array([L, 1, L // 2 + 1, L - 1, 0, 3, 2][:R], dtype=np.int32)
    ds, dnv = backend.upload(s), backend.upload(nv)
    zero_filled = backend.read(backend.launch_softmax_rows(ds, R, L, n_valid=dnv), np.float32, (R, L))
    sentinel = np.full((R, L), -7.25, np.float32)
    valid = np.arange(L)[None, :] < nv[:, None]
    out = backend.upload(sentinel)
    backend.launch_softmax_rows_valid(ds, R, L, out, n_valid=dnv)
    got = backend.read(out, np.float32, (R, L))
    o16 = backend.upload(np.full((R, L), 0x1234, np.uint16))
    backend.launch_softmax_rows_valid(ds, R, L, o16, out_dtype=AGN_F16, n_valid=dnv)
    got16 = backend.read(o16, np.uint16, (R, L))
    inplace = backend.upload(s)
    backend.launch_softmax_rows_valid(inplace, R, L, inplace, n_valid=dnv)
    got_ip = backend.read(inplace, np.float32, (R, L))
    # the zero-filling entry points still zero-fill after a call of the other form (no hidden state)
    again = backend.read(backend.launch_softmax_rows(ds, R, L, out=backend.upload(sentinel), n_valid=dnv), np.float32, (R, L))
    assert np.array_equal(again.view(np.uint32), zero_filled.view(np.uint32))
    assert np.array_equal(got[valid].view(np.uint32), zero_filled[valid].view(np.uint32)) and np.all(got[~valid] == -7.25)
    assert np.array_equal(got16[valid], zero_filled.astype(np.float16).view(np.uint16)[valid]) and np.all(got16[~valid] == 0x1234)
    assert np.array_equal(got_ip[valid].view(np.uint32), zero_filled[valid].view(np.uint32))
    assert np.array_equal(got_ip[~valid].view(np.uint32), s[~valid].view(np.uint32))  # the scores past the valid length survive


@pytest.mark.parametrize("heads,L", [(3, 2048), (2, 1028), (1, 4096), (2, 1100)])
def test_softmax_square_causal_row_pairs(backend, heads, L):
    """Square causal matrices of more than 1024 columns run rows i and L-1-i in one CTA: every form of the op
    (zero-filled, valid entries only, 16-bit rows, unnormalised + sums, scaled, in place) against the oracle."""
    s = synth.causal_scores(1, heads, L)
    nv = np.tile(np.arange(1, L + 1, dtype=np.int32), heads)
    ref = orc.softmax_rows(s, nv, max(1, orc.max_threads()))
    ds = backend.upload(s)
    got = backend.read(backend.launch_softmax_rows(ds, heads * L, L, causal_period=L), np.float32, s.shape)
    assert backend.last_kernel == "softmax_causal_pair"
    assert synth.max_rel_to_row_scale(got, ref) <= 1e-5
    upper = np.triu(np.ones((L, L), dtype=bool), k=1)
    assert not got[:, upper].any()
    # the CTA-per-row kernel gives the same values to within the tolerance (different reduction tree)
    backend.set_option("softmax_causal_pair", 0)
    try:
        per_row = backend.read(backend.launch_softmax_rows(ds, heads * L, L, causal_period=L), np.float32, s.shape)
        assert backend.last_kernel != "softmax_causal_pair"
    finally:
        backend.set_option("softmax_causal_pair", 1)
    assert synth.max_rel_to_row_scale(per_row, got) <= 2e-6
    # valid entries only: the tail keeps the sentinel, the valid part is bit-identical to the zero-filled form
    out = backend.upload(np.full(s.shape, -7.25, np.float32))
    backend.launch_softmax_rows_valid(ds, heads * L, L, out, causal_period=L)
    assert backend.last_kernel == "softmax_causal_pair"
    g2 = backend.read(out, np.float32, s.shape)
    assert np.array_equal(g2[:, ~upper].view(np.uint32), got[:, ~upper].view(np.uint32)) and np.all(g2[:, upper] == -7.25)
    # bf16 rows = the f32 result rounded to nearest even
    o16 = backend.launch_softmax_rows_scaled_out16(ds, heads * L, L, 1.0, AGN_BF16, causal_period=L)
    g16 = backend.read(o16, np.uint16, s.shape)
    assert np.array_equal(g16, to_bf16_bits(got).reshape(s.shape))
    # unnormalised weights and sums with a score scale (the reference kernel's form)
    sums = backend.empty(4 * heads * L)
    wts = backend.read(backend.launch_softmax_rows_scaled(ds, heads * L, L, 0.125, sums=sums, causal_period=L), np.float32, s.shape)
    sm = backend.read(sums, np.float32, (heads, L))
    ref_scaled = orc.softmax_rows(s * np.float32(0.125), nv, max(1, orc.max_threads()))
    assert synth.max_rel_to_row_scale(wts / sm[:, :, None], ref_scaled) <= 1e-5
    assert np.allclose(wts.sum(axis=2, dtype=np.float64), sm, rtol=1e-5)
    # in place
    inplace = backend.upload(s)
    backend.launch_softmax_rows(inplace, heads * L, L, out=inplace, causal_period=L)
    assert np.array_equal(backend.read(inplace, np.float32, s.shape).view(np.uint32), got.view(np.uint32))
