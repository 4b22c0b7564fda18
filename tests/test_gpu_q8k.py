"""Q8_K activation rows (quantize_row_q8_k, src/quant/q8_k.rs:49-92) on the GPU.

The quantiser's outputs are integers and one f32 per block produced by two IEEE divisions, so the
bar is the oracle's bytes exactly: d as bit patterns, qs and bsums as integers, for ordinary rows,
ragged rows (zero-padded last block), unaligned rows, and the values where implementations differ
(ties between +a and -a, products that end in .5, NaN, infinities, a subnormal maximum).

SiLU·mul with the quantiser on the end computes its f32 value with the same function as the unfused
kernel, so it must equal `quantize(unfused f32 output)` byte for byte.  The fused norms hold a row
in another thread mapping than the f32 norm kernel (a warp owns whole blocks), so the sum of
squares is added in another order: against `quantize(GPU f32 norm)` and against the oracle's own
chain (whose f32 values differ from the GPU's by up to 1e-5 of the row scale) d agrees to 1e-5
relative, a q differs by at most one step in a small fraction of the positions, and bsums are
exactly the group sums of the qs that were written."""
import json
from pathlib import Path

import numpy as np
import pytest

from agention_infer_b200 import BackendError, synth
from oracle import oracle as orc
from tests.test_gpu_guard_bands import Guarded, guarded_like

pytestmark = pytest.mark.gpu
THREADS = max(1, orc.max_threads())
KA = json.loads((Path(__file__).parent / "golden" / "reference_known_answers.json").read_text())


def read_q8k(backend, bufs, T, n):
    nb = (n + 255) // 256
    d, qs, bs = bufs
    return (backend.read(d, np.float32, (T, nb)), backend.read(qs, np.int8, (T, nb * 256)),
            backend.read(bs, np.int16, (T, nb * 16)))


def assert_same(got, want, what=""):
    assert np.array_equal(got[0].view(np.uint32), want[0].view(np.uint32)), f"{what}: d differs"
    assert np.array_equal(got[1], want[1]), f"{what}: qs differs at {np.argwhere(got[1] != want[1])[:4].tolist()}"
    assert np.array_equal(got[2], want[2]), f"{what}: bsums differs"


def gpu_quantize(backend, x):
    x = np.ascontiguousarray(x, dtype=np.float32)
    T, n = x.shape
    return read_q8k(backend, backend.launch_quantize_rows_q8_k(backend.upload(x), T, n), T, n)


@pytest.mark.parametrize("T,n", [(512, 2048), (37, 3584), (4096, 256), (5, 100), (3, 257), (7, 1000), (4, 1023), (1, 1),
                                 (2, 18944), (3, 40000)])
def test_quantize_rows_bit_exact(backend, T, n):
    x = synth.activations(3, "x", (T, n)) * np.float32(3.0)
    assert_same(gpu_quantize(backend, x), orc.quantize_rows_q8_k(x, THREADS), f"T={T} n={n}")
    assert backend.last_kernel == "quantize_rows_q8_k"


def test_quantize_rows_unaligned_input(backend):
    """Rows that start 4 bytes off a 16-byte boundary, and a row length that is not a multiple of 4."""
    for T, n in ((6, 512), (5, 1001)):
        x = synth.activations(3, "x", (T, n))
        g = Guarded(backend, x.nbytes, skew=4).put(x)
        got = read_q8k(backend, backend.launch_quantize_rows_q8_k(g.ptr, T, n), T, n)
        assert_same(got, orc.quantize_rows_q8_k(x), f"skewed T={T} n={n}")


def test_reference_unit_test_inputs(backend):  # src/quant/q8_k.rs:97-139
    for name in ("q8_k_roundtrip_error", "q8_k_bsums", "q8_k_all_zero", "q8_k_partial_block"):
        x = np.array(KA[name]["x_bits"], dtype=np.uint32).view(np.float32)[None]
        got = gpu_quantize(backend, x)
        assert_same(got, orc.quantize_rows_q8_k(x), name)
    x = np.array(KA["q8_k_roundtrip_error"]["x_bits"], dtype=np.uint32).view(np.float32)
    d, qs, _ = gpu_quantize(backend, x[None])
    assert np.abs(d[0, 0] * qs[0].astype(np.float32) - x).max() < KA["q8_k_roundtrip_error"]["dequant_abs_err_below"]


def tie_and_rounding_rows():
    rows = []
    def row():
        r = np.zeros(512, np.float32); rows.append(r); return r
    r = row(); r[2], r[9] = -4.0, 4.0; r[0] = 1.0                     # -a before +a, two lanes of one half
    r = row(); r[2], r[9] = 4.0, -4.0; r[0] = 1.0                     # +a before -a
    r = row(); r[4], r[5] = 3.0, -3.0                                 # inside one lane's float4
    r = row(); r[5], r[4] = 3.0, -3.0
    r = row(); r[130], r[7] = 5.0, -5.0; r[256 + 200], r[256 + 3] = -2.0, 2.0   # across the two halves of a block
    r = row(); r[7], r[130] = 5.0, -5.0; r[256 + 3], r[256 + 200] = -2.0, 2.0
    r = row(); r[255], r[0] = -1.0, 1.0; r[256:] = 0.25                # first and last element
    r = row(); r[0] = -127.0; r[1:9] = [0.5, 1.5, -0.5, -2.5, 126.5, -126.5, 0.49999997, -0.49999997]  # iscale = 1
    r = row(); r[0] = 127.0; r[1:7] = [0.5, 1.5, -0.5, 2.5, -126.5, 126.49999]  # iscale = -1
    r = row(); r[:] = 0.0                                              # nothing above 0
    r = row(); r[3] = np.nan; r[10] = 2.0; r[300] = np.nan             # NaN never wins the scan; quantises to 0
    r = row(); r[:256] = np.nan                                        # a block of NaN only
    r = row(); r[5] = np.inf; r[6] = 1.0; r[256 + 9] = -np.inf; r[256 + 1] = np.inf
    r = row(); r[7] = 1e-41; r[9] = -1e-42                             # subnormal maximum: iscale overflows
    r = row(); r[1] = -0.0; r[2] = 0.0
    r = row(); r[:] = 3.4e38; r[17] = -3.4e38
    return np.stack(rows)


def test_ties_rounding_and_special_values_bit_exact(backend):
    x = tie_and_rounding_rows()
    with np.errstate(all="ignore"):
        want = orc.quantize_rows_q8_k(x)
    assert_same(gpu_quantize(backend, x), want, "special rows")
    # the same rows through the element-wise kernel (row length not a multiple of 4)
    y = np.ascontiguousarray(x[:, :511])
    assert_same(gpu_quantize(backend, y), orc.quantize_rows_q8_k(y), "special rows, scalar loads")


def test_every_half_integer_product_rounds_away_from_zero(backend):
    """iscale = 1 (max = -127): every k + 0.5 and its two f32 neighbours, |k| <= 126."""
    k = np.arange(-126, 127, dtype=np.float32)
    vals = np.concatenate([k + np.float32(0.5), np.nextafter(k + np.float32(0.5), np.float32(np.inf)),
                           np.nextafter(k + np.float32(0.5), np.float32(-np.inf))])
    vals = vals[np.abs(vals) < 127.0]
    n_rows = -(-vals.size // 255)
    padded = np.zeros(n_rows * 255, np.float32)
    padded[: vals.size] = vals
    x = np.empty((n_rows, 256), np.float32)
    x[:, 0] = -127.0
    x[:, 1:] = padded.reshape(n_rows, 255)
    assert_same(gpu_quantize(backend, x), orc.quantize_rows_q8_k(x), "half-integer products")


def q8k_close_to_chain(got, want, what):
    """GPU fused output against the oracle's norm -> quantise chain."""
    d, qs, bs = got
    wd, wq, wb = want
    assert np.all(np.abs(d - wd) <= 1e-5 * np.abs(wd) + 1e-30), what
    diff = np.abs(qs.astype(np.int32) - wq.astype(np.int32))
    assert diff.max() <= 1, what
    assert (diff != 0).mean() < 2e-3, f"{what}: {(diff != 0).mean():.2e} of the positions differ"
    assert np.array_equal(bs, qs.reshape(qs.shape[0], -1, 16).astype(np.int16).sum(axis=2)), what


@pytest.mark.parametrize("bpw", [0, 1, 4])
@pytest.mark.parametrize("T,H", [(512, 2048), (300, 3584), (64, 4096), (9, 256), (5, 8192), (3, 12288), (2, 32768), (1, 3584)])
def test_rms_norm_q8_k(backend, T, H, bpw):
    x, w = synth.activations(2, "x", (T, H)), synth.norm_weight(2, "w", H)
    dx, dw = backend.upload(x), backend.upload(w)
    normed = backend.launch_rms_norm(dx, dw, T, H, 1e-6)
    two = read_q8k(backend, backend.launch_quantize_rows_q8_k(normed, T, H), T, H)
    backend.set_option("rms_q8k_bpw", bpw)  # blocks per warp: by row length (0), or forced
    try:
        fused = read_q8k(backend, backend.launch_rms_norm_q8_k(dx, dw, T, H, 1e-6), T, H)
    finally:
        backend.set_option("rms_q8k_bpw", 0)
    assert backend.last_kernel == "rms_norm_q8_k"
    q8k_close_to_chain(fused, two, f"rms_norm_q8_k T={T} H={H} vs the two launches")
    q8k_close_to_chain(fused, orc.quantize_rows_q8_k(orc.rms_norm_rows(x, w, 1e-6, THREADS), THREADS), "vs oracle chain")


@pytest.mark.parametrize("T,H", [(512, 2048), (300, 3584), (7, 4096), (3, 16384)])
def test_add_residual_rms_norm_q8_k(backend, T, H):
    x, dl, w = synth.activations(2, "x", (T, H)), synth.activations(2, "delta", (T, H)), synth.norm_weight(2, "w", H)
    dx, dd, dw = backend.upload(x), backend.upload(dl), backend.upload(w)
    new_x, normed = backend.launch_add_residual_rms_norm(dx, dd, dw, T, H, 1e-5)
    two = read_q8k(backend, backend.launch_quantize_rows_q8_k(normed, T, H), T, H)
    new_x2, bufs = backend.launch_add_residual_rms_norm_q8_k(dx, dd, dw, T, H, 1e-5)
    q8k_close_to_chain(read_q8k(backend, bufs, T, H), two, f"add_residual_rms_norm_q8_k T={T} H={H} vs the two launches")
    a, b = backend.read(new_x, np.float32, (T, H)), backend.read(new_x2, np.float32, (T, H))
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
    assert np.array_equal(a.view(np.uint32), (x + dl).view(np.uint32))  # one f32 addition: exact against numpy
    nx, nm = orc.add_residual_rms_norm_rows(x, dl, w, 1e-5, THREADS)
    q8k_close_to_chain(read_q8k(backend, bufs, T, H), orc.quantize_rows_q8_k(nm, THREADS), "vs oracle chain")


@pytest.mark.parametrize("T,I", [(64, 8192), (33, 18944), (1, 256), (3, 14336)])
def test_silu_mul_q8_k_equals_the_two_launches(backend, T, I):
    g, u = synth.activations(2, "gate", (T, I)), synth.activations(2, "up", (T, I))
    dg, du = backend.upload(g), backend.upload(u)
    prod = backend.launch_silu_mul(dg, du, T * I)
    two = read_q8k(backend, backend.launch_quantize_rows_q8_k(prod, T, I), T, I)
    fused = read_q8k(backend, backend.launch_silu_mul_q8_k(dg, du, T, I), T, I)
    assert backend.last_kernel == "silu_mul_q8_k"
    assert_same(fused, two, f"silu_mul_q8_k T={T} I={I}")
    q8k_close_to_chain(fused, orc.quantize_rows_q8_k(orc.silu_mul(g, u, THREADS), THREADS), "vs oracle chain")


def test_fused_forms_with_special_values(backend):
    """NaN / inf / zero rows through the fused kernels: still the two launches' bytes."""
    T, H = 6, 512
    x = synth.activations(2, "x", (T, H))
    x[1] = 0.0; x[2, 5] = np.nan; x[3, 7] = np.inf; x[4, :256] = 0.0; x[5, 3], x[5, 300] = 9.0, -9.0
    w = synth.norm_weight(2, "w", H)
    dx, dw = backend.upload(x), backend.upload(w)
    two = read_q8k(backend, backend.launch_quantize_rows_q8_k(backend.launch_rms_norm(dx, dw, T, H, 1e-6), T, H), T, H)
    fused = read_q8k(backend, backend.launch_rms_norm_q8_k(dx, dw, T, H, 1e-6), T, H)
    finite = [0, 1, 4, 5]  # rows 2 (a NaN) and 3 (an infinity) have a NaN or zero scale factor: every value NaN or 0
    q8k_close_to_chain(tuple(a[finite] for a in fused), tuple(a[finite] for a in two), "rms_norm_q8_k special")
    assert_same(tuple(a[[2, 3]] for a in fused), tuple(a[[2, 3]] for a in two), "rms_norm_q8_k NaN / inf rows")
    two = read_q8k(backend, backend.launch_quantize_rows_q8_k(backend.launch_silu_mul(dx, dx, T * H), T, H), T, H)
    assert_same(read_q8k(backend, backend.launch_silu_mul_q8_k(dx, dx, T, H), T, H), two, "silu_mul_q8_k special")


def test_q8_k_writes_stay_inside(backend):
    for T, n in ((5, 3584), (3, 100), (2, 1001)):
        nb = (n + 255) // 256
        x = synth.activations(2, "x", (T, n))
        gx = guarded_like(backend, x)
        d, qs, bs = Guarded(backend, 4 * T * nb), Guarded(backend, 256 * T * nb), Guarded(backend, 32 * T * nb)
        backend.launch_quantize_rows_q8_k(gx.ptr, T, n, out=(d.ptr, qs.ptr, bs.ptr))
        if n % 256 == 0:
            w = guarded_like(backend, synth.norm_weight(2, "w", n))
            nx = Guarded(backend, x.nbytes)
            backend.launch_rms_norm_q8_k(gx.ptr, w.ptr, T, n, 1e-6, out=(d.ptr, qs.ptr, bs.ptr))
            backend.launch_add_residual_rms_norm_q8_k(gx.ptr, gx.ptr, w.ptr, T, n, 1e-6, new_x=nx.ptr, out=(d.ptr, qs.ptr, bs.ptr))
            backend.launch_silu_mul_q8_k(gx.ptr, gx.ptr, T, n, out=(d.ptr, qs.ptr, bs.ptr))
            nx.check("new_x"); w.check("w")
        for g, name in ((d, "d"), (qs, "qs"), (bs, "bsums"), (gx, "x")):
            g.check(f"{name} T={T} n={n}")


def test_q8_k_argument_errors(backend):
    x = backend.upload(synth.activations(2, "x", (2, 512)))
    w = backend.upload(synth.norm_weight(2, "w", 512))
    out = (backend.empty(64), backend.empty(2048), backend.empty(256))
    with pytest.raises(BackendError, match="multiple of 256"):
        backend.launch_rms_norm_q8_k(x, w, 2, 500, 1e-6, out=out)
    with pytest.raises(BackendError, match="multiple of 256"):
        backend.launch_silu_mul_q8_k(x, x, 2, 384, out=out)
    with pytest.raises(BackendError, match="aligned"):
        backend.launch_quantize_rows_q8_k(x, 2, 512, out=(out[0], out[1].data_ptr() + 2, out[2]))
    with pytest.raises(BackendError, match="aligned"):
        backend.launch_rms_norm_q8_k(x.data_ptr() + 4, w, 1, 256, 1e-6, out=out)
    with pytest.raises(BackendError):
        backend.launch_quantize_rows_q8_k(x, 2, 0, out=out)
    backend.launch_quantize_rows_q8_k(x, 0, 512, out=out)  # T = 0: nothing to do
    backend.sync()


def test_fuzz_quantize_rows(backend):
    """Seeded random shapes: ragged lengths, rows off a 16-byte boundary, magnitudes over twelve decades, and a
    sprinkling of exact zeros, ties and non-finite values."""
    r = np.random.default_rng(815)
    for it in range(60):
        T = int(r.integers(1, 9))
        n = int(r.choice([1, 3, 4, 15, 16, 17, 100, 255, 256, 257, 511, 512, 640, 1000, 1024, 1028, 3584, 4100]))
        x = (r.standard_normal((T, n)) * 10.0 ** r.integers(-6, 6, size=(T, 1))).astype(np.float32)
        x[r.random((T, n)) < 0.05] = 0.0
        if n > 8:
            j = r.integers(0, n, size=4)
            x[0, j[0]], x[0, j[1]] = np.abs(x[0]).max() + 1, -(np.abs(x[0]).max() + 1)  # a +a / -a tie for the block maximum
            if it % 5 == 0:
                x[T - 1, j[2]] = np.nan
            if it % 7 == 0:
                x[T - 1, j[3]] = np.inf
        off = int(r.integers(0, 4))
        g = Guarded(backend, x.nbytes, skew=4 * off).put(x)
        with np.errstate(all="ignore"):
            want = orc.quantize_rows_q8_k(x)
        got = read_q8k(backend, backend.launch_quantize_rows_q8_k(g.ptr, T, n), T, n)
        assert_same(got, want, f"fuzz it={it} T={T} n={n} off={off}")


def test_q8_k_ops_in_a_recorded_graph(backend):
    """The fused producers recorded once and replayed on new inputs: the replay's bytes are the eager call's."""
    be = backend
    T, H, I = 8, 3584, 18944
    w = synth.norm_weight(3, "w", H)
    dx, dd, dnx, dg, du, dw = be.empty(4 * T * H), be.empty(4 * T * H), be.empty(4 * T * H), be.empty(4 * T * I), be.empty(4 * T * I), be.upload(w)
    qa = (be.empty(4 * T * H // 256), be.empty(T * H), be.empty(2 * T * H // 16))
    qb = (be.empty(4 * T * I // 256), be.empty(T * I), be.empty(2 * T * I // 16))

    def chain():
        be.launch_add_residual_rms_norm_q8_k(dx, dd, dw, T, H, 1e-6, new_x=dnx, out=qa)
        be.launch_silu_mul_q8_k(dg, du, T, I, out=qb)

    def load(salt):
        a = {n: synth.activations(3, n, s, salt=salt) for n, s in (("x", (T, H)), ("delta", (T, H)), ("gate", (T, I)), ("up", (T, I)))}
        for buf, n in ((dx, "x"), (dd, "delta"), (dg, "gate"), (du, "up")):
            be.copy_h2d(buf, a[n])
        be.sync()
        return a

    load(0)
    be.graph_begin()
    chain()
    g = be.graph_end()
    try:
        for salt in (1, 2):
            a = load(salt)
            be.graph_launch(g)
            rep_a, rep_b = read_q8k(be, qa, T, H), read_q8k(be, qb, T, I)
            nx = be.read(dnx, np.float32, (T, H))
            chain()
            assert_same(read_q8k(be, qa, T, H), rep_a, "replayed add_residual_rms_norm_q8_k")
            assert_same(read_q8k(be, qb, T, I), rep_b, "replayed silu_mul_q8_k")
            assert np.array_equal(nx.view(np.uint32), (a["x"] + a["delta"]).view(np.uint32))
            q8k_close_to_chain(rep_b, orc.quantize_rows_q8_k(orc.silu_mul(a["gate"], a["up"], THREADS), THREADS), "replay vs oracle chain")
    finally:
        be.graph_destroy(g)


def test_quantize_random_blocks_over_the_whole_exponent_range_bit_exact(backend):
    """131,072 blocks with magnitudes from 1e-44 to 3e38 (subnormal maxima, whose iscale overflows, up to maxima whose
    iscale is almost subnormal); half of them hold multiples of max / 254, so that iscale * v lands on or next to k and
    k + 0.5."""
    r = np.random.default_rng(2612)
    T, nb = 2048, 64
    mag = (10.0 ** r.uniform(-44, 38.5, size=(T, nb, 1))).astype(np.float32)
    base = r.standard_normal((T, nb, 256)).astype(np.float32)
    half_steps = r.integers(-254, 255, size=(T, nb, 256)).astype(np.float32) * np.float32(0.5)
    pick = r.random((T, nb, 1)) < 0.5
    sign = np.where(r.random((T, nb)) < 0.5, np.float32(-1.0), np.float32(1.0))
    with np.errstate(all="ignore"):
        vals = np.where(pick, half_steps / np.float32(127.0), base / np.float32(5.0))
        vals[..., 0] = np.where(pick[..., 0], sign, vals[..., 0])  # the block maximum of the structured blocks, either sign
        x = (vals * mag).astype(np.float32).reshape(T, nb * 256)
    x[~np.isfinite(x)] = 0.0
    with np.errstate(all="ignore"):
        want = orc.quantize_rows_q8_k(x, THREADS)
    assert_same(gpu_quantize(backend, x), want, "random blocks, whole exponent range")
