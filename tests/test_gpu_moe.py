"""GPU parity of the MoE routing ops (router softmax + top-2, gather of rows by expert)
against the CPU oracle.  Expert indices, offsets and the permutation are exact; the routing
weights are within 1e-5 of the row scale like the other float ops."""
import numpy as np
import pytest

from agention_infer_b200 import BackendError, synth
from oracle import oracle as orc

pytestmark = pytest.mark.gpu
TOL = 1e-5


@pytest.mark.parametrize("T,E", [(8192, 8), (1, 8), (1000, 4), (77, 64), (5, 2), (300, 16)])
def test_router_top2(backend, T, E):
    logits = synth.activations(5, "logits", (T, E))
    if E > 2:
        logits[0, :2] = logits[0, 2]  # a three-way tie: lower indices win
    ref_idx, ref_w = orc.router_top2(logits)
    idx, w = backend.router_top2(backend.upload(logits), T, E)
    assert np.array_equal(backend.read(idx, np.int32, (T, 2)), ref_idx)
    assert synth.max_rel_to_row_scale(backend.read(w, np.float32, (T, 2)), ref_w) <= TOL


@pytest.mark.parametrize("small_sort", [1, 0])
@pytest.mark.parametrize("T,H,E", [(8192, 4096, 8), (1, 64, 8), (1000, 130, 4), (513, 256, 64), (2048, 100, 3), (2049, 64, 8),
                                   (16385, 64, 8), (17, 32, 1), (40000, 32, 16), (2048, 64, 64), (33, 16, 5)])
def test_gather_rows_by_expert(backend, T, H, E, small_sort):
    """Both sorts: one CTA for up to 4096 pairs (T <= 2048), three kernels beyond or with the option off."""
    x = synth.activations(5, "x", (T, H))
    logits = synth.activations(5, "logits", (T, max(E, 2)))
    idx, _ = orc.router_top2(logits)
    idx = np.ascontiguousarray(idx % E)
    ref_out, ref_off, ref_tok, ref_slot = orc.gather_rows_by_expert(x, idx, E)
    backend.set_option("moe_small_sort", small_sort)
    try:
        out, off, tok, slot = backend.gather_rows_by_expert(backend.upload(x), backend.upload(idx), T, H, E)
    finally:
        backend.set_option("moe_small_sort", 1)
    assert np.array_equal(backend.read(off, np.int32, (E + 1,)), ref_off)
    assert np.array_equal(backend.read(tok, np.int32, (2 * T,)), ref_tok)
    assert np.array_equal(backend.read(slot, np.int32, (2 * T,)), ref_slot)
    got = backend.read(out, np.float32, (2 * T, H))
    assert np.array_equal(got.view(np.uint32), ref_out.view(np.uint32))


def test_gather_twice_reuses_the_workspace(backend):
    T, H, E = 3000, 64, 8
    x = synth.activations(5, "x", (T, H))
    dx = backend.upload(x)
    for salt in (0, 1):
        idx, _ = orc.router_top2(synth.activations(5, "logits", (T, E), salt=salt))
        ref = orc.gather_rows_by_expert(x, idx, E)
        got = backend.gather_rows_by_expert(dx, backend.upload(idx), T, H, E)
        assert np.array_equal(backend.read(got[0], np.float32, (2 * T, H)), ref[0])
        assert np.array_equal(backend.read(got[1], np.int32, (E + 1,)), ref[1])


def test_per_expert_silu_over_routed_rows(backend):
    # the expert-sorted gate/up rows form one contiguous [2T, I] array: one silu_mul launch
    T, I, E = 256, 1024, 8
    idx, _ = orc.router_top2(synth.activations(5, "logits", (T, E)))
    gate = synth.activations(5, "gate", (2 * T, I)); up = synth.activations(5, "up", (2 * T, I))
    out = backend.launch_silu_mul(backend.upload(gate), backend.upload(up), 2 * T * I)
    assert synth.max_rel_to_row_scale(backend.read(out, np.float32, (2 * T, I)), orc.silu_mul(gate, up)) <= TOL


@pytest.mark.parametrize("small_sort", [1, 0])
def test_gather_bad_expert_index_is_reported(backend, small_sort):
    T, H, E = 40, 32, 4
    x = synth.activations(5, "x", (T, H))
    idx = np.zeros((T, 2), np.int32); idx[:, 1] = 1; idx[7, 0] = 9; idx[20, 1] = -3
    backend.set_option("moe_small_sort", small_sort)
    try:
        out, off, tok, slot = backend.gather_rows_by_expert(backend.upload(x), backend.upload(idx), T, H, E)
    finally:
        backend.set_option("moe_small_sort", 1)
    with pytest.raises(BackendError) as e:
        backend.sync()
    assert e.value.status == 4
    backend.sync()
    # the two bad pairs are dropped: 78 rows placed, the last two slots marked empty, the rest in order
    tok_h = backend.read(tok, np.int32, (2 * T,))
    assert backend.read(off, np.int32, (E + 1,)).tolist() == [0, 39, 78, 78, 78]
    assert tok_h[78:].tolist() == [-1, -1]
    assert tok_h[:39].tolist() == [t for t in range(T) if t != 7] and tok_h[39:78].tolist() == [t for t in range(T) if t != 20]


def test_moe_argument_errors(backend):
    with pytest.raises(BackendError):
        backend.router_top2(backend.empty(64), 4, 1)
    with pytest.raises(BackendError):
        backend.gather_rows_by_expert(backend.empty(64), backend.empty(64), 4, 4, 65)
