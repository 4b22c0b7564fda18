"""The allocation-free gather-by-expert entry point, for hosts that cannot call cudaMalloc
(the GPU's memory already belongs to their own arena, or an allocation in the serving loop
would stall every stream).  It is called through the C ABI twice in a row, with different
sizes and routing, and every output must equal the regular entry point's bit for bit: the
second call sees the scratch array as the first one left it.

The file name sorts after every other test file on purpose: pytest collects it last, so a run
that stops at the first failure has already run all the other tests before this one."""
import ctypes as C

import numpy as np
import pytest

from agention_infer_b200 import _abi, synth
from oracle import oracle as orc

pytestmark = pytest.mark.gpu


def _noalloc(lib, be, dx, didx, T, H, E):
    out = be.empty(8 * T * H); off = be.empty(4 * (E + 1)); tok = be.empty(8 * T); slot = be.empty(8 * T)
    err = C.create_string_buffer(256)
    st = lib.agn_gather_rows_by_expert_noalloc_f32(be.stream(), dx.ptr, didx.ptr, T, H, E, out.ptr, off.ptr, tok.ptr,
                                                   slot.ptr, err, len(err))
    assert st == _abi.AGN_OK, err.value.decode()
    return out, off, tok, slot


def test_noalloc_matches_regular_entry_point_twice_in_a_row(backend):
    lib = _abi.load()
    H, E = 256, 8
    for call, T in enumerate((3000, 1111)):  # the second, smaller call runs over stale scratch contents
        x = synth.activations(5, "x", (T, H), salt=call)
        idx, _ = orc.router_top2(synth.activations(5, "logits", (T, E), salt=call))
        dx, didx = backend.upload(x), backend.upload(idx)
        want = backend.gather_rows_by_expert(dx, didx, T, H, E)
        got = _noalloc(lib, backend, dx, didx, T, H, E)
        shapes = [((2 * T, H), np.float32), ((E + 1,), np.int32), ((2 * T,), np.int32), ((2 * T,), np.int32)]
        for g, w, (shape, dt) in zip(got, want, shapes):
            a, b = backend.read(g, dt, shape), backend.read(w, dt, shape)
            assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
        # and against the oracle, so that both entry points cannot be wrong together
        ref = orc.gather_rows_by_expert(x, idx, E)
        assert np.array_equal(backend.read(got[0], np.float32, (2 * T, H)), ref[0])
        assert np.array_equal(backend.read(got[1], np.int32, (E + 1,)), ref[1])


def test_noalloc_rejects_sizes_beyond_the_built_in_scratch(backend):
    lib = _abi.load()
    err = C.create_string_buffer(256)
    T, E = 5_000_000, 8  # needs 256 + 9766*8*4 bytes > 256 KiB
    st = lib.agn_gather_rows_by_expert_noalloc_f32(backend.stream(), 1, 1, T, 64, E, 1, 1, 1, 1, err, len(err))
    assert st == _abi.AGN_EINVAL
    assert b"scratch" in err.value and b"limit" in err.value
    st = lib.agn_gather_rows_by_expert_noalloc_f32(backend.stream(), 1, 1, 16, 64, 65, 1, 1, 1, 1, err, len(err))
    assert st == _abi.AGN_EINVAL


def test_noalloc_out_of_range_expert_drops_the_pair(backend):
    """An expert index outside [0, n_experts) drops that (token, slot) pair: offsets[E] = 2T - dropped,
    the unused tail of src_token is -1, the status stays AGN_OK; everything else as the oracle."""
    lib = _abi.load()
    T, H, E = 700, 128, 8
    x = synth.activations(5, "x", (T, H))
    idx, _ = orc.router_top2(synth.activations(5, "logits", (T, E)))
    idx = idx.copy()
    bad = [(3, 0), (3, 1), (250, 1), (699, 0)]
    for t, s_ in bad:
        idx[t, s_] = E if s_ else -1
    dx, didx = backend.upload(x), backend.upload(idx)
    out, off, tok, slot = _noalloc(lib, backend, dx, didx, T, H, E)
    backend.sync()  # nothing is reported through a context either
    n_ok = 2 * T - len(bad)
    offsets = backend.read(off, np.int32, (E + 1,))
    src_token = backend.read(tok, np.int32, (2 * T,))
    src_slot = backend.read(slot, np.int32, (2 * T,))
    rows = backend.read(out, np.float32, (2 * T, H))
    assert offsets[0] == 0 and offsets[E] == n_ok and np.all(np.diff(offsets) >= 0)
    assert np.all(src_token[n_ok:] == -1)
    # the kept pairs in stable (expert, token, slot) order
    keep = [(int(idx[t, s_]), t, s_) for t in range(T) for s_ in range(2) if 0 <= idx[t, s_] < E]
    keep.sort()
    assert np.array_equal(src_token[:n_ok], np.array([k[1] for k in keep], np.int32))
    assert np.array_equal(src_slot[:n_ok], np.array([k[2] for k in keep], np.int32))
    assert np.array_equal(rows[:n_ok].view(np.uint32), x[src_token[:n_ok]].view(np.uint32))
    counts = np.bincount([k[0] for k in keep], minlength=E)
    assert np.array_equal(np.diff(offsets), counts)


def test_noalloc_zero_tokens_is_the_warm_up_call(backend):
    """T = 0 resolves the scratch address (the start-up call the header asks for) and zeroes offsets."""
    lib = _abi.load()
    E = 8
    off = backend.upload(np.full(E + 1, 77, np.int32))
    err = C.create_string_buffer(256)
    st = lib.agn_gather_rows_by_expert_noalloc_f32(backend.stream(), None, None, 0, 64, E, None, off.ptr, None, None, err, len(err))
    assert st == _abi.AGN_OK, err.value.decode()
    assert not backend.read(off, np.int32, (E + 1,)).any()
