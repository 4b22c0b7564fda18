"""The allocation-free gather-by-expert entry point, for hosts that cannot call cudaMalloc
(the GPU's memory already belongs to their own arena, or an allocation in the serving loop
would stall every stream).  It is called through the C ABI twice in a row, with different
sizes and routing, and every output must equal the regular entry point's bit for bit: the
second call sees the scratch array as the first one left it."""
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
