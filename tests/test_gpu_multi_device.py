"""Two contexts on two GPUs in one process: independent streams and memory, same results.
Needs at least two visible devices (skipped on a one-GPU box)."""
import numpy as np
import pytest

from agention_infer_b200 import AGN_Q4_K, BackendError, CudaBackend, synth
from oracle import oracle as orc

pytestmark = pytest.mark.gpu


def _second_backend():
    try:
        return CudaBackend(1)
    except BackendError:
        pytest.skip("only one GPU is visible")


def test_two_contexts_two_devices_interleaved(backend):
    be1 = _second_backend()
    try:
        T, H, I = 700, 2048, 4096
        x = synth.activations(1, "x", (T, H)); w = synth.norm_weight(1, "w", H)
        g = synth.activations(1, "gate", (T, I)); u = synth.activations(1, "up", (T, I))
        table = synth.quant_table(AGN_Q4_K, 300, H, cfg_index=1); ids = synth.token_ids(1, T, 300)
        bufs = []
        for be in (backend, be1):  # enqueue everything on both devices before reading anything back
            dx, dw = be.upload(x), be.upload(w)
            o1 = be.launch_rms_norm(dx, dw, T, H, 1e-5)
            o2 = be.launch_silu_mul(be.upload(g), be.upload(u), T * I)
            o3 = be.get_rows(AGN_Q4_K, be.upload(table), table.nbytes, 300, H, be.upload(ids), T)
            bufs.append((be, o1, o2, o3))
        st, rows = orc.get_rows(AGN_Q4_K, table, 300, H, ids)
        for be, o1, o2, o3 in bufs:
            assert synth.max_rel_to_row_scale(be.read(o1, np.float32, (T, H)), orc.rms_norm_rows(x, w, 1e-5)) <= 1e-5
            assert synth.max_rel_to_row_scale(be.read(o2, np.float32, (T, I)), orc.silu_mul(g, u)) <= 1e-5
            assert np.array_equal(be.read(o3, np.float32, (T, H)).view(np.uint32), rows.view(np.uint32))
        a = backend.read(bufs[0][1], np.float32, (T, H)); b = be1.read(bufs[1][1], np.float32, (T, H))
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32))  # both GPUs agree bit for bit
    finally:
        be1.close()


def test_events_and_copies_follow_their_own_context(backend):
    """Events, copies and syncs of a context act on that context's device whatever the last op left current: time
    a kernel on device 1 right after work on device 0, and the other way round."""
    be1 = _second_backend()
    try:
        T, H = 512, 2048
        x = synth.activations(1, "x", (T, H)); w = synth.norm_weight(1, "w", H)
        ref = orc.rms_norm_rows(x, w, 1e-5)
        for first, second in ((backend, be1), (be1, backend)):
            d0x, d0w = first.upload(x), first.upload(w)
            first.launch_rms_norm(d0x, d0w, T, H, 1e-5)  # leaves `first`'s device current
            dx, dw = second.upload(x), second.upload(w)
            first.launch_rms_norm(d0x, d0w, T, H, 1e-5)  # ... again, right before the events of `second`
            e0, e1 = second.event(), second.event()
            second.record(e0)
            out = second.launch_rms_norm(dx, dw, T, H, 1e-5)
            second.record(e1)
            second.sync()
            assert 0.0 < second.elapsed_ms(e0, e1) < 1000.0
            assert synth.max_rel_to_row_scale(second.read(out, np.float32, (T, H)), ref) <= 1e-5
            second.destroy_event(e0); second.destroy_event(e1)
            first.sync()
    finally:
        be1.close()
