"""The one kind of device-side wait the kernels have — a poll of a shared-memory barrier that a
bulk copy completes — gives up after a bounded number of polls, raises a device flag, and the
host reads AGN_ETIMEOUT at the next agn_sync.  Nothing faults or hangs: the test makes the wait
run out on a barrier that nothing ever signals (the context option "test_idle_barrier_wait"),
after the row's own copy has landed, with the poll limit lowered to a few thousand."""
import numpy as np
import pytest

from agention_infer_b200 import AGN_Q4_K, BackendError, _abi, synth
from oracle import oracle as orc

pytestmark = pytest.mark.gpu


def test_a_wait_that_runs_out_is_reported_once_and_the_context_stays_usable(backend):
    vocab, H, T = 8, 256, 1
    table = synth.quant_table(AGN_Q4_K, vocab, H)
    ids = np.array([5], dtype=np.uint32)
    _, ref = orc.get_rows(AGN_Q4_K, table, vocab, H, ids)
    dtab, dids = backend.upload(table), backend.upload(ids)
    sentinel = np.full((T, H), -7.25, np.float32)
    out = backend.upload(sentinel)
    backend.set_option("mbar_spin_limit", 4000)
    backend.set_option("test_idle_barrier_wait", 1)
    try:
        backend.get_rows(AGN_Q4_K, dtab, table.nbytes, vocab, H, dids, T, out=out)
        assert backend.last_kernel == "get_rows"
        with pytest.raises(BackendError) as e:
            backend.sync()
        assert e.value.status == _abi.AGN_ETIMEOUT and "wait" in str(e.value)
    finally:
        backend.set_option("test_idle_barrier_wait", 0)
        backend.set_option("mbar_spin_limit", 1 << 22)
    backend.sync()  # reported once
    # the launch that gave up wrote nothing: its output is invalid, as the message says
    assert np.array_equal(backend.read(out, np.float32, (T, H)), sentinel)
    # and the same context runs the same op correctly afterwards
    backend.get_rows(AGN_Q4_K, dtab, table.nbytes, vocab, H, dids, T, out=out)
    assert np.array_equal(backend.read(out, np.float32, (T, H)).view(np.uint32), ref.view(np.uint32))


def test_option_ranges(backend):
    with pytest.raises(BackendError):
        backend.set_option("mbar_spin_limit", 0)
    with pytest.raises(BackendError):
        backend.set_option("rms_ring", 99)
    with pytest.raises(BackendError):
        backend.set_option("softmax_leave_tail", 1)  # no context-wide switch: agn_softmax_rows_valid_f32 is the entry point
