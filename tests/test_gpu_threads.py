"""Several host threads, one context each, on the same GPU at the same time: the library keeps no
state outside a context (`Backend: Send + Sync` in the reference, src/ops/mod.rs:93; here one
context per thread, calls on one context serialised by its owner), so concurrent use must give
the single-threaded results."""
import threading

import numpy as np
import pytest

from agention_infer_b200 import AGN_Q4_K, AGN_ROPE_NEOX, CudaBackend, synth
from oracle import oracle as orc

pytestmark = pytest.mark.gpu


def test_four_threads_four_contexts_one_device():
    T, H, I, nq, nkv, hd, vocab = 257, 1024, 2048, 8, 2, 128, 200
    x, w = synth.activations(2, "x", (T, H)), synth.norm_weight(2, "w", H)
    g, u = synth.activations(2, "gate", (T, I)), synth.activations(2, "up", (T, I))
    q, k = synth.activations(2, "q", (T, nq * hd)), synth.activations(2, "k", (T, nkv * hd))
    pos = synth.positions(3, T, True)
    table = synth.quant_table(AGN_Q4_K, vocab, H, cfg_index=2); ids = synth.token_ids(2, T, vocab)
    ref = {"rms": orc.rms_norm_rows(x, w, 1e-6), "silu": orc.silu_mul(g, u),
           "q": orc.rope_rows(q, nq, hd, hd, pos, 1e6, 1.0, orc.NEOX), "k": orc.rope_rows(k, nkv, hd, hd, pos, 1e6, 1.0, orc.NEOX),
           "rows": orc.get_rows(AGN_Q4_K, table, vocab, H, ids)[1]}
    errors = []

    def worker(n):
        try:
            be = CudaBackend(0)
            try:
                dx, dw, dg, du = be.upload(x), be.upload(w), be.upload(g), be.upload(u)
                dt, di, dp = be.upload(table), be.upload(ids), be.upload(pos)
                for it in range(20):
                    o1 = be.launch_rms_norm(dx, dw, T, H, 1e-6)
                    o2 = be.launch_silu_mul(dg, du, T * I)
                    dq, dk = be.upload(q), be.upload(k)
                    be.launch_rope_qk(dq, dk, T, nq, nkv, hd, hd, dp, 1e6, 1.0, AGN_ROPE_NEOX)
                    o3 = be.get_rows(AGN_Q4_K, dt, table.nbytes, vocab, H, di, T)
                    assert synth.max_rel_to_row_scale(be.read(o1, np.float32, (T, H)), ref["rms"]) <= 1e-5
                    assert synth.max_rel_to_row_scale(be.read(o2, np.float32, (T, I)), ref["silu"]) <= 1e-5
                    assert synth.max_rel_to_row_scale(be.read(dq, np.float32, (T, nq * hd)), ref["q"]) <= 1e-5
                    assert synth.max_rel_to_row_scale(be.read(dk, np.float32, (T, nkv * hd)), ref["k"]) <= 1e-5
                    assert np.array_equal(be.read(o3, np.float32, (T, H)).view(np.uint32), ref["rows"].view(np.uint32))
                    for b in (o1, o2, o3, dq, dk):
                        b.free()
            finally:
                be.close()
        except BaseException as e:  # noqa: BLE001 - reported to the main thread
            errors.append((n, repr(e)))

    threads = [threading.Thread(target=worker, args=(n,)) for n in range(4)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout=300)
    assert not any(t.is_alive() for t in threads)
    assert errors == []
