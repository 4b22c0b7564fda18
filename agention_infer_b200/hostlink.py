"""Host-link probe: what pinned host <-> device copies reach on this machine, per GPU, with 1, 2, 4
... GPUs copying at the same time.

The host-slice entry points (`agn_host_*`) are bound by this link, not by HBM, and on a
multi-GPU box by whatever the GPUs share on the host side (memory controllers, root complexes).
The probe moves plain pinned buffers through the library's own copy entry points
(`agn_host_alloc`, `agn_memcpy_h2d`, `agn_memcpy_d2h`: one `cudaMemcpyAsync` each) with no kernel
in between, so its figures are the ceiling for any staging scheme:

    python -m agention_infer_b200.hostlink --gpus 8 [--mb 256] [--reps 8]

One process per GPU; for every number of active GPUs n in {1, 2, 4, ...} the first n processes
copy at the same time (host-to-device alone, device-to-host alone, both directions on two
streams) while the others idle.  Prints one JSON object: per n, the mean and the slowest
per-GPU GB/s of each of the three cases.
"""
from __future__ import annotations

import argparse
import json
import multiprocessing as mp
import time


def _worker(rank: int, world: int, mb: int, reps: int, barrier, out_q) -> None:
    import numpy as np

    from .backend import CudaBackend
    up, down = CudaBackend(rank), CudaBackend(rank)  # one context (one stream) per direction
    n = mb << 20
    h_in, h_out = up.pinned((n,), np.uint8), down.pinned((n,), np.uint8)
    h_in[:] = 1
    d_in, d_out = up.empty(n), down.empty(n)

    def run(h2d: bool, d2h: bool) -> float:
        up.sync(); down.sync()
        t0 = time.perf_counter()
        for _ in range(reps):
            if h2d:
                up.copy_h2d(d_in, h_in)
            if d2h:
                down.copy_d2h(h_out, d_out)
        up.sync(); down.sync()
        return reps * n / (time.perf_counter() - t0) / 1e9  # GB/s per direction

    run(True, True)  # warm-up
    res = {}
    active = 1
    while active <= world:
        for case, (a, b) in (("h2d", (True, False)), ("d2h", (False, True)), ("both_per_direction", (True, True))):
            barrier.wait()
            if rank < active:
                res[f"{active}:{case}"] = run(a, b)
            barrier.wait()
        active *= 2
    out_q.put((rank, res))
    up.free_pinned(h_in); down.free_pinned(h_out)
    up.close(); down.close()


def probe(gpus: int, mb: int = 256, reps: int = 8) -> dict:
    ctx = mp.get_context("spawn")
    barrier, q = ctx.Barrier(gpus, timeout=300), ctx.Queue()  # a worker that dies breaks the barrier instead of hanging the rest
    procs = [ctx.Process(target=_worker, args=(r, gpus, mb, reps, barrier, q)) for r in range(gpus)]
    for p in procs:
        p.start()
    got = dict(q.get(timeout=600) for _ in procs)
    for p in procs:
        p.join(timeout=60)
    table = {}
    active = 1
    while active <= gpus:
        row = {}
        for case in ("h2d", "d2h", "both_per_direction"):
            vals = [got[r][f"{active}:{case}"] for r in range(active)]
            row[case] = {"mean_gbs_per_gpu": round(sum(vals) / len(vals), 2), "min_gbs_per_gpu": round(min(vals), 2),
                         "sum_gbs": round(sum(vals), 1)}
        table[str(active)] = row
        active *= 2
    return {"probe": "pinned cudaMemcpyAsync through agn_memcpy_h2d / agn_memcpy_d2h, no kernel", "buffer_mb": mb,
            "reps": reps, "gpus": gpus, "active_gpus": table}


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--mb", type=int, default=256, help="bytes per copy, MiB")
    ap.add_argument("--reps", type=int, default=8)
    a = ap.parse_args()
    print(json.dumps(probe(a.gpus, a.mb, a.reps)))


if __name__ == "__main__":
    main()
