"""Row sharding and the measurement collectives, on CPU with the gloo backend, world size 2:
each rank runs the oracle on its shard; the concatenation must equal the unsharded result,
the max-over-ranks reduction must return the slowest rank's time on every rank."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent

from agention_infer_b200 import sharding, synth  # noqa: E402


@pytest.mark.parametrize("T,world", [(0, 4), (1, 2), (7, 8), (4096, 8), (65536, 3), (5, 5)])
def test_shards_partition_the_rows(T, world):
    parts = sharding.all_shards(T, world)
    assert parts[0][0] == 0 and parts[-1][1] == T
    assert all(a[1] == b[0] for a, b in zip(parts, parts[1:]))
    sizes = [b - a for a, b in parts]
    assert max(sizes) - min(sizes) <= 1


def test_checksums_combine_over_shards():
    a = synth.activations(1, "x", (37, 20))
    whole = sharding.checksum(a)
    parts = [sharding.checksum(a[s:e]) for s, e in sharding.all_shards(37, 3)]
    assert sharding.combine_checksums(parts) == whole
    b = a.copy(); b[5, 5] += 1
    assert sharding.checksum(b) != whole


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, T, H, q):
    sys.path.insert(0, str(ROOT))
    import torch.distributed as dist
    from oracle import oracle as orc
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        x = synth.activations(2, "x", (T, H)); w = synth.norm_weight(2, "w", H)
        s, e = sharding.shard_rows(T, rank, world)
        mine = orc.rms_norm_rows(x[s:e], w, 1e-6)
        slowest = sharding.max_over_ranks(10.0 + rank)
        sums = sharding.gather_objects(sharding.checksum(mine))
        dist.barrier()
        q.put((rank, slowest, sums, sharding.checksum(orc.rms_norm_rows(x, w, 1e-6))))
    finally:
        dist.destroy_process_group()


def test_two_ranks_sharded_equals_unsharded():
    world, T, H = 2, 33, 256
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, T, H, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, slowest, sums, whole in res:
        assert slowest == 10.0 + world - 1
        assert sharding.combine_checksums(sums) == whole


def _liveness_worker(rank, world, port, q):
    sys.path.insert(0, str(ROOT))
    import datetime

    import torch.distributed as dist
    store = dist.TCPStore("127.0.0.1", port, world, is_master=(rank == 0), timeout=datetime.timedelta(seconds=30))
    sharding.rendezvous(store, "step0", rank, world, timeout_s=20)
    if rank == 2:
        q.put((rank, "left"))  # this rank leaves between steps (host-side failure, nothing in flight)
        return
    try:
        sharding.rendezvous(store, "step1", rank, world, timeout_s=1.5)
        q.put((rank, "no failure seen"))
    except sharding.RankFailure as e:
        q.put((rank, e.missing))
    if rank == 0:
        import time
        time.sleep(1.0)  # keep the store alive until the others have polled it


def test_a_rank_that_leaves_between_steps_is_named_by_the_others():
    world = 3
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_liveness_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert res[2] == "left"
    assert res[0] == [2] and res[1] == [2]
