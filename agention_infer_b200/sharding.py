"""Token-row sharding across the GPUs of one box.

Every layer op is independent per token row, so the rows of a batch are split into
contiguous blocks, one per rank, and no data-path collective is needed.  Norm weights, the
RoPE table and the quantised embedding table are replicated.  The only communication is
for measurement and verification: a barrier, a max over the ranks' elapsed times, and a
gather of small per-rank checksums.
"""
from __future__ import annotations

from typing import List, Sequence, Tuple

import numpy as np


def shard_rows(T: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous block [start, stop) of rank `rank` out of `world`; the first T % world
    ranks take one extra row, so every row is owned exactly once for any T >= 0."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world of {world}")
    base, extra = divmod(T, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def all_shards(T: int, world: int) -> List[Tuple[int, int]]:
    return [shard_rows(T, r, world) for r in range(world)]


def checksum(a: np.ndarray) -> Tuple[int, int, int]:
    """Order-sensitive 64-bit checksum of an array's bytes (sum of u32 words weighted by
    position modulo 2^64); concatenating shards reproduces the whole-array value through
    `combine_checksums`."""
    w = np.ascontiguousarray(a).view(np.uint8).reshape(-1)
    pad = (-w.size) % 4
    if pad:
        w = np.concatenate([w, np.zeros(pad, np.uint8)])
    u = w.view(np.uint32).astype(np.uint64)
    idx = np.arange(1, u.size + 1, dtype=np.uint64)
    with np.errstate(over="ignore"):
        return int((u * idx).sum(dtype=np.uint64)), int(u.sum(dtype=np.uint64)), int(u.size)


def combine_checksums(parts: Sequence[Tuple[int, int, int]]) -> Tuple[int, int, int]:
    """Checksum of the concatenation from the per-shard (weighted, plain, words) triples."""
    M = 1 << 64
    weighted = plain = words = 0
    for wsum, psum, n in parts:
        weighted = (weighted + wsum + (words % M) * psum) % M
        plain = (plain + psum) % M
        words += n
    return weighted, plain, words


def max_over_ranks(value: float, group=None) -> float:
    """Max of a host scalar over all ranks (torch.distributed all_reduce MAX); identity when
    no process group is initialised."""
    import torch
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()):
        return float(value)
    dev = "cuda" if dist.get_backend(group) == "nccl" else "cpu"
    t = torch.tensor([value], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())


class RankFailure(RuntimeError):
    """Some ranks did not reach a rendezvous in time; `.missing` lists them."""

    def __init__(self, tag: str, missing):
        super().__init__(f"ranks {sorted(missing)} did not reach '{tag}' in time")
        self.missing = sorted(missing)


def rendezvous(store, tag: str, rank: int, world: int, timeout_s: float = 30.0, poll_s: float = 0.05) -> None:
    """Host-side liveness check between steps: every rank posts a key in the key-value store
    and waits, with a limit, for the keys of all the others.  A rank that has died or hangs on
    the host is reported by name (RankFailure) instead of blocking the next collective.  It
    runs with no kernel or collective in flight, so no GPU work is ever abandoned."""
    import time
    store.set(f"{tag}/{rank}", b"1")
    deadline = time.monotonic() + timeout_s
    missing = set(range(world)) - {rank}
    while missing:
        for r in list(missing):
            if store.check([f"{tag}/{r}"]):
                missing.discard(r)
        if not missing:
            break
        if time.monotonic() > deadline:
            raise RankFailure(tag, missing)
        time.sleep(poll_s)


def gather_objects(obj, group=None) -> list:
    """All ranks' small Python objects (checksums, parity figures), in rank order."""
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()):
        return [obj]
    out = [None] * dist.get_world_size(group)
    dist.all_gather_object(out, obj, group=group)
    return out
