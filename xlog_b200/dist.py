"""Host-side plumbing for several ranks (one process per GPU) over ``torch.distributed``.

The data path of a multi-rank fixpoint (partition, all-to-all, termination vote) runs inside
libxlb.so over NCCL.  This module holds what the host program does around it: the owner
function (bit-identical to the device's), slicing inputs, distributing the communicator id and
gathering shards for inspection.  ``exchange_by_owner`` restates the library's exchange
bookkeeping (count matrix, variable all-to-all) on host arrays so it can be exercised with the
gloo backend where no GPU is present.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

_M1 = np.uint64(0xFF51AFD7ED558CCD)
_M2 = np.uint64(0xC4CEB9FE1A85EC53)
_S = np.uint64(33)


def mix64(x: np.ndarray) -> np.ndarray:
    """The 64-bit finaliser the library hashes join keys with (xk::mix64)."""
    with np.errstate(over="ignore"):
        x = np.asarray(x, dtype=np.uint64).copy()
        x ^= x >> _S
        x *= _M1
        x ^= x >> _S
        x *= _M2
        x ^= x >> _S
    return x


def owner_of(keys: np.ndarray, world: int) -> np.ndarray:
    """Owner rank of every join-key value: ``mix64(key) mod world`` (xlb_owner_of)."""
    return (mix64(keys) % np.uint64(world)).astype(np.int64)


def shard_bounds(rows: int, rank: int, world: int) -> tuple[int, int]:
    """The contiguous slice of an input relation that ``rank`` loads."""
    return rows * rank // world, rows * (rank + 1) // world


def init_comm(provider, rank: int, world: int, device=None) -> None:
    """Create the library's NCCL communicator: rank 0 draws the id, torch.distributed carries its
    128 bytes to every rank, every rank joins.  Needs an initialised process group."""
    import torch
    import torch.distributed as dist

    lib = provider._lib
    t = torch.zeros(128, dtype=torch.uint8, device=device if device is not None else "cpu")
    if rank == 0:
        buf = (C.c_uint8 * 128)()
        provider._check(lib.xlb_comm_unique_id(buf))
        t.copy_(torch.tensor(list(buf), dtype=torch.uint8))
    dist.broadcast(t, 0)
    arr = (C.c_uint8 * 128)(*t.cpu().tolist())
    provider._check(lib.xlb_comm_init(provider._ctx, arr, rank, world))


class ExchangeCountError(RuntimeError):
    """A rank's send counts do not add up to the rows it holds: nothing was exchanged."""


def exchange_by_owner(rows: np.ndarray, keys: np.ndarray, world: int, _send_counts=None) -> np.ndarray:
    """Send every packed row to ``owner_of(key)``; returns the rows this rank receives, grouped by
    source rank.  Same steps as the library's exchange: stable partition by owner, all-gather of the
    send counts, variable-size all-to-all.

    Every rank's count row travels with the number of rows that rank holds; a row that does not add
    up to it is caught by **every** rank from the gathered matrix, before any rank posts a receive
    sized by it, so a bad count ends the exchange with the same error everywhere instead of leaving
    the other ranks waiting in the all-to-all.  (``_send_counts`` lets a test put a wrong row in.)"""
    import torch
    import torch.distributed as dist

    rows = np.asarray(rows, dtype=np.uint64)
    own = owner_of(keys, world)
    order = np.argsort(own, kind="stable")
    part = rows[order]
    send = np.bincount(own, minlength=world).astype(np.int64)
    if _send_counts is not None:
        send = np.asarray(_send_counts, dtype=np.int64)
    counts = [torch.zeros(world + 1, dtype=torch.int64) for _ in range(world)]
    dist.all_gather(counts, torch.from_numpy(np.append(send, len(rows)).astype(np.int64)))
    bad = [r for r in range(world) if int(counts[r][:world].sum()) != int(counts[r][world]) or int(counts[r][:world].min()) < 0]
    if bad:
        raise ExchangeCountError(f"send counts of rank(s) {bad} do not add up to their row counts")
    rank = dist.get_rank()
    recv = [int(counts[r][rank]) for r in range(world)]
    out = torch.empty(sum(recv), dtype=torch.int64)
    dist.all_to_all_single(out, torch.from_numpy(part.view(np.int64).copy()), recv, send.tolist())
    return out.numpy().view(np.uint64)


def allreduce_sum(v: int) -> int:
    """The termination vote: sum of the ranks' new-tuple counts."""
    import torch
    import torch.distributed as dist

    t = torch.tensor([v], dtype=torch.int64)
    dist.all_reduce(t)
    return int(t.item())


def gather_shards(cols: list[np.ndarray]) -> list[np.ndarray]:
    """All ranks' shards of a relation, concatenated and sorted by all columns (on every rank)."""
    import torch.distributed as dist

    parts = [None] * dist.get_world_size()
    dist.all_gather_object(parts, [np.asarray(c) for c in cols])
    cat = [np.concatenate([p[i] for p in parts]) for i in range(len(cols))]
    order = np.lexsort(tuple(reversed(cat))) if cat and len(cat[0]) else np.arange(0)
    return [c[order] for c in cat]
