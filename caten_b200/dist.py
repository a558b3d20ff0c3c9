"""Multi-GPU plumbing: one process per GPU, sequences sharded, weights replicated.

Sequences of a batch never interact (attention is per sequence, external/llm/layers.lisp:35-51;
the KV cache is indexed by batch row, layers.lisp:25-33), so the batch is cut into contiguous
slices, one per rank, and no collective runs on the data path.  ``torch.distributed`` is used for
exactly two things: broadcasting the packed weight arena from rank 0 at load, and gathering the
generated token ids.  The reference has no distributed component; there is no counterpart.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional, Tuple

import numpy as np

from .synthetic import Packed

ALIGN = 256


def shard_batch(batch: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous slice (first sequence, count) of rank ``rank``; earlier ranks take the remainder."""
    if world < 1 or not (0 <= rank < world):
        raise ValueError("shard_batch: bad rank/world")
    base, rem = divmod(batch, world)
    nb = base + (1 if rank < rem else 0)
    b0 = rank * base + min(rank, rem)
    return b0, nb


@dataclass
class Entry:
    offset: int
    nbytes: int
    ggml_type: int      # -1: plain fp32 array
    shape: Tuple[int, ...]


class Stub:
    """Shape/type of a state-dict entry whose bytes live in the device arena."""

    def __init__(self, e: Entry):
        self.shape = e.shape
        self.ggml_type = e.ggml_type
        if e.ggml_type >= 0:
            self.rows, self.cols = e.shape


def pack_arena(sd: dict) -> Tuple[np.ndarray, Dict[str, Entry]]:
    """Lays every entry of a state dict out in one byte arena (256-byte aligned slots)."""
    index, off = {}, 0
    for k, v in sd.items():
        nbytes = v.data.nbytes if isinstance(v, Packed) else np.asarray(v).astype(np.float32, copy=False).nbytes
        index[k] = Entry(off, nbytes, v.ggml_type if isinstance(v, Packed) else -1,
                         (v.rows, v.cols) if isinstance(v, Packed) else tuple(np.asarray(v).shape))
        off += (nbytes + ALIGN - 1) // ALIGN * ALIGN
    arena = np.zeros(off, np.uint8)
    for k, v in sd.items():
        e = index[k]
        src = v.data if isinstance(v, Packed) else np.ascontiguousarray(v, dtype=np.float32).view(np.uint8).reshape(-1)
        arena[e.offset:e.offset + e.nbytes] = src.reshape(-1)
    return arena, index


def unpack_arena(arena: np.ndarray, index: Dict[str, Entry]) -> dict:
    """Inverse of :func:`pack_arena` on a host arena (used by the CPU tests)."""
    sd = {}
    for k, e in index.items():
        raw = arena[e.offset:e.offset + e.nbytes]
        sd[k] = Packed(e.ggml_type, e.shape[0], e.shape[1], raw.copy()) if e.ggml_type >= 0 else raw.copy().view(np.float32).reshape(e.shape)
    return sd


def broadcast_state_dict(sd: Optional[dict], device, src: int = 0):
    """Rank ``src`` passes its state dict, the others None.  Returns (arena tensor on ``device``,
    index).  Works with the nccl backend (CUDA device) and with gloo (CPU)."""
    import torch
    import torch.distributed as dist

    rank = dist.get_rank()
    if rank == src:
        arena_np, index = pack_arena(sd)
        meta = [index, int(arena_np.size)]
    else:
        arena_np, meta = None, [None, None]
    dist.broadcast_object_list(meta, src=src)
    index, size = meta
    if rank == src:
        arena = torch.from_numpy(arena_np).to(device)
    else:
        arena = torch.empty(size, dtype=torch.uint8, device=device)
    dist.broadcast(arena, src=src)
    return arena, index


def device_views(arena, index: Dict[str, Entry]):
    """(stub state dict, {key: device pointer}) for :class:`caten_b200.gpt2.GPT2`."""
    base = arena.data_ptr()
    return {k: Stub(e) for k, e in index.items()}, {k: base + e.offset for k, e in index.items()}


def gather_ids(local_ids, batch: int, world: int):
    """local_ids: torch int64 [steps, nb_local] on every rank -> [steps, batch] (on all ranks).
    Slices may differ in size by one; they are padded to the largest for the collective."""
    import torch
    import torch.distributed as dist

    steps = local_ids.shape[0]
    nb_max = max(shard_batch(batch, world, r)[1] for r in range(world))
    pad = torch.zeros((steps, nb_max), dtype=torch.int64, device=local_ids.device)
    pad[:, :local_ids.shape[1]] = local_ids
    out = [torch.empty_like(pad) for _ in range(world)]
    dist.all_gather(out, pad)
    cols = [out[r][:, :shard_batch(batch, world, r)[1]] for r in range(world)]
    return torch.cat(cols, dim=1)


# ---------------------------------------------------------------------------------------------------
# The same two collectives through the library's own C ABI (`caten_b200_dist_*`: NCCL calls on the
# context's stream), i.e. the path a host without torch.distributed takes.  The 128-byte group id
# and the arena index are small host objects; how they travel between the processes is the host's
# business (`exchange` below: any callable that returns rank 0's object on every rank).
# ---------------------------------------------------------------------------------------------------
def capi_group_init(rt, rank: int, world: int, exchange) -> None:
    """Joins ``world`` processes into one group.  ``exchange(obj_or_None)`` must return, on every
    rank, the object rank 0 passed (e.g. a broadcast over the launcher's rendezvous store)."""
    import ctypes as C

    from . import _lib as L
    ident = None
    if world > 1 and rank == 0:
        buf = C.create_string_buffer(L.DIST_ID_BYTES)
        L.check(None, rt.lib.caten_b200_dist_unique_id(buf))
        ident = bytes(buf.raw)
    ident = exchange(ident) if world > 1 else None
    L.check(rt.ctx, rt.lib.caten_b200_dist_init(rt.ctx, int(rank), int(world), ident))


def capi_broadcast_state_dict(rt, sd: Optional[dict], rank: int, exchange, src: int = 0):
    """Rank ``src`` passes its state dict, the others None.  Returns (device arena buffer, index);
    the arena holds every tensor's bytes and may be closed once the weights are uploaded."""
    from . import _lib as L
    if rank == src:
        arena_np, index = pack_arena(sd)
        meta = (index, int(arena_np.size))
    else:
        arena_np, meta = None, None
    index, size = exchange(meta)
    arena = rt.open_buffer((size,), np.uint8)
    if rank == src:
        L.check(rt.ctx, rt.lib.caten_b200_h2d(rt.ctx, arena.ptr, arena_np.ctypes.data, arena_np.nbytes))
    L.check(rt.ctx, rt.lib.caten_b200_dist_bcast_weights(rt.ctx, arena.ptr, size, src))
    rt.sync()
    return arena, index


def arena_views(arena_ptr: int, index: Dict[str, Entry]):
    """(stub state dict, {key: device pointer}) for an arena at device address ``arena_ptr``."""
    return {k: Stub(e) for k, e in index.items()}, {k: arena_ptr + e.offset for k, e in index.items()}


def assemble_gathered(flat: np.ndarray, steps: int, batch: int, world: int) -> np.ndarray:
    """``flat``: [world, steps * nb_max] as `caten_b200_dist_gather_ids` returns it (every rank's
    [steps, nb_local] block padded to the widest slice) -> [steps, batch] in sequence order."""
    nb_max = max(shard_batch(batch, world, r)[1] for r in range(world))
    blocks = np.asarray(flat).reshape(world, steps, nb_max)
    return np.concatenate([blocks[r][:, :shard_batch(batch, world, r)[1]] for r in range(world)], axis=1)


def capi_gather_ids(rt, local_ids: np.ndarray, batch: int, world: int) -> np.ndarray:
    """local_ids: int64 [steps, nb_local] on every rank -> [steps, batch] on every rank."""
    from . import _lib as L
    steps = local_ids.shape[0]
    nb_max = max(shard_batch(batch, world, r)[1] for r in range(world))
    pad = np.zeros((steps, nb_max), np.int64)
    pad[:, :local_ids.shape[1]] = local_ids
    src = rt.transfer_from_array(pad)
    dst = rt.open_buffer((world, steps * nb_max), np.int64)
    L.check(rt.ctx, rt.lib.caten_b200_dist_gather_ids(rt.ctx, src.ptr, steps * nb_max, dst.ptr))
    out = assemble_gathered(dst.numpy(), steps, batch, world)
    src.close(); dst.close()
    return out
