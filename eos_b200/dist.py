"""Host logic of the multi-GPU layout: one process per GPU, no collective on the encoder's data path, one
all-gather of per-shard top-k keys for scoring.

The reference has no multi-GPU layer (docs/consumer-subquadratic-gpu-spec.md:28 rules it out); the sharding below
keeps its result order: document ids are global row indices, shards are contiguous id ranges, and the merged list
is ordered by score descending, then id ascending (runtime/retrieval_eval.go:1153-1161).
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Tuple

import numpy as np

from . import _lib


def shard_bounds(n_total: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous row range [lo, hi) of `rank`; the last ranks may be short or empty."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError(f"bad rank {rank} for world size {world}")
    shard = (n_total + world - 1) // world
    lo = min(n_total, rank * shard)
    return lo, min(n_total, lo + shard)


def batch_bounds(batch: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous slice of a batch for data-parallel encoding (sequences are independent)."""
    return shard_bounds(batch, world, rank)


def encode_keys(ids: np.ndarray, scores: np.ndarray) -> np.ndarray:
    """The sortable 64-bit key of a (score, id) candidate as the kernels exchange it:
    (order-preserving bits of the f32 score << 32) | (0xffffffff - id); larger = better; 0 = empty (id < 0)."""
    ids = np.asarray(ids, dtype=np.int64)
    u = np.asarray(scores, dtype=np.float32).view(np.uint32).astype(np.uint64)
    neg = (u & np.uint64(0x80000000)) != 0
    ordered = np.where(neg, (~u) & np.uint64(0xFFFFFFFF), u | np.uint64(0x80000000))
    keys = (ordered << np.uint64(32)) | (np.uint64(0xFFFFFFFF) - ids.astype(np.uint64) & np.uint64(0xFFFFFFFF))
    return np.where(ids < 0, np.uint64(0), keys)


def decode_keys(keys: np.ndarray) -> Tuple[np.ndarray, np.ndarray]:
    """Inverse of encode_keys: (ids int64 with -1 for empty, scores f32 with -inf for empty)."""
    keys = np.asarray(keys).astype(np.uint64)
    o = (keys >> np.uint64(32)).astype(np.uint32)
    bits = np.where((o & np.uint32(0x80000000)) != 0, o & np.uint32(0x7FFFFFFF), ~o)
    scores = bits.astype(np.uint32).view(np.float32).copy()
    ids = (np.uint64(0xFFFFFFFF) - (keys & np.uint64(0xFFFFFFFF))).astype(np.int64)
    empty = keys == 0
    ids[empty] = -1
    scores[empty] = -np.inf
    return ids, scores


NCCL_ID_BYTES = 128


def new_comm_id() -> bytes:
    """The 128-byte NCCL id (rank 0 makes it and hands it to every other rank by whatever channel the host has)."""
    buf = C.create_string_buffer(NCCL_ID_BYTES)
    _lib.call("eos_b200_comm_unique_id", buf)
    return buf.raw


class Comm:
    """The library's own communicator over the GPUs of a sharded corpus (one process per GPU): the collectives of
    Corpus.score_topk_sharded are issued by the library through it, so the host needs no collective library."""

    def __init__(self, runtime, rank: int, world: int, comm_id: bytes):
        if len(comm_id) != NCCL_ID_BYTES:
            raise ValueError("comm_id must be the 128 bytes of new_comm_id()")
        self.rt, self.rank, self.world = runtime, int(rank), int(world)
        self.handle = C.c_void_p()
        buf = C.create_string_buffer(comm_id, NCCL_ID_BYTES)
        _lib.call("eos_b200_comm_init", runtime.handle, self.rank, self.world, buf, C.byref(self.handle))
        runtime._adopt(self)

    def merge_keys(self, d_keys: int, q_count: int, k: int, d_ids: int, d_scores: int, stream: Optional[int] = None) -> None:
        """Collective: all-gather of every rank's key lists [q_count, k] and the merge into the global top-k."""
        _lib.call("eos_b200_comm_merge_keys", self.handle, d_keys, int(q_count), int(k), d_ids, d_scores, stream)

    def close(self) -> None:
        if self.handle:
            _lib.lib().eos_b200_comm_destroy(self.handle)
            self.handle = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
