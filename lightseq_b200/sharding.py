"""Host-side batch sharding for replica-parallel inference.

The reference serves "eight A100" as eight independent single-GPU model objects (README.md:83): requests are
independent, so the batch dimension is partitioned and no data-path collective exists. ``shard_batch`` sorts the
sentences by source length and deals them round-robin so that every rank gets the same number of sentences and a
similar padded length; ``merge_results`` puts the per-rank outputs back in request order.
"""
from __future__ import annotations

from typing import List, Sequence, Tuple

import numpy as np


def shard_batch(ids: np.ndarray, pad_id: int, world_size: int) -> List[Tuple[np.ndarray, np.ndarray]]:
    """ids int32 [B, S] right-padded. Returns, per rank, (row indices into ids, trimmed sub-batch)."""
    if world_size < 1:
        raise ValueError("world_size must be positive")
    ids = np.asarray(ids)
    if ids.ndim != 2:
        raise ValueError("ids must be [batch, seq_len]")
    lens = (ids != pad_id).sum(axis=1)
    order = np.argsort(-lens, kind="stable")
    out = []
    for r in range(world_size):
        rows = order[r::world_size]
        if rows.size == 0:
            out.append((rows, ids[:0, :1]))
            continue
        width = max(int(lens[rows].max()), 1)
        out.append((rows, np.ascontiguousarray(ids[rows, :width])))
    return out


def merge_results(batch: int, shards: Sequence[Tuple[np.ndarray, np.ndarray, np.ndarray]], end_id: int):
    """shards: per rank (row indices, tokens [b, 1, L_r], scores [b, 1]). Returns tokens [batch, 1, max L] padded
    with ``end_id`` and scores [batch, 1] in the original request order."""
    width = max((t.shape[2] for _, t, _ in shards if t.size), default=0)
    tokens = np.full((batch, 1, width), end_id, dtype=np.int32)
    scores = np.zeros((batch, 1), dtype=np.float32)
    for rows, t, s in shards:
        if len(rows) == 0:
            continue
        tokens[rows, :, : t.shape[2]] = t
        scores[rows] = s
    return tokens, scores
