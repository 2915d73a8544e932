"""Host-side batch sharding for replica-parallel inference.

The reference serves "eight A100" as eight independent single-GPU model objects (README.md:83): requests are
independent, so the batch dimension is partitioned and no data-path collective exists. ``shard_batch`` sorts the
sentences by source length and deals them round-robin so that every rank gets the same number of sentences and a
similar padded length; ``merge_results`` puts the per-rank outputs back in request order.
"""
from __future__ import annotations

import ctypes
from concurrent.futures import ThreadPoolExecutor
from typing import List, Optional, Sequence, Tuple

import numpy as np


def shard_batch(ids: np.ndarray, pad_id: int, world_size: int, trim: bool = True) -> List[Tuple[np.ndarray, np.ndarray]]:
    """ids int32 [B, S] right-padded. Returns, per rank, (row indices into ids, sub-batch). With ``trim`` every
    sub-batch is cut to its own longest sentence (less padded work; the decode-length cap, source length + extra,
    then follows the shard's width as it would for any smaller request); without it every shard keeps the full
    width and each sentence's result is bit-identical to the unsharded run."""
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
        width = max(int(lens[rows].max()), 1) if trim else ids.shape[1]
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


class ReplicaRunner:
    """One request batch over several GPUs of one host: a full model replica, one host thread and one stream per
    GPU; ``infer`` splits the batch with ``shard_batch``, runs the shards concurrently (the native calls release
    the GIL) and merges the results in request order. No collective: the shards are independent.

        runner = ReplicaRunner("model.ls100", max_batch_size=128, devices=[0, 1, 2, 3])
        tokens, scores = runner.infer(ids, pad_id=1, end_id=2)
    """

    def __init__(self, weight_path: str, max_batch_size: int, devices: Sequence[int], model: str = "QuantTransformer"):
        if not devices:
            raise ValueError("devices must not be empty")
        self.devices = list(devices)
        self._rt = ctypes.CDLL("libcudart.so.12", mode=ctypes.RTLD_GLOBAL)
        # one single-thread executor per device: the thread that created a replica is the one that runs it
        self._pools = [ThreadPoolExecutor(max_workers=1, thread_name_prefix=f"ls100-gpu{d}") for d in self.devices]
        per_gpu = (max_batch_size + len(self.devices) - 1) // len(self.devices)

        def make(dev):
            from . import inference as lsi

            if self._rt.cudaSetDevice(ctypes.c_int(dev)) != 0:
                raise RuntimeError(f"cudaSetDevice({dev}) failed")
            return getattr(lsi, model)(weight_path, per_gpu)

        self.models = [p.submit(make, d).result() for p, d in zip(self._pools, self.devices)]
        self.per_gpu = per_gpu

    def infer(self, ids: np.ndarray, pad_id: int, end_id: int, trim: bool = True):
        ids = np.ascontiguousarray(ids, dtype=np.int32)
        shards = shard_batch(ids, pad_id, len(self.devices), trim)
        futs = [p.submit(m.infer, sub) if len(rows) else None for p, m, (rows, sub) in zip(self._pools, self.models, shards)]
        outs = []
        for (rows, _), f in zip(shards, futs):
            if f is None:
                continue
            tok, sc = f.result()
            outs.append((rows, tok, sc))
        return merge_results(ids.shape[0], outs, end_id)

    def close(self):
        for p, m in zip(self._pools, list(self.models)):
            p.submit(lambda: None).result()
        self.models = []
        for p in self._pools:
            p.shutdown()
