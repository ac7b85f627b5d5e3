"""Batch sharding across GPUs: images are independent on this path, so a global batch is cut into
contiguous per-rank slices, each rank runs the whole graph on its slice, and only the compacted
detections come back to rank 0.  There is no collective on the data path.

The reference emits detections layer by layer and, inside a layer, image by image
(Model::detections, include/Model.h:1062-1109).  With contiguous slices the global order is
therefore, for each detector head in layer order, rank 0's records, then rank 1's, ...; records
carry global image numbers (Runner(batch_id_offset=...)).
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import numpy as np


def shard_range(global_batch: int, rank: int, world: int) -> Tuple[int, int]:
    """[first, last) image of `rank`: contiguous slices, the first `global_batch % world` ranks get one more."""
    if not (0 <= rank < world) or global_batch < 0:
        raise ValueError("bad rank / world / batch")
    base, extra = divmod(global_batch, world)
    first = rank * base + min(rank, extra)
    return first, first + base + (1 if rank < extra else 0)


def split_heads(records: np.ndarray, head_ends: Sequence[int]) -> List[np.ndarray]:
    """Cuts a runner's flat record array at the running counts noted after each detector head."""
    out, start = [], 0
    for end in head_ends:
        out.append(records[start:end])
        start = end
    return out


def merge_shards(per_rank_heads: Sequence[Sequence[np.ndarray]]) -> np.ndarray:
    """per_rank_heads[r][h] = records of head h from rank r (ranks hold ascending image slices).
    Returns the records in the order a single process running the whole batch would emit them."""
    if not per_rank_heads:
        raise ValueError("no shards")
    n_heads = len(per_rank_heads[0])
    if any(len(h) != n_heads for h in per_rank_heads):
        raise ValueError("shards disagree on the number of detector heads")
    parts = [per_rank_heads[r][h] for h in range(n_heads) for r in range(len(per_rank_heads))]
    parts = [p for p in parts if len(p)]
    return np.concatenate(parts) if parts else per_rank_heads[0][0][:0]


def gather_detections(heads: Sequence[np.ndarray], group=None, dst: int = 0) -> Optional[np.ndarray]:
    """Host-side gather over a torch.distributed group (any backend): every rank passes its per-head
    record arrays; `dst` receives the merged global array, the others None.  A rank whose forward
    failed passes an Exception instead and the gather re-raises it on `dst`."""
    import torch.distributed as dist
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    payload = heads if isinstance(heads, Exception) else [np.ascontiguousarray(h) for h in heads]
    gathered = [None] * world if rank == dst else None
    dist.gather_object(payload, gathered, dst=dst, group=group)
    if rank != dst:
        return None
    for r, item in enumerate(gathered):
        if isinstance(item, Exception):
            raise RuntimeError(f"rank {r} failed: {item}") from item
    return merge_shards(gathered)
