"""Host-side logic of the multi-GPU path on CPU: slice arithmetic, the per-head merge, and a
world-size-2 gloo gather (including a rank that fails)."""
import os
import socket

import numpy as np
import pytest
import torch.distributed as dist
import torch.multiprocessing as mp

from pixienn_b200 import sharding
from pixienn_b200.ops import DET_DTYPE


def test_shard_ranges_cover_the_batch():
    for gb in (0, 1, 7, 64, 65):
        for world in (1, 2, 3, 8):
            spans = [sharding.shard_range(gb, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == gb
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        sharding.shard_range(8, 2, 2)


def fake_records(head, images):
    """Deterministic records: three per (head, image)."""
    out = np.zeros(3 * len(images), DET_DTYPE)
    for k, img in enumerate(images):
        for j in range(3):
            out[3 * k + j] = (img, head, j, 1, 0.5 + 0.01 * j, j, img, head * 100 + j)
    return out


def test_merge_equals_single_process_order():
    whole = [fake_records(h, range(6)) for h in range(3)]
    shards = [[fake_records(h, range(*sharding.shard_range(6, r, 4))) for h in range(3)] for r in range(4)]
    assert sharding.merge_shards(shards).tobytes() == np.concatenate(whole).tobytes()
    flat = np.concatenate(whole)
    ends = np.cumsum([len(w) for w in whole])
    assert [a.tobytes() for a in sharding.split_heads(flat, ends)] == [w.tobytes() for w in whole]
    with pytest.raises(ValueError):
        sharding.merge_shards([[whole[0]], [whole[0], whole[1]]])


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, fail_rank, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        if rank == fail_rank:
            payload = RuntimeError("device lost")            # a failed replica reports instead of hanging the gather
        else:
            payload = [fake_records(h, range(*sharding.shard_range(5, rank, world))) for h in range(2)]
        try:
            merged = sharding.gather_detections(payload)
            if rank == 0:
                q.put(("ok", merged.tobytes()))
        except RuntimeError as e:
            if rank == 0:
                q.put(("error", str(e)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("fail_rank", [-1, 1])
def test_gloo_gather_world_size_2(fail_rank):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, fail_rank, q)) for r in range(2)]
    for p in procs:
        p.start()
    kind, value = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    if fail_rank < 0:
        want = np.concatenate([fake_records(h, range(5)) for h in range(2)]).tobytes()
        assert kind == "ok" and value == want
    else:
        assert kind == "error" and "rank 1 failed" in value
