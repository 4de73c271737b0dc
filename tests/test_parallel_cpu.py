"""Multi-rank host logic (lane sharding, token gather) on the gloo backend, world size 2 and 3,
plus the failure path: a rank that never joins makes the gather time out with an error."""
from __future__ import annotations

import os
import socket
import sys
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

REPO = Path(__file__).resolve().parents[1]


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, total: int, absent_rank: int, q):
    sys.path.insert(0, str(REPO))
    from __graft_entry__ import load_package
    par = load_package().parallel
    if rank == absent_rank:
        q.put((rank, "absent"))
        return
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    import datetime
    try:
        dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
    except Exception as e:                      # rendezvous never completes when a rank is missing
        q.put((rank, "error:" + type(e).__name__))
        return
    first, count = par.shard_lanes(total, world, rank)
    mine = torch.arange(first, first + count, dtype=torch.int32) * 10 + 1
    try:
        out = par.gather_tokens(mine, total, dst=0)
        q.put((rank, None if out is None else out.tolist()))
    except Exception as e:
        q.put((rank, "error:" + type(e).__name__))
    finally:
        dist.destroy_process_group()


def _run(world: int, total: int, absent_rank: int = -1):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, total, absent_rank, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
    return res


def test_shard_lanes_covers_every_lane_once(pkg):
    par = pkg.parallel
    for total in (0, 1, 7, 128, 4032):
        for world in (1, 2, 3, 8):
            spans = [par.shard_lanes(total, world, r) for r in range(world)]
            assert spans[0][0] == 0 and sum(c for _, c in spans) == total
            for (f0, c0), (f1, _) in zip(spans, spans[1:]):
                assert f1 == f0 + c0
            assert max(c for _, c in spans) - min(c for _, c in spans) <= 1
    with pytest.raises(ValueError):
        par.shard_lanes(8, 2, 2)


@pytest.mark.parametrize("world,total", [(2, 8), (2, 7), (3, 10)])
def test_gather_tokens_gloo(world, total):
    res = _run(world, total)
    assert res[0] == [i * 10 + 1 for i in range(total)]
    assert all(res[r] is None for r in range(1, world))


def test_missing_rank_is_reported_not_hung():
    res = _run(2, 8, absent_rank=1)
    assert res[1] == "absent"
    assert isinstance(res[0], str) and res[0].startswith("error:")
