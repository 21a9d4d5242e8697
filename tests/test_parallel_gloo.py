"""world_size-2 check of the data-parallel plumbing on CPU (gloo): disjoint shards, max-over-ranks
timings, rank-ordered gather of token ids."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, global_batch, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from flash_stu_2_b200 import parallel
    s, e = parallel.shard_range(global_batch, world, rank)
    ids = torch.arange(s, e).view(-1, 1).repeat(1, 3) * 10 + torch.arange(3)
    full = parallel.gather_token_ids(ids, global_batch)
    times = parallel.max_over_ranks([1.0 + rank, 5.0 - rank])
    q.put((rank, s, e, full.tolist(), times))
    dist.destroy_process_group()


def test_two_rank_sharding_and_reductions():
    world, gb = 2, 5
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, gb, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    (r0, s0, e0, full0, t0), (r1, s1, e1, full1, t1) = res
    assert (s0, e0, s1, e1) == (0, 3, 3, 5)
    want = [[b * 10 + j for j in range(3)] for b in range(gb)]
    assert full0 == want and full1 == want
    assert t0 == [2.0, 5.0] and t1 == [2.0, 5.0]


def test_shard_ranges_cover_batch():
    from flash_stu_2_b200 import parallel
    for gb in (1, 7, 8, 32, 33):
        for world in (1, 2, 4, 8):
            spans = [parallel.shard_range(gb, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == gb
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))


def _leaver(rank, world, port, fport, q, mode):
    """Rank `world-1` leaves after step 1, between steps, with nothing in flight.  mode 'fence': the others meet a
    host-side StepFence before the next collective and must raise RankLost; mode 'timeout': they go straight into
    the collective, which a short process-group timeout / the closed connection must end with an error."""
    import datetime
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import sys
    sys.path.insert(0, ROOT)
    from flash_stu_2_b200 import parallel
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
    store = dist.TCPStore("127.0.0.1", fport, world, is_master=(rank == 0), timeout=datetime.timedelta(seconds=20),
                          wait_for_workers=False)
    fence = parallel.StepFence(store, world, timeout_s=1.5)
    outcome = "finished"
    try:
        for step in range(4):
            if mode == "fence":
                fence.arrive(step)
            t = torch.ones(4) * (rank + 1)
            dist.all_reduce(t)
            assert float(t[0]) == world * (world + 1) / 2
            if rank == world - 1 and step == 1:
                outcome = "left"
                break
    except parallel.RankLost as e:
        outcome = f"RankLost at fence: {e}"
    except Exception as e:  # the collective itself failed (peer gone / timeout)
        outcome = f"collective error: {type(e).__name__}"
    q.put((rank, outcome))
    q.close()
    q.join_thread()          # the report is on its way before the process disappears
    if outcome != "left":
        time.sleep(0.5)
    os._exit(0)              # no goodbye to the process group: a lost rank is simply gone


import time

import pytest


@pytest.mark.parametrize("mode", ["fence", "timeout"])
def test_a_rank_leaving_between_steps_makes_the_others_raise(mode):
    world = 3
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port, fport = _free_port(), _free_port()
    procs = [ctx.Process(target=_leaver, args=(r, world, port, fport, q, mode)) for r in range(world)]
    t0 = time.monotonic()
    for p in procs:
        p.start()
    res = dict(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=30)
    assert res[world - 1] == "left"
    for r in range(world - 1):
        if mode == "fence":
            assert res[r].startswith("RankLost at fence"), res
        else:
            assert res[r].startswith("collective error"), res
    assert time.monotonic() - t0 < 100   # nobody hung
