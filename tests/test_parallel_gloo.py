"""world_size-2 check of the data-parallel plumbing on CPU (gloo): disjoint shards, max-over-ranks
timings, rank-ordered gather of token ids."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


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
