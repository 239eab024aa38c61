"""Host-side sharding logic and the two-scalar reduction, on CPU with gloo (world size 2)."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from pe_ablations_b200 import eval as E


def test_shard_range_partitions_exactly():
    for n in (1, 7, 8, 64, 65):
        for w in (1, 2, 3, 4, 8):
            seen = []
            for r in range(w):
                seen += list(E.shard_range(n, w, r))
            assert seen == list(range(n))
            sizes = [len(E.shard_range(n, w, r)) for r in range(w)]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        E.shard_range(4, 2, 2)


def test_shard_heads_keeps_gqa_groups_together():
    q, kv = E.shard_heads(16, 4, 2, 1)
    assert list(kv) == [2, 3] and list(q) == list(range(8, 16))
    q, kv = E.shard_heads(16, 16, 8, 3)
    assert list(q) == [6, 7] == list(kv)
    with pytest.raises(ValueError):
        E.shard_heads(16, 4, 8, 0)


def test_perplexity_of_uniform_model():
    import math
    assert abs(E.perplexity(100 * math.log(32000.0), 100) - 32000.0) < 1e-6
    assert E.perplexity(0.0, 0.0) == float("inf")


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # rank r "evaluates" its shard of 5 fake sequences whose NLL sums are known
        per_seq_nll = torch.tensor([10.0, 20.0, 30.0, 40.0, 50.0], dtype=torch.float64)
        mine = E.shard_range(5, world, rank)
        nll = per_seq_nll[mine.start:mine.stop].sum()
        cnt = torch.tensor(float(len(mine) * 7))
        tot_nll, tot_cnt = E.reduce_loss_sums(nll, cnt)
        q.put((rank, tot_nll, tot_cnt, len(mine)))
    finally:
        dist.destroy_process_group()


def test_two_rank_reduction_gloo():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, nll, cnt, n in res:
        assert nll == 150.0 and cnt == 35.0
    assert sorted(r[3] for r in res) == [2, 3]
