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


# ---- failures made on the host: no GPU faults, traps or hangs ------------------------------------
def _worker_lost_rank(rank, world, port, q):
    """Step 1 completes on both ranks; rank 1 then leaves (between steps, nothing in flight) and
    rank 0's next reduction has to give up by itself."""
    import time

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    one = torch.tensor(1.0, dtype=torch.float64)
    nll, cnt = E.reduce_loss_sums(one * (rank + 1), one, timeout_s=30.0)
    assert (nll, cnt) == (3.0, 2.0)
    if rank == 1:
        q.put((rank, "left", 0.0))
        q.close()
        q.join_thread()                   # the message is out before the process disappears
        os._exit(0)                       # gone without a goodbye: no destroy_process_group
    t0 = time.monotonic()
    try:
        E.reduce_loss_sums(one, one, timeout_s=5.0)
        q.put((rank, "no error", time.monotonic() - t0))
    except RuntimeError as e:
        q.put((rank, f"raised: {e}", time.monotonic() - t0))
    q.close()
    q.join_thread()
    os._exit(0)


def test_survivor_raises_when_a_rank_leaves_between_steps():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker_lost_rank, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = dict((r[0], r[1:]) for r in (q.get(timeout=120) for _ in range(2)))
    for p in procs:
        p.join(timeout=60)
    assert res[1][0] == "left"
    msg, waited = res[0]
    assert msg.startswith("raised:") and "reduction failed or timed out" in msg, msg
    assert waited < 20.0, waited          # the 5 s limit, not the process group's default of minutes


def _worker_bad_status(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        one = torch.tensor(1.0, dtype=torch.float64)
        # rank 1's kernels "reported an expired wait": a fake status code, injected on the host
        try:
            E.reduce_loss_sums(one, one, timeout_s=30.0, status=0x40000000 if rank == 1 else 0)
            q.put((rank, "no error"))
        except RuntimeError as e:
            q.put((rank, f"raised: {e}"))
        # the group is still usable afterwards
        nll, cnt = E.reduce_loss_sums(one, one, timeout_s=30.0, status=0)
        q.put((rank, (nll, cnt)))
    finally:
        dist.destroy_process_group()


def test_every_rank_raises_when_one_rank_reports_expired_waits():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker_bad_status, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in range(4)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    first = {r: m for r, m in res if isinstance(m, str)}
    second = {r: m for r, m in res if not isinstance(m, str)}
    assert all(m.startswith("raised:") and "expired waits" in m for m in first.values()), first
    assert len(first) == 2 and second == {0: (2.0, 2.0), 1: (2.0, 2.0)}


def test_single_process_reduction_raises_on_a_status_code():
    one = torch.tensor(1.0, dtype=torch.float64)
    assert E.reduce_loss_sums(one * 3, one) == (3.0, 1.0)
    with pytest.raises(RuntimeError, match="expired waits"):
        E.reduce_loss_sums(one, one, status=2)
