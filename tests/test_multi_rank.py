"""Host-side multi-rank logic on CPU ranks (gloo, world_size 2): sharding, gather order, and a
missing rank surfacing as an error instead of a hang."""
import datetime
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from triton_snn_fusion_b200.parallel import gather_logits, shard_range


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _fake_logits(start, stop, classes=7):
    idx = torch.arange(start, stop, dtype=torch.float32).unsqueeze(1)
    return idx * 10.0 + torch.arange(classes, dtype=torch.float32).unsqueeze(0)


def _worker_gather(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=30))
    try:
        start, stop = shard_range(16, rank, world)
        out = gather_logits(_fake_logits(start, stop))
        ok = torch.equal(out, _fake_logits(0, 16))
        pre = torch.empty(16, 7)
        out2 = gather_logits(_fake_logits(start, stop), out=pre)
        ok = ok and out2 is pre and torch.equal(pre, _fake_logits(0, 16))
        q.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


def test_shard_range():
    assert shard_range(512, 0, 8) == (0, 64) and shard_range(512, 7, 8) == (448, 512)
    assert [shard_range(6, r, 3) for r in range(3)] == [(0, 2), (2, 4), (4, 6)]
    with pytest.raises(ValueError):
        shard_range(10, 0, 4)
    with pytest.raises(ValueError):
        shard_range(8, 2, 2)


def test_gather_single_process_is_identity():
    x = torch.randn(4, 3)
    assert gather_logits(x) is x


def test_gather_order_two_gloo_ranks():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker_gather, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert results == [(0, True), (1, True)]


def _worker_lonely(port, q):
    # rank 0 of a 2-rank job whose peer never starts: rendezvous must fail within the timeout
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    try:
        dist.init_process_group("gloo", rank=0, world_size=2, timeout=datetime.timedelta(seconds=3))
        gather_logits(torch.zeros(2, 2))
        q.put("no error")
    except Exception as exc:  # noqa: BLE001 - any rendezvous / collective error is the expected outcome
        q.put(type(exc).__name__)


def test_missing_rank_is_an_error_not_a_hang():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    p = ctx.Process(target=_worker_lonely, args=(_free_port(), q))
    p.start()
    outcome = q.get(timeout=120)
    p.join(timeout=60)
    assert outcome != "no error"
