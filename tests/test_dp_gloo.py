"""The gradient exchange on CPU ranks (gloo, world size 2): sums, bucket boundaries, failure on the host."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from causal_tuner_b200.dp import GradientExchange, exchange_gradients, shard_rows


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def worker(rank, world, port, bucket_bytes, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.manual_seed(100 + rank)
        shapes = [(16, 64), (96, 16), (16, 64), (8, 16), (5, 3)]
        gradients = [torch.randn(*shape) for shape in shapes]
        strided = torch.randn(6, 10)[:, ::2]          # a non-contiguous gradient view
        local = [g.clone() for g in gradients] + [strided.clone()]
        count = exchange_gradients(gradients + [strided], bucket_bytes=bucket_bytes)
        gathered = [None] * world
        dist.all_gather_object(gathered, [t.tolist() for t in local])
        expected = [sum(torch.tensor(gathered[r][i]) for r in range(world)) for i in range(len(local))]
        ok = all(torch.allclose(a, e, rtol=0, atol=1e-6) for a, e in zip(gradients + [strided], expected))
        results[rank] = (ok, count)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("bucket_bytes,collectives", [(1 << 30, 1), (4096, 4), (1, 6)])
def test_exchange_sums_over_two_ranks(bucket_bytes, collectives):
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(worker, args=(2, free_port(), bucket_bytes, results), nprocs=2, join=True)
    assert dict(results) == {0: (True, collectives), 1: (True, collectives)}


def failing_worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import datetime
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
    try:
        if rank == 1:
            results[rank] = "left before the collective"   # a rank that never joins the exchange
            return
        try:
            exchange_gradients([torch.ones(4)])
            results[rank] = "no error"
        except Exception as error:  # the survivor learns of it through the process-group timeout
            results[rank] = type(error).__name__
    finally:
        try:
            dist.destroy_process_group()
        except Exception:
            pass


def test_missing_rank_surfaces_as_an_error_on_the_survivor():
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(failing_worker, args=(2, free_port(), results), nprocs=2, join=True)
    assert results[1] == "left before the collective"
    assert results[0] != "no error"


def test_single_process_is_a_no_op():
    gradient = torch.randn(4, 4)
    before = gradient.clone()
    assert exchange_gradients([gradient]) == 0
    assert torch.equal(gradient, before)
    with pytest.raises(TypeError):
        GradientExchange().add(torch.zeros(2, dtype=torch.bfloat16))


def test_row_sharding_covers_every_row_once():
    for total, world in ((8, 2), (7, 3), (4, 8), (0, 2)):
        spans = [shard_rows(total, r, world) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == total
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
    with pytest.raises(ValueError):
        shard_rows(4, 2, 2)
