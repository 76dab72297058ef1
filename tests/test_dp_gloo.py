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


class _ToyDecoder(torch.nn.Module):
    """Stands in for CausalLM on CPU ranks: a few trainable matrices between the batch and the 'hidden'
    output, with the attributes Trainer.update reads."""

    def __init__(self):
        super().__init__()
        torch.manual_seed(7)
        self.first = torch.nn.Parameter(torch.randn(6, 8))
        self.second = torch.nn.Parameter(torch.randn(8, 3))
        self.third = torch.nn.Parameter(torch.randn(3, 5))
        self.lm_head = torch.nn.Linear(5, 11, bias=False).requires_grad_(False)
        self.runtime = type("R", (), {"compute_dtype": torch.float32})()
        self.model = type("M", (), {"norm": type("N", (), {"weight": torch.zeros(1)})()})()
        self.fail = False

    def forward(self, batch):
        if self.fail:
            raise MemoryError("injected on the host")
        x = torch.nn.functional.one_hot(batch["input_ids"] % 6, 6).float()
        return x @ self.first @ self.second @ self.third


def trainer_worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import datetime
    from causal_tuner_b200 import _lib, training
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=30))
    try:
        # CPU ranks: the CUDA-only loss and the device check are replaced; the exchange logic is what runs.
        training.projection_loss = lambda hidden, head, targets, weights, **kw: (hidden @ head.T).square().sum()
        _lib.check_device = lambda *a, **k: None
        model = _ToyDecoder()
        optimizer = torch.optim.AdamW([p for p in model.parameters() if p.requires_grad], lr=1e-3)
        trainer = training.Trainer(model, optimizer, device="cpu", bucket_bytes=64)   # several buckets
        ids = torch.arange(12).reshape(2, 6) + rank
        batch = {"input_ids": ids, "attention_mask": torch.ones_like(ids)}
        first = trainer.update([batch])
        grads = [p.grad.clone() for p in model.parameters() if p.requires_grad]
        model.fail = rank == 1                      # rank 1 raises inside its forward pass
        try:
            trainer.update([batch])
            outcome = "no error"
        except Exception as error:
            outcome = f"{type(error).__name__}: {error}"
        model.fail = False
        again = trainer.update([batch])             # the ranks are still in step: the next update works
        gathered = [None] * world
        dist.all_gather_object(gathered, [g.tolist() for g in grads])
        same = all(torch.equal(torch.tensor(gathered[0][i]), torch.tensor(gathered[r][i]))
                   for r in range(world) for i in range(len(grads)))
        results[rank] = (first["collectives"], outcome, again["collectives"], same, first["loss"] == first["loss"])
    finally:
        dist.destroy_process_group()


def test_a_rank_that_raises_mid_update_stops_every_rank_and_the_next_update_still_works():
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(trainer_worker, args=(2, free_port(), results), nprocs=2, join=True)
    for rank in (0, 1):
        collectives, outcome, again, same, finite = results[rank]
        assert collectives == again and collectives >= 3        # buckets + the scalar all-reduce, every update
        assert same and finite                                  # both ranks hold the same summed gradients
    assert results[1][1].startswith("MemoryError")
    assert results[0][1].startswith("RuntimeError: Another rank failed")


def test_bucket_plan_is_a_function_of_the_shapes():
    from causal_tuner_b200.dp import BucketPlan
    shapes = [(4, 8), (8, 4), (2, 2), (16,), (3, 5)]
    plan = BucketPlan(shapes, "cpu", bucket_bytes=64)
    assert [plan.slot[i][0] for i in range(5)] == [2, 1, 1, 0, 0]       # reverse parameter order, >= 64 bytes each
    assert sum(b.numel() for b in plan.buffers) == sum(torch.Size(s).numel() for s in shapes)
    assert all(plan.view(i).shape == torch.Size(s) for i, s in enumerate(shapes))
    other = BucketPlan(shapes, "cpu", bucket_bytes=64)
    assert plan.slot == other.slot and plan.members == other.members
    with pytest.raises(ValueError):
        BucketPlan(shapes, "cpu", bucket_bytes=0)


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


def test_balanced_assignment_evens_out_attention_cost():
    from causal_tuner_b200.dp import balance_rows, row_costs
    generator = torch.Generator().manual_seed(5)
    rows, width, world = 16, 512, 4
    segments = torch.zeros(rows, width, dtype=torch.long)
    for row in range(rows):
        cursor, index = 0, 1
        while cursor < width:
            size = int(torch.randint(8, width + 1, (), generator=generator)) if row % 2 else width
            segments[row, cursor:cursor + size] = index
            cursor, index = cursor + size, index + 1
    mask = torch.ones_like(segments)
    costs = row_costs(mask, segments, width=width)
    assert max(costs) == pytest.approx(width + width / 12)        # one full-width document
    assignment = balance_rows(costs, world)
    assert sorted(r for rows_ in assignment for r in rows_) == list(range(rows))
    assert all(len(rows_) == rows // world for rows_ in assignment)
    load = lambda members: sum(costs[r] for r in members)
    contiguous = [list(range(*shard_rows(rows, r, world))) for r in range(world)]
    assert max(map(load, assignment)) <= max(map(load, contiguous))
    assert max(map(load, assignment)) - min(map(load, assignment)) <= max(costs) - min(costs)
    assert assignment == balance_rows(list(costs), world)          # same on every rank
    # ragged: 7 rows over 3 ranks -> at most 3 each; padding tokens cost nothing
    ragged = balance_rows([5., 1., 1., 1., 4., 1., 3.], 3)
    assert [len(m) for m in ragged] == [3, 2, 2] or max(len(m) for m in ragged) <= 3
    assert row_costs(torch.zeros(2, 8, dtype=torch.long)) == [0.0, 0.0]
    with pytest.raises(ValueError):
        balance_rows([1.0], 0)
