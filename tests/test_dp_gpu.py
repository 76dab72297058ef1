"""Data-parallel optimizer update on two GPUs (NCCL) against single-GPU accumulation over the same rows."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def build(golden_path, device):
    from test_step_gpu import load_model, batch_of
    from causal_tuner_b200.modeling.model import Runtime
    with np.load(golden_path) as data:
        g = {key: data[key] for key in data.files}
    runtime = Runtime(rank=16, base_dtype=torch.float32, train_dtype=torch.float32, compute_dtype=torch.float32,
                      attention="vanilla", checkpoint=False)
    torch.cuda.set_device(device)
    return load_model(g, runtime, nf4=False), batch_of(g)


def worker(rank, world, port, golden_path, results):
    import sys
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from causal_tuner_b200.training import Trainer, make_optimizer
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        model, batch = build(golden_path, rank)
        model = model.to(f"cuda:{rank}")
        mine = {k: v[rank:rank + 1] for k, v in batch.items()}          # one packed row per rank
        trainer = Trainer(model, make_optimizer(model, learning_rate=1e-4), device=f"cuda:{rank}", bucket_bytes=1 << 16)
        metrics = trainer.update([mine])
        results[rank] = (metrics["loss"], metrics["collectives"],
                         [p.grad.cpu().numpy() for p in model.adapter_parameters()])
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_ranks_match_single_gpu_accumulation():
    from conftest import GOLDEN
    from causal_tuner_b200.training import Trainer, make_optimizer
    path = os.path.join(GOLDEN, "step_tiny_b1.npz")
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(worker, args=(2, free_port(), path, results), nprocs=2, join=True)
    model, batch = build(path, 0)
    halves = [{k: v[i:i + 1] for k, v in batch.items()} for i in range(2)]
    single = Trainer(model, make_optimizer(model, learning_rate=1e-4), device="cuda:0").update(halves)
    for rank in (0, 1):
        loss, collectives, grads = results[rank]
        assert abs(loss - single["loss"]) / single["loss"] < 1e-6
        assert collectives > 1          # several buckets, launched while the backward pass was running
        for actual, parameter in zip(grads, model.adapter_parameters()):
            torch.testing.assert_close(torch.from_numpy(actual), parameter.grad.cpu(), rtol=2e-4, atol=1e-7)
