"""Golden fixture of one whole optimizer step of the tiny decoder, produced by the REFERENCE on CPU.

    PYTHONPATH=<reference>/src python tests/golden/make_golden_step.py [--dtype bfloat16]

Configuration (fp32 everywhere, "vanilla" attention): 2 layers, hidden 256, 4 query heads + 1 shared
KV head, head_dim 64, SwiGLU MLP 688, vocab 1024, RoPE theta 1e4 (partial rotary factor left at the
reference default 0.5), RMSNorm eps 1e-5. Every frozen matrix (projections, embedding, head) is
N(0, 0.02) rounded through NF4 (64-element blocks, fp32 absmax) and stored packed; the reference
loads the decoded values because its NF4 path refuses non-CUDA devices (modeling/lora.py:44-45).
LoRA rank 16, A ~ N(0, 0.02); B = 0 in step_tiny_b0.npz and B ~ N(0, 0.02) in step_tiny_b1.npz.
Batch: 2 packed rows of 512 tokens, ids uniform over the vocabulary, documents of U[32, 256] tokens
laid end to end. One `Trainer.update(step=0, total_steps=1)` with AdamW lr 1e-4 (training/engine.py:41-111).
With --dtype bfloat16 the same step (variant B != 0 only) runs with bf16 compute - frozen weights stored in
fp32 and cast to bf16 at use, fp32 adapters, gradients and optimizer state - and is written to
step_tiny_bf16.npz: the reference's own bf16 arithmetic on the CPU, which is what a bf16 GPU step is held
against.
Recorded: loss, gradient norm, every adapter gradient (after the division by the total weight and
before clipping is NOT observable, so the clipped .grad is recorded) and every adapter after the step.
"""

import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))

from causal_tuner.arguments import parse_args
from causal_tuner.modeling.config import ModelConfig
from causal_tuner.modeling.model import CausalLM
from causal_tuner.train import runtime_from_args
from causal_tuner.training.engine import Trainer, make_optimizer
from causal_tuner_b200.quant import quantize_nf4
from oracle import nf4 as oracle_nf4


def make_batch(generator, rows=2, length=512, vocab=1024):
    ids = torch.randint(0, vocab, (rows, length), generator=generator)
    segments = torch.zeros(rows, length, dtype=torch.long)
    for row in range(rows):
        cursor, index = 0, 1
        while cursor < length:
            size = int(torch.randint(32, 257, (1,), generator=generator))
            segments[row, cursor:cursor + size] = index
            cursor += size
            index += 1
    return {"input_ids": ids, "attention_mask": torch.ones_like(ids), "segment_ids": segments}


def main():
    bf16 = "--dtype" in sys.argv and sys.argv[sys.argv.index("--dtype") + 1] == "bfloat16"
    args = parse_args(["--repo-id", "fixture", "--dataset-name", "fixture", "--dtype", "bfloat16" if bf16 else "float32",
                       "--param-dtype", "float32", "--lora-rank", "16", "--attn-mechanism", "vanilla",
                       "--learning-rate", "1e-4", "--warmup-steps", "0"])
    config = ModelConfig(hidden_size=256, intermediate_size=688, vocab_size=1024, num_hidden_layers=2,
                         num_attention_heads=4, head_dim=64, rope_theta=1e4, rms_norm_eps=1e-5, pad_token_id=0,
                         eos_token_id=1)
    for variant in ((1,) if bf16 else (0, 1)):
        generator = torch.Generator().manual_seed(20240 + variant)
        model = CausalLM(config, runtime_from_args(args), "cpu")
        record = {}
        with torch.no_grad():
            for name, parameter in model.named_parameters():
                key = name.replace(".", "__")
                if name.endswith("lora_A"):
                    parameter.copy_(torch.randn(parameter.shape, generator=generator) * .02)
                    record["a__" + key] = parameter.float().numpy().copy()
                elif name.endswith("lora_B"):
                    parameter.copy_(torch.randn(parameter.shape, generator=generator) * (.02 if variant else 0.))
                    record["b__" + key] = parameter.float().numpy().copy()
                elif parameter.ndim == 2:       # frozen matrix: N(0, .02) through NF4
                    packed, state = quantize_nf4(torch.randn(parameter.shape, generator=generator) * .02, blocksize=64)
                    decoded = oracle_nf4.decode(packed.numpy(), state.absmax.numpy(), state.code.numpy(),
                                                parameter.numel(), 64)
                    parameter.copy_(torch.from_numpy(decoded).reshape(parameter.shape))
                    record["q__" + key] = packed.reshape(-1).numpy()
                    record["s__" + key] = state.absmax.numpy()
                elif name.endswith("bias"):
                    parameter.copy_(torch.randn(parameter.shape, generator=generator) * .02)
                    record["v__" + key] = parameter.float().numpy().copy()
                else:                            # norm weights
                    parameter.copy_(torch.rand(parameter.shape, generator=generator) + .5)
                    record["v__" + key] = parameter.float().numpy().copy()
        batch = make_batch(generator)
        record["input_ids"], record["segment_ids"] = batch["input_ids"].numpy(), batch["segment_ids"].numpy()
        optimizer = make_optimizer(model, args)
        metrics = Trainer(model, optimizer, args, device="cpu").update([batch], step=0, total_steps=1)
        record["loss"], record["grad_norm"] = np.float64(metrics["loss"]), np.float64(metrics["grad_norm"])
        record["effective_weight"], record["valid_tokens"] = np.float64(metrics["effective_weight"]), metrics["valid_tokens"]
        for name, parameter in model.named_parameters():
            if parameter.requires_grad:
                key = name.replace(".", "__")
                record["g__" + key] = parameter.grad.float().numpy().copy()
                record["u__" + key] = parameter.detach().float().numpy().copy()
        path = os.path.join(HERE, "step_tiny_bf16.npz" if bf16 else f"step_tiny_b{variant}.npz")
        np.savez_compressed(path, **record)
        print(path, os.path.getsize(path) // 1024, "KiB", "loss", metrics["loss"], "norm", metrics["grad_norm"])


if __name__ == "__main__":
    main()
