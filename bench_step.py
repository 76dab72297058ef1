"""Training-step workloads of bench.py: one optimizer update of an NF4 + rank-256 LoRA MQA decoder.

step7b (BASELINE.json configs[4]): 32 layers, hidden 4096, 32 query heads + 1 KV head, head_dim 128,
SwiGLU MLP 14336, vocab 49152, RoPE theta 1e6; per-GPU batch of 4 packed rows of 4096 tokens.
step1b (configs[3]): 24 layers, hidden 2048, 16 heads, head_dim 128, MLP 8192; 8 rows of 4096 per GPU.
Random-init frozen base packed to NF4 (64-element blocks, fp32 absmax), fp32 adapters, gradients
and Adam state, bf16 compute, FlashAttention-2 for attention (kept as the reference has it), token
ids uniform over the vocabulary, document lengths log-uniform in [64, 4096] laid end to end.
"""

import math
import os
import time

import torch

WORKLOADS = {
    "step7b": dict(config=dict(hidden_size=4096, intermediate_size=14336, vocab_size=49152, num_hidden_layers=32,
                               num_attention_heads=32, head_dim=128, rope_theta=1e6),
                   rows=4, length=4096, reference="BASELINE.json configs[4]"),
    "step1b": dict(config=dict(hidden_size=2048, intermediate_size=8192, vocab_size=49152, num_hidden_layers=24,
                               num_attention_heads=16, head_dim=128, rope_theta=1e6),
                   rows=8, length=4096, reference="BASELINE.json configs[3]"),
}
RANK = 256
CPU_SAMPLE_TOKENS = 512


def step_flops(config, tokens, rank=RANK):
    """Algorithmic FLOP of one update: sum over the seven projections of 4TKN + 6TKr + 6TNr per layer,
    plus the frozen head (logits and hidden gradient, 4THV). Attention is not counted."""
    h, i, d, v = config["hidden_size"], config["intermediate_size"], config["head_dim"], config["vocab_size"]
    shapes = [(h, h), (h, d), (h, d), (h, h), (h, i), (h, i), (i, h)]
    per_token = sum(4 * k * n + 6 * k * rank + 6 * n * rank for k, n in shapes)
    return config["num_hidden_layers"] * per_token * tokens + 4 * tokens * h * v


def synthetic_batch(rows, length, vocab, seed):
    """Packed rows: ids uniform over the vocabulary, documents of log-uniform length in [64, 4096]."""
    generator = torch.Generator().manual_seed(seed)
    ids = torch.randint(0, vocab, (rows, length), generator=generator)
    segments = torch.zeros(rows, length, dtype=torch.long)
    low, high = math.log(64), math.log(4096)
    for row in range(rows):
        cursor, index = 0, 1
        while cursor < length:
            size = int(math.exp(low + (high - low) * float(torch.rand((), generator=generator))))
            segments[row, cursor:cursor + size] = index
            cursor += size
            index += 1
    return {"input_ids": ids, "attention_mask": torch.ones_like(ids), "segment_ids": segments}


def build_model(name, device, mlp_cache_gib=0, keep_low_rank=False):
    from causal_tuner_b200.modeling.config import ModelConfig
    from causal_tuner_b200.modeling.model import CausalLM, Runtime
    spec = WORKLOADS[name]
    torch.manual_seed(2024)   # identical replica on every rank
    runtime = Runtime(rank=RANK, checkpoint=False, attention="flash_attention_2",
                      mlp_cache_budget_bytes=int(mlp_cache_gib * 2**30) or None, keep_low_rank=keep_low_rank)
    model = CausalLM(ModelConfig(**spec["config"]), runtime, device)
    with torch.no_grad():
        model.model.embed_tokens.weight.normal_(std=.02)
        model.lm_head.weight.normal_(std=.02)
        for parameter_name, parameter in model.named_parameters():
            if parameter_name.endswith("lora_B"):
                parameter.normal_(std=.01)   # non-zero so that gradients reach lora_A
    model.install_nf4(blocksize=64, nested=False)
    return model


# ---- CPU leg: the unmodified reference (oracle/_ref) on its own CPU branch ---------------------------
class ReferenceCpuStep:
    """The reference's `CausalLM` + `Trainer.update` (training/engine.py:41-111), installed unmodified in
    oracle/_ref, on the host cores: the workload's full architecture (all layers, head, AdamW over every
    adapter), its non-CUDA branch (dense bf16 base weights because its NF4 path refuses non-CUDA devices,
    modeling/lora.py:44-45; "vanilla" attention, kernels/reference.py:19-27, which caps a call at
    batch x heads x length^2 <= 2^23 scores). A step is one whole optimizer update on ONE packed row of
    CPU_SAMPLE_TOKENS tokens - a bounded sample of the workload's rows; per-token cost is what scales."""

    def __init__(self, name, threads):
        from oracle import ref_bridge
        ref_bridge.load()
        from causal_tuner.modeling.config import ModelConfig
        from causal_tuner.modeling.model import CausalLM, Runtime
        torch.set_num_threads(threads)
        self.spec = WORKLOADS[name]
        config = ModelConfig(pad_token_id=0, eos_token_id=1, **self.spec["config"])
        runtime = Runtime(rank=RANK, attention="vanilla", checkpoint=False)
        torch.manual_seed(2024)
        started = time.perf_counter()
        # Built on the meta device and filled from one random block per parameter: drawing 7e9 normal
        # samples on the host would take minutes and the timed arithmetic does not depend on the values.
        self.model = CausalLM(config, runtime, "meta").to_empty(device="cpu")
        block = torch.randn(1 << 20)
        with torch.no_grad():
            for parameter_name, parameter in self.model.named_parameters():
                scale = 1.0 if "norm" in parameter_name else (.01 if parameter_name.endswith("lora_B") else .02)
                flat = parameter.view(-1)
                source = (block * scale).to(parameter.dtype)
                if "norm" in parameter_name:
                    source = source.abs() + .5
                for start in range(0, flat.numel(), source.numel()):
                    stop = min(start + source.numel(), flat.numel())
                    flat[start:stop] = source[:stop - start]
        self.build_seconds = time.perf_counter() - started
        self.trainer = ref_bridge.reference_trainer(self.model, "cpu", loss_token_budget=128)
        self.updates = 0
        self.resize(CPU_SAMPLE_TOKENS)

    def resize(self, tokens):
        """Use one packed row of `tokens` tokens per update (a slow host gets a smaller sample)."""
        self.tokens = tokens
        self.batch = synthetic_batch(1, tokens, self.spec["config"]["vocab_size"], seed=1000)

    def step(self):
        metrics = self.trainer.update([dict(self.batch)], step=self.updates, total_steps=1 << 20)
        self.updates += 1
        return metrics

    def sample_text(self, steps):
        c = self.spec["config"]
        return (f"{steps} whole optimizer updates of the reference's own CausalLM/Trainer (oracle/_ref, unmodified) on the host "
                f"cores: all {c['num_hidden_layers']} layers + head + AdamW, bf16 compute with dense base weights and "
                f"'vanilla' attention (its non-CUDA branch), one packed row of {self.tokens} of the workload's "
                f"{self.spec['rows'] * self.spec['length']} tokens per update (so AdamW's per-update cost is spread over "
                f"{self.tokens} tokens instead of {self.spec['rows'] * self.spec['length']}); model built in "
                f"{self.build_seconds:.0f} s")


def reference_cpu_available():
    from oracle import ref_bridge
    return ref_bridge.available()


# ---- CPU leg when oracle/_ref is absent: the oracle's restatement on a bounded sample -------------------
class CpuLayerSample:
    """One decoder layer and the head of the workload on CPU_SAMPLE_TOKENS tokens, forward and backward
    through oracle/model.py (the restatement of the reference's CPU branch). A whole step costs
    `layers` times the layer plus the head; tokens/s is scaled accordingly."""

    def __init__(self, name, threads):
        from oracle import model as oracle_model
        torch.set_num_threads(threads)
        self.oracle, self.spec = oracle_model, WORKLOADS[name]
        c = self.spec["config"]
        generator = torch.Generator().manual_seed(99)
        h, i, d = c["hidden_size"], c["intermediate_size"], c["head_dim"]
        shapes = {"self_attn.q_proj": (h, h, True), "self_attn.k_proj": (d, h, True), "self_attn.v_proj": (d, h, True),
                  "self_attn.o_proj": (h, h, False), "mlp.gate_proj": (i, h, False), "mlp.up_proj": (i, h, False),
                  "mlp.down_proj": (h, i, False)}
        dtype = torch.bfloat16
        params = {"L.input_layernorm.weight": torch.ones(h, dtype=dtype),
                  "L.post_attention_layernorm.weight": torch.ones(h, dtype=dtype)}
        for key, (outer, inner, bias) in shapes.items():
            params[f"L.{key}.weight"] = (torch.randn(outer, inner, generator=generator) * .02).to(dtype)
            params[f"L.{key}.lora_A"] = (torch.randn(RANK, inner, generator=generator) * .02).requires_grad_(True)
            params[f"L.{key}.lora_B"] = (torch.randn(outer, RANK, generator=generator) * .01).requires_grad_(True)
            if bias:
                params[f"L.{key}.bias"] = torch.zeros(outer, dtype=dtype)
        self.params, self.dtype = params, dtype
        self.head = (torch.randn(c["vocab_size"], h, generator=generator) * .02).to(dtype)
        self.x = torch.randn(1, CPU_SAMPLE_TOKENS, h, generator=generator).to(dtype).requires_grad_(True)
        self.segments = torch.ones(1, CPU_SAMPLE_TOKENS, dtype=torch.int32)
        self.segments[:, CPU_SAMPLE_TOKENS // 2:] = 2
        half = int(d * 0.5) // 2
        angle = torch.arange(CPU_SAMPLE_TOKENS).float()[None, :, None] * torch.rand(half)
        self.cosine, self.sine = angle.cos().to(dtype), angle.sin().to(dtype)
        self.targets = torch.randint(0, c["vocab_size"], (CPU_SAMPLE_TOKENS,), generator=generator)
        self.trainable = [p for p in params.values() if p.requires_grad]

    def layer_seconds(self):
        c = self.spec["config"]
        start = time.perf_counter()
        y = self.oracle.layer(self.params, "L", self.x, self.cosine, self.sine, self.segments, c["num_attention_heads"],
                              c["head_dim"], 1e-6, self.dtype)
        torch.autograd.grad(y, (self.x, *self.trainable), torch.ones_like(y))
        return time.perf_counter() - start

    def head_seconds(self):
        start = time.perf_counter()
        hidden = self.x.detach().flatten(0, 1).requires_grad_(True)
        logits = torch.nn.functional.linear(hidden, self.head).float()
        loss = torch.nn.functional.cross_entropy(logits, self.targets, reduction="sum")
        torch.autograd.grad(loss, hidden)
        return time.perf_counter() - start

    def tokens_per_second(self, passes):
        self.layer_seconds()   # warm-up
        layer = min(self.layer_seconds() for _ in range(passes))
        head = min(self.head_seconds() for _ in range(max(1, passes)))
        layers = self.spec["config"]["num_hidden_layers"]
        return CPU_SAMPLE_TOKENS / (layers * layer + head), layer, head


def cpu_estimate(name, passes=3):
    threads = os.cpu_count() or 1
    sample = CpuLayerSample(name, threads)
    rate, layer, head = sample.tokens_per_second(passes)
    layers = WORKLOADS[name]["config"]["num_hidden_layers"]
    text = (f"one decoder layer ({layer:.2f} s) and the head ({head:.2f} s) of the workload, forward+backward on "
            f"{CPU_SAMPLE_TOKENS} tokens in bf16, best of {passes}; a step costs {layers} layers + head, so tokens/s = "
            f"{CPU_SAMPLE_TOKENS} / ({layers} x layer + head); oracle/model.py restating the reference CPU branch "
            f"(modeling/model.py:150-156, modeling/lora.py:29-39)")
    return {"value": rate, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": text}
