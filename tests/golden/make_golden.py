"""Generate the golden fixtures in this directory by running the REFERENCE's own code.

Run in a container where the reference checkout is importable:

    TRITON_INTERPRET=1 PYTHONPATH=<reference>/src python tests/golden/make_golden.py

* nf4_*.npz        - the reference's Triton kernel `_decode` (kernels/nf4_cuda.py:9-29) executed
                     by the Triton interpreter on CPU tensors, fp32 storage and fp32 output (the
                     interpreter's float->bf16 conversion truncates instead of rounding to nearest
                     even, so 16-bit outputs are not recorded);
* projection_*.npz - `Projection.forward` CPU branch (modeling/lora.py:29-39) + torch autograd;
* mlp_*.npz        - `MLP.untiled` CPU branch (modeling/model.py:127-131) + torch autograd;
* rope_*.npz       - `rotate` CPU branch (modeling/rotary.py:16-24), values and input gradient.

The fixtures are committed; nothing at test time imports the reference.
"""

import os
import sys

os.environ.setdefault("TRITON_INTERPRET", "1")

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))


def f32(t):
    return t.detach().float().contiguous().numpy()


def nf4_cases():
    import triton
    import triton.language as tl
    from causal_tuner.kernels import nf4_cuda
    from causal_tuner_b200.quant import quantize_nf4
    cases = [((71, 96), bs, nested) for bs in (64, 128, 4096) for nested in (False, True)]
    cases += [((17, 19), 64, False), ((17, 19), 64, True)]
    for index, (shape, blocksize, nested) in enumerate(cases):
        torch.manual_seed(100 + index)
        packed, state = quantize_nf4(torch.randn(*shape), blocksize=blocksize, nested=nested)
        n = shape[0] * shape[1]
        out = torch.empty(n, dtype=torch.float32)
        rows = max(1, 4096 // blocksize)
        auxiliary = state.state2 if nested else state
        # Same launch as dequantize_nf4 (kernels/nf4_cuda.py:38-42) minus the CUDA-only launch cache.
        nf4_cuda._decode[(triton.cdiv(n, rows * blocksize),)](
            packed.reshape(-1), state.absmax, state.code, auxiliary.code, auxiliary.absmax,
            state.offset if nested else state.absmax, out, N=n, GROUP=blocksize,
            SCALE_GROUP=auxiliary.blocksize, NESTED=nested, STORAGE_DTYPE=tl.float32, ROWS=rows)
        record = dict(packed=packed.reshape(-1).numpy(), absmax=state.absmax.numpy(), code=state.code.numpy(),
                      n=n, rows=shape[0], cols=shape[1], blocksize=blocksize, nested=int(nested), out=out.numpy())
        if nested:
            record.update(code2=auxiliary.code.numpy(), absmax2=auxiliary.absmax.numpy(),
                          offset=state.offset.numpy(), blocksize2=auxiliary.blocksize)
        np.savez_compressed(os.path.join(HERE, f"nf4_{shape[0]}x{shape[1]}_b{blocksize}_n{int(nested)}.npz"), **record)


def projection_cases():
    from causal_tuner.modeling.lora import Projection
    for name, dtype, (inputs, outputs, rank, bias, rows) in (
            ("fp32_small", torch.float32, (32, 24, 4, True, (2, 7))),
            ("fp32_odd", torch.float32, (68, 32, 5, False, (1, 13))),
            ("bf16_small", torch.bfloat16, (32, 24, 4, True, (2, 7))),
            ("bf16_wide", torch.bfloat16, (256, 192, 16, True, (3, 50)))):
        torch.manual_seed(7)
        module = Projection(inputs, outputs, bias=bias, rank=rank, base_dtype=dtype, compute_dtype=dtype, device="cpu")
        torch.nn.init.normal_(module.lora_B, std=.05)
        if bias:
            torch.nn.init.normal_(module.bias, std=.1)
        x = torch.randn(*rows, inputs, dtype=dtype, requires_grad=True)
        y = module(x)
        dy = torch.randn_like(y)
        dx, da, db = torch.autograd.grad(y, (x, module.lora_A, module.lora_B), dy)
        record = dict(x=f32(x), weight=f32(module.weight), a=f32(module.lora_A), b=f32(module.lora_B), dy=f32(dy),
                      y=f32(y), dx=f32(dx), da=f32(da), db=f32(db), bf16=int(dtype == torch.bfloat16))
        if bias:
            record["bias"] = f32(module.bias)
        np.savez_compressed(os.path.join(HERE, f"projection_{name}.npz"), **record)


def mlp_cases():
    from causal_tuner.modeling.config import ModelConfig
    from causal_tuner.modeling.model import MLP, Runtime
    for name, dtype in (("fp32", torch.float32), ("bf16", torch.bfloat16)):
        torch.manual_seed(11)
        module = MLP(ModelConfig.tiny(), Runtime(rank=4, base_dtype=dtype, compute_dtype=dtype), "cpu")
        for key, parameter in module.named_parameters():
            if "lora_B" in key:
                torch.nn.init.normal_(parameter, std=.1)
        x = torch.randn(2, 7, 32, dtype=dtype, requires_grad=True)
        y = module.untiled(x)
        dy = torch.randn_like(y)
        names = [n for n, p in module.named_parameters() if p.requires_grad]
        grads = torch.autograd.grad(y, (x, *(p for p in module.parameters() if p.requires_grad)), dy)
        record = dict(x=f32(x), dy=f32(dy), y=f32(y), dx=f32(grads[0]), bf16=int(dtype == torch.bfloat16))
        for key, parameter in module.named_parameters():
            record["p_" + key.replace(".", "_")] = f32(parameter)
        for key, grad in zip(names, grads[1:]):
            record["g_" + key.replace(".", "_")] = f32(grad)
        np.savez_compressed(os.path.join(HERE, f"mlp_{name}.npz"), **record)


def rope_cases():
    from causal_tuner.modeling.rotary import rotate
    for name, dtype, heads, head_dim, rotary_dim in (("fp32_h4_d8", torch.float32, 4, 8, 4),
                                                     ("bf16_h4_d8", torch.bfloat16, 4, 8, 4),
                                                     ("bf16_h3_d128", torch.bfloat16, 3, 128, 64)):
        torch.manual_seed(13)
        x = torch.randn(2, 7, heads, head_dim, dtype=dtype, requires_grad=True)
        angles = torch.arange(14).reshape(2, 7, 1) * 60000 * torch.rand(rotary_dim // 2)
        cosine, sine = angles.cos().to(dtype), angles.sin().to(dtype)
        y = rotate(x, cosine, sine)
        dy = torch.randn_like(y)
        dx, = torch.autograd.grad(y, x, dy)
        np.savez_compressed(os.path.join(HERE, f"rope_{name}.npz"), x=f32(x), cosine=f32(cosine), sine=f32(sine),
                            y=f32(y), dy=f32(dy), dx=f32(dx), bf16=int(dtype == torch.bfloat16))


if __name__ == "__main__":
    nf4_cases()
    projection_cases()
    mlp_cases()
    rope_cases()
    print(sorted(f for f in os.listdir(HERE) if f.endswith(".npz")))
