"""B200-native (sm_100a) kernels behind causal-tuner's fused projection / SwiGLU-MLP operators.

The sub-packages mirror the reference's module layout for the hot path only:

* ``causal_tuner_b200.kernels.linear``   - ``project_group`` and its primitives
* ``causal_tuner_b200.kernels.mlp_cuda`` - ``tiled_lora_mlp`` and its primitives
* ``causal_tuner_b200.kernels.nf4_cuda`` - ``dequantize_nf4``
* ``causal_tuner_b200.kernels.core_cuda``- adjacent-pair RoPE used inside the projection op
* ``causal_tuner_b200.modeling``         - ``Projection``, ``MLP``, ``Runtime``

Every operator enqueues hand-written CUDA kernels from ``libct_b200.so`` through its
C ABI (``include/ct_b200.h``). There is no CPU path: importing works anywhere, calling
an operator needs a CUDA device and the built library.
"""

__version__ = "0.1.0"
