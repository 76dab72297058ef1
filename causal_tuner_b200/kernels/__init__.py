"""Operator layer: same module and function names as the reference's ``causal_tuner.kernels``."""
