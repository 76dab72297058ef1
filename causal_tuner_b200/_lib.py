"""ctypes binding of libct_b200.so (the C ABI declared in include/ct_b200.h)."""

import ctypes
import os
import threading

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIBRARY_PATH = os.path.join(_HERE, "libct_b200.so")

F32, BF16, F16 = 0, 1, 2
PATH_AUTO, PATH_SIMT, PATH_TCGEN05 = 0, 1, 2
OK, ERR_ARG, ERR_UNSUPPORTED, ERR_CUDA, ERR_DEVICE = 0, -1, -2, -3, -4

_DTYPES = {torch.float32: F32, torch.bfloat16: BF16, torch.float16: F16}

_P, _I, _L, _F = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_float

# name -> (restype, argtypes); one entry per declaration in include/ct_b200.h
SIGNATURES = {
    "ct_abi_version": (_I, []),
    "ct_launch_count": (_L, []),
    "ct_tcgen05_launch_count": (_L, []),
    "ct_check_device": (_I, [_P]),
    "ct_selftest_bounded_wait": (_I, [_L, _P]),
    "ct_last_error": (ctypes.c_char_p, []),
    "ct_timing_enable": (_I, [_I]),
    "ct_timing_collect": (_I, [_P, _P, _P]),
    "ct_nf4_decode": (_I, [_P, _P, _P, _P, _P, _P, _P, _L, _I, _I, _I, _I, _I, _P]),
    "ct_nf4_decode_transposed": (_I, [_P, _P, _P, _P, _P, _P, _P, _L, _L, _L, _I, _I, _I, _I, _I, _P]),
    "ct_nf4_decode_chunks": (_I, [_P, _P, _P, _P, _P, _P, _P, _L, _I, _I, _I, _I, _I, _L, _L, _P]),
    "ct_cast": (_I, [_P, _I, _L, _P, _I, _L, _L, _L, _P]),
    "ct_matmul": (_I, [_P, _L, _L, _P, _L, _L, _P, _L, _L, _L, _L, _I, _I, _I, _I, _P]),
    "ct_matmul_nf4": (_I, [_P, _L, _P, _P, _P, _P, _L, _L, _L, _L, _I, _I, _P]),
    "ct_gated_forward": (_I, [_P, _L, _P, _L, _P, _P, _L, _P, _P, _P, _P, _P, _L, _L, _L, _L, _L, _L, _I, _P]),
    "ct_gated_backward": (_I, [_P, _L, _P, _L, _P, _P, _L, _P, _P, _P, _P, _P, _P, _L, _L, _L, _L, _L, _L, _I, _P]),
    "ct_gated_input_gradient": (_I, [_P, _P, _L, _P, _L, _P, _P, _L, _P, _P, _P, _L, _L, _L, _L, _L, _L, _I, _I, _P]),
    "ct_input_gradient_swiglu": (_I, [_P, _L, _P, _L, _P, _P, _L, _P, _P, _L, _P, _P, _P, _L, _L, _L, _L, _L, _I, _P]),
    "ct_forward_linear": (_I, [_P, _L, _P, _L, _P, _P, _P, _P, _L, _P, _L, _P, _L, _L, _L, _L, _L, _I, _I, _P]),
    "ct_input_gradient": (_I, [_P, _L, _P, _L, _L, _P, _P, _P, _L, _P, _L, _L, _L, _L, _L, _I, _I, _I, _P]),
    "ct_input_gradient_group": (_I, [_I, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _L, _P, _P, _L, _L, _I, _I, _I, _P]),
    "ct_parameter_gradients_workspace": (_L, [_L, _L, _L, _L, _I, _I]),
    "ct_parameter_gradients": (_I, [_P, _L, _P, _L, _P, _L, _P, _L, _P, _P, _L, _L, _L, _L, _I, _I, _P, _I, _P]),
    "ct_parameter_gradients_noalloc_capacity": (_L, []),
    "ct_parameter_gradients_noalloc": (_I, [_P, _L, _P, _L, _P, _L, _P, _L, _P, _P, _L, _L, _L, _L, _I, _I, _I, _P]),
    "ct_swiglu": (_I, [_P, _P, _P, _P, _P, _P, _L, _I, _I, _P]),
    "ct_rope": (_I, [_P, _P, _P, _P, _L, _I, _I, _I, _I, _I, _P]),
    "ct_accumulate_workspace": (_L, [_L, _L, _L, _I, _I]),
    "ct_accumulate": (_I, [_P, _L, _P, _L, _P, _L, _L, _L, _I, _I, _P, _I, _P]),
    "ct_token_gradients_group_workspace": (_L, [_I, _P, _P, _L, _I, _I]),
    "ct_token_gradients_group": (_I, [_I, _P, _P, _P, _P, _P, _P, _P, _L, _P, _I, _P, _I, _P]),
    "ct_cast_many": (_I, [_I, _P, _P, _P, _I, _I, _P]),
    "ct_position_values": (_I, [_P, _P, _P, _P, _L, _I, _I, _P]),
    "ct_add_inplace": (_I, [_P, _P, _L, _I, _P]),
    "ct_rmsnorm_forward": (_I, [_P, _P, _P, _P, _L, _L, ctypes.c_float, _I, _I, _P]),
    "ct_rmsnorm_backward": (_I, [_P, _P, _P, _P, _P, _L, _L, _I, _I, _P]),
    "ct_rmsnorm_backward_add": (_I, [_P, _P, _P, _P, _P, _P, _L, _L, _I, _I, _P]),
    "ct_rmsnorm_backward_from_output": (_I, [_P, _P, _P, _P, _P, _P, _L, _L, _I, _I, _P]),
    "ct_rmsnorm_weight_gradient": (_I, [_P, _P, _P, _P, _P, _P, _L, _L, _L, _I, _I, _P]),
    "ct_rmsnorm_weight_reduce": (_I, [_P, _L, _L, _P, _I, _P]),
    "ct_weighted_ce": (_I, [_P, _P, _P, _P, _L, _L, _I, _I, _P]),
    "ct_nf4_encode": (_I, [_P, _L, _I, _I, _P, _P, _P, _P]),
    "ct_nf4_nest": (_I, [_P, _L, _I, _P, _P, _P, _P, _P]),
    "ct_grad_norm_workspace": (_L, [_I]),
    "ct_grad_norm": (_I, [_I, _P, _P, _P, _F, _P, _P, _P]),
    "ct_adamw_update": (_I, [_I, _P, _P, _P, _P, _P, _P, _P, _P, _F, _F, _F, _F, _L, _I, _P]),
}


class LibraryMissing(RuntimeError):
    """libct_b200.so has not been built; there is no other implementation to fall back to."""


_lock = threading.Lock()
_library = None
# GEMM path used by the operators: PATH_AUTO in production; tests pin PATH_SIMT / PATH_TCGEN05.
gemm_path = PATH_AUTO


def load():
    """Load the shared library once and attach the prototypes."""
    global _library
    if _library is not None:
        return _library
    with _lock:
        if _library is None:
            if not os.path.exists(LIBRARY_PATH):
                raise LibraryMissing(
                    f"{LIBRARY_PATH} is missing. Build it with `python -m causal_tuner_b200.build` "
                    "(needs nvcc); the operators have no CPU or PyTorch fallback.")
            library = ctypes.CDLL(LIBRARY_PATH)
            for name, (restype, argtypes) in SIGNATURES.items():
                function = getattr(library, name)
                function.restype, function.argtypes = restype, argtypes
            _library = library
    return _library


def check(code):
    if code != OK:
        message = load().ct_last_error().decode(errors="replace")
        kind = {ERR_ARG: ValueError, ERR_UNSUPPORTED: NotImplementedError}.get(code, RuntimeError)
        raise kind(f"libct_b200 error {code}: {message}")


def code_of(dtype):
    try:
        return _DTYPES[dtype]
    except KeyError:
        raise TypeError(f"libct_b200 supports float32, bfloat16 and float16 tensors, not {dtype}") from None


def pointer(tensor):
    return None if tensor is None else tensor.data_ptr()


def require_cuda(*tensors):
    for tensor in tensors:
        if tensor is not None and not tensor.is_cuda:
            raise RuntimeError("causal_tuner_b200 operators run on CUDA tensors only; there is no CPU path")


def stream_of(tensor):
    """Raw handle of the current stream of the tensor's device."""
    return torch.cuda.current_stream(tensor.device).cuda_stream


class on_device:
    """Make the tensor's device current for the duration of a launch (no-op when it already is)."""

    def __init__(self, tensor):
        self.index = tensor.device.index
        self.guard = None

    def __enter__(self):
        if self.index is not None and self.index != torch.cuda.current_device():
            self.guard = torch.cuda.device(self.index)
            self.guard.__enter__()
        return self

    def __exit__(self, *exc):
        if self.guard is not None:
            self.guard.__exit__(*exc)
        return False


def check_device(tensor=None):
    """Synchronise and raise if a kernel reported a bounded-wait timeout or CUDA reports an error."""
    stream = torch.cuda.current_stream().cuda_stream if tensor is None else stream_of(tensor)
    check(load().ct_check_device(stream))


def launch_count():
    return int(load().ct_launch_count())


def tcgen05_launch_count():
    return int(load().ct_tcgen05_launch_count())


def timing_enable(on=True):
    """Start (or stop) recording CUDA-event times of every tcgen05 GEMM launch."""
    check(load().ct_timing_enable(int(bool(on))))


def timing_collect():
    """(total device ms, total algorithmic FLOP, launches) of the tcgen05 GEMM since timing_enable."""
    ms, flops, count = ctypes.c_double(), ctypes.c_double(), ctypes.c_int64()
    check(load().ct_timing_collect(ctypes.byref(ms), ctypes.byref(flops), ctypes.byref(count)))
    return ms.value, flops.value, count.value
