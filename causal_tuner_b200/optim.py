"""AdamW whose step also divides the gradients by the supervision weight and clips them.

The reference ends an update with four multi-tensor passes over the adapter gradients:
`torch._foreach_div_(grads, denominator)`, `clip_grad_norm_`, the clip multiply and the fused
`torch.optim.AdamW.step()` (training/engine.py:97-107). `FusedAdamW.scale_clip_step` does the
same arithmetic in two passes (`ct_grad_norm`, `ct_adamw_update`) and takes the denominator as a device
scalar, so the host does not wait for it. It is a `torch.optim.AdamW` in every other respect
(param_groups, state with `step` / `exp_avg` / `exp_avg_sq`, state_dict, zero_grad), and `step()`
without scaling or clipping is the same call with a divisor of one and no norm limit.
"""

import ctypes

import torch

from . import _lib


class FusedAdamW(torch.optim.AdamW):
    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=1e-2):
        super().__init__(params, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, foreach=False, fused=False)
        self._one = None
        self.last_norm = None

    @staticmethod
    def supports(parameters):
        """fp32 CUDA parameters on one device, each contiguous."""
        parameters = list(parameters)
        return bool(parameters) and all(
            p.is_cuda and p.dtype == torch.float32 and p.is_contiguous() and p.device == parameters[0].device
            for p in parameters)

    def _state_of(self, param):
        state = self.state[param]
        if not state:
            state["step"] = torch.zeros((), dtype=torch.float32)
            state["exp_avg"] = torch.zeros_like(param, memory_format=torch.preserve_format)
            state["exp_avg_sq"] = torch.zeros_like(param, memory_format=torch.preserve_format)
        return state

    @torch.no_grad()
    def scale_clip_step(self, divisor=None, max_norm=0.0, *, write_grads=True):
        """g /= divisor; clip to `max_norm` (0 = no limit); AdamW step. Returns a device tensor
        [norm of g / divisor, clip coefficient]. A non-finite norm leaves parameters, moments and
        gradients untouched; call `rollback()` after reading one to take back the step counters."""
        groups = [(group, [p for p in group["params"] if p.grad is not None]) for group in self.param_groups]
        parameters = [p for _, members in groups for p in members]
        self._stepped = []
        if not parameters:
            return torch.zeros(2)
        if not self.supports(parameters) or any(p.grad.dtype != torch.float32 or not p.grad.is_contiguous()
                                                for p in parameters):
            raise TypeError("FusedAdamW steps contiguous fp32 CUDA parameters and gradients on one device")
        device = parameters[0].device
        if divisor is None:
            if self._one is None or self._one.device != device:
                self._one = torch.ones((), device=device, dtype=torch.float32)
            divisor = self._one
        if divisor.device != device or divisor.dtype != torch.float32 or divisor.numel() != 1:
            raise TypeError("divisor must be one fp32 value on the parameters' device")
        library = _lib.load()
        norm = torch.empty(2, device=device, dtype=torch.float32)
        pointers = lambda tensors: (ctypes.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])
        extents = lambda tensors: (ctypes.c_int64 * len(tensors))(*[t.numel() for t in tensors])
        with _lib.on_device(parameters[0]):
            stream = _lib.stream_of(parameters[0])
            workspace = torch.empty(max(library.ct_grad_norm_workspace(len(parameters)), 4), device=device,
                                    dtype=torch.uint8)
            _lib.check(library.ct_grad_norm(len(parameters), pointers([p.grad for p in parameters]),
                                            extents(parameters), divisor.data_ptr(), float(max_norm),
                                            norm.data_ptr(), workspace.data_ptr(), stream))
            for group, members in groups:
                if not members:
                    continue
                if group.get("amsgrad") or group.get("maximize"):
                    raise NotImplementedError("FusedAdamW has no amsgrad / maximize variant")
                states = [self._state_of(p) for p in members]
                steps = {int(state["step"]) for state in states}
                if len(steps) != 1:
                    raise RuntimeError("parameters of one group must have taken the same number of steps")
                beta1, beta2 = group["betas"]
                decay = (ctypes.c_float * len(members))(*([float(group["weight_decay"])] * len(members)))
                _lib.check(library.ct_adamw_update(
                    len(members), pointers([p.grad for p in members]), pointers(members),
                    pointers([state["exp_avg"] for state in states]),
                    pointers([state["exp_avg_sq"] for state in states]), extents(members), decay,
                    divisor.data_ptr(), norm.data_ptr(), float(group["lr"]), float(beta1), float(beta2),
                    float(group["eps"]), steps.pop() + 1, int(bool(write_grads)), stream))
                for state in states:
                    state["step"] += 1
                self._stepped.extend(states)
        self.last_norm = norm
        return norm

    def rollback(self):
        """Undo the step counters of the last call (used when its norm turned out not to be finite)."""
        for state in getattr(self, "_stepped", []):
            state["step"] -= 1
        self._stepped = []

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        self.scale_clip_step(None, 0.0, write_grads=False)
        return loss
