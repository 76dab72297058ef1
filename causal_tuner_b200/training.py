"""One optimizer update over weighted micro-batches, with the data-parallel gradient exchange.

Follows the reference's training/engine.py:10-111 (`make_optimizer`, `Trainer.update`): per
micro-batch forward, tiled lm_head loss, backward; then gradients are divided by the total
supervision weight, clipped, and AdamW steps. The reference is single-device; with
torch.distributed initialised every rank runs its own micro-batches and, between the last
backward and the division (training/engine.py:90-97), the fp32 adapter gradients, the total
weight and the total loss are summed across ranks - which makes the update equal to
single-device accumulation over the concatenated batch (up to fp32 summation order).
"""

import torch
import torch.distributed as dist

from . import _lib
from .dp import BucketPlan, PlannedExchange
from .optim import FusedAdamW
from .kernels.loss import active_rows, projection_loss
from .segments import prediction_targets


def make_optimizer(model, *, learning_rate=2e-5, weight_decay=0.0, betas=(0.9, 0.999), eps=1e-8):
    """AdamW over the trainable parameters; weight decay on matrices only (training/engine.py:10-16).
    fp32 CUDA adapters get the optimizer whose step also scales and clips (optim.py)."""
    parameters = [p for p in model.parameters() if p.requires_grad]
    groups = [{"params": group, "weight_decay": weight_decay if decay else 0.0}
              for decay in (True, False) if (group := [p for p in parameters if (p.ndim > 1) == decay])]
    if FusedAdamW.supports(parameters):
        return FusedAdamW(groups, lr=learning_rate, betas=betas, eps=eps, weight_decay=weight_decay)
    return torch.optim.AdamW(groups, lr=learning_rate, betas=betas, eps=eps, weight_decay=weight_decay,
                             foreach=False, fused=all(p.is_cuda for p in parameters))


class Trainer:
    def __init__(self, model, optimizer, *, device, max_grad_norm=1.0, loss_token_budget=4096, group=None,
                 bucket_bytes=64 << 20):
        self.model, self.optimizer, self.device = model, optimizer, device
        self.max_grad_norm, self.loss_token_budget = max_grad_norm, loss_token_budget
        self.group, self.bucket_bytes = group, bucket_bytes
        self._plan = None

    def update(self, batches, *, learning_rate=None):
        self.model.train()
        self.optimizer.zero_grad(set_to_none=True)
        total_loss = torch.zeros((), device=self.device, dtype=torch.float32)
        total_weight = torch.zeros_like(total_loss)
        microbatches, valid_tokens = 0, 0
        batches = list(batches)
        parameters = [p for group in self.optimizer.param_groups for p in group["params"]]
        distributed = dist.is_available() and dist.is_initialized() and dist.get_world_size(self.group) > 1
        exchange, hooks, failure = None, [], None
        if distributed:
            shapes = [tuple(p.shape) for p in parameters]
            if self._plan is None or self._plan.shapes != shapes:
                self._plan = BucketPlan(shapes, self.device, self.bucket_bytes)
            position = {param: index for index, param in enumerate(parameters)}
        try:
            for index, batch in enumerate(batches):
                if distributed and index == len(batches) - 1:
                    # Last micro-batch: every gradient is final as soon as autograd has accumulated it, so it
                    # is copied into its bucket right away and complete buckets are all-reduced under the rest
                    # of the backward pass (a 16-bit gradient is widened by that copy and rounded once after).
                    exchange = PlannedExchange(self._plan, self.group)
                    hooks = [p.register_post_accumulate_grad_hook(
                        lambda param, exchange=exchange: exchange.add(position[param], param.grad)) for p in parameters]
                microbatches += 1
                valid_tokens += int(batch["attention_mask"].sum())
                targets, weights = prediction_targets(batch)
                rows = active_rows(weights, self.device)
                targets, weights = targets.to(self.device), weights.to(self.device)
                batch = {k: v.to(self.device) if torch.is_tensor(v) else v for k, v in batch.items()}
                hidden = self.model(batch)
                loss = projection_loss(hidden, self.model.lm_head.weight, targets, weights,
                                       token_budget=self.loss_token_budget,
                                       compute_dtype=self.model.runtime.compute_dtype,
                                       reuse_hidden=not self.model.model.norm.weight.requires_grad, rows=rows)
                del hidden
                loss.backward()
                total_loss.add_(loss.detach())
                total_weight.add_(weights.sum())
                del loss, batch
            if microbatches == 0:
                raise ValueError("An optimizer update requires at least one microbatch")
            for param in parameters:
                if param.grad is None:
                    raise RuntimeError("A trainable parameter has no gradient; the graph is disconnected")
        except Exception as error:      # told to the other ranks below, then raised again
            failure = error
        finally:
            for hook in hooks:          # never leave hooks behind: the next update builds its own exchange
                hook.remove()
        collectives = 0
        if distributed:
            # The loss, the weight and a failure flag travel in the last, small all-reduce. A rank whose
            # forward or backward raised still launches every bucket (contents irrelevant) so that the
            # collectives of its peers complete; every rank then sees the flag and raises before stepping.
            scalars = torch.stack((total_loss, total_weight, torch.full_like(total_loss, 0.0 if failure is None else 1.0)))
            if exchange is None:
                exchange = PlannedExchange(self._plan, self.group)
            if failure is not None:
                exchange.flush()
            summed = exchange.finish(scalars)
            collectives = exchange.collectives
            if failure is None and scalars[2].item() > 0:
                failure = RuntimeError("Another rank failed during this update; no optimizer step was taken")
            if failure is None:
                for param, value in zip(parameters, summed):
                    if param.grad.dtype == torch.float32:
                        param.grad = value            # a view of the persistent bucket: no copy back
                    else:
                        param.grad.copy_(value)
                total_loss, total_weight = scalars[0], scalars[1]
        if failure is not None:
            raise failure
        denominator = total_weight.clamp_min(1.0)
        if learning_rate is not None:
            for group in self.optimizer.param_groups:
                group["lr"] = learning_rate
        if (isinstance(self.optimizer, FusedAdamW) and FusedAdamW.supports(parameters)
                and all(p.grad.dtype == torch.float32 and p.grad.is_contiguous() for p in parameters)):
            # Divide, measure, clip and step in two passes over the gradients; the denominator stays on
            # the device. A non-finite norm steps nothing and is raised below, as the reference does
            # before its optimizer step.
            norm = self.optimizer.scale_clip_step(denominator, self.max_grad_norm or 0.0)[0]
            if not torch.isfinite(norm):
                self.optimizer.rollback()
                if self.max_grad_norm:
                    raise RuntimeError("The total norm of the gradients is non-finite, so it cannot be clipped")
                raise FloatingPointError("Non-finite gradient norm")
        else:
            # A Python scalar keeps the multi-tensor path (a tensor divisor is applied gradient by gradient).
            torch._foreach_div_([param.grad for param in parameters], float(denominator))
            if self.max_grad_norm:
                norm = torch.nn.utils.clip_grad_norm_(parameters, self.max_grad_norm, error_if_nonfinite=True,
                                                      foreach=all(p.is_cuda for p in parameters))
            else:
                norm = torch.sqrt(sum(p.grad.float().norm().square() for p in parameters))
                if not torch.isfinite(norm):
                    raise FloatingPointError("Non-finite gradient norm")
            self.optimizer.step()
        _lib.check_device()   # a kernel that gave up on a bounded wait must not pass as a finished step
        return {"loss": (total_loss / denominator).item(), "effective_weight": total_weight.item(),
                "grad_norm": norm.item(), "microbatches": microbatches, "valid_tokens": valid_tokens,
                "collectives": collectives}
