"""AdamW for the training benchmark, as one kernel launch per eight tensors (``csrc/optim.cu``).

``FusedAdamW`` has the four methods a training loop calls (``zero_grad``, ``step``, ``state_dict``, ``load_state_dict``)
and the update rule of ``torch.optim.AdamW`` (decoupled weight decay, bias-corrected moments). Unlike torch's fused form it
keeps both moments in float32 for bfloat16 parameters, and its checkpoints restore them bit for bit. Parameters must be
contiguous CUDA tensors in bfloat16 or float32 whose gradients have the same type.

The reference has no optimizer (it benchmarks a loss step only, scalingcontrasts.cu:294-311).
"""
from __future__ import annotations

from typing import Dict, Iterable, List, Tuple

import torch


class FusedAdamW:
    def __init__(self, params: Iterable[torch.Tensor], lr: float = 1e-3, betas: Tuple[float, float] = (0.9, 0.999),
                 eps: float = 1e-8, weight_decay: float = 1e-2) -> None:
        self.params: List[torch.Tensor] = list(params)
        if not self.params:
            raise ValueError("FusedAdamW needs at least one parameter")
        for p in self.params:
            if not p.is_cuda or p.dtype not in (torch.bfloat16, torch.float32) or not p.is_contiguous():
                raise ValueError("FusedAdamW takes contiguous CUDA parameters in bfloat16 or float32")
        if not (0.0 <= betas[0] < 1.0 and 0.0 <= betas[1] < 1.0) or lr < 0.0 or eps < 0.0 or weight_decay < 0.0:
            raise ValueError("FusedAdamW: lr, eps and weight_decay must not be negative and betas must lie in [0, 1)")
        self.lr, self.betas, self.eps, self.weight_decay = float(lr), (float(betas[0]), float(betas[1])), float(eps), float(weight_decay)
        self.steps = 0
        self.exp_avg = [torch.zeros(p.shape, dtype=torch.float32, device=p.device) for p in self.params]
        self.exp_avg_sq = [torch.zeros(p.shape, dtype=torch.float32, device=p.device) for p in self.params]
        # torch.optim-style view for code that reads or schedules the learning rate
        self.param_groups = [{"params": self.params, "lr": self.lr, "betas": self.betas, "eps": self.eps,
                              "weight_decay": self.weight_decay}]

    def zero_grad(self, set_to_none: bool = True) -> None:
        for p in self.params:
            if p.grad is None:
                continue
            if set_to_none:
                p.grad = None
            else:
                p.grad.detach_()
                p.grad.zero_()

    @torch.no_grad()
    def step(self) -> None:
        from ._ext import native

        group = self.param_groups[0]
        entries = []
        for p, m, v in zip(self.params, self.exp_avg, self.exp_avg_sq):
            g = p.grad
            if g is None:
                continue
            if g.dtype != p.dtype or g.device != p.device:
                raise ValueError("FusedAdamW: a gradient's type and device must match its parameter's")
            if not g.is_contiguous():
                g = g.contiguous()
            entries.append((p.data_ptr(), g.data_ptr(), m.data_ptr(), v.data_ptr(), p.numel(), p.dtype == torch.bfloat16, g))
        if not entries:
            return
        self.steps += 1
        stream = torch.cuda.current_stream(self.params[0].device).cuda_stream
        native().adamw_step([entry[:6] for entry in entries], float(group["lr"]), float(group["betas"][0]), float(group["betas"][1]),
                            float(group["eps"]), float(group["weight_decay"]), self.steps, stream)

    def state_dict(self) -> Dict[str, object]:
        group = self.param_groups[0]
        return {"steps": self.steps, "lr": group["lr"], "betas": tuple(group["betas"]), "eps": group["eps"],
                "weight_decay": group["weight_decay"], "exp_avg": [m.clone() for m in self.exp_avg],
                "exp_avg_sq": [v.clone() for v in self.exp_avg_sq]}

    def load_state_dict(self, state: Dict[str, object]) -> None:
        if len(state["exp_avg"]) != len(self.params) or len(state["exp_avg_sq"]) != len(self.params):
            raise ValueError("FusedAdamW: the checkpoint holds a different number of tensors")
        for mine, theirs in zip(self.exp_avg + self.exp_avg_sq, list(state["exp_avg"]) + list(state["exp_avg_sq"])):
            if tuple(mine.shape) != tuple(theirs.shape):
                raise ValueError("FusedAdamW: a moment's shape differs from its parameter's")
            mine.copy_(theirs.to(device=mine.device, dtype=torch.float32))
        self.steps = int(state["steps"])
        group = self.param_groups[0]
        group["lr"], group["betas"] = float(state["lr"]), (float(state["betas"][0]), float(state["betas"][1]))
        group["eps"], group["weight_decay"] = float(state["eps"]), float(state["weight_decay"])
