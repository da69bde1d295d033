"""The one-tower projector of the headline training step: ``Linear(in, mid) -> GELU -> Linear(mid, out)`` in bfloat16
with Xavier-uniform weights and zero biases. Its matrix products are plain library GEMMs (torch / cuBLAS); the
hand-written kernels of this library live in the loss and the collectives.

The reference has no model (README.md:83-84 of the reference lists PyTorch only as a baseline); this is the tower the
training benchmark puts in front of the loss.
"""
from __future__ import annotations

import torch
from torch import nn


class Projector(nn.Module):
    def __init__(self, in_features: int = 1024, mid_features: int = 3072, out_features: int = 768,
                 dtype: torch.dtype = torch.bfloat16, device=None, seed: int = 0) -> None:
        super().__init__()
        self.fc1 = nn.Linear(in_features, mid_features, dtype=dtype, device=device)
        self.act = nn.GELU()
        self.fc2 = nn.Linear(mid_features, out_features, dtype=dtype, device=device)
        generator = torch.Generator(device="cpu").manual_seed(seed)
        with torch.no_grad():
            for layer in (self.fc1, self.fc2):
                weight = torch.empty(layer.weight.shape, dtype=torch.float32)
                nn.init.xavier_uniform_(weight, generator=generator)
                layer.weight.copy_(weight.to(dtype))
                layer.bias.zero_()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.fc2(self.act(self.fc1(x)))

    def flops_per_row(self) -> int:
        """Multiply-add flops of forward plus backward per input row (three GEMM passes per layer)."""
        return 6 * (self.fc1.in_features * self.fc1.out_features + self.fc2.in_features * self.fc2.out_features)
