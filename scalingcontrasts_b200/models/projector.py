"""The one-tower projector of the headline training step: ``Linear(in, mid) -> GELU -> Linear(mid, out)`` in bfloat16
with Xavier-uniform weights and zero biases.

Its matrix products are plain library GEMMs (torch / cuBLAS, biases folded into the forward GEMMs' epilogues). What sits
between them is this library's own (``csrc/tower.cu``): on a GPU the module runs as one autograd function whose
activation is a single vectorised pass, and whose backward computes ``dz = dh * gelu'(z)`` and the first layer's bias
gradient in one pass over the activations and the second layer's bias gradient in one pass over the incoming gradient,
both summed in a fixed order (the step stays bit-reproducible). On CPU tensors, in other dtypes or without the
extension it is the plain ``nn`` composition.

The reference has no model (README.md:83-84 of the reference lists PyTorch only as a baseline); this is the tower the
training benchmark puts in front of the loss.
"""
from __future__ import annotations

import torch
from torch import nn


class _FusedTower(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight1, bias1, weight2, bias2, landing):
        from .._ext import native

        ctx.landing = landing
        ext, stream = native(), torch.cuda.current_stream().cuda_stream
        z = torch.addmm(bias1, x, weight1.t())
        h = torch.empty_like(z)
        ext.gelu_forward(z.data_ptr(), h.data_ptr(), z.numel(), torch.cuda.get_device_properties(x.device).multi_processor_count,
                         stream)
        y = torch.addmm(bias2, h, weight2.t())
        ctx.save_for_backward(x, weight1, weight2, z, h)
        return y

    @staticmethod
    def backward(ctx, dy):
        from .._ext import native

        x, weight1, weight2, z, h = ctx.saved_tensors
        ext, stream = native(), torch.cuda.current_stream().cuda_stream
        dy = dy.contiguous()
        rows, mid, out = x.shape[0], weight1.shape[0], weight2.shape[0]
        partials = torch.empty(int(ext.tower_partial_blocks(rows)) * max(mid, out), dtype=torch.float32, device=x.device)

        def landing(name, shape):
            # Where a parameter's gradient should be produced: a fresh alias of the buffer a gradient reducer named (so
            # that autograd adopts it as `.grad` and nothing is copied afterwards), or new memory.
            target = None if ctx.landing is None else ctx.landing.get(name)
            if target is not None and tuple(target.shape) == tuple(shape) and target.dtype == dy.dtype:
                return target.view(target.shape)
            return torch.empty(shape, dtype=dy.dtype, device=x.device)

        dbias2 = landing("fc2.bias", (out,))
        ext.column_sums(dy.data_ptr(), partials.data_ptr(), dbias2.data_ptr(), rows, out, stream)
        dweight2 = torch.mm(dy.t(), h, out=landing("fc2.weight", (out, mid)))
        dh = dy @ weight2
        dbias1 = landing("fc1.bias", (mid,))
        ext.gelu_backward_bias(dh.data_ptr(), z.data_ptr(), dh.data_ptr(), partials.data_ptr(), dbias1.data_ptr(), rows, mid, stream)
        dweight1 = torch.mm(dh.t(), x, out=landing("fc1.weight", (mid, x.shape[1])))  # dh now holds dz (written in place)
        dx = dh @ weight1 if ctx.needs_input_grad[0] else None
        return dx, dweight1, dbias1, dweight2, dbias2, None


class Projector(nn.Module):
    def __init__(self, in_features: int = 1024, mid_features: int = 3072, out_features: int = 768,
                 dtype: torch.dtype = torch.bfloat16, device=None, seed: int = 0, fused: bool = True) -> None:
        super().__init__()
        self.fc1 = nn.Linear(in_features, mid_features, dtype=dtype, device=device)
        self.act = nn.GELU()
        self.fc2 = nn.Linear(mid_features, out_features, dtype=dtype, device=device)
        self.fused = fused
        # Optional: parameter name -> buffer in which that parameter's gradient should be produced (a gradient reducer's
        # bucket slots, see GradientReducer.landing_buffers); used by the fused path only.
        self.gradient_landing = None
        generator = torch.Generator(device="cpu").manual_seed(seed)
        with torch.no_grad():
            for layer in (self.fc1, self.fc2):
                weight = torch.empty(layer.weight.shape, dtype=torch.float32)
                nn.init.xavier_uniform_(weight, generator=generator)
                layer.weight.copy_(weight.to(dtype))
                layer.bias.zero_()

    def _can_fuse(self, x: torch.Tensor) -> bool:
        if not (self.fused and x.is_cuda and x.dim() == 2 and x.dtype == torch.bfloat16 and x.is_contiguous()):
            return False
        if self.fc1.weight.dtype != torch.bfloat16 or self.fc1.out_features % 8 or self.fc2.out_features % 8:
            return False
        from .._ext import available

        return available()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self._can_fuse(x):
            return _FusedTower.apply(x, self.fc1.weight, self.fc1.bias, self.fc2.weight, self.fc2.bias, self.gradient_landing)
        return self.fc2(self.act(self.fc1(x)))

    def flops_per_row(self) -> int:
        """Multiply-add flops of forward plus backward per input row (three GEMM passes per layer)."""
        return 6 * (self.fc1.in_features * self.fc1.out_features + self.fc2.in_features * self.fc2.out_features)
