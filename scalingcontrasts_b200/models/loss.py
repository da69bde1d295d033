"""``MatryoshkaSigmoidLoss``: the streamed loss as a torch module with learnable temperature and bias.

``logit_scale`` (the log of the logit scale, initialised to log 10) and ``logit_bias`` (initialised to -10) are 0-d
parameters under the names open_clip's SigLIP models use, so a checkpoint's ``state_dict`` keeps that layout. The
forward pass runs the whole box step (publish, barrier, streamed scoring of every peer's block, summands all-reduce)
and already holds the embedding gradient when it returns; ``backward`` only scales it by the incoming gradient. The two
scalar gradients come from the all-reduced summands, so they are identical on every rank and need no further reduction;
the embedding gradient is final per row. Gradients of upstream parameters must therefore be summed across ranks, not
averaged.

On CPU tensors the module evaluates the same loss with ``CpuStreamedLoss`` over a gloo group or a single process.

The reference has no module, optimizer or autograd (its torch baseline hard-codes 10 and -10, baseline_torch.py:73-74);
this is the framework layer around its ``StreamedLoss`` contract (scalingcontrasts.cuh:1179-1197).
"""
from __future__ import annotations

import math
from typing import Optional

import torch
from torch import nn

from ..config import DEFAULT_BETA, DEFAULT_BIAS, LossSpec, REFERENCE_SPEC, SUMMAND_SLOTS
from ..ladder import Matryoshka


class _DeviceLoss(torch.autograd.Function):
    @staticmethod
    def forward(ctx, embeddings, logit_scale, logit_bias, module):
        engine = module.engine
        scalars = module._scalars
        scalars[0] = logit_scale.detach().float().exp()
        scalars[1] = logit_bias.detach().float()
        source = embeddings.detach()
        if source.dtype != torch.bfloat16:
            source = source.to(torch.bfloat16)
        source = source.contiguous()
        gradient, summands = engine.step(source, scalars=scalars)
        kept = summands.clone()  # the payload is rewritten by the next step
        ctx.save_for_backward(gradient, kept)
        ctx.input_dtype = embeddings.dtype
        ctx.unit_upstream = bool(module.unit_upstream)
        module.last_summands = kept
        return kept[0].clone()

    @staticmethod
    def backward(ctx, grad_output):
        gradient, summands = ctx.saved_tensors
        if ctx.unit_upstream:
            # The caller promised `loss.backward()` with nothing after the loss: the upstream gradient is one, and a pass
            # over the row gradients that multiplies them by it (25 MB in, 25 MB out per step) is left out.
            return gradient.to(ctx.input_dtype), summands[2], summands[1], None
        scaled = gradient * grad_output.to(gradient.dtype)
        return scaled.to(ctx.input_dtype), summands[2] * grad_output, summands[1] * grad_output, None


class _HostLoss(torch.autograd.Function):
    """CPU twin: every rank gathers the world's blocks over the group and streams them through the CPU loss."""

    @staticmethod
    def forward(ctx, embeddings, logit_scale, logit_bias, module):
        import torch.distributed as dist

        from ..cpu.streamed import CpuStreamedLoss

        block = embeddings.detach().contiguous()
        rows, hidden = block.shape
        distributed = dist.is_available() and dist.is_initialized()
        world = dist.get_world_size(module.group) if distributed else 1
        rank = dist.get_rank(module.group) if distributed else 0
        if world > 1:
            blocks = [torch.empty_like(block) for _ in range(world)]
            dist.all_gather(blocks, block, group=module.group)
        else:
            blocks = [block]
        beta, bias = float(logit_scale.detach().exp()), float(logit_bias.detach())
        precision = torch.float64 if block.dtype == torch.float64 else torch.float32
        loss = CpuStreamedLoss(rows, hidden, module.ladder, module.spec, precision)
        loss.begin(block)
        for p in range(world):
            peer = (rank + p) % world
            loss.score(block, blocks[peer], rank * rows, peer * rows, beta, bias, world * rows)
        gradient, summands = loss.finish(block, torch.empty(rows, hidden, dtype=precision),
                                         torch.zeros(SUMMAND_SLOTS, dtype=precision))
        if world > 1:
            dist.all_reduce(summands, op=dist.ReduceOp.SUM, group=module.group)
        ctx.save_for_backward(gradient, summands)
        ctx.input_dtype = embeddings.dtype
        module.last_summands = summands
        return summands[0].clone()

    @staticmethod
    def backward(ctx, grad_output):
        gradient, summands = ctx.saved_tensors
        return (gradient * grad_output).to(ctx.input_dtype), summands[2] * grad_output, summands[1] * grad_output, None


class MatryoshkaSigmoidLoss(nn.Module):
    """One-set sigmoid contrastive loss over Matryoshka prefixes, streamed across the GPUs of a box."""

    def __init__(self, rows: int, hidden: int, prefixes: int = 5, ladder: Optional[Matryoshka] = None,
                 spec: LossSpec = REFERENCE_SPEC, domain=None, group=None, device=None,
                 init_logit_scale: float = math.log(DEFAULT_BETA), init_logit_bias: float = DEFAULT_BIAS) -> None:
        super().__init__()
        self.rows, self.hidden = rows, hidden
        self.ladder = ladder if ladder is not None else Matryoshka.halvings(hidden, prefixes)
        self.spec, self.group, self.domain = spec, group, domain
        device = torch.device(device) if device is not None else (
            domain.device if domain is not None and hasattr(domain, "device") else torch.device("cpu"))
        self.logit_scale = nn.Parameter(torch.tensor(init_logit_scale, dtype=torch.float32, device=device))
        self.logit_bias = nn.Parameter(torch.tensor(init_logit_bias, dtype=torch.float32, device=device))
        self.last_summands: Optional[torch.Tensor] = None
        # Set by a caller that differentiates the loss itself with an upstream gradient of one (``loss.backward()``): the
        # GPU path then hands the row gradients on without scaling them. Anything that scales or combines the loss before
        # differentiating must leave it False.
        self.unit_upstream = False
        self.engine = None
        if device.type == "cuda":
            from ..parallel.box import BoxLoss

            device_domain = domain if domain is not None and hasattr(domain, "alloc") else None
            self.engine = BoxLoss(rows, hidden, self.ladder, spec, device_domain, device)
            self.register_buffer("_scalars", torch.zeros(2, dtype=torch.float32, device=device), persistent=False)

    def forward(self, embeddings: torch.Tensor) -> torch.Tensor:
        if tuple(embeddings.shape) != (self.rows, self.hidden):
            raise ValueError(f"embeddings must be [{self.rows}, {self.hidden}], got {tuple(embeddings.shape)}")
        if embeddings.is_cuda:
            if self.engine is None:
                raise RuntimeError("this module was built for the CPU; construct it with device='cuda'")
            return _DeviceLoss.apply(embeddings, self.logit_scale, self.logit_bias, self)
        return _HostLoss.apply(embeddings, self.logit_scale, self.logit_bias, self)

    def prefix_losses(self) -> Optional[torch.Tensor]:
        """Per-prefix losses of the last forward (world sums), narrowest first."""
        if self.last_summands is None:
            return None
        return self.last_summands[4:4 + self.ladder.count]

    def cells_per_step(self, world: int) -> int:
        """Cells this rank scores in one step: rows x world rows x prefixes."""
        return self.rows * self.rows * world * self.ladder.count

    def extra_repr(self) -> str:
        return f"rows={self.rows}, hidden={self.hidden}, ends={self.ladder.ends}, positives={self.spec.positives}"

