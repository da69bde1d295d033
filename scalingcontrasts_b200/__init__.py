"""B200-native contrastive-training primitives: a streamed, row-owned, one-set Matryoshka sigmoid loss, NVSwitch
multimem collectives, an RDMA rail interface and the benchmark modes around them.

The public surface follows ashvardanian/ScalingContrasts (``Domain`` + ``StreamedLoss``, scalingcontrasts.mojo:36-41 of
its README) with a torch layer on top: ``MatryoshkaSigmoidLoss`` (an ``nn.Module`` over an ``autograd.Function``), a
projector model, a gradient reducer and a trainer.
"""
from .config import LossSpec, PAIRS_SPEC, REFERENCE_SPEC, Settings  # noqa: F401
from .ladder import Matryoshka  # noqa: F401

__version__ = "0.1.0"

_LAZY = {
    "Domain": ("scalingcontrasts_b200.parallel.domain", "Domain"),
    "PeerDomain": ("scalingcontrasts_b200.parallel.domain", "PeerDomain"),
    "MultimemDomain": ("scalingcontrasts_b200.parallel.domain", "MultimemDomain"),
    "HostDomain": ("scalingcontrasts_b200.parallel.domain", "HostDomain"),
    "StreamedLoss": ("scalingcontrasts_b200.ops.streamed_loss", "StreamedLoss"),
    "CpuStreamedLoss": ("scalingcontrasts_b200.cpu.streamed", "CpuStreamedLoss"),
    "MatryoshkaSigmoidLoss": ("scalingcontrasts_b200.models.loss", "MatryoshkaSigmoidLoss"),
    "Projector": ("scalingcontrasts_b200.models.projector", "Projector"),
    "GradientReducer": ("scalingcontrasts_b200.parallel.reducer", "GradientReducer"),
    "ContrastiveTrainer": ("scalingcontrasts_b200.trainer", "ContrastiveTrainer"),
    "FusedAdamW": ("scalingcontrasts_b200.optim", "FusedAdamW"),
    "RdmaRail": ("scalingcontrasts_b200.parallel.rail", "RdmaRail"),
}


def __getattr__(name):
    target = _LAZY.get(name)
    if target is None:
        raise AttributeError(name)
    import importlib

    return getattr(importlib.import_module(target[0]), target[1])
