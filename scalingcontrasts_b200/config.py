"""Frozen configuration records shared by the CPU and GPU paths and by the command line.

``LossSpec`` states which cells are positives and how the diagonal is treated; ``Settings`` mirrors the reference
binary's flags (scalingcontrasts.cu:40-45, 580-603) and adds the ones a multi-process torch framework needs.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field, replace
from typing import Optional, Tuple

from .ladder import Matryoshka

COSINE_FLOOR = 1e-2  # a norm product at or below this reads as a zero cosine (scalingcontrasts.cuh:50-51)
INVERSE_COSINE_FLOOR = 1.0 / COSINE_FLOOR
DEFAULT_BETA = 10.0  # SigLIP's initial logit scale exp(t), t = log 10
DEFAULT_BIAS = -10.0  # SigLIP's initial logit bias
SUMMAND_SLOTS = 12  # loss, bias-grad, log-beta-grad, pad, then one loss per prefix (8 slots)

_POSITIVES = ("self", "pairs")
_DIAGONALS = ("own", "negative", "skip")


@dataclass(frozen=True)
class LossSpec:
    """Targets of the one-set sigmoid loss.

    ``positives="self"`` is the reference's rule: the only positive of row i is its own copy (i, i), whose cosine is
    taken as exactly one and which moves no embedding (scalingcontrasts.cuh:874-893).
    ``positives="pairs"`` makes global rows 2m and 2m+1 each other's positive; the partner cell carries a real cosine
    and a real gradient.

    ``diagonal`` says what cell (i, i) is: ``"own"`` a positive with cosine one, ``"negative"`` a negative with cosine
    one (the literal reading of "every other cell is a negative"), ``"skip"`` not a cell at all.
    """

    positives: str = "self"
    diagonal: Optional[str] = None

    def __post_init__(self) -> None:
        if self.positives not in _POSITIVES:
            raise ValueError(f"positives must be one of {_POSITIVES}, got {self.positives!r}")
        diagonal = self.diagonal
        if diagonal is None:
            diagonal = "own" if self.positives == "self" else "negative"
            object.__setattr__(self, "diagonal", diagonal)
        if diagonal not in _DIAGONALS:
            raise ValueError(f"diagonal must be one of {_DIAGONALS}, got {diagonal!r}")

    @property
    def pairs(self) -> bool:
        return self.positives == "pairs"

    def code(self) -> int:
        """The packed form the native kernels take: bit 0 pairs, bits 1-2 diagonal (0 own, 1 negative, 2 skip)."""
        return (1 if self.pairs else 0) | (_DIAGONALS.index(self.diagonal) << 1)


REFERENCE_SPEC = LossSpec("self")
PAIRS_SPEC = LossSpec("pairs")


@dataclass(frozen=True)
class Settings:
    """One run of a benchmark mode. Defaults are the reference's (scalingcontrasts.cu:40-45)."""

    mode: str = "box"
    rows: int = 1024
    hidden: int = 1024
    prefixes: int = 5
    gpus: int = 0  # 0: every visible device (box/oracle/collectives) or the simulated world size (simulate)
    windows: int = 10
    max_mib: int = 128
    min_kib: int = 1024
    repeats: int = 1000
    host: int = 0
    hosts: int = 1
    nics: str = ""
    exchange: str = ""
    positives: str = "self"
    diagonal: Optional[str] = None
    inputs: str = "keyed"  # "keyed": splitmix64 uniform; "normal": seeded N(0,1)
    seed: int = 0
    warm: int = 20
    steps: int = 100
    beta: float = DEFAULT_BETA
    bias: float = DEFAULT_BIAS
    device: str = "cuda"
    ends: Tuple[int, ...] = field(default_factory=tuple)

    def ladder(self) -> Matryoshka:
        return Matryoshka(self.ends) if self.ends else Matryoshka.halvings(self.hidden, self.prefixes)

    def spec(self) -> LossSpec:
        return LossSpec(self.positives, self.diagonal)

    def with_(self, **changes) -> "Settings":
        return replace(self, **changes)

    def validate(self) -> None:
        if self.windows < 0 or (self.windows == 0 and self.mode != "hosts"):
            raise ValueError("--windows must be positive")
        for name in ("rows", "hidden", "prefixes", "max_mib", "repeats", "hosts"):
            if getattr(self, name) <= 0:
                raise ValueError(f"--{name.replace('_', '-')} must be positive")
        if self.host < 0 or self.host >= self.hosts:
            raise ValueError("--host must lie in [0, --hosts)")
        if self.inputs not in ("keyed", "normal"):
            raise ValueError("--inputs must be keyed or normal")
        self.spec()
        self.ladder()


def log_beta(beta: float) -> float:
    return math.log(beta)
