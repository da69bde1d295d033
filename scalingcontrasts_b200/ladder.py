"""Matryoshka prefix ladder.

A ladder is an ascending list of prefix widths ("ends"), narrowest first. Band ``b`` owns the channels
``[begin(b), ends[b])`` and prefix ``b`` is the first ``ends[b]`` channels of an embedding. The widest end equals
the hidden size. Up to eight prefixes are supported, which is what one tile's tensor-memory budget holds.

Parity: the reference's ``matryoshka_t`` (scalingcontrasts.cuh:120-140) and Mojo ``Matryoshka``
(scalingcontrasts.mojo:936-1004). Unlike the reference, band edges may sit on any multiple of 16 channels (one bf16
tensor-core K-step) rather than 64, so H=768 with five halvings (48/96/192/384/768) is a legal ladder.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Iterable, Sequence, Tuple

MAX_PREFIXES = 8
EDGE_MULTIPLE = 16
HIDDEN_MULTIPLE = 64


@dataclass(frozen=True)
class Matryoshka:
    """Ascending prefix ends, narrowest first."""

    ends: Tuple[int, ...]

    def __post_init__(self) -> None:
        ends = tuple(int(e) for e in self.ends)
        object.__setattr__(self, "ends", ends)
        if not 1 <= len(ends) <= MAX_PREFIXES:
            raise ValueError(f"a ladder holds 1..{MAX_PREFIXES} prefixes, got {len(ends)}")
        previous = 0
        for end in ends:
            if end <= previous:
                raise ValueError(f"prefix ends must ascend strictly, got {ends}")
            previous = end

    # -- construction ---------------------------------------------------------------------------------------
    @staticmethod
    def halvings(hidden: int, count: int) -> "Matryoshka":
        """``ends[p] = hidden >> (count-1-p)``: the widest prefix is the whole embedding, each next one half of it."""
        if count < 1 or count > MAX_PREFIXES:
            raise ValueError(f"a ladder holds 1..{MAX_PREFIXES} prefixes, got {count}")
        ends = tuple(hidden >> (count - 1 - p) for p in range(count))
        if ends[0] <= 0:
            raise ValueError(f"hidden={hidden} cannot be halved {count - 1} times")
        return Matryoshka(ends)

    @staticmethod
    def of(ends: Iterable[int]) -> "Matryoshka":
        return Matryoshka(tuple(sorted(int(e) for e in ends)))

    # -- queries --------------------------------------------------------------------------------------------
    @property
    def count(self) -> int:
        return len(self.ends)

    @property
    def hidden(self) -> int:
        return self.ends[-1]

    def prefixes(self) -> Tuple[int, ...]:
        return self.ends

    def begin(self, band: int) -> int:
        return 0 if band == 0 else self.ends[band - 1]

    def end(self, band: int) -> int:
        return self.ends[band]

    def width(self, band: int) -> int:
        return self.ends[band] - self.begin(band)

    def band_of(self, channel: int) -> int:
        for band, end in enumerate(self.ends):
            if channel < end:
                return band
        raise IndexError(channel)

    def padded(self) -> Sequence[int]:
        """The ends padded with zeros to MAX_PREFIXES, the form the native kernels take."""
        return list(self.ends) + [0] * (MAX_PREFIXES - len(self.ends))

    # -- validation for the tensor-core kernels ------------------------------------------------------------
    def check_device_shape(self, rows: int, hidden: int) -> None:
        """Raises ValueError unless (rows, hidden, ladder) is a shape the sm_100a kernels tile exactly."""
        if hidden != self.hidden:
            raise ValueError(f"the widest prefix {self.hidden} must equal hidden {hidden}")
        if hidden % HIDDEN_MULTIPLE:
            raise ValueError(f"hidden {hidden} must be a multiple of {HIDDEN_MULTIPLE}")
        if rows <= 0 or rows % 128:
            raise ValueError(f"rows {rows} must be a positive multiple of 128")
        for end in self.ends:
            if end % EDGE_MULTIPLE:
                raise ValueError(f"band edge {end} must be a multiple of {EDGE_MULTIPLE}")

    def mma_depth_per_cell(self) -> int:
        """Tensor-core depth units per scored cell, forward plus backward, of this library's kernels: every
        channel once forward (bands accumulate in their own tensor-memory slots) and once backward."""
        return 2 * self.hidden
