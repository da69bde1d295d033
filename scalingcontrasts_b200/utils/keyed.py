"""Keyed, reproducible inputs: the CPU twins of the device generators.

Every value is a pure function of its index through the splitmix64 finalizer, so any rank of any run can regenerate
any other rank's data and check a collective's sums without moving them. Parity: ``splitmix64``,
``keyed_embeddings_cuda_``, ``keyed_integers_cuda_``, ``keyed_fractions_cuda_`` (scalingcontrasts.cu:48-82).
Seeded N(0,1) inputs are provided beside them for the configurations that ask for normal embeddings.
"""
from __future__ import annotations

import numpy as np
import torch

_M1 = np.uint64(0xBF58476D1CE4E5B9)
_M2 = np.uint64(0x94D049BB133111EB)


def splitmix64(values: np.ndarray) -> np.ndarray:
    """The splitmix64 finalizer over an array of uint64 keys (wrapping arithmetic)."""
    v = np.asarray(values, dtype=np.uint64).copy()
    with np.errstate(over="ignore"):
        v = (v ^ (v >> np.uint64(30))) * _M1
        v = (v ^ (v >> np.uint64(27))) * _M2
        v = v ^ (v >> np.uint64(31))
    return v


def keyed_embeddings(rows: int, hidden: int, salt: int, scale: float, dtype=torch.bfloat16) -> torch.Tensor:
    """``[rows, hidden]`` values in ``[-scale/2, scale/2)``; key ``(salt*rows + row)*hidden + channel``."""
    with np.errstate(over="ignore"):
        row = (np.uint64(salt) * np.uint64(rows) + np.arange(rows, dtype=np.uint64))[:, None]
        key = row * np.uint64(hidden) + np.arange(hidden, dtype=np.uint64)[None, :]
    bits = splitmix64(key) >> np.uint64(40)
    # float32 arithmetic in the same order as the device kernel: exact conversion, exact scale by 2^-24, subtract, scale
    unit = bits.astype(np.float32) * np.float32(2.0**-24) - np.float32(0.5)
    values = unit * np.float32(scale)
    return torch.from_numpy(values).to(dtype)


def keyed_integers(scalars: int, members: int, member: int, first: int = 0) -> torch.Tensor:
    """Small integers (< 2**12) as float32: sums of up to 2**12 of them are exact in any order."""
    with np.errstate(over="ignore"):
        key = (np.arange(first, first + scalars, dtype=np.uint64)) * np.uint64(members) + np.uint64(member)
    return torch.from_numpy((splitmix64(key) >> np.uint64(52)).astype(np.float32))


def keyed_integer_sums(scalars: int, members: int, first: int = 0) -> torch.Tensor:
    """The exact sum over members of ``keyed_integers`` for each scalar."""
    total = torch.zeros(scalars, dtype=torch.float32)
    for member in range(members):
        total += keyed_integers(scalars, members, member, first)
    return total


def keyed_fractions(scalars: int, members: int, member: int, first: int = 0) -> torch.Tensor:
    """Fractions in ``[-0.5, 0.5)`` whose sums round, so a change of summation order shows in the bits."""
    with np.errstate(over="ignore"):
        key = (np.arange(first, first + scalars, dtype=np.uint64)) * np.uint64(members) + np.uint64(member)
    bits = splitmix64(key) >> np.uint64(40)
    return torch.from_numpy(bits.astype(np.float32) * np.float32(2.0**-24) - np.float32(0.5))


def normal_embeddings(rows: int, hidden: int, seed: int, rank: int = 0, dtype=torch.bfloat16,
                      normalize: bool = True) -> torch.Tensor:
    """Seeded N(0,1) rows, optionally L2-normalised over the full width (the loss renormalises every prefix)."""
    generator = torch.Generator(device="cpu").manual_seed(int(seed) * 1_000_003 + int(rank))
    values = torch.randn(rows, hidden, generator=generator, dtype=torch.float32)
    if normalize:
        values = torch.nn.functional.normalize(values, dim=-1)
    return values.to(dtype)


def make_embeddings(kind: str, rows: int, hidden: int, rank: int, seed: int, scale: float,
                    dtype=torch.bfloat16) -> torch.Tensor:
    if kind == "keyed":
        return keyed_embeddings(rows, hidden, rank, scale, dtype)
    if kind == "normal":
        return normal_embeddings(rows, hidden, seed, rank, dtype)
    raise ValueError(f"unknown input kind {kind!r}")
