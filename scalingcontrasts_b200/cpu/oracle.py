"""Float64 oracle of the one-set Matryoshka sigmoid loss over a whole world of rows.

This is the definition every other path is checked against. For band k with prefix width ``ends[k]`` and N rows:

    n_k(i)   = ||v_i[:ends[k]]||                      cos_k(i,j) = <v_i, v_j>_k / (n_k(i) n_k(j)) if that product > 1e-2
    z(i,j)   = +1 for a positive cell, -1 otherwise   s = z (beta cos + bias)
    L        = sum_k sum_i sum_j  (1/N) softplus(-s)

The gradient with respect to row i collects both the cell (i, j) where it is the query and the mirror cell (j, i) where
it is the candidate; they are equal, which is the factor two the row-owned device kernels apply locally.

Parity: ``oracle_loss`` (scalingcontrasts.cu:133-170) for ``LossSpec("self")``. ``oracle_loops`` restates it as plain
loops (also compiled as a C++ twin in csrc/oracle_cpu.cpp) to cross-check the vectorised form.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from ..config import COSINE_FLOOR, LossSpec, REFERENCE_SPEC
from ..ladder import Matryoshka


@dataclass
class OracleResult:
    loss: float
    band_losses: torch.Tensor  # [K] float64
    gradient: torch.Tensor  # [N, H] float64
    bias_grad: float
    log_beta_grad: float


def cell_targets(n: int, spec: LossSpec, row_base: int = 0, column_base: int = 0, columns: Optional[int] = None):
    """Returns (z, weight_mask, own) for a block of cells: rows ``row_base..+n``, columns ``column_base..+columns``.

    ``z`` is +1/-1, ``weight_mask`` is 0 where the cell is skipped, ``own`` marks the diagonal cells whose cosine is
    pinned to one and which move no embedding.
    """
    columns = n if columns is None else columns
    rows_index = torch.arange(row_base, row_base + n).unsqueeze(1)
    columns_index = torch.arange(column_base, column_base + columns).unsqueeze(0)
    own = rows_index == columns_index
    z = torch.full((n, columns), -1.0, dtype=torch.float64)
    mask = torch.ones((n, columns), dtype=torch.float64)
    if spec.pairs:
        z = torch.where((rows_index ^ 1) == columns_index, torch.ones_like(z), z)
    if spec.diagonal == "own":
        z = torch.where(own, torch.ones_like(z), z)
    elif spec.diagonal == "skip":
        mask = torch.where(own, torch.zeros_like(mask), mask)
    return z, mask, own


def oracle(world: torch.Tensor, ladder: Matryoshka, beta: float, bias: float,
           spec: LossSpec = REFERENCE_SPEC) -> OracleResult:
    """Vectorised float64 evaluation over the whole world ``[N, H]``."""
    v = world.detach().to(torch.float64).cpu()
    n, hidden = v.shape
    if hidden != ladder.hidden:
        raise ValueError(f"hidden {hidden} != ladder's widest prefix {ladder.hidden}")
    weight = 1.0 / n
    z, mask, own = cell_targets(n, spec)
    gradient = torch.zeros_like(v)
    band_losses = torch.zeros(ladder.count, dtype=torch.float64)
    bias_grad = 0.0
    log_beta_grad = 0.0
    for band, width in enumerate(ladder.ends):
        p = v[:, :width]
        norms = p.square().sum(dim=1).sqrt()
        denominator = norms[:, None] * norms[None, :]
        active = denominator > COSINE_FLOOR
        dots = p @ p.T
        cosine = torch.where(active, dots / torch.where(active, denominator, torch.ones_like(denominator)),
                             torch.zeros_like(dots))
        cosine = torch.where(own, torch.ones_like(cosine), cosine)
        logit = beta * cosine
        s = z * (logit + bias)
        cell_loss = weight * mask * torch.nn.functional.softplus(-s)
        band_losses[band] = cell_loss.sum()
        cell_grad = -weight * mask * z * torch.sigmoid(-s)  # dL/d(logit)
        bias_grad += float(cell_grad.sum())
        log_beta_grad += float((cell_grad * logit).sum())
        moving = active & ~own
        a = torch.where(moving, cell_grad, torch.zeros_like(cell_grad))
        inverse_norms = torch.where(norms > 0, 1.0 / norms, torch.zeros_like(norms))
        inverse_denominator = inverse_norms[:, None] * inverse_norms[None, :]
        first = (a * inverse_denominator) @ p
        second = (a * cosine).sum(dim=1, keepdim=True) * inverse_norms[:, None].square() * p
        gradient[:, :width] += 2.0 * beta * (first - second)
    return OracleResult(float(band_losses.sum()), band_losses, gradient, bias_grad, log_beta_grad)


def oracle_loops(world: torch.Tensor, ladder: Matryoshka, beta: float, bias: float,
                 spec: LossSpec = REFERENCE_SPEC) -> OracleResult:
    """The same evaluation as explicit loops over ordered pairs, adding each cell's gradient to both of its rows.
    O(K N^2 H) in Python: for small worlds only."""
    v = world.detach().to(torch.float64).cpu()
    n, _ = v.shape
    weight = 1.0 / n
    gradient = torch.zeros_like(v)
    band_losses = torch.zeros(ladder.count, dtype=torch.float64)
    bias_grad = 0.0
    log_beta_grad = 0.0
    for band, width in enumerate(ladder.ends):
        p = v[:, :width]
        norms = p.square().sum(dim=1).sqrt()
        for i in range(n):
            for j in range(n):
                diagonal = i == j
                if diagonal and spec.diagonal == "skip":
                    continue
                denominator = float(norms[i] * norms[j])
                active = denominator > COSINE_FLOOR
                dot = float(p[i] @ p[j])
                cosine = 1.0 if diagonal else (dot / denominator if active else 0.0)
                target = -1.0
                if spec.pairs and (i ^ 1) == j:
                    target = 1.0
                if diagonal and spec.diagonal == "own":
                    target = 1.0
                logit = beta * cosine
                s = target * (logit + bias)
                band_losses[band] += weight * float(torch.nn.functional.softplus(torch.tensor(-s, dtype=torch.float64)))
                cell_grad = -weight * target * float(torch.sigmoid(torch.tensor(-s, dtype=torch.float64)))
                bias_grad += cell_grad
                log_beta_grad += cell_grad * logit
                if diagonal or not active:
                    continue
                scaled = cell_grad * beta
                gradient[i, :width] += scaled * (p[j] / denominator - cosine * p[i] / float(norms[i] ** 2))
                gradient[j, :width] += scaled * (p[i] / denominator - cosine * p[j] / float(norms[j] ** 2))
    return OracleResult(float(band_losses.sum()), band_losses, gradient, bias_grad, log_beta_grad)


def relative_l2(measured: torch.Tensor, expected: torch.Tensor) -> float:
    """``sqrt(sum (m - e)^2 / sum e^2)``: the reference's gradient error measure (scalingcontrasts.cu:459-466)."""
    m = measured.detach().to(torch.float64).cpu()
    e = expected.detach().to(torch.float64).cpu()
    denominator = float(e.square().sum())
    if denominator == 0.0:
        return float((m - e).square().sum().sqrt())
    return float(((m - e).square().sum() / denominator).sqrt())
