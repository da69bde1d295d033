"""CPU twin of the streamed, row-owned loss: same ``begin / score / finish`` contract as the device object, written
with plain torch operations in a chosen precision (float32 by default).

A rank owns ``rows`` query rows. ``score`` is called once per candidate block, in any order; the per-row accumulators
(query gradient, row summands, per-band self coefficients) persist between calls, so memory does not grow with the
number of blocks. ``finish`` folds the L2-normalisation's self term into the gradient and reduces the row summands.

This mirrors the device algebra exactly (raw-dot gradient, per-band coefficient, suffix-summed gradient per band) so a
disagreement between the two paths localises to a kernel, not to a formula. Parity: ``streamed_loss_t``
(scalingcontrasts.cuh:1179-1302) and the cell math at scalingcontrasts.cuh:874-898.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from ..config import INVERSE_COSINE_FLOOR, LossSpec, REFERENCE_SPEC, SUMMAND_SLOTS
from ..ladder import Matryoshka


def prefix_inverse_norms(rows: torch.Tensor, ladder: Matryoshka, dtype=torch.float32) -> torch.Tensor:
    """``[K, R]`` inverse norms of every prefix; zero where the prefix is all zeros (scalingcontrasts.cuh:672-686)."""
    squares = rows.to(dtype).square()
    running = torch.zeros(rows.shape[0], dtype=dtype, device=rows.device)
    out = torch.empty(ladder.count, rows.shape[0], dtype=dtype, device=rows.device)
    for band in range(ladder.count):
        running = running + squares[:, ladder.begin(band):ladder.end(band)].sum(dim=1)
        out[band] = torch.where(running > 0, running.rsqrt(), torch.zeros_like(running))
    return out


class CpuStreamedLoss:
    """One rank's streamed loss state in plain torch operations (on the CPU by default; any torch device works, which
    is how the device kernels' intermediates are checked in place)."""

    def __init__(self, rows: int, hidden: int, ladder: Matryoshka, spec: LossSpec = REFERENCE_SPEC,
                 dtype: torch.dtype = torch.float32, device="cpu", keep_cubes: bool = False) -> None:
        if ladder.hidden != hidden:
            raise ValueError(f"the widest prefix {ladder.hidden} must equal hidden {hidden}")
        self.rows, self.hidden, self.ladder, self.spec, self.dtype = rows, hidden, ladder, spec, dtype
        self.device = torch.device(device)
        k = ladder.count
        options = dict(dtype=dtype, device=self.device)
        self.query_inverse_norms = torch.zeros(k, rows, **options)
        self.query_gradient = torch.zeros(rows, hidden, **options)
        self.row_loss = torch.zeros(k, rows, **options)
        self.row_bias_grad = torch.zeros(rows, **options)
        self.row_log_beta_grad = torch.zeros(rows, **options)
        self.self_coefficients = torch.zeros(k, rows, **options)
        self.keep_cubes = keep_cubes
        self.last_cubes = None  # [K, R, C] suffix-summed raw-dot gradients of the last score(), when kept
        self.last_prefix_dots = None
        self._begun = False

    def bytes(self) -> int:
        tensors = (self.query_inverse_norms, self.query_gradient, self.row_loss, self.row_bias_grad,
                   self.row_log_beta_grad, self.self_coefficients)
        return sum(t.numel() * t.element_size() for t in tensors)

    # -- contract -------------------------------------------------------------------------------------------
    def begin(self, queries: torch.Tensor) -> None:
        self._check(queries)
        self.query_inverse_norms = prefix_inverse_norms(queries, self.ladder, self.dtype)
        for t in (self.query_gradient, self.row_loss, self.row_bias_grad, self.row_log_beta_grad,
                  self.self_coefficients):
            t.zero_()
        self._begun = True

    def score(self, queries: torch.Tensor, candidates: torch.Tensor, query_base: int, candidate_base: int,
              beta: float, bias: float, live: int) -> None:
        if not self._begun:
            raise RuntimeError("score() before begin()")
        self._check(queries)
        dtype = self.dtype
        q = queries.to(dtype)
        c = candidates.to(dtype)
        columns = c.shape[0]
        weight = 1.0 / float(live)
        candidate_inverse_norms = prefix_inverse_norms(candidates, self.ladder, dtype)
        row_index = torch.arange(query_base, query_base + self.rows, device=self.device).unsqueeze(1)
        column_index = torch.arange(candidate_base, candidate_base + columns, device=self.device).unsqueeze(0)
        own = row_index == column_index
        z = torch.full((self.rows, columns), -1.0, dtype=dtype, device=self.device)
        mask = torch.ones((self.rows, columns), dtype=dtype, device=self.device)
        if self.keep_cubes:
            self.last_cubes = torch.zeros(self.ladder.count, self.rows, columns, dtype=dtype, device=self.device)
            self.last_prefix_dots = torch.zeros(self.ladder.count, self.rows, columns, dtype=dtype, device=self.device)
        if self.spec.pairs:
            z = torch.where((row_index ^ 1) == column_index, torch.ones_like(z), z)
        if self.spec.diagonal == "own":
            z = torch.where(own, torch.ones_like(z), z)
        elif self.spec.diagonal == "skip":
            mask = torch.where(own, torch.zeros_like(mask), mask)
        suffix = torch.zeros(self.rows, columns, dtype=dtype, device=self.device)
        for band in reversed(range(self.ladder.count)):
            end = self.ladder.end(band)
            dots = q[:, :end] @ c[:, :end].T
            inverse_denominator = torch.clamp(
                self.query_inverse_norms[band][:, None] * candidate_inverse_norms[band][None, :],
                max=INVERSE_COSINE_FLOOR)
            floored = inverse_denominator >= INVERSE_COSINE_FLOOR
            cosine = torch.where(floored, torch.zeros_like(dots), dots * inverse_denominator)
            logit = beta * torch.where(own, torch.ones_like(cosine), cosine)
            s = z * (logit + bias)
            decay = torch.exp(-s.abs())
            complement = torch.where(s >= 0, decay, torch.ones_like(decay)) / (1.0 + decay)
            cell_grad = -weight * mask * z * complement
            self.row_loss[band] += (weight * mask * (torch.clamp(-s, min=0) + torch.log1p(decay))).sum(dim=1)
            self.row_bias_grad += cell_grad.sum(dim=1)
            self.row_log_beta_grad += (cell_grad * logit).sum(dim=1)
            raw_grad = torch.where(own | floored, torch.zeros_like(cell_grad),
                                   2.0 * beta * cell_grad * inverse_denominator)
            self.self_coefficients[band] += (raw_grad * dots).sum(dim=1)
            suffix = suffix + raw_grad
            if self.keep_cubes:
                self.last_cubes[band] = suffix
                self.last_prefix_dots[band] = dots
            begin = self.ladder.begin(band)
            self.query_gradient[:, begin:end] += suffix @ c[:, begin:end]

    def finish(self, queries: torch.Tensor, gradient_out: Optional[torch.Tensor] = None,
               summands: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
        """Returns ``(gradient [R,H], summands [SUMMAND_SLOTS])``; summands are this rank's share and are meant to be
        summed (not averaged) across ranks."""
        if not self._begun:
            raise RuntimeError("finish() before begin()")
        q = queries.to(self.dtype)
        fold = torch.zeros(self.rows, self.hidden, dtype=self.dtype, device=self.device)
        for band in range(self.ladder.count):
            term = self.self_coefficients[band] * self.query_inverse_norms[band].square()
            fold[:, :self.ladder.end(band)] += term[:, None]
        gradient = self.query_gradient - fold * q
        if gradient_out is None:
            gradient_out = torch.empty(self.rows, self.hidden, dtype=queries.dtype, device=self.device)
        gradient_out.copy_(gradient.to(gradient_out.dtype))
        if summands is None:
            summands = torch.zeros(SUMMAND_SLOTS, dtype=torch.float32, device=self.device)
        summands.zero_()
        summands[0] = float(self.row_loss.sum())
        summands[1] = float(self.row_bias_grad.sum())
        summands[2] = float(self.row_log_beta_grad.sum())
        for band in range(self.ladder.count):
            summands[4 + band] = float(self.row_loss[band].sum())
        self._begun = False
        return gradient_out, summands

    def _check(self, queries: torch.Tensor) -> None:
        if tuple(queries.shape) != (self.rows, self.hidden):
            raise ValueError(f"queries must be [{self.rows}, {self.hidden}], got {tuple(queries.shape)}")


def simulate_world(blocks, ladder: Matryoshka, beta: float, bias: float, spec: LossSpec = REFERENCE_SPEC,
                   dtype: torch.dtype = torch.float32, order=None):
    """Runs every rank of a world in-process: rank r owns ``blocks[r]`` and scores every block. Returns the per-rank
    gradients and the world's summed summands. ``order(rank)`` may return any permutation of the block indices."""
    world = len(blocks)
    rows, hidden = blocks[0].shape
    live = world * rows
    gradients = []
    total = torch.zeros(SUMMAND_SLOTS, dtype=torch.float64)
    for rank in range(world):
        loss = CpuStreamedLoss(rows, hidden, ladder, spec, dtype)
        loss.begin(blocks[rank])
        sequence = list(range(world)) if order is None else list(order(rank))
        for peer in sequence:
            loss.score(blocks[rank], blocks[peer], rank * rows, peer * rows, beta, bias, live)
        gradient, summands = loss.finish(blocks[rank], torch.empty(rows, hidden, dtype=dtype))
        gradients.append(gradient)
        total += summands.to(torch.float64)
    return gradients, total
