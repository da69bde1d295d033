"""The streamed, row-owned Matryoshka sigmoid loss on one B200: ``begin``, then ``score`` once per candidate block in
any order, then ``finish``.

A rank owns ``rows`` query rows. Each ``score`` runs, on the calling stream,

1. (unless the caller supplies them) the candidates' prefix inverse norms and per-tile maxima,
2. (fused form only) a transpose of the candidates (its gradient GEMM reads them K-major),
3. the fused tile kernel (tcgen05): segment dots of every band in tensor memory, sigmoid loss, per-row partial sums, and
   the per-band suffix-summed gradient of a work item (a strip of 128 rows against a run of candidate tiles) as
   bfloat16 patches in a per-CTA scratch buffer, which the same CTA folds into the query gradient with a tensor-core
   GEMM while its epilogue warps already score the next item: no ``[K, R, R]`` gradient cube exists. Optionally the
   same launch pulls the next block from a peer's memory into local staging,
4. the deterministic fold of the partials.

The default is the two-kernel form (``fused=False``; the only one for ladders of seven or eight prefixes): the forward
kernel writes the bfloat16 gradient cube ``[K, R, R]`` and a separate backward tile kernel folds it, reading the candidates
as they lie in memory (an MN-major tensor-core operand, no transposed copy). The fused form saves the cube's memory
(0.59 GB of scratch instead of 2.86 GB at 16384 rows) and is about a fifth slower there, because its GEMM has room for only
two shared-memory stages beside the score pass; so it is a choice, not the default.

``finish`` folds the L2-normalisation's self term, casts the gradient to bfloat16 and reduces the row summands into
``summands`` (any device float32 span of ``SUMMAND_SLOTS`` values, a domain payload included):
``[loss, d/d bias, d/d log(beta), 0, loss of prefix 0, ..., loss of prefix 7]``. Summands are this rank's share: sum
them across ranks. The embedding gradient is final as computed (the owner applies a cell and its mirror), so no
gradient crosses GPUs.

Scratch memory is allocated once, in ``__init__``, and is independent of the number of blocks scored.

Parity: ``streamed_loss_t`` (scalingcontrasts.cuh:1179-1324) and Mojo ``StreamedLoss`` (scalingcontrasts.mojo:1560-1781).
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Optional, Tuple

import torch

from .._ext import native
from ..config import LossSpec, REFERENCE_SPEC, SUMMAND_SLOTS
from ..ladder import Matryoshka


@dataclass
class PullRequest:
    """Up to two contiguous spans to copy (peer memory -> local memory) inside the next forward launch."""

    src0: int = 0
    dst0: int = 0
    bytes0: int = 0
    src1: int = 0
    dst1: int = 0
    bytes1: int = 0


class BlockNorms:
    """Inverse prefix norms ``[K, R]`` of a block followed by their per-64-row maxima ``[K, R/64]`` in one contiguous
    float32 buffer, so that a block's norms travel with it as a single span."""

    def __init__(self, prefixes: int, rows: int, storage: Optional[torch.Tensor] = None, device=None) -> None:
        self.prefixes, self.rows = prefixes, rows
        self.scalars = BlockNorms.scalars_for(prefixes, rows)
        if storage is None:
            storage = torch.empty(self.scalars, dtype=torch.float32, device=device)
        if storage.numel() != self.scalars or storage.dtype != torch.float32:
            raise ValueError("BlockNorms storage has the wrong size or dtype")
        self.storage = storage
        self.inverse = storage[:prefixes * rows].view(prefixes, rows)
        self.tile_max = storage[prefixes * rows:prefixes * rows + prefixes * (rows // 64)].view(prefixes, rows // 64)

    @staticmethod
    def scalars_for(prefixes: int, rows: int) -> int:
        """Scalars of the buffer, rounded up to whole 16-byte vectors so that the span can be pulled as one."""
        return -(-(prefixes * rows + prefixes * (rows // 64)) // 4) * 4

    @property
    def nbytes(self) -> int:
        return self.scalars * 4


def _stream(stream) -> int:
    return (torch.cuda.current_stream() if stream is None else stream).cuda_stream


def compute_block_norms(rows: torch.Tensor, ladder: Matryoshka, norms: BlockNorms, copy_to: Optional[torch.Tensor] = None,
                        stream=None) -> None:
    """Fills ``norms`` for the bfloat16 block ``rows``; optionally copies the block to ``copy_to`` in the same pass
    (used to publish a block into symmetric memory)."""
    _check_block(rows)
    copy_pointer = 0
    if copy_to is not None:
        if copy_to.shape != rows.shape or copy_to.dtype != torch.bfloat16 or not copy_to.is_contiguous():
            raise ValueError("copy_to must match the block")
        copy_pointer = copy_to.data_ptr()
    native().prefix_norms(rows.data_ptr(), copy_pointer, norms.inverse.data_ptr(), norms.tile_max.data_ptr(),
                          rows.shape[0], rows.shape[1], list(ladder.ends), _stream(stream))


def _check_block(block: torch.Tensor) -> None:
    if block.dtype != torch.bfloat16 or block.dim() != 2 or not block.is_contiguous() or not block.is_cuda:
        raise ValueError("a block must be a contiguous CUDA bfloat16 matrix")
    if block.data_ptr() % 16:
        raise ValueError("a block must start on a 16-byte boundary")


class StreamedLoss:
    """One rank's streamed loss state on a GPU. See the module docstring for the contract."""

    def __init__(self, rows: int, hidden: int, ladder: Matryoshka, spec: LossSpec = REFERENCE_SPEC, device=None,
                 candidate_rows: Optional[int] = None, budget_s: float = 2.0, backward_split: int = 0,
                 fused: Optional[bool] = None, tiles_per_run: Optional[int] = None,
                 transpose_candidates: Optional[bool] = None, overlap_backward: Optional[bool] = None,
                 backward_multiprocessors: Optional[int] = None) -> None:
        ladder.check_device_shape(rows, hidden)
        self.rows, self.hidden, self.ladder, self.spec = rows, hidden, ladder, spec
        self.candidate_rows = rows if candidate_rows is None else candidate_rows
        if self.candidate_rows % 128:
            raise ValueError("candidate blocks must hold a multiple of 128 rows")
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.budget_ns = int(budget_s * 1e9)
        properties = torch.cuda.get_device_properties(self.device)
        self.multiprocessors = properties.multi_processor_count
        k, ext = ladder.count, native()
        supported = bool(ext.forward_fused_supported(hidden, k))
        if fused and not supported:
            raise ValueError("the fused kernel takes ladders of at most six prefixes")
        if fused is None and os.environ.get("SC_LOSS_FUSED", "") in ("0", "1"):
            fused = os.environ["SC_LOSS_FUSED"] == "1" and supported  # A/B switch for measurements
        self.fused = False if fused is None else bool(fused)
        chooser = ext.forward_choose_tiles_per_run_fused if self.fused else ext.forward_choose_tiles_per_run
        self.tiles_per_run = int(chooser(rows, self.candidate_rows, self.multiprocessors))
        if tiles_per_run is not None:
            if tiles_per_run < 1 or (self.candidate_rows // 64) % tiles_per_run or (self.fused and tiles_per_run > 16):
                raise ValueError("tiles_per_run must divide the candidate tiles (and be at most 16 for the fused kernel)")
            self.tiles_per_run = int(tiles_per_run)
        self.partial_slots = int(ext.forward_partial_slots(self.candidate_rows, self.tiles_per_run))
        self.quantities = int(ext.forward_quantities(k))
        # One CTA per output tile keeps the gradient fold a plain read-modify-write, hence bit-reproducible; a larger
        # split divides the candidate range between CTAs that add with atomics (faster for tiny blocks, order-dependent).
        self.backward_split = max(1, int(backward_split))
        f32 = dict(dtype=torch.float32, device=self.device)
        bf16 = dict(dtype=torch.bfloat16, device=self.device)
        self.query_norms = BlockNorms(k, rows, device=self.device)
        self.candidate_norms = BlockNorms(k, self.candidate_rows, device=self.device)
        self.query_gradient = torch.zeros(rows, hidden, **f32)
        self.row_accumulators = torch.zeros(self.quantities, rows, **f32)
        self.partials = torch.empty(self.partial_slots, self.quantities, rows, **f32)
        if self.fused:
            # Gradient patches of the items in flight: two buffers per CTA, independent of the block's size.
            scratch = int(ext.forward_fused_scratch_bytes(k, self.tiles_per_run, self.multiprocessors))
            self.similarity_gradients = torch.empty(scratch // 2, **bf16)
        else:
            self.similarity_gradients = torch.empty(k, rows, self.candidate_rows, **bf16)
        # The backward kernel reads the candidates as they lie in memory (an MN-major tensor-core operand); the K-major
        # form with a transposed copy per block remains for the fused kernel, for blocks narrower than 64 channels, and
        # on request (``transpose_candidates=True`` or SC_LOSS_TRANSPOSE=1).
        if transpose_candidates is None:
            transpose_candidates = os.environ.get("SC_LOSS_TRANSPOSE", "0") == "1"
        self.transpose_candidates = bool(transpose_candidates) or self.fused or hidden < 64
        self.transposed_candidates = (torch.empty(hidden, self.candidate_rows, **bf16) if self.transpose_candidates
                                      else torch.empty(0, **bf16))
        self.status = torch.zeros(8, dtype=torch.int32, device=self.device)
        # What never changes between blocks lives in a native plan, so that scoring a block is one call into C++.
        self._plan = ext.LossPlan(rows, self.candidate_rows, hidden, list(ladder.ends), self.tiles_per_run, self.partial_slots,
                                  self.quantities, self.backward_split, spec.code(), self.fused,
                                  self.similarity_gradients.data_ptr(), self.similarity_gradients.numel() * 2,
                                  self.transposed_candidates.data_ptr(), self.query_gradient.data_ptr(),
                                  self.partials.data_ptr(), self.row_accumulators.data_ptr(), self.status.data_ptr(),
                                  self.budget_ns, self.multiprocessors)
        self._plan.transpose_candidates = self.transpose_candidates
        # With ``overlap_backward`` a block's gradient GEMM runs on a second stream, on a few multiprocessors, beside the
        # next block's forward kernel (whose grid shrinks by as many), and a step's last one runs alone in finish(). It
        # takes a second gradient cube, and the caller must leave a block's candidates in place until the block after
        # next has been handed to score() (or finish() was called). Results are bit-identical to the in-line order.
        # Measured on a power-capped B200 it gains nothing (8 blocks of 16384 rows: 15.1 ms at 20 multiprocessors for the
        # backward, 15.7 at 28, 16.9 at 40, against 15.3 in line), so it is off unless asked for.
        if overlap_backward is None:
            overlap_backward = os.environ.get("SC_LOSS_OVERLAP", "0") == "1"
        self.overlap_backward = bool(overlap_backward) and not self.transpose_candidates
        self.similarity_gradients_alt = torch.empty(0, **bf16)
        if self.overlap_backward:
            if backward_multiprocessors is None:
                backward_multiprocessors = int(os.environ.get("SC_LOSS_BACKWARD_SMS", "0")) or round(self.multiprocessors * 0.2)
            self.backward_multiprocessors = max(1, min(int(backward_multiprocessors), self.multiprocessors - 1))
            self.similarity_gradients_alt = torch.empty_like(self.similarity_gradients)
            self._plan.enable_overlap(self.similarity_gradients_alt.data_ptr(), self.backward_multiprocessors)
        self._begun = False
        self._query_norms_view: Optional[BlockNorms] = None

    # ------------------------------------------------------------------------------------------------------
    def bytes(self) -> int:
        """Bytes of scratch this object holds; does not grow with the number of blocks scored."""
        tensors = (self.query_norms.storage, self.candidate_norms.storage, self.query_gradient, self.row_accumulators,
                   self.partials, self.similarity_gradients, self.similarity_gradients_alt, self.transposed_candidates,
                   self.status)
        return sum(t.numel() * t.element_size() for t in tensors)

    def begin(self, queries: torch.Tensor, stream=None, query_norms: Optional[BlockNorms] = None) -> None:
        """Clears the per-row accumulators and takes the queries' prefix norms (computed here unless supplied)."""
        self._check_queries(queries)
        with torch.cuda.stream(stream) if stream is not None else _NullContext():
            self.query_gradient.zero_()
            self.row_accumulators.zero_()
        if query_norms is None:
            compute_block_norms(queries, self.ladder, self.query_norms, stream=stream)
            self._query_norms_view = self.query_norms
        else:
            self._query_norms_view = query_norms
        self._plan.begin_step()
        self._begun = True

    def score(self, queries: torch.Tensor, candidates: torch.Tensor, query_base: int, candidate_base: int, beta: float,
              bias: float, live: int, stream=None, *, candidate_norms: Optional[BlockNorms] = None,
              scalars: Optional[torch.Tensor] = None, pull_next: Optional[PullRequest] = None) -> None:
        """Scores one candidate block (local memory) against this rank's rows.

        ``scalars``, when given, is a device float32 ``[beta, bias]`` that overrides the two host floats, so learnable
        values never visit the host. ``pull_next`` rides in the forward launch: the copy it names overlaps this block's
        scoring."""
        if not self._begun:
            raise RuntimeError("score() before begin()")
        self._check_queries(queries)
        _check_block(candidates)
        if tuple(candidates.shape) != (self.candidate_rows, self.hidden):
            raise ValueError(f"candidates must be [{self.candidate_rows}, {self.hidden}]")
        if candidate_norms is None:
            compute_block_norms(candidates, self.ladder, self.candidate_norms, stream=stream)
            candidate_norms = self.candidate_norms
        pull = pull_next or PullRequest()
        qn = self._query_norms_view
        self._plan.score(queries.data_ptr(), candidates.data_ptr(), qn.inverse.data_ptr(), candidate_norms.inverse.data_ptr(),
                         candidate_norms.tile_max.data_ptr(), int(query_base), int(candidate_base), float(beta), float(bias),
                         float(live), 0 if scalars is None else scalars.data_ptr(), pull.src0, pull.dst0, pull.bytes0,
                         pull.src1, pull.dst1, pull.bytes1, _stream(stream))

    def finish(self, queries: torch.Tensor, gradient_out: Optional[torch.Tensor] = None,
               summands: Optional[torch.Tensor] = None, stream=None) -> Tuple[torch.Tensor, torch.Tensor]:
        if not self._begun:
            raise RuntimeError("finish() before begin()")
        self._check_queries(queries)
        if gradient_out is None:
            gradient_out = torch.empty(self.rows, self.hidden, dtype=torch.bfloat16, device=self.device)
        _check_block(gradient_out)
        if summands is None:
            summands = torch.empty(SUMMAND_SLOTS, dtype=torch.float32, device=self.device)
        if summands.dtype != torch.float32 or summands.numel() < SUMMAND_SLOTS or not summands.is_contiguous():
            raise ValueError(f"summands must be a contiguous float32 span of at least {SUMMAND_SLOTS} values")
        ext, s = native(), _stream(stream)
        qn = self._query_norms_view
        self._plan.join(s)
        ext.finalize(queries.data_ptr(), qn.inverse.data_ptr(), self.row_accumulators.data_ptr(),
                     self.query_gradient.data_ptr(), gradient_out.data_ptr(), self.rows, self.hidden, list(self.ladder.ends), s)
        ext.sum_summands(self.row_accumulators.data_ptr(), summands.data_ptr(), self.rows, self.ladder.count, s)
        self._begun = False
        return gradient_out, summands

    def check(self) -> None:
        """Raises if a tile kernel's bounded wait ran out (reads the status block: synchronises)."""
        words = [int(v) & 0xFFFFFFFF for v in self.status.cpu().tolist()]
        if words[0] != 0:
            raise RuntimeError(f"streamed loss kernel gave up: code {words[0]} at site {words[1]} "
                               f"(detail {words[2]}, parity {words[3]}, barrier {words[4]:#x}, block {words[5]}, "
                               f"thread {words[6]})")

    def _check_queries(self, queries: torch.Tensor) -> None:
        _check_block(queries)
        if tuple(queries.shape) != (self.rows, self.hidden):
            raise ValueError(f"queries must be [{self.rows}, {self.hidden}], got {tuple(queries.shape)}")


class _NullContext:
    def __enter__(self):
        return None

    def __exit__(self, *args):
        return False


def keyed_embeddings_device(rows: int, hidden: int, salt: int, scale: float, device=None) -> torch.Tensor:
    """The device twin of ``utils.keyed.keyed_embeddings`` (bit-identical values)."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    out = torch.empty(rows, hidden, dtype=torch.bfloat16, device=device)
    native().keyed_embeddings(out.data_ptr(), rows, hidden, int(salt), float(scale), _stream(None))
    return out
