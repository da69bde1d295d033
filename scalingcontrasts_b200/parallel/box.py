"""The intra-box data-parallel loss step: every GPU owns ``rows`` rows and scores them against every GPU's block.

One step on a rank, all on one stream and without a host synchronisation:

1. publish: one pass computes the block's prefix norms and copies the block into the rank's symmetric replica, so that
   peers find embeddings and norms side by side;
2. a domain barrier says "everyone's block is complete";
3. ``begin``, then one ``score`` per peer in the staggered order ``(rank + p) mod S`` (so the eight GPUs never all pull
   from the same peer at once); the forward launch that scores block ``p`` also pulls block ``p+1`` from its owner's
   replica into one of two local staging buffers with plain peer loads, so the NVLink transfer overlaps the scoring;
4. ``finish`` writes the rank's summands straight into the domain payload, and the all-reduce sums them across ranks;
   its entry and exit rounds double as the fence that says "everyone has finished reading my block".

``simulate`` plays one rank of a larger world on a single GPU by scoring the own block ``S`` times under shifted
candidate bases (timing and memory only; block 0 holds the own copies).

Parity: ``step_box`` (scalingcontrasts.cu:294-311), ``run_simulate`` (scalingcontrasts.cu:377-394); the staging pull
replaces the reference's serial ``cudaMemcpyAsync`` (scalingcontrasts.cuh:1262-1265).
"""
from __future__ import annotations

import os

from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import torch

from ..config import LossSpec, REFERENCE_SPEC, SUMMAND_SLOTS
from ..ladder import Matryoshka
from ..ops.streamed_loss import BlockNorms, PullRequest, StreamedLoss, compute_block_norms
from ..utils.trace import phase


def _check_gradient(gradient: torch.Tensor, rows: int, hidden: int) -> None:
    if (gradient.dtype != torch.bfloat16 or tuple(gradient.shape) != (rows, hidden) or not gradient.is_contiguous()
            or not gradient.is_cuda):
        raise ValueError(f"the gradient must be a contiguous CUDA bfloat16 tensor of shape [{rows}, {hidden}]")


@dataclass
class SourceBlock:
    """Where one candidate block lives: in this GPU's memory (``embeddings`` / ``norms`` given), or in a domain member's
    replica at the two offsets, from where it is pulled into local staging before it is scored."""

    candidate_base: int
    embeddings: Optional[torch.Tensor] = None
    norms: Optional[BlockNorms] = None
    member: int = -1
    embeddings_offset: int = 0
    norms_offset: int = 0

    @property
    def local(self) -> bool:
        return self.embeddings is not None


class BoxLoss:
    """One rank's engine for box-wide loss steps. ``domain`` may be None for a single, unconnected GPU."""

    def __init__(self, rows: int, hidden: int, ladder: Matryoshka, spec: LossSpec = REFERENCE_SPEC, domain=None,
                 device=None, budget_s: float = 2.0, overlap_backward: Optional[bool] = None) -> None:
        self.rows, self.hidden, self.ladder, self.spec, self.domain = rows, hidden, ladder, spec, domain
        self.device = domain.device if domain is not None else (
            torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device))
        # On request (or SC_LOSS_OVERLAP=1) each block's gradient GEMM runs beside the next block's forward kernel (see
        # StreamedLoss). Off by default: on a power-capped B200 the two kernels side by side took as long as one after
        # the other (15.1 against 15.3 ms for eight 16384-row blocks at the best split), for twice the gradient cube.
        if overlap_backward is None:
            overlap_backward = os.environ.get("SC_LOSS_OVERLAP", "0") == "1"
        self.loss = StreamedLoss(rows, hidden, ladder, spec, self.device, budget_s=budget_s, overlap_backward=overlap_backward)
        # Staging buffers for peers' blocks: with the overlap a block is still read by its gradient GEMM while the block
        # after it is scored and the one after that is pulled, hence three.
        self._slots = 3 if self.loss.overlap_backward else 2
        k = ladder.count
        block_bytes = rows * hidden * 2
        if domain is not None:
            if domain.payload_scalars < SUMMAND_SLOTS:
                raise ValueError(f"the domain's payload must hold at least {SUMMAND_SLOTS} scalars")
            self._embeddings_offset = domain.alloc(block_bytes)
            self._norms_offset = domain.alloc(BlockNorms.scalars_for(k, rows) * 4)
            self.embeddings = domain.tensor(self._embeddings_offset, (rows, hidden), torch.bfloat16)
            norms_storage = domain.tensor(self._norms_offset, (BlockNorms.scalars_for(k, rows),), torch.float32)
            self.summands = domain.payload()[:SUMMAND_SLOTS]
            self.members, self.member = domain.members, domain.member
        else:
            self.embeddings = torch.empty(rows, hidden, dtype=torch.bfloat16, device=self.device)
            norms_storage = torch.empty(BlockNorms.scalars_for(k, rows), dtype=torch.float32, device=self.device)
            self.summands = torch.zeros(SUMMAND_SLOTS, dtype=torch.float32, device=self.device)
            self.members, self.member = 1, 0
        self.norms = BlockNorms(k, rows, norms_storage)
        self.staged = [torch.empty(rows, hidden, dtype=torch.bfloat16, device=self.device) for _ in range(self._slots)]
        self.staged_norms = [BlockNorms(k, rows, device=self.device) for _ in range(self._slots)]
        self.gradient = torch.empty(rows, hidden, dtype=torch.bfloat16, device=self.device)
        self._cursor = 0
        self.use_graphs = False
        self._graphs = {}

    @staticmethod
    def heap_bytes(rows: int, hidden: int, prefixes: int) -> int:
        """Symmetric heap a ``BoxLoss`` takes from its domain."""
        return rows * hidden * 2 + BlockNorms.scalars_for(prefixes, rows) * 4 + 1024

    def bytes(self) -> int:
        own = sum(t.numel() * t.element_size() for t in self.staged) + sum(n.nbytes for n in self.staged_norms)
        return self.loss.bytes() + own + self.gradient.numel() * 2

    def _pull(self, block: SourceBlock, slot: int) -> PullRequest:
        return PullRequest(self.domain.address(block.embeddings_offset, block.member), self.staged[slot].data_ptr(),
                           self.rows * self.hidden * 2, self.domain.address(block.norms_offset, block.member),
                           self.staged_norms[slot].storage.data_ptr(), self.staged_norms[slot].nbytes)

    def score_sequence(self, blocks: Sequence[SourceBlock], query_base: int, live: int, beta: float, bias: float,
                       scalars: Optional[torch.Tensor] = None, stream=None) -> None:
        """Scores ``blocks`` in order. A block in a peer's replica is pulled into a staging buffer by the forward launch of
        the block before it, so only a remote block in first position costs a launch of its own. The staging buffers are
        used in rotation across calls, so that a buffer is written again only once every kernel reading it has finished
        (two buffers when the gradient GEMM runs in line, three when it overlaps the next block's forward)."""
        from .._ext import native

        ahead = None  # the staging slot that the previous block's launch filled with this block
        for index, block in enumerate(blocks):
            if block.local:
                candidates, norms = block.embeddings, block.norms
            else:
                if ahead is None:
                    ahead = self._take_slot()
                    request = self._pull(block, ahead)
                    native().pull(request.src0, request.dst0, request.bytes0, request.src1, request.dst1, request.bytes1,
                                  self.loss.multiprocessors, (torch.cuda.current_stream() if stream is None else stream).cuda_stream)
                candidates, norms = self.staged[ahead], self.staged_norms[ahead]
            following = blocks[index + 1] if index + 1 < len(blocks) else None
            pull, ahead = None, None
            if following is not None and not following.local:
                ahead = self._take_slot()
                pull = self._pull(following, ahead)
            with phase(f"score block at {block.candidate_base}" + (" + pull of the next" if pull is not None else "")):
                self.loss.score(self.embeddings, candidates, query_base, block.candidate_base, beta, bias, live, stream,
                                candidate_norms=norms, scalars=scalars, pull_next=pull)

    def _take_slot(self) -> int:
        self._cursor = (self._cursor + 1) % self._slots
        return self._cursor

    # ------------------------------------------------------------------------------------------------------
    def _core(self, beta: float, bias: float, scalars: Optional[torch.Tensor], gradient: torch.Tensor, reduce: bool,
              stream) -> None:
        """Everything of a step after the publish pass. It touches only buffers this object (or its domain) owns plus
        ``scalars`` and ``gradient``, which is what makes it replayable as a CUDA graph."""
        members, member, rows = self.members, self.member, self.rows
        if self.domain is not None:
            with phase("barrier: every block is published"):
                self.domain.barrier(stream)
        self.loss.begin(self.embeddings, stream, query_norms=self.norms)
        blocks: List[SourceBlock] = [SourceBlock(member * rows, self.embeddings, self.norms)]
        for p in range(1, members):
            peer = (member + p) % members
            blocks.append(SourceBlock(peer * rows, member=peer, embeddings_offset=self._embeddings_offset,
                                      norms_offset=self._norms_offset))
        self.score_sequence(blocks, member * rows, members * rows, beta, bias, scalars, stream)
        with phase("finish: self term, cast, summands"):
            self.loss.finish(self.embeddings, gradient, self.summands, stream)
        if self.domain is not None:
            # Either collective closes the step: its rounds are also the fence that says "every peer has finished
            # reading my block", without which the next step's publish could overwrite a block still being pulled.
            if reduce:
                self.domain.all_reduce(SUMMAND_SLOTS, stream)
            else:
                self.domain.barrier(stream)

    def step(self, queries: torch.Tensor, beta: float = 10.0, bias: float = -10.0, scalars: Optional[torch.Tensor] = None,
             gradient_out: Optional[torch.Tensor] = None, stream=None, reduce: bool = True,
             graph: Optional[bool] = None) -> Tuple[torch.Tensor, torch.Tensor]:
        """Runs one step; returns ``(gradient [R,H] bf16, summands [SUMMAND_SLOTS] f32)``. With ``reduce`` the summands
        are the world's sums on return (stream order); without it they are this rank's share and a barrier closes the
        step instead.

        With ``graph`` (default: the object's ``use_graphs``) everything after the publish pass is captured once per
        argument set as a CUDA graph and replayed afterwards, so a step costs the host two launches however many
        blocks it scores; the first call of an argument set runs eagerly, the second captures. Every member of the
        domain must make the same choice in the same step."""
        with phase("publish: prefix norms + copy into symmetric memory"):
            compute_block_norms(queries, self.ladder, self.norms, copy_to=self.embeddings, stream=stream)
        gradient = self.gradient if gradient_out is None else gradient_out
        _check_gradient(gradient, self.rows, self.hidden)
        if (self.use_graphs if graph is None else graph) and stream is None:
            self._replay(float(beta), float(bias), scalars, gradient, bool(reduce))
        else:
            self._core(beta, bias, scalars, gradient, reduce, stream)
        return gradient, self.summands

    def _replay(self, beta: float, bias: float, scalars: Optional[torch.Tensor], gradient: torch.Tensor, reduce: bool) -> None:
        from .._ext import native

        key = (beta, bias, 0 if scalars is None else scalars.data_ptr(), gradient.data_ptr(), reduce)
        entry = self._graphs.get(key)
        if entry is None:
            # First use: run eagerly (loads every kernel, fills the tensor-map cache) and remember that it happened.
            self._core(beta, bias, scalars, gradient, reduce, None)
            if len(self._graphs) >= 8:
                self._graphs.clear()
            self._graphs[key] = False
            return
        if entry is False:
            ext = native()
            graph = torch.cuda.CUDAGraph()
            before = ext.launch_count()
            with torch.cuda.graph(graph):
                self._core(beta, bias, scalars, gradient, reduce, None)
            # The launchers counted their kernels while capturing, although nothing ran: that count stands for the replay
            # that follows, and later replays add it themselves. `scalars` and `gradient` are kept alive with the graph.
            self._graphs[key] = (graph, int(ext.launch_count() - before), scalars, gradient)
            graph.replay()
            return
        entry[0].replay()
        native().note_launches(entry[1])

    def simulate(self, queries: torch.Tensor, world: int, beta: float = 10.0, bias: float = -10.0, stream=None,
                 pull: bool = True) -> Tuple[torch.Tensor, torch.Tensor]:
        """One rank of a ``world``-GPU step on this GPU alone: the own block stands in for every peer's."""
        rows = self.rows
        compute_block_norms(queries, self.ladder, self.norms, copy_to=self.embeddings, stream=stream)
        self.loss.begin(self.embeddings, stream, query_norms=self.norms)
        for block in range(world):
            if block == 0 or not pull:
                candidates, norms = self.embeddings, self.norms
            else:
                candidates, norms = self.staged[(block - 1) % self._slots], self.staged_norms[(block - 1) % self._slots]
            request = None
            if pull and block + 1 < world:
                slot = block % self._slots
                request = PullRequest(self.embeddings.data_ptr(), self.staged[slot].data_ptr(), rows * self.hidden * 2,
                                      self.norms.storage.data_ptr(), self.staged_norms[slot].storage.data_ptr(),
                                      self.staged_norms[slot].nbytes)
            self.loss.score(self.embeddings, candidates, 0, block * rows, beta, bias, world * rows, stream,
                            candidate_norms=norms, pull_next=request)
        self.loss.finish(self.embeddings, self.gradient, self.summands, stream)
        return self.gradient, self.summands

    def check(self) -> None:
        self.loss.check()
        if self.domain is not None:
            self.domain.check()
