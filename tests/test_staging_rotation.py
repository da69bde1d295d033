"""Host-side order of the staging buffers that peers' blocks are pulled into (``BoxLoss.score_sequence``), checked on CPU
with the device calls replaced by recorders: a buffer may be written by a pull only when no kernel that is still running
reads it. In line (two buffers) that is the block being scored; with the gradient GEMM overlapped (three buffers) also the
block before it, whose GEMM runs beside this block's forward."""
from __future__ import annotations

import random
from types import SimpleNamespace

import pytest

from scalingcontrasts_b200.ops.streamed_loss import PullRequest
from scalingcontrasts_b200.parallel import box as box_module
from scalingcontrasts_b200.parallel.box import BoxLoss, SourceBlock


class _Recorder:
    multiprocessors = 1

    def __init__(self):
        self.steps = []  # per scored block: (slot read or None, slots filled ahead of it, slots written while it is scored)
        self.pending_writes = []

    # stands in for the native module: a pull launched by itself, ahead of the block it feeds
    def pull(self, src0, dst0, bytes0, src1, dst1, bytes1, multiprocessors, stream):
        self.pending_writes.append(dst0)

    # stands in for StreamedLoss.score
    def score(self, queries, candidates, query_base, candidate_base, beta, bias, live, stream, *, candidate_norms, scalars,
              pull_next):
        ahead = list(self.pending_writes)
        self.pending_writes.clear()
        during = [pull_next.dst0] if pull_next is not None else []
        self.steps.append((candidates if isinstance(candidates, int) else None, ahead, during))


def _engine(slots: int, recorder: _Recorder) -> BoxLoss:
    engine = object.__new__(BoxLoss)
    engine._slots, engine._cursor = slots, 0
    engine.staged = list(range(slots))        # a staging buffer is represented by its slot number
    engine.staged_norms = list(range(slots))
    engine.embeddings = "own"
    engine.loss = recorder
    engine._pull = lambda block, slot: PullRequest(src0=1, dst0=slot, bytes0=16)
    return engine


@pytest.mark.parametrize("slots,readers", [(2, 1), (3, 2)])
def test_a_pull_never_overwrites_a_buffer_that_a_running_kernel_reads(monkeypatch, slots, readers):
    recorder = _Recorder()
    monkeypatch.setattr("scalingcontrasts_b200._ext.native", lambda: recorder)
    engine = _engine(slots, recorder)
    generator = random.Random(7)
    stream = SimpleNamespace(cuda_stream=0)
    for _ in range(50):  # sequences as the box step and the hosts step form them, and arbitrary mixes, back to back
        length = generator.randint(1, 9)
        blocks = [SourceBlock(128 * i, "local", "norms") if generator.random() < 0.3 else
                  SourceBlock(128 * i, member=1, embeddings_offset=0, norms_offset=0) for i in range(length)]
        engine.score_sequence(blocks, 0, 1024, 10.0, -10.0, None, stream)
    assert len(recorder.steps) > 100
    def reads(first, last):
        return {recorder.steps[k][0] for k in range(max(0, first), last + 1)} - {None}

    for index, (read, ahead, during) in enumerate(recorder.steps):
        # a pull inside block i's forward launch runs beside that forward and, overlapped, beside block i-1's GEMM
        assert not (set(during) & reads(index - readers + 1, index)), (index, during)
        # a pull launched ahead of block i follows block i-1's forward in stream order; in line nothing else is running,
        # overlapped the GEMMs of blocks i-1 and i-2 may be
        if readers == 2:
            assert not (set(ahead) & reads(index - 2, index - 1)), (index, ahead)
        # and a remote block is scored from the buffer its pull was aimed at
        if read is not None:
            aimed = ahead + (recorder.steps[index - 1][2] if index else [])
            assert read in aimed, (index, read, aimed)


def test_module_is_importable_without_a_gpu():
    assert hasattr(box_module, "BoxLoss")
