"""``ContrastiveTrainer``: the headline training step as one public call.

A step is: projector forward on a batch of rows, the box-wide Matryoshka sigmoid loss (streamed over every GPU's
block), backward through the projector with the parameter gradients all-reduced on a side stream while backward still
runs, and the optimizer update. Batches come from pinned host memory: ``feed`` starts the host-to-device copy of a batch
on a copy stream (so the copy of batch t+1 hides under step t), ``step`` consumes the oldest fed batch and starts the
device-to-host copy of its loss into pinned memory.

The reference benchmarks a loss step only (scalingcontrasts.cu:294-311); a model, an optimizer and checkpoints are what
a training framework adds around it.
"""
from __future__ import annotations

from collections import deque
from typing import Deque, Dict, Optional, Tuple

import torch

from .config import LossSpec, REFERENCE_SPEC
from .ladder import Matryoshka
from .models.loss import MatryoshkaSigmoidLoss
from .models.projector import Projector
from .parallel.reducer import GradientReducer
from .utils.trace import phase


class ContrastiveTrainer:
    def __init__(self, rows: int, in_features: int = 1024, mid_features: int = 3072, hidden: int = 768, prefixes: int = 5,
                 spec: LossSpec = REFERENCE_SPEC, lr: float = 1e-4, weight_decay: float = 0.0, group=None, device=None,
                 seed: int = 0, multicast: Optional[bool] = None, optimizer: str = "adamw", graphs: bool = True) -> None:
        from .parallel.box import BoxLoss
        from .parallel.domain import Domain

        self.rows, self.in_features, self.hidden = rows, in_features, hidden
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.ladder = Matryoshka.halvings(hidden, prefixes)
        self.projector = Projector(in_features, mid_features, hidden, torch.bfloat16, self.device, seed)
        heap = BoxLoss.heap_bytes(rows, hidden, prefixes) + GradientReducer.heap_bytes(self.projector.parameters())
        self.domain = Domain.create(payload_scalars=16, heap_bytes=heap, group=group, device=self.device, multicast=multicast)
        self.world, self.rank = self.domain.members, self.domain.member
        self.loss = MatryoshkaSigmoidLoss(rows, hidden, prefixes, self.ladder, spec, self.domain, group, self.device)
        # The loss step after its publish pass is the same kernel sequence over the same buffers every time: replayed as
        # a CUDA graph it costs the host two launches however many peers are scored.
        self.loss.engine.use_graphs = graphs
        self.loss.unit_upstream = True  # step_on_device() calls loss.backward() on the bare loss
        # Every rank's loss is the world's sum and row gradients are final, so parameter gradients are summed.
        self.reducer = GradientReducer(self.projector.parameters(), self.domain, scale=1.0)
        self.projector.gradient_landing = self.reducer.landing_buffers(self.projector) or None
        parameters = list(self.projector.parameters()) + list(self.loss.parameters())
        if optimizer == "adamw":
            from .optim import FusedAdamW

            self.optimizer = FusedAdamW(parameters, lr=lr, weight_decay=weight_decay)  # one own launch per step
        elif optimizer == "adamw-torch":
            self.optimizer = torch.optim.AdamW(parameters, lr=lr, weight_decay=weight_decay, fused=True)
        elif optimizer == "sgd":
            self.optimizer = torch.optim.SGD(parameters, lr=lr, momentum=0.9)
        else:
            raise ValueError("optimizer must be adamw, adamw-torch or sgd")
        self.steps_done = 0
        self._copy_stream = torch.cuda.Stream(device=self.device)
        self._slots = [torch.empty(rows, in_features, dtype=torch.bfloat16, device=self.device) for _ in range(2)]
        self._slot_free = [torch.cuda.Event() for _ in range(2)]
        self._fed: Deque[Tuple[int, torch.cuda.Event]] = deque()
        self._next_slot = 0
        self._loss_host = torch.zeros(2, 16, dtype=torch.float32).pin_memory()
        # Status words of the tile kernels and of the two collective channels travel to the host with every loss, so a
        # wait that ran out (a peer that stopped) surfaces one step later without an extra synchronisation.
        self._status_sources = [self.loss.engine.loss.status]
        if hasattr(self.domain, "status_view"):
            self._status_sources += [self.domain.status_view(0), self.domain.status_view(1)]
        self._status_host = torch.zeros(2, len(self._status_sources), 8, dtype=torch.int32).pin_memory()
        # One report per step: the summands and the status blocks are gathered into one device buffer by the library's
        # span-copy kernel (two spans per launch) and cross to the host as a single copy.
        self._report = torch.zeros(16 + 8 * len(self._status_sources), dtype=torch.int32, device=self.device)
        self._report_host = torch.zeros(2, self._report.numel(), dtype=torch.int32).pin_memory()
        self._loss_events = [torch.cuda.Event(), torch.cuda.Event()]
        self._loss_pending: Deque[int] = deque()
        for event in self._slot_free:
            event.record()

    # -- data path --------------------------------------------------------------------------------------------
    def feed(self, batch: torch.Tensor) -> None:
        """Starts the host-to-device copy of one batch (pinned ``[rows, in_features]`` bfloat16) on the copy stream."""
        if batch.device.type != "cpu" or tuple(batch.shape) != (self.rows, self.in_features) or batch.dtype != torch.bfloat16:
            raise ValueError(f"a batch is a host bfloat16 tensor of shape [{self.rows}, {self.in_features}]")
        if len(self._fed) >= 2:
            raise RuntimeError("at most two batches may be in flight; call step() before feeding a third")
        slot = self._next_slot
        self._next_slot ^= 1
        self._copy_stream.wait_event(self._slot_free[slot])
        with torch.cuda.stream(self._copy_stream):
            self._slots[slot].copy_(batch, non_blocking=True)
            landed = torch.cuda.Event()
            landed.record(self._copy_stream)
        self._fed.append((slot, landed))

    def step(self, batch: Optional[torch.Tensor] = None) -> Optional[float]:
        """Runs one training step on the oldest fed batch (feeding ``batch`` first when given). Returns the loss of the
        previous step, whose device-to-host copy has had a whole step to land, or None on the first call."""
        if batch is not None:
            self.feed(batch)
        if not self._fed:
            raise RuntimeError("step() without a fed batch")
        slot, landed = self._fed.popleft()
        torch.cuda.current_stream().wait_event(landed)
        loss = self.step_on_device(self._slots[slot])
        self._slot_free[slot].record()
        previous = self._collect_loss()
        index = self.steps_done % 2
        self._gather_report()
        self._report_host[index].copy_(self._report, non_blocking=True)
        self._loss_events[index].record()
        self._loss_pending.append(index)
        return previous

    def _gather_report(self) -> None:
        from ._ext import native

        ext, stream = native(), torch.cuda.current_stream().cuda_stream
        base = self._report.data_ptr()
        spans = [(self.loss.last_summands.data_ptr(), base, 48)]
        spans += [(source.data_ptr(), base + 64 + 32 * position, 32) for position, source in enumerate(self._status_sources)]
        for first in range(0, len(spans), 2):
            a = spans[first]
            b = spans[first + 1] if first + 1 < len(spans) else (0, 0, 0)
            ext.pull(a[0], a[1], a[2], b[0], b[1], b[2], 1, stream)

    def step_on_device(self, x: torch.Tensor) -> torch.Tensor:
        """One step on a batch that already lives on the device; returns the loss as a device scalar."""
        self.optimizer.zero_grad(set_to_none=True)
        with phase("projector forward"):
            embeddings = self.projector(x)
        with phase("loss step"):
            loss = self.loss(embeddings)
        with phase("backward + overlapped gradient all-reduce"):
            loss.backward()
            self.reducer.wait()
        with phase("optimizer"):
            self.optimizer.step()
        self.steps_done += 1
        return loss

    def _collect_loss(self) -> Optional[float]:
        if not self._loss_pending:
            return None
        index = self._loss_pending.popleft()
        self._loss_events[index].synchronize()
        report = self._report_host[index]
        self._loss_host[index, :12] = report[:12].view(torch.float32)
        self._status_host[index] = report[16:].view(len(self._status_sources), 8)
        codes = self._status_host[index, :, 0].tolist()
        if any(codes):
            names = ["loss kernels", "loss collectives", "gradient reducer"]
            failed = ", ".join(f"{names[i]}: {self._status_host[index, i].tolist()}" for i, code in enumerate(codes) if code)
            raise RuntimeError(f"a bounded device wait ran out during a training step ({failed})")
        return float(self._loss_host[index, 0])

    def last_loss(self) -> Optional[float]:
        """The newest loss (synchronises on its copy)."""
        value = None
        while self._loss_pending:
            value = self._collect_loss()
        return value

    # -- accounting -------------------------------------------------------------------------------------------
    def cells_per_step(self) -> int:
        return self.loss.cells_per_step(self.world)

    def h2d_bytes_per_step(self) -> int:
        return self.rows * self.in_features * 2

    def d2h_bytes_per_step(self) -> int:
        return self._report.numel() * 4

    # -- checkpoints ------------------------------------------------------------------------------------------
    def state_dict(self) -> Dict[str, object]:
        return {"projector": self.projector.state_dict(), "loss": self.loss.state_dict(),
                "optimizer": self.optimizer.state_dict(), "step": self.steps_done,
                "ladder": list(self.ladder.ends)}

    def load_state_dict(self, state: Dict[str, object]) -> None:
        self.projector.load_state_dict(state["projector"])
        self.loss.load_state_dict(state["loss"])
        self.optimizer.load_state_dict(state["optimizer"])
        self.steps_done = int(state["step"])

    def check(self) -> None:
        self.loss.engine.check()

    def close(self) -> None:
        torch.cuda.synchronize(self.device)
        self.reducer.remove()
        self.domain.close()

