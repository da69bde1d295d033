"""The cross-box rail: one connection between a GPU of this host and the same-numbered GPU of another host.

``RdmaRail`` keeps the reference's interface and ordering rules: ``local`` is the endpoint record to publish,
``connect`` takes the peer's record, ``post_embeddings(parity)`` writes this GPU's block into the peer's landing buffer
of that parity (two buffers alternate between steps, so a block may land while the previous one is still being read),
``post_summands`` writes one row of loss summands into the peer's host-side table, ``await_landed`` consumes one
completion. ``exchange_endpoint`` is the filesystem rendezvous: a record is written as ``*.partial`` and renamed, the
counterpart is polled every 10 ms with a two-minute deadline.

This box has one host and no RDMA NIC (no libibverbs, no ``/sys/class/infiniband``), so the only transport built here
is the loopback one (``csrc/rail.cpp``): device-to-device copies into memory the peer exported, completions through a
shared-memory queue. A verbs transport would implement the same five calls; real-NIC behaviour is untested here.

Parity: ``rdma_rail_t`` / ``rdma_endpoint_t`` (scalingcontrasts.cuh:419-646), ``exchange_endpoint``
(scalingcontrasts.cu:224-249).
"""
from __future__ import annotations

import errno
import os
import time
import uuid
from typing import List, Optional, Sequence

import torch

from .._ext import native

RENDEZVOUS_DEADLINE_S = 120.0
RENDEZVOUS_POLL_S = 0.010


class RailError(RuntimeError):
    pass


class RdmaRail:
    """One rail over the loopback transport."""

    def __init__(self, embeddings: torch.Tensor, landing: torch.Tensor, hosts: int, host: int,
                 packet_sequence: Optional[int] = None, name: Optional[str] = None) -> None:
        if embeddings.dim() != 2 or not embeddings.is_contiguous() or not embeddings.is_cuda:
            raise ValueError("embeddings must be a contiguous CUDA matrix [R, H]")
        rows, hidden = embeddings.shape
        if tuple(landing.shape) != (2, rows, hidden) or landing.dtype != embeddings.dtype or not landing.is_contiguous():
            raise ValueError("landing must be a contiguous [2, R, H] tensor of the embeddings' dtype")
        self.embeddings, self.landing = embeddings, landing
        self.hosts, self.host = hosts, host
        self.block_bytes = rows * hidden * embeddings.element_size()
        self.mailbox = name or f"/sc-rail-{os.getpid()}-{uuid.uuid4().hex[:12]}"
        sequence = packet_sequence if packet_sequence is not None else int.from_bytes(os.urandom(3), "little")
        self._native = native().LoopbackRail(embeddings.device.index, embeddings.data_ptr(), self.block_bytes,
                                             landing.data_ptr(), hosts, host, self.mailbox, sequence)

    @property
    def local(self) -> bytes:
        """The endpoint record to hand to the peer."""
        return self._native.local_endpoint()

    def connect(self, endpoint: bytes) -> None:
        self._native.connect(endpoint)

    def post_embeddings(self, parity: int, stream=None) -> None:
        stream = torch.cuda.current_stream(self.embeddings.device) if stream is None else stream
        self._native.post_embeddings(int(parity), stream.cuda_stream)

    def post_summands(self, host: int, values: Sequence[float]) -> None:
        self._native.post_summands(int(host), [float(v) for v in values])

    def await_landed(self, timeout_s: float = 30.0) -> int:
        """Blocks until one completion arrives and returns its immediate data (the byte count). Raises ``RailError`` on a
        timeout or an error completion."""
        try:
            return int(self._native.await_landed(float(timeout_s)))
        except RuntimeError as error:
            raise RailError(str(error)) from error

    def read_summands(self, host: int, count: int = 4) -> List[float]:
        return list(self._native.read_summands(int(host), int(count)))

    def inject_completion_error(self, status: int) -> None:
        """Host-side fault injection: the next completion this side produces reports ``status`` instead of success."""
        self._native.inject_completion_error(int(status))

    def drain(self) -> None:
        self._native.drain()

    def close(self) -> None:
        self._native.close()


def exchange_endpoint(directory: str, own_host: int, remote_host: int, gpu: int, record: bytes,
                      deadline_s: float = RENDEZVOUS_DEADLINE_S) -> bytes:
    """Publishes ``record`` as ``endpoint-<own>-<remote>-<gpu>`` and returns the counterpart
    ``endpoint-<remote>-<own>-<gpu>``; raises ``TimeoutError`` (``ETIMEDOUT``) when it does not show up in time."""
    os.makedirs(directory, exist_ok=True)
    mine = os.path.join(directory, f"endpoint-{own_host}-{remote_host}-{gpu}")
    theirs = os.path.join(directory, f"endpoint-{remote_host}-{own_host}-{gpu}")
    with open(mine + ".partial", "wb") as handle:
        handle.write(record)
        handle.flush()
        os.fsync(handle.fileno())
    os.replace(mine + ".partial", mine)
    expected = len(record)
    deadline = time.monotonic() + deadline_s
    while True:
        try:
            with open(theirs, "rb") as handle:
                data = handle.read()
            if len(data) == expected:
                return data
        except FileNotFoundError:
            pass
        if time.monotonic() > deadline:
            raise TimeoutError(errno.ETIMEDOUT, f"endpoint {theirs} never appeared")
        time.sleep(RENDEZVOUS_POLL_S)
