"""Domains: the collective interface of one box (barrier, reduce-scatter, all-reduce over a symmetric payload).

Three implementations share one interface:

* ``MultimemDomain`` - every GPU's replica is bound to one NVSwitch multicast object; the collectives are single
  kernels built on ``multimem.ld_reduce / st / red``. One process per GPU: physical allocations and the multicast
  object cross processes as POSIX file descriptors over a Unix socket (``SCM_RIGHTS``), rendezvous through the
  ``torch.distributed`` store.
* ``PeerDomain`` - the same replicas mapped peer to peer without a multicast object; arrivals are remote atomics and
  reductions read every peer in member order. Used where the fabric has no multicast, or when it is switched off.
* ``HostDomain`` - CPU tensors and a ``gloo`` group (or a single process): the twin used by CPU ranks and tests.

``Domain.create`` picks the first that the machine supports. Beside the payload, a GPU domain is a small symmetric
heap: ``alloc`` hands out offsets that mean the same thing in every member's replica, ``tensor`` views them.

Every device-side wait is bounded (``budget_s``); when one runs out the kernel records it in the member's status
block and later collectives return at once. ``check()`` turns a recorded failure into a Python exception.

Parity: ``multimem_domain_t`` (scalingcontrasts.cuh:244-410), Mojo ``Collective`` / ``MultimemDomain`` /
``PeerDomain`` (scalingcontrasts.mojo:308-385, 388-548, 732-873).
"""
from __future__ import annotations

import os
import socket
import struct
import time
import uuid
from typing import List, Optional, Sequence

import torch

from .._ext import native

CONTROL_REGION = 4096  # bytes reserved at the start of every replica for the control block
LATENCY_SLOT_BYTES = 64 << 10  # largest payload of the one-round all-reduce
LATENCY_CHANNELS = 4  # control channels that own a staging area for it
_TYPE_CODES = {torch.float32: 0, torch.bfloat16: 1}
_DTYPE_NAMES = {torch.float32: "float32", torch.bfloat16: "bfloat16", torch.int32: "int32", torch.uint8: "uint8",
                torch.int64: "int64"}

STATUS_NAMES = {0: "ok", 1: "timeout in a collective (a member never arrived)",
                2: "timeout in a tile kernel's pipeline", 3: "bad argument"}


class DomainError(RuntimeError):
    """A device-side wait ran out, or the domain could not be formed."""


def default_budget_s() -> float:
    return float(os.environ.get("SC_WAIT_BUDGET_MS", "2000")) / 1000.0


# ---------------------------------------------------------------------------------------------------------------
# host-side rendezvous helpers (no GPU involved)
# ---------------------------------------------------------------------------------------------------------------
class StoreRendezvous:
    """Barriers and small broadcasts through the torch.distributed key-value store; works for any backend."""

    _serial = 0

    def __init__(self, group=None, timeout_s: float = 120.0) -> None:
        import torch.distributed as dist

        self.group = group
        self.timeout_s = timeout_s
        if dist.is_available() and dist.is_initialized():
            self.rank = dist.get_rank(group)
            self.world = dist.get_world_size(group)
            self.store = dist.distributed_c10d._get_default_store()
            ranks = dist.get_process_group_ranks(group) if group is not None else list(range(self.world))
            self.prefix = "sc/" + "-".join(str(r) for r in ranks[:4]) + f"/{len(ranks)}/"
        else:
            self.rank, self.world, self.store, self.prefix = 0, 1, None, "sc/"

    def _key(self, name: str) -> str:
        return self.prefix + name

    def next_tag(self, name: str) -> str:
        StoreRendezvous._serial += 1
        return f"{name}#{StoreRendezvous._serial}"

    def barrier(self, tag: str) -> None:
        if self.world == 1:
            return
        key = self._key("barrier/" + tag)
        self.store.add(key, 1)
        deadline = time.monotonic() + self.timeout_s
        while int(self.store.add(key, 0)) < self.world:
            if time.monotonic() > deadline:
                raise DomainError(f"rendezvous barrier {tag!r} timed out: a rank never joined")
            time.sleep(0.001)

    def broadcast(self, tag: str, value: Optional[bytes]) -> bytes:
        if self.world == 1:
            return value or b""
        key = self._key("bcast/" + tag)
        if self.rank == 0:
            self.store.set(key, value or b"")
        self.store.wait([key])
        return bytes(self.store.get(key))

    def all_agree(self, tag: str, ok: bool) -> bool:
        """True iff every rank reports ok."""
        if self.world == 1:
            return ok
        key = self._key("agree/" + tag)
        self.store.add(key, 1 if ok else 0)
        self.barrier(tag + "/b")
        return int(self.store.add(key, 0)) == self.world


def _exchange_descriptors(rendezvous: StoreRendezvous, own_descriptor: int, make_multicast) -> tuple:
    """Member 0 collects every member's descriptor over a Unix socket and hands everyone the full list, plus the
    multicast object's descriptor when ``make_multicast`` (called on member 0 only) returns one.
    Returns ``(descriptors by member, multicast descriptor or -1)``; the caller closes them."""
    world, rank = rendezvous.world, rendezvous.rank
    if world == 1:
        multicast = make_multicast() if make_multicast is not None else -1
        return [own_descriptor], multicast
    tag = rendezvous.next_tag("fds")
    name = rendezvous.broadcast(tag, uuid.uuid4().hex.encode() if rank == 0 else None).decode()
    address = "\0sc-domain-" + name
    if rank == 0:
        server = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
        server.bind(address)
        server.listen(world)
        server.settimeout(rendezvous.timeout_s)
        rendezvous.barrier(tag + "/listening")
        descriptors: List[int] = [-1] * world
        descriptors[0] = own_descriptor
        connections = {}
        try:
            for _ in range(world - 1):
                connection, _ = server.accept()
                connection.settimeout(rendezvous.timeout_s)
                message, received, _, _ = socket.recv_fds(connection, 16, 1)
                peer = struct.unpack("i", message[:4])[0]
                descriptors[peer] = received[0]
                connections[peer] = connection
            multicast = make_multicast() if make_multicast is not None else -1
            outgoing = list(descriptors) + ([multicast] if multicast >= 0 else [])
            for peer, connection in connections.items():
                socket.send_fds(connection, [struct.pack("ii", world, 1 if multicast >= 0 else 0)], outgoing)
        finally:
            for connection in connections.values():
                connection.close()
            server.close()
        return descriptors, multicast
    rendezvous.barrier(tag + "/listening")
    client = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
    client.settimeout(rendezvous.timeout_s)
    client.connect(address)
    try:
        socket.send_fds(client, [struct.pack("i", rank)], [own_descriptor])
        message, received, _, _ = socket.recv_fds(client, 16, world + 1)
        count, has_multicast = struct.unpack("ii", message[:8])
        if count != world or len(received) != world + has_multicast:
            raise DomainError("descriptor exchange returned a malformed reply")
        multicast = received[world] if has_multicast else -1
        os.close(received[rank])  # a duplicate of our own
        descriptors = list(received[:world])
        descriptors[rank] = own_descriptor
        return descriptors, multicast
    finally:
        client.close()


# ---------------------------------------------------------------------------------------------------------------
# the interface
# ---------------------------------------------------------------------------------------------------------------
class Domain:
    """Collective interface; see the module docstring. Use ``Domain.create``."""

    members: int
    member: int
    payload_scalars: int

    @staticmethod
    def create(payload_scalars: int = 16, heap_bytes: int = 0, group=None, device=None, multicast: Optional[bool] = None,
               budget_s: Optional[float] = None) -> "Domain":
        """Forms a domain over the ranks of ``group`` (default: the whole job). On CUDA devices this is a
        ``MultimemDomain`` when every member supports multicast (and ``multicast`` is not False), else a
        ``PeerDomain``; on the CPU a ``HostDomain``."""
        if device is None:
            device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
        device = torch.device(device)
        if device.type == "cpu":
            return HostDomain(payload_scalars, group)
        if multicast is None:
            multicast = os.environ.get("SC_MULTICAST", "1") != "0"
        return DeviceDomain._form(payload_scalars, heap_bytes, group, device, multicast, budget_s)

    # collectives -----------------------------------------------------------------------------------------
    def payload(self, member: Optional[int] = None) -> torch.Tensor:
        raise NotImplementedError

    def barrier(self, stream=None) -> None:
        raise NotImplementedError

    def all_reduce(self, scalars: Optional[int] = None, stream=None) -> None:
        raise NotImplementedError

    def reduce_scatter(self, shard_scalars: int, stream=None) -> None:
        raise NotImplementedError

    def check(self) -> None:
        pass

    def close(self) -> None:
        pass

    def replica_bytes(self) -> int:
        raise NotImplementedError


class DeviceDomain(Domain):
    """Symmetric memory on GPUs; ``MultimemDomain`` and ``PeerDomain`` differ only in how the kernels reach peers."""

    uses_multicast = False

    def __init__(self) -> None:  # use _form
        self._native = None

    @classmethod
    def _form(cls, payload_scalars: int, heap_bytes: int, group, device: torch.device, want_multicast: bool,
              budget_s: Optional[float]) -> "DeviceDomain":
        ext = native()
        rendezvous = StoreRendezvous(group)
        payload_bytes = -(-payload_scalars * 4 // 256) * 256
        heap_end = CONTROL_REGION + payload_bytes + int(heap_bytes)
        heap_end = -(-heap_end // 256) * 256
        # Staging area of the one-round all-reduce: per channel two sets (used alternately) of one slot per member.
        total = heap_end + LATENCY_CHANNELS * 2 * rendezvous.world * LATENCY_SLOT_BYTES
        index = device.index if device.index is not None else torch.cuda.current_device()
        torch.cuda.set_device(index)
        supported = bool(ext.NativeDomain.multicast_supported(index)) if want_multicast else False
        want = rendezvous.all_agree(rendezvous.next_tag("mc-supported"), supported) if want_multicast else False
        handle = ext.NativeDomain(index, rendezvous.rank, rendezvous.world, total, want)
        own = handle.export_replica()
        multicast_ok = want
        notes: List[str] = [] if want else (["multicast not requested"] if not want_multicast else
                                            ["a member's device reports no multicast support"])
        descriptors: Sequence[int] = []
        multicast_descriptor = -1

        def make_multicast() -> int:
            nonlocal multicast_ok
            if not want:
                return -1
            try:
                return handle.create_multicast()
            except RuntimeError as error:
                multicast_ok = False
                notes.append(str(error))
                return -1

        try:
            descriptors, multicast_descriptor = _exchange_descriptors(rendezvous, own, make_multicast)
            for peer, descriptor in enumerate(descriptors):
                if peer != rendezvous.rank:
                    handle.import_replica(peer, descriptor)
            if want:
                try:
                    if rendezvous.rank != 0:
                        if multicast_descriptor < 0:
                            raise RuntimeError("member 0 could not create the multicast object")
                        handle.import_multicast(multicast_descriptor)
                    elif multicast_descriptor < 0:
                        raise RuntimeError("multicast object creation failed")
                    handle.add_device()
                except RuntimeError as error:
                    multicast_ok = False
                    notes.append(str(error))
                multicast_ok = rendezvous.all_agree(rendezvous.next_tag("mc-added"), multicast_ok)
        finally:
            for descriptor in descriptors:
                if descriptor >= 0:
                    os.close(descriptor)
            if multicast_descriptor >= 0:
                os.close(multicast_descriptor)
        handle.map_replicas()
        if want and multicast_ok:
            try:
                handle.bind_multicast()
            except RuntimeError as error:
                multicast_ok = False
                notes.append(str(error))
            multicast_ok = rendezvous.all_agree(rendezvous.next_tag("mc-bound"), multicast_ok)
        handle.zero_own()
        ext.preload_kernels()
        torch.cuda.synchronize(index)
        rendezvous.barrier(rendezvous.next_tag("zeroed"))

        domain = MultimemDomain() if (want and multicast_ok) else PeerDomain()
        domain._native = handle
        domain.multicast_notes = notes  # why a peer domain was formed where a multimem one was asked for
        domain._rendezvous = rendezvous
        domain.device = torch.device("cuda", index)
        domain.members, domain.member = rendezvous.world, rendezvous.rank
        domain.payload_scalars = payload_scalars
        domain._payload_offset = CONTROL_REGION
        domain._heap_next = CONTROL_REGION + payload_bytes
        domain._heap_end = heap_end
        domain._latency_offset = heap_end
        domain.budget_s = default_budget_s() if budget_s is None else budget_s
        domain._control = ext.make_control(handle, 0, int(domain.budget_s * 1e9), domain.uses_multicast)
        domain._channels = {0: domain._control}
        domain.multiprocessors = torch.cuda.get_device_properties(index).multi_processor_count
        domain.stride = handle.stride()
        domain._closed = False
        return domain

    # memory ----------------------------------------------------------------------------------------------
    def replica_bytes(self) -> int:
        return int(self._native.stride())

    def alloc(self, nbytes: int, align: int = 256) -> int:
        """Reserves ``nbytes`` of the symmetric heap and returns its offset. Every member must make the same calls in
        the same order, so that an offset names the same region in every replica."""
        offset = -(-self._heap_next // align) * align
        if offset + nbytes > self._heap_end:
            raise DomainError(f"symmetric heap exhausted: wanted {nbytes} bytes at {offset}, heap ends at {self._heap_end}")
        self._heap_next = offset + nbytes
        return offset

    def address(self, offset: int, member: Optional[int] = None) -> int:
        return int(self._native.replica(self.member if member is None else member)) + offset

    def multicast_address(self, offset: int) -> int:
        return int(self._native.multicast()) + offset if self.uses_multicast else 0

    def tensor(self, offset: int, shape: Sequence[int], dtype: torch.dtype, member: Optional[int] = None) -> torch.Tensor:
        """A view of ``shape`` at ``offset`` of a member's replica (this member's by default). Views of a peer's replica
        are peer memory: read them with this library's kernels or plain elementwise torch ops, never hand them to a
        library GEMM or attention kernel."""
        return native().tensor_from_pointer(self.address(offset, member), list(shape), _DTYPE_NAMES[dtype], self.device.index)

    def payload(self, member: Optional[int] = None) -> torch.Tensor:
        return self.tensor(self._payload_offset, (self.payload_scalars,), torch.float32, member)

    # collectives -----------------------------------------------------------------------------------------
    @staticmethod
    def _stream(stream) -> int:
        return (torch.cuda.current_stream() if stream is None else stream).cuda_stream

    def channel(self, index: int):
        """Control block ``index`` (0..15). Collectives that may be in flight at the same time (say the loss step on one
        stream and the gradient reducer on another) must use different channels; within a channel every member issues
        the same collectives in the same order on one stream."""
        if not 0 <= index < CONTROL_REGION // int(native().CONTROL_BYTES):
            raise ValueError("channel index out of range")
        if index not in self._channels:
            self._channels[index] = native().make_control(self._native, index * int(native().CONTROL_BYTES),
                                                          int(self.budget_s * 1e9), self.uses_multicast)
        return self._channels[index]

    def barrier(self, stream=None, channel: int = 0) -> None:
        native().barrier(self.channel(channel), self._stream(stream))

    def all_reduce(self, scalars: Optional[int] = None, stream=None, *, offset: Optional[int] = None,
                   dtype: torch.dtype = torch.float32, scale: float = 1.0, channel: int = 0,
                   latency: Optional[bool] = None) -> None:
        """In place over the first ``scalars`` elements of the payload (or of the heap region at ``offset``). Payloads
        of up to 64 KiB take the one-round latency form (every member sums the members' staged vectors itself, in
        member order) unless ``latency`` is False; larger ones are reduced and broadcast by the switch in two rounds."""
        scalars = self.payload_scalars if scalars is None else scalars
        byte_offset = self._payload_offset if offset is None else offset
        nbytes = scalars * (4 if dtype == torch.float32 else 2)
        if nbytes <= LATENCY_SLOT_BYTES and channel < LATENCY_CHANNELS and latency is not False:
            slots = self._latency_offset + channel * 2 * self.members * LATENCY_SLOT_BYTES
            native().all_reduce_small(self.channel(channel), byte_offset, scalars, _TYPE_CODES[dtype], float(scale), slots,
                                      LATENCY_SLOT_BYTES, self._stream(stream))
            return
        native().all_reduce(self.channel(channel), byte_offset, scalars, _TYPE_CODES[dtype], float(scale),
                            self.multiprocessors, self._stream(stream))

    def collective_path(self) -> str:
        """How the last collective launched by this process reached its peers: ``multimem`` or ``peer``."""
        return {1: "multimem", 0: "peer"}.get(int(native().last_collective_path()), "none")

    def reduce_scatter(self, shard_scalars: int, stream=None, *, offset: Optional[int] = None,
                       dtype: torch.dtype = torch.float32, scale: float = 1.0, out: Optional[torch.Tensor] = None,
                       channel: int = 0) -> None:
        """Member m ends with the reduced elements ``[m*shard, (m+1)*shard)`` in its own replica, or in ``out``
        (float32, scaled) when given."""
        out_pointer = 0
        if out is not None:
            if out.dtype != torch.float32 or not out.is_contiguous() or out.numel() < shard_scalars:
                raise ValueError("reduce_scatter: out must be a contiguous float32 tensor of at least one shard")
            out_pointer = out.data_ptr()
        native().reduce_scatter(self.channel(channel), self._payload_offset if offset is None else offset, shard_scalars,
                                _TYPE_CODES[dtype], float(scale), out_pointer, self.multiprocessors, self._stream(stream))

    def expect_arrivals(self, arrivals: int, stream=None) -> None:
        """Waits for arrivals this member does not contribute: with nobody arriving, the bounded wait runs out and the
        status block records it. A host-driven way to exercise the timeout path."""
        native().expect_arrivals(self._control, arrivals, self._stream(stream))

    # status ----------------------------------------------------------------------------------------------
    def status_address(self) -> int:
        return self.address(int(native().STATUS_OFFSET))

    def status_words(self) -> List[int]:
        view = native().tensor_from_pointer(self.status_address(), [8], "int32", self.device.index)
        return [int(v) & 0xFFFFFFFF for v in view.cpu().tolist()]

    def status_view(self, channel: int = 0) -> torch.Tensor:
        """The eight status words of a channel as a device tensor (for callers that copy them out with their results)."""
        address = self.address(channel * int(native().CONTROL_BYTES) + int(native().STATUS_OFFSET))
        return native().tensor_from_pointer(address, [8], "int32", self.device.index)

    def set_budget(self, seconds: float) -> None:
        self.budget_s = seconds
        for control in self._channels.values():
            control.set_budget_ns(int(seconds * 1e9))

    def channel_status_words(self, channel: int) -> List[int]:
        address = self.address(channel * int(native().CONTROL_BYTES) + int(native().STATUS_OFFSET))
        view = native().tensor_from_pointer(address, [8], "int32", self.device.index)
        return [int(v) & 0xFFFFFFFF for v in view.cpu().tolist()]

    def check(self) -> None:
        for channel in sorted(self._channels):
            words = self.channel_status_words(channel)
            if words[0] != 0:
                raise DomainError(
                    f"member {self.member}, channel {channel}: {STATUS_NAMES.get(words[0], words[0])} at site {words[1]} "
                    f"(target {words[2]}, seen {words[3]}, detail {words[4]}, block {words[5]}, thread {words[6]})")

    def reset(self) -> None:
        """Clears a recorded failure and re-synchronises the round with the arrivals seen so far. Every member must call
        it at a quiescent point (no collective in flight anywhere)."""
        torch.cuda.synchronize(self.device)
        ext = native()
        base = self.address(0)
        words = ext.tensor_from_pointer(base, [CONTROL_REGION // 4], "int32", self.device.index)
        for channel in self._channels:
            first = channel * int(ext.CONTROL_BYTES) // 4
            flag = int(words[first + int(ext.FLAG_OFFSET) // 4].item())
            words[first + int(ext.ROUND_OFFSET) // 4] = flag
            words[first + int(ext.FINISHED_OFFSET) // 4] = 0
            words[first + int(ext.STATUS_OFFSET) // 4:first + int(ext.STATUS_OFFSET) // 4 + 8] = 0
        torch.cuda.synchronize(self.device)

    def host_barrier(self, name: str = "user") -> None:
        self._rendezvous.barrier(self._rendezvous.next_tag(name))

    def close(self) -> None:
        if getattr(self, "_closed", True):
            return
        self._closed = True
        torch.cuda.synchronize(self.device)
        try:
            self._rendezvous.barrier(self._rendezvous.next_tag("closing"))
        except Exception:
            pass  # a member that already left must not keep the others from releasing their memory
        self._native.close()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class MultimemDomain(DeviceDomain):
    """Replicas bound to an NVSwitch multicast object; collectives reduce inside the switch."""

    uses_multicast = True


class PeerDomain(DeviceDomain):
    """Replicas mapped peer to peer; collectives use remote atomics and peer loads and stores."""

    uses_multicast = False


class HostDomain(Domain):
    """CPU twin over a gloo group (or one process). The payload is a CPU float32 tensor per member."""

    def __init__(self, payload_scalars: int = 16, group=None) -> None:
        import torch.distributed as dist

        self._dist = dist if dist.is_available() and dist.is_initialized() else None
        self.group = group
        self.members = self._dist.get_world_size(group) if self._dist else 1
        self.member = self._dist.get_rank(group) if self._dist else 0
        self.payload_scalars = payload_scalars
        self._payload = torch.zeros(payload_scalars, dtype=torch.float32)
        self.device = torch.device("cpu")

    def replica_bytes(self) -> int:
        return self._payload.numel() * 4

    def payload(self, member: Optional[int] = None) -> torch.Tensor:
        if member not in (None, self.member):
            raise DomainError("a host domain only exposes its own replica")
        return self._payload

    def barrier(self, stream=None) -> None:
        if self._dist:
            self._dist.barrier(self.group)

    def all_reduce(self, scalars: Optional[int] = None, stream=None) -> None:
        scalars = self.payload_scalars if scalars is None else scalars
        if self._dist:
            view = self._payload[:scalars]
            self._dist.all_reduce(view, op=self._dist.ReduceOp.SUM, group=self.group)

    def reduce_scatter(self, shard_scalars: int, stream=None) -> None:
        if not self._dist:
            return
        total = self._payload[:shard_scalars * self.members].clone()
        self._dist.all_reduce(total, op=self._dist.ReduceOp.SUM, group=self.group)
        begin = self.member * shard_scalars
        self._payload[begin:begin + shard_scalars] = total[begin:begin + shard_scalars]
