"""The inter-box data-parallel loss step: boxes exchange their blocks over rails while each box scores its own GPUs'
blocks, then every GPU also scores the blocks that landed on its box.

One step on a rank (host ``h``, local GPU ``g`` of ``G``), in the reference's order:

1. no drain is needed: the landing buffer of this step's parity was last read by the remote rank two steps ago, and
   that rank's post of the step in between, whose completion this rank consumed then, ran on the remote stream after
   those reads (the reference synchronises its devices here because it has no such ordering to lean on);
2. the block is published into the box's symmetric memory and posted on every rail (to GPU ``g`` of every other host)
   into the landing buffer of this step's parity; the writes fly while
3. the rank scores the box's own blocks (the box step);
4. for every rail the rank waits for the remote block to land, copies it (with its prefix norms) into symmetric memory
   where the box's other GPUs can reach it over NVLink, and the box meets on a domain barrier;
5. the rank scores every landed block of every remote host, pulling its peers' landed blocks over NVLink;
6. ``finish``, and the summands are all-reduced inside the box;
7. the box's sum crosses the rails as one row per host (GPU 0's rails); every host adds the rows in host order, so all
   hosts hold bit-identical totals, and the totals are spread to the box's GPUs. Only GPU 0 of a box waits on the host
   for this (an event on its stream, not a device-wide synchronise); the others enqueue the closing all-reduce and go on.

With the loopback transport the "hosts" are groups of GPUs of one box. Parity: ``step_hosts`` (scalingcontrasts.cu:313-368),
``make_cluster`` (scalingcontrasts.cu:260-292).
"""
from __future__ import annotations

import os
import tempfile
from typing import List, Optional, Tuple

import torch

from ..config import LossSpec, REFERENCE_SPEC, SUMMAND_SLOTS
from ..ladder import Matryoshka
from ..ops.streamed_loss import BlockNorms, compute_block_norms
from .box import BoxLoss, SourceBlock
from .rail import RdmaRail, exchange_endpoint


class _null_context:
    def __enter__(self):
        return None

    def __exit__(self, *arguments):
        return False


class HostsLoss(BoxLoss):
    """One rank's engine for steps that span several hosts. ``domain`` is the rank's box domain."""

    def __init__(self, rows: int, hidden: int, ladder: Matryoshka, spec: LossSpec, domain, host: int, hosts: int,
                 exchange: str, rail_timeout_s: float = 30.0) -> None:
        super().__init__(rows, hidden, ladder, spec, domain)
        self.host, self.hosts, self.exchange, self.rail_timeout_s = host, hosts, exchange, rail_timeout_s
        self.remote_hosts = [h for h in range(hosts) if h != host]
        k = ladder.count
        block_bytes = rows * hidden * 2
        norm_bytes = BlockNorms.scalars_for(k, rows) * 4
        # Landed blocks live in symmetric memory so that the box's other GPUs can pull them: [remote][parity].
        self._landed_offsets = [[(domain.alloc(block_bytes), domain.alloc(norm_bytes)) for _ in range(2)]
                                for _ in self.remote_hosts]
        self.landed = [[(domain.tensor(e, (rows, hidden), torch.bfloat16),
                         BlockNorms(k, rows, domain.tensor(n, (BlockNorms.scalars_for(k, rows),), torch.float32)))
                        for e, n in parities] for parities in self._landed_offsets]
        # What a rail writes into: plain device memory, exportable to the peer's process.
        self.landings = [torch.zeros(2, rows, hidden, dtype=torch.bfloat16, device=self.device) for _ in self.remote_hosts]
        self.rails: List[RdmaRail] = []
        for index, remote in enumerate(self.remote_hosts):
            rail = RdmaRail(self.embeddings, self.landings[index], hosts, host)
            record = exchange_endpoint(exchange, host, remote, self.member, rail.local)
            rail.connect(record)
            self.rails.append(rail)
        self.steps = 0
        self._host_summands = torch.zeros(SUMMAND_SLOTS, dtype=torch.float32).pin_memory()
        self._host_total = torch.zeros(SUMMAND_SLOTS, dtype=torch.float32).pin_memory()
        self._summands_ready = torch.cuda.Event()

    @staticmethod
    def heap_bytes_for(rows: int, hidden: int, prefixes: int, hosts: int) -> int:
        per_block = rows * hidden * 2 + BlockNorms.scalars_for(prefixes, rows) * 4 + 512
        return BoxLoss.heap_bytes(rows, hidden, prefixes) + 2 * (hosts - 1) * per_block + 4096

    def step(self, queries: torch.Tensor, beta: float = 10.0, bias: float = -10.0, scalars: Optional[torch.Tensor] = None,
             gradient_out: Optional[torch.Tensor] = None, stream=None) -> Tuple[torch.Tensor, torch.Tensor]:
        """One step across the hosts; the summands on return are always the world's sums (there is no unreduced form:
        the closing all-reduce is also what spreads the hosts' totals inside the box)."""
        members, member, rows, hosts = self.members, self.member, self.rows, self.hosts
        parity = self.steps % 2
        world_rows = hosts * members * rows
        rank_base = (self.host * members + member) * rows
        # 2. publish and post
        compute_block_norms(queries, self.ladder, self.norms, copy_to=self.embeddings, stream=stream)
        for rail in self.rails:
            rail.post_embeddings(parity, stream)
        # 3. the box's own blocks
        self.domain.barrier(stream)
        self.loss.begin(self.embeddings, stream, query_norms=self.norms)
        blocks = [SourceBlock(rank_base, self.embeddings, self.norms)]
        for p in range(1, members):
            peer = (member + p) % members
            blocks.append(SourceBlock((self.host * members + peer) * rows, member=peer,
                                      embeddings_offset=self._embeddings_offset, norms_offset=self._norms_offset))
        self.score_sequence(blocks, rank_base, world_rows, beta, bias, scalars, stream)
        # 4. wait for the remote blocks, make them reachable inside the box
        for index, rail in enumerate(self.rails):
            landed_bytes = rail.await_landed(self.rail_timeout_s)
            if landed_bytes != rows * self.hidden * 2:
                raise RuntimeError(f"rail delivered {landed_bytes} bytes, expected {rows * self.hidden * 2}")
            embeddings, norms = self.landed[index][parity]
            compute_block_norms(self.landings[index][parity], self.ladder, norms, copy_to=embeddings, stream=stream)
        self.domain.barrier(stream)
        # 5. the landed blocks of every remote host, from every GPU of this box
        blocks = []
        for index, remote in enumerate(self.remote_hosts):
            for p in range(members):
                peer = (member + p) % members
                base = (remote * members + peer) * rows
                if peer == member:
                    embeddings, norms = self.landed[index][parity]
                    blocks.append(SourceBlock(base, embeddings, norms))
                else:
                    offsets = self._landed_offsets[index][parity]
                    blocks.append(SourceBlock(base, member=peer, embeddings_offset=offsets[0], norms_offset=offsets[1]))
        self.score_sequence(blocks, rank_base, world_rows, beta, bias, scalars, stream)
        # 6. finish and the box's sum
        gradient = self.gradient if gradient_out is None else gradient_out
        self.loss.finish(self.embeddings, gradient, self.summands, stream)
        self.domain.all_reduce(SUMMAND_SLOTS, stream)
        # 7. hosts' sums in host order
        if member == 0:
            current = torch.cuda.current_stream(self.device) if stream is None else stream
            with torch.cuda.stream(current):
                self._host_summands.copy_(self.summands, non_blocking=True)
                self._summands_ready.record(current)
            self._summands_ready.synchronize()
            for rail in self.rails:
                rail.post_summands(self.host, self._host_summands.tolist())
            for rail in self.rails:
                rail.await_landed(self.rail_timeout_s)
            self._host_total.zero_()
            for host in range(hosts):  # host order on every host: bit-identical totals everywhere
                if host == self.host:
                    self._host_total += self._host_summands
                else:
                    rail = self.rails[self.remote_hosts.index(host)]
                    self._host_total += torch.tensor(rail.read_summands(host, SUMMAND_SLOTS), dtype=torch.float32)
            with torch.cuda.stream(current):
                self.summands.copy_(self._host_total, non_blocking=True)
        else:
            with torch.cuda.stream(stream) if stream is not None else _null_context():
                self.summands.zero_()
        self.domain.all_reduce(SUMMAND_SLOTS, stream)
        self.steps += 1
        return gradient, self.summands

    def close(self) -> None:
        torch.cuda.synchronize(self.device)
        for rail in self.rails:
            rail.close()


def run_hosts_mode(context) -> None:
    """``hosts`` mode of the command line: ``--hosts`` logical hosts of ``--gpus`` GPUs each on this box, loopback
    rails between them. One timing row like ``box``; with ``--windows 0`` an oracle row instead."""
    import torch.distributed as dist

    from ..cpu import oracle, relative_l2
    from ..utils.keyed import make_embeddings
    from ..utils.timing import time_windows
    from .domain import Domain

    s = context.settings
    hosts = s.hosts
    if hosts < 2:
        raise SystemExit("hosts mode needs --hosts >= 2")
    if context.world % hosts:
        raise SystemExit("the number of ranks must be a multiple of --hosts")
    per_host = context.world // hosts
    host, local = context.rank // per_host, context.rank % per_host
    groups = [dist.new_group(list(range(h * per_host, (h + 1) * per_host))) for h in range(hosts)]
    ladder = s.ladder()
    exchange = s.exchange
    if not exchange:
        holder = [tempfile.mkdtemp(prefix="sc-rails-") if context.rank == 0 else None]
        dist.broadcast_object_list(holder, src=0)
        exchange = holder[0]
    domain = Domain.create(payload_scalars=16, heap_bytes=HostsLoss.heap_bytes_for(s.rows, s.hidden, ladder.count, hosts),
                           group=groups[host], device=context.device, multicast=context.multicast)
    engine = HostsLoss(s.rows, s.hidden, ladder, s.spec(), domain, host, hosts, exchange)
    oracle_run = s.windows == 0 or s.mode == "oracle"
    scale = 1.0 if oracle_run else 0.1
    block = make_embeddings(s.inputs, s.rows, s.hidden, context.rank, s.seed, scale).to(context.device)
    gradient, summands = engine.step(block, s.beta, s.bias)
    context.barrier()
    engine.check()
    if oracle_run:
        blocks = [torch.empty_like(block) for _ in range(context.world)]
        gradients = [torch.empty_like(gradient) for _ in range(context.world)]
        losses = [torch.empty_like(summands) for _ in range(context.world)]
        dist.all_gather(blocks, block)
        dist.all_gather(gradients, gradient.clone())
        dist.all_gather(losses, summands.clone())
        if context.rank == 0:
            expected = oracle(torch.cat([b.cpu() for b in blocks]), ladder, s.beta, s.bias, s.spec())
            error = relative_l2(torch.cat([g.float().cpu() for g in gradients]), expected.gradient)
            first = losses[0][0].view(torch.int32).item()
            disagreeing = sum(1 for other in losses if other[0].view(torch.int32).item() != first)
            context.emit(f"oracle,{s.rows},{s.hidden},{ladder.count},{context.world},{expected.loss:.9e},"
                         f"{float(losses[0][0]):.9e},{error:.3e},{disagreeing}")
    else:
        timing = time_windows(lambda: engine.step(block, s.beta, s.bias), s.windows, 3, context.device)
        engine.check()
        cells = s.rows * s.rows * context.world * ladder.count
        from ..cli import _roofline_columns

        context.emit(f"hosts,{s.rows},{s.hidden},{ladder.count},{context.world},{engine.bytes()},{timing.min_ms:.4f},"
                     f"{timing.median_ms:.4f},{cells / timing.min_ms / 1e6:.1f},"
                     f"{_roofline_columns(s.rows, context.world, s.hidden, timing.min_ms)}")
    context.barrier()
    engine.close()
    domain.close()
    if context.rank == 0 and not s.exchange:
        for name in os.listdir(exchange):
            os.unlink(os.path.join(exchange, name))
        os.rmdir(exchange)
