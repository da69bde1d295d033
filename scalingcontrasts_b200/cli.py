"""Benchmark and verification modes, one CSV row per measurement:

    python -m scalingcontrasts_b200.cli oracle      --rows 128 --hidden 768 --prefixes 5 --gpus 8
    python -m scalingcontrasts_b200.cli box         --rows 4096 --hidden 768 --prefixes 5 --gpus 8
    python -m scalingcontrasts_b200.cli simulate    --rows 4096 --hidden 768 --prefixes 5 --gpus 72
    python -m scalingcontrasts_b200.cli collectives --gpus 8 --min-kib 1 --max-mib 128 --repeats 20
    python -m scalingcontrasts_b200.cli hosts       --rows 1024 --hosts 2 --gpus 4 --exchange /tmp/rails
    python -m scalingcontrasts_b200.cli train       --rows 16384 --gpus 8 --warm 20 --steps 100

Rows keep the reference's leading columns so that they paste into the same tables, with device-timed columns added at
the end:

    simulate,R,H,K,S,bytes,min_ms,median_ms,gcells_per_s,roofline_ms,fraction_of_roofline,peaks
    box|hosts,R,H,K,world,bytes,min_ms,median_ms,gcells_per_s_per_gpu,roofline_ms,fraction_of_roofline,peaks
    oracle,R,H,K,ranks,exact_loss,measured_loss,rel_grad_err,disagreeing
    barrier,count,stride,min_us,median_us
    reduce_scatter|all_reduce|all_reduce_two_round,count,bytes,min_us,median_us,algbw,busbw,path
    validation|validation_one_round,count,bytes,wrong_scatter,wrong_sums,repeats,differing,path
    train,R,H,K,world,min_ms,median_ms,gcells_per_s

Multi-GPU modes run one process per GPU. Under ``torchrun`` the ranks are taken from the environment; otherwise the
command starts ``--gpus`` worker processes itself. Every time is measured with CUDA events on the launching stream
and is the maximum over ranks; bus bandwidth follows the nccl-tests convention (all-reduce ``bytes/t * 2(n-1)/n``,
reduce-scatter ``bytes/t * (n-1)/n`` with ``bytes`` the whole per-GPU payload).

Parity: the modes and flags of ``scalingcontrasts.cu:377-605`` and ``cli.mojo:574-791``. Unknown flags are rejected with
exit status 2 like the reference's parser.
"""
from __future__ import annotations

import argparse
import math
import os
import socket
import sys
from typing import List, Optional

from .config import Settings

MODES = ("oracle", "simulate", "box", "hosts", "collectives", "train")
STEP_CALLS = 3  # loss steps per timed window (scalingcontrasts.cu:33)
COLLECTIVE_CALLS = 20  # collectives per timed window (scalingcontrasts.cu:34)
ORACLE_SCALE = 1.0  # unit-scale keyed inputs keep the narrowest prefixes off the cosine floor
BENCHMARK_SCALE = 0.1


def build_parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(prog="scalingcontrasts_b200", description=__doc__,
                                     formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("mode", choices=MODES)
    defaults = Settings()
    parser.add_argument("--rows", type=int, default=defaults.rows)
    parser.add_argument("--hidden", type=int, default=defaults.hidden)
    parser.add_argument("--prefixes", type=int, default=defaults.prefixes)
    parser.add_argument("--ends", type=str, default="", help="explicit ascending prefix ends, comma separated")
    parser.add_argument("--gpus", type=int, default=0, help="GPUs to use (simulate: size of the simulated world)")
    parser.add_argument("--windows", type=int, default=defaults.windows, help="timed windows (hosts mode: 0 prints an oracle row)")
    parser.add_argument("--max-mib", type=int, default=defaults.max_mib)
    parser.add_argument("--min-kib", type=int, default=defaults.min_kib)
    parser.add_argument("--repeats", type=int, default=defaults.repeats)
    parser.add_argument("--host", type=int, default=0)
    parser.add_argument("--hosts", type=int, default=1)
    parser.add_argument("--nics", type=str, default="")
    parser.add_argument("--exchange", type=str, default="")
    parser.add_argument("--positives", choices=["self", "pairs"], default="self")
    parser.add_argument("--diagonal", choices=["own", "negative", "skip"], default=None)
    parser.add_argument("--inputs", choices=["keyed", "normal"], default="keyed")
    parser.add_argument("--seed", type=int, default=0)
    parser.add_argument("--warm", type=int, default=defaults.warm)
    parser.add_argument("--steps", type=int, default=defaults.steps)
    parser.add_argument("--device", choices=["cuda", "cpu"], default="cuda")
    parser.add_argument("--no-multicast", action="store_true", help="form a peer domain even where multicast exists")
    parser.add_argument("--no-graphs", action="store_true", help="enqueue every step kernel by kernel instead of replaying a CUDA graph")
    parser.add_argument("--header", action="store_true")
    return parser


def settings_from(arguments: argparse.Namespace) -> Settings:
    ends = tuple(int(e) for e in arguments.ends.split(",")) if arguments.ends else ()
    settings = Settings(mode=arguments.mode, rows=arguments.rows, hidden=arguments.hidden, prefixes=arguments.prefixes,
                        gpus=arguments.gpus, windows=arguments.windows, max_mib=arguments.max_mib, min_kib=arguments.min_kib,
                        repeats=arguments.repeats, host=arguments.host, hosts=arguments.hosts, nics=arguments.nics,
                        exchange=arguments.exchange, positives=arguments.positives, diagonal=arguments.diagonal,
                        inputs=arguments.inputs, seed=arguments.seed, warm=arguments.warm, steps=arguments.steps,
                        device=arguments.device, ends=ends)
    settings.validate()
    return settings


# ---------------------------------------------------------------------------------------------------------------
# process plumbing
# ---------------------------------------------------------------------------------------------------------------
def _free_port() -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as probe:
        probe.bind(("127.0.0.1", 0))
        return probe.getsockname()[1]


def _worker(local_rank: int, world: int, port: int, argv: List[str]) -> None:
    os.environ.update({"RANK": str(local_rank), "LOCAL_RANK": str(local_rank), "WORLD_SIZE": str(world),
                       "MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port)})
    run(argv)


def _world_for(settings: Settings, multicast: bool) -> int:
    if "WORLD_SIZE" in os.environ:
        return int(os.environ["WORLD_SIZE"])
    if settings.mode == "simulate":
        return 1
    if settings.device == "cpu":
        return max(settings.gpus, 1)
    import torch

    visible = torch.cuda.device_count()
    return settings.gpus if settings.gpus > 0 else max(visible, 1)


def main(argv: Optional[List[str]] = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    parser = build_parser()
    arguments = parser.parse_args(argv)  # unknown flags exit with status 2
    settings = settings_from(arguments)
    world = _world_for(settings, not arguments.no_multicast)
    if world > 1 and "RANK" not in os.environ:
        import torch.multiprocessing as mp

        mp.start_processes(_worker, args=(world, _free_port(), argv), nprocs=world, join=True, start_method="spawn")
        return 0
    run(argv)
    return 0


def run(argv: List[str]) -> None:
    arguments = build_parser().parse_args(argv)
    settings = settings_from(arguments)
    context = RankContext(settings, multicast=not arguments.no_multicast, graphs=not arguments.no_graphs)
    try:
        if arguments.header and context.rank == 0:
            print(HEADERS[settings.mode], flush=True)
        {"oracle": run_oracle, "simulate": run_simulate, "box": run_box, "hosts": run_hosts,
         "collectives": run_collectives, "train": run_train}[settings.mode](context)
    finally:
        context.close()


HEADERS = {
    "simulate": "mode,rows,hidden,prefixes,world,bytes,min_ms,median_ms,gcells_per_s,roofline_ms,fraction_of_roofline,peaks",
    "box": "mode,rows,hidden,prefixes,world,bytes,min_ms,median_ms,gcells_per_s_per_gpu,roofline_ms,fraction_of_roofline,peaks",
    "hosts": "mode,rows,hidden,prefixes,world,bytes,min_ms,median_ms,gcells_per_s_per_gpu,roofline_ms,fraction_of_roofline,peaks",
    "oracle": "mode,rows,hidden,prefixes,ranks,exact_loss,measured_loss,rel_grad_err,disagreeing",
    "collectives": "mode,count,bytes,min_us,median_us,algbw,busbw,path",
    "train": "mode,rows,hidden,prefixes,world,min_ms,median_ms,gcells_per_s",
}


class RankContext:
    """What every mode needs: rank, world, device, an initialised process group when there are several ranks."""

    def __init__(self, settings: Settings, multicast: bool = True, graphs: bool = True) -> None:
        import torch
        import torch.distributed as dist

        self.settings, self.multicast, self.graphs = settings, multicast, graphs
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.cuda = settings.device == "cuda"
        if self.cuda:
            torch.cuda.set_device(self.local_rank)
            self.device = torch.device("cuda", self.local_rank)
        else:
            self.device = torch.device("cpu")
        self._owns_group = False
        if self.world > 1 and not dist.is_initialized():
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            if self.cuda:
                os.environ.setdefault("NCCL_NVLS_ENABLE", "0")  # NCCL is bootstrap only; the domain owns the multicast
                dist.init_process_group("nccl", device_id=self.device)
            else:
                dist.init_process_group("gloo")
            self._owns_group = True

    def emit(self, row: str) -> None:
        if self.rank == 0:
            print(row, flush=True)

    def barrier(self) -> None:
        import torch
        import torch.distributed as dist

        if self.cuda:
            torch.cuda.synchronize(self.device)
        if self.world > 1:
            dist.barrier()

    def close(self) -> None:
        import torch.distributed as dist

        if self._owns_group and dist.is_initialized():
            dist.destroy_process_group()


def _embeddings(context: RankContext, scale: float, rank: Optional[int] = None):
    from .utils.keyed import make_embeddings

    s = context.settings
    block = make_embeddings(s.inputs, s.rows, s.hidden, context.rank if rank is None else rank, s.seed, scale)
    return block.to(context.device)


def _box_engine(context: RankContext):
    from .parallel.box import BoxLoss
    from .parallel.domain import Domain

    s = context.settings
    ladder = s.ladder()
    ladder.check_device_shape(s.rows, s.hidden)
    domain = Domain.create(payload_scalars=16, heap_bytes=BoxLoss.heap_bytes(s.rows, s.hidden, ladder.count),
                           device=context.device, multicast=context.multicast)
    engine = BoxLoss(s.rows, s.hidden, ladder, s.spec(), domain)
    engine.use_graphs = context.graphs
    return engine, domain


def _roofline_columns(rows: int, world: int, hidden: int, min_ms: float) -> str:
    """``roofline_ms,fraction,source``: the step's bound (tensor time at the measured sustained peak, which is the one
    that applies to steps timed in a long run, or peer pulls at link bandwidth, whichever is slower) and how much of it
    the measured time reaches. The source names the denominator: ``measured-sustained`` or ``fallback-sustained``."""
    from .utils.roofline import load_peaks, loss_step_roofline_ms

    peaks = load_peaks()
    bound = loss_step_roofline_ms(rows, world, hidden, peaks, sustained=True)
    return f"{bound:.4f},{bound / min_ms:.3f},{peaks.source}-sustained"


def _time(context: RankContext, step, windows: int, calls: int):
    from .utils.timing import time_windows

    return time_windows(step, windows, calls, context.device if context.cuda else None)


# ---------------------------------------------------------------------------------------------------------------
# modes
# ---------------------------------------------------------------------------------------------------------------
def run_simulate(context: RankContext) -> None:
    """One rank of a ``--gpus``-GPU world on a single GPU: time and memory only."""
    from .parallel.box import BoxLoss

    s = context.settings
    world = max(s.gpus, 1)
    ladder = s.ladder()
    engine = BoxLoss(s.rows, s.hidden, ladder, s.spec(), None, context.device)
    block = _embeddings(context, BENCHMARK_SCALE)
    engine.simulate(block, world, s.beta, s.bias)
    context.barrier()
    engine.check()
    timing = _time(context, lambda: engine.simulate(block, world, s.beta, s.bias), s.windows, STEP_CALLS)
    engine.check()
    cells = s.rows * s.rows * world * ladder.count
    context.emit(f"simulate,{s.rows},{s.hidden},{ladder.count},{world},{engine.bytes()},{timing.min_ms:.4f},"
                 f"{timing.median_ms:.4f},{cells / timing.min_ms / 1e6:.1f},{_roofline_columns(s.rows, world, s.hidden, timing.min_ms)}")


def run_box(context: RankContext) -> None:
    s = context.settings
    engine, domain = _box_engine(context)
    block = _embeddings(context, BENCHMARK_SCALE)
    engine.step(block, s.beta, s.bias)
    context.barrier()
    engine.check()
    timing = _time(context, lambda: engine.step(block, s.beta, s.bias), s.windows, STEP_CALLS)
    engine.check()
    cells = s.rows * s.rows * context.world * engine.ladder.count
    context.emit(f"box,{s.rows},{s.hidden},{engine.ladder.count},{context.world},{engine.bytes()},{timing.min_ms:.4f},"
                 f"{timing.median_ms:.4f},{cells / timing.min_ms / 1e6:.1f},"
                 f"{_roofline_columns(s.rows, context.world, s.hidden, timing.min_ms)}")
    domain.close()


def run_oracle(context: RankContext) -> None:
    """One step, then the whole world's loss and gradient against the float64 evaluation on rank 0."""
    import torch
    import torch.distributed as dist

    from .cpu import oracle, relative_l2, simulate_world

    s = context.settings
    ladder = s.ladder()
    scale = ORACLE_SCALE
    if context.cuda:
        engine, domain = _box_engine(context)
        block = _embeddings(context, scale)
        gradient, summands = engine.step(block, s.beta, s.bias)
        context.barrier()
        engine.check()
        gradient, summands = gradient.clone(), summands.clone()
        if context.world > 1:
            blocks = [torch.empty_like(block) for _ in range(context.world)]
            gradients = [torch.empty_like(gradient) for _ in range(context.world)]
            losses = [torch.empty_like(summands) for _ in range(context.world)]
            dist.all_gather(blocks, block)
            dist.all_gather(gradients, gradient)
            dist.all_gather(losses, summands)
        else:
            blocks, gradients, losses = [block], [gradient], [summands]
        domain.close()
        measured_gradient = torch.cat([g.float().cpu() for g in gradients])
        measured_loss = float(losses[0][0])
        disagreeing = sum(1 for other in losses if other[0].view(torch.int32).item() != losses[0][0].view(torch.int32).item())
        world_rows = torch.cat([b.cpu() for b in blocks])
    else:
        ranks = max(s.gpus, 1)
        blocks = [_embeddings(context, scale, rank).float() for rank in range(ranks)]
        gradients, total = simulate_world(blocks, ladder, s.beta, s.bias, s.spec())
        measured_gradient, measured_loss, disagreeing = torch.cat(gradients), float(total[0]), 0
        world_rows = torch.cat(blocks)
    if context.rank == 0:
        expected = oracle(world_rows, ladder, s.beta, s.bias, s.spec())
        error = relative_l2(measured_gradient, expected.gradient)
        ranks = world_rows.shape[0] // s.rows
        context.emit(f"oracle,{s.rows},{s.hidden},{ladder.count},{ranks},{expected.loss:.9e},{measured_loss:.9e},"
                     f"{error:.3e},{disagreeing}")


def run_collectives(context: RankContext) -> None:
    import torch

    from ._ext import native
    from .parallel.domain import Domain, LATENCY_SLOT_BYTES

    s = context.settings
    ext = native()
    max_scalars = s.max_mib * (1 << 20) // 4
    domain = Domain.create(payload_scalars=max_scalars, device=context.device, multicast=context.multicast)
    count = domain.members
    stream = torch.cuda.current_stream().cuda_stream
    for _ in range(3):
        domain.barrier()
    context.barrier()
    timing = _time(context, domain.barrier, s.windows, COLLECTIVE_CALLS)
    context.emit(f"barrier,{count},{domain.stride},{timing.min_ms * 1e3:.2f},{timing.median_ms * 1e3:.2f}")
    scalars = max(s.min_kib * 1024 // 4, 4 * count)
    while scalars <= max_scalars:
        shard = scalars // count // 4 * 4
        payload_bytes = shard * count * 4
        calls = [("reduce_scatter", lambda: domain.reduce_scatter(shard), (count - 1) / count),
                 ("all_reduce", lambda: domain.all_reduce(shard * count), 2 * (count - 1) / count)]
        if payload_bytes <= LATENCY_SLOT_BYTES:
            # the row above took the one-round latency form; this one is the two-round form at the same size
            calls.append(("all_reduce_two_round", lambda: domain.all_reduce(shard * count, latency=False), 2 * (count - 1) / count))
        for name, call, factor in calls:
            call()
            context.barrier()
            timing = _time(context, call, s.windows, COLLECTIVE_CALLS)
            algbw = payload_bytes / (timing.min_ms * 1e6)
            context.emit(f"{name},{count},{payload_bytes},{timing.min_ms * 1e3:.2f},{timing.median_ms * 1e3:.2f},"
                         f"{algbw:.2f},{algbw * factor:.2f},{domain.collective_path()}")
        scalars *= 2
    domain.check()
    # validation: exact keyed integers, then bit-for-bit repeats of an all-reduce whose sums round
    payload = domain.payload()
    total = max_scalars // count // 4 * 4 * count
    shard = total // count
    counters = torch.zeros(3, dtype=torch.int64, device=context.device)
    ext.keyed_integers(payload.data_ptr(), total, 0, count, domain.member, stream)
    domain.reduce_scatter(shard)
    ext.count_wrong_sums(payload.data_ptr() + domain.member * shard * 4, shard, domain.member * shard, count,
                         counters.data_ptr(), stream)
    domain.barrier()
    ext.keyed_integers(payload.data_ptr(), total, 0, count, domain.member, stream)
    domain.all_reduce(total)
    ext.count_wrong_sums(payload.data_ptr(), total, 0, count, counters.data_ptr() + 8, stream)
    reference = torch.empty(total, dtype=torch.float32, device=context.device)
    for repeat in range(s.repeats):
        domain.barrier()
        ext.keyed_fractions(payload.data_ptr(), total, 0, count, domain.member, stream)
        domain.all_reduce(total)
        if repeat == 0:
            reference.copy_(payload[:total])
        else:
            ext.count_differences(payload.data_ptr(), reference.data_ptr(), total, counters.data_ptr() + 16, stream)
    context.barrier()
    domain.check()
    import torch.distributed as dist

    if context.world > 1:
        dist.all_reduce(counters)
    wrong_scatter, wrong_sums, differing = (int(v) for v in counters.cpu().tolist())
    context.emit(f"validation,{count},{total * 4},{wrong_scatter},{wrong_sums},{s.repeats},{differing},{domain.collective_path()}")
    # the same two checks for the one-round latency form, at its largest size
    small = min(LATENCY_SLOT_BYTES // 4, max_scalars) // 4 * 4
    counters.zero_()
    domain.barrier()
    ext.keyed_integers(payload.data_ptr(), small, 0, count, domain.member, stream)
    domain.all_reduce(small)
    ext.count_wrong_sums(payload.data_ptr(), small, 0, count, counters.data_ptr() + 8, stream)
    for repeat in range(s.repeats):
        domain.barrier()
        ext.keyed_fractions(payload.data_ptr(), small, 0, count, domain.member, stream)
        domain.all_reduce(small)
        if repeat == 0:
            reference[:small].copy_(payload[:small])
        else:
            ext.count_differences(payload.data_ptr(), reference.data_ptr(), small, counters.data_ptr() + 16, stream)
    context.barrier()
    domain.check()
    if context.world > 1:
        dist.all_reduce(counters)
    _, wrong_sums, differing = (int(v) for v in counters.cpu().tolist())
    context.emit(f"validation_one_round,{count},{small * 4},0,{wrong_sums},{s.repeats},{differing},{domain.collective_path()}")
    domain.close()


def run_train(context: RankContext) -> None:
    import torch

    from .trainer import ContrastiveTrainer

    s = context.settings
    trainer = ContrastiveTrainer(s.rows, hidden=s.hidden, prefixes=s.prefixes, spec=s.spec(), device=context.device,
                                 seed=s.seed, multicast=context.multicast, graphs=context.graphs)
    generator = torch.Generator().manual_seed(s.seed * 7919 + context.rank)
    batches = [torch.randn(s.rows, trainer.in_features, generator=generator).to(torch.bfloat16).to(context.device)
               for _ in range(4)]
    state = {"step": 0}

    def step() -> None:
        trainer.step_on_device(batches[state["step"] % 4])
        state["step"] += 1

    for _ in range(max(s.warm, 3)):
        step()
    context.barrier()
    trainer.check()
    windows = max(1, math.ceil(s.steps / 10))
    timing = _time(context, step, windows, 10)
    trainer.check()
    cells = trainer.cells_per_step() * context.world
    context.emit(f"train,{s.rows},{s.hidden},{s.prefixes},{context.world},{timing.min_ms:.4f},{timing.median_ms:.4f},"
                 f"{cells / timing.min_ms / 1e6:.1f}")
    trainer.close()


def run_hosts(context: RankContext) -> None:
    from .parallel.hosts import run_hosts_mode

    run_hosts_mode(context)


if __name__ == "__main__":
    sys.exit(main())
