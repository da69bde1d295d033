"""Headline benchmark: the training step of the named configuration, device-timed, one JSON line from rank 0.

    python bench.py --gpus 1 --steps 100 --warmup 20
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29500 \
        bench.py --gpus 8 --steps 100 --warmup 20

Configuration (the reference's headline metric on this framework's flagship step): a one-tower projector
(bfloat16, Linear 1024 -> 3072, GELU, Linear 3072 -> 768, Xavier init) on R = 16384 random N(0,1) rows per GPU, the
K = 5 Matryoshka sigmoid loss streamed over every GPU's block, backward, the projector gradients' all-reduce on a side
stream, and an AdamW update. Metric: scored cells per second summed over the job, where one rank scores
R x (N R) x K cells per step. Weak scaling in rows per GPU (work per GPU grows with N because every rank scores every
peer's block).

Two numbers are measured on the same objects: ``value`` times K steps on batches that already sit on the device
(CUDA events, maximum over ranks, a barrier and a synchronise on both sides); ``e2e`` times K calls of the public
``ContrastiveTrainer.step`` path fed from pinned host memory, with the host-to-device copy of every step's batch and
the device-to-host read of every step's loss inside the timed region.

Beside the number the line carries its evidence: ``oracle`` (a 128-rows-per-rank step with pair positives over the same
ranks, run before anything is timed and checked against the float64 evaluation: relative loss and gradient error, ranks
whose loss bits differ), ``ranks_disagreeing_on_loss`` after the timed steps, ``multicast_kernels`` (which form the
collective launcher of this process used last), ``loss_step_ms`` / ``loss_ms_per_block`` / ``non_loss_ms`` (the loss
step timed alone, outside the timed regions), ``clocks`` sampled on every rank through both timed regions, and
``ms_times_sm_mhz`` so that a power-capped run can be compared with an uncapped one.

``--impl reference`` is the reference arm. The reference is a C++/CUDA/Mojo tree without a Python package, so it cannot
be installed into ``baseline/_ref``; the arm prints its ``unavailable`` line.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import time

IDLE_BEFORE_E2E_S = 2.0  # the end-to-end region starts from an idle GPU, like the device-timed region before it
PUBLISHED_GCELLS_PER_GPU = 275.0  # reference README: 8 x B300, H=1024, K=5, R=16384 (loss step only)


def parse() -> argparse.Namespace:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=100)
    parser.add_argument("--warmup", type=int, default=20)
    parser.add_argument("--impl", choices=["ours", "reference"], default="ours")
    parser.add_argument("--rows", type=int, default=16384)
    parser.add_argument("--in-features", type=int, default=1024)
    parser.add_argument("--mid-features", type=int, default=3072)
    parser.add_argument("--hidden", type=int, default=768)
    parser.add_argument("--prefixes", type=int, default=5)
    parser.add_argument("--no-e2e", action="store_true")
    return parser.parse_args()


def reference_arm(arguments: argparse.Namespace) -> None:
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({
            "impl": "reference",
            "unavailable": "reference is a C++23/CUDA/Mojo tree with no setup.py or pyproject.toml (pip: 'not installable'); "
                           "its CUDA build needs nvcc >= 13.1, a network fetch of NumKong and libibverbs, its Python "
                           "baselines need open_clip / jax, none of which exist on this image"}), flush=True)


def respawn_under_torchrun(arguments: argparse.Namespace) -> int:
    """``python bench.py --gpus N`` without a launcher: start the N ranks ourselves."""
    port = 29500 + (os.getpid() % 2000)
    command = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={arguments.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.abspath(__file__)] + sys.argv[1:]
    return subprocess.call(command)


def main() -> int:
    arguments = parse()
    if arguments.impl == "reference":
        reference_arm(arguments)
        return 0
    if arguments.gpus > 1 and "RANK" not in os.environ:
        return respawn_under_torchrun(arguments)

    import torch
    import torch.distributed as dist

    from scalingcontrasts_b200 import _ext
    from scalingcontrasts_b200.trainer import ContrastiveTrainer
    from scalingcontrasts_b200.utils.clocks import ClockSampler

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != arguments.gpus:
        raise SystemExit(f"--gpus {arguments.gpus} but WORLD_SIZE={world}")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        # NCCL only carries the barrier and the max-over-ranks here; keep it off the switch's multicast resources, which
        # the library's own domain binds.
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=device)
    ext = _ext.native()  # raises when the extension is missing: no silent fallback

    def fence() -> None:
        torch.cuda.synchronize(device)
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize(device)

    def gather_objects(value):
        if world == 1:
            return [value]
        values = [None] * world
        dist.all_gather_object(values, value)
        return values

    # ---- correctness of this job's ranks, before anything is timed -----------------------------------------------
    oracle_block = small_oracle(rank, world, device, arguments.hidden, arguments.prefixes)

    rows, steps, warmup = arguments.rows, arguments.steps, max(arguments.warmup, 3)
    trainer = ContrastiveTrainer(rows, arguments.in_features, arguments.mid_features, arguments.hidden, arguments.prefixes,
                                 device=device, seed=0)
    generator = torch.Generator(device="cpu").manual_seed(1234 + rank)
    rotation = 4  # 4 x 33.5 MB of inputs > 126 MB of L2, on top of a ~3 GB working set per step
    host_batches = [torch.randn(rows, arguments.in_features, generator=generator).to(torch.bfloat16).pin_memory()
                    for _ in range(rotation)]
    device_batches = [batch.to(device) for batch in host_batches]

    # ---- device-timed steps on resident batches ---------------------------------------------------------------
    for step in range(warmup):
        trainer.step_on_device(device_batches[step % rotation])
    fence()
    trainer.check()
    sampler = ClockSampler(local_rank).start()  # every rank samples its own GPU, across both timed regions
    launches_before = ext.launch_count()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for step in range(steps):
        trainer.step_on_device(device_batches[step % rotation])
    stop.record()
    fence()
    elapsed_ms = start.elapsed_time(stop)
    launches = ext.launch_count() - launches_before
    trainer.check()
    final_loss = float(trainer.loss.last_summands[0])
    # every rank must hold the same loss, bit for bit (the summands are all-reduced inside the step)
    loss_bits = gather_objects(int(trainer.loss.last_summands[0].view(torch.int32).item()))
    ranks_disagreeing_on_loss = sum(1 for bits in loss_bits if bits != loss_bits[0])

    # ---- end to end through the public step(): pinned host batches in, loss out, every step --------------------
    e2e_ms = None
    if not arguments.no_e2e:
        # Both timed regions start from the same state: the GPU idles for a moment, then the region's own warm-up steps run.
        # Without the pause the second region inherits the heat and the power-cap history of the first and reads 3-5 % slower
        # for that alone (alternating the regions on one GPU showed it; the pause is reported in `config`).
        torch.cuda.synchronize()
        time.sleep(IDLE_BEFORE_E2E_S)
    device_region_end = sampler.mark()
    if not arguments.no_e2e:
        trainer.feed(host_batches[0])
        for step in range(3):
            trainer.feed(host_batches[(step + 1) % rotation])
            trainer.step()
        trainer.last_loss()
        fence()
        start.record()
        for step in range(steps):
            trainer.feed(host_batches[(step + 1) % rotation])  # the copy for the next step flies under this one
            trainer.step()
        trainer.last_loss()  # the last step's loss has reached the host
        stop.record()
        fence()
        e2e_ms = start.elapsed_time(stop)
    e2e_clock = sampler.region(device_region_end).get("sm_mhz")
    device_clock = sampler.region(0, device_region_end).get("sm_mhz")
    clocks = sampler.stop()

    # ---- the loss step alone (outside the timed regions), to separate the blocks' cost from projector and optimizer ----
    engine = trainer.loss.engine
    embeddings = trainer.projector(device_batches[0]).detach()
    for _ in range(3):
        engine.step(embeddings, scalars=trainer.loss._scalars)
    fence()
    loss_steps = max(3, min(steps, 20))
    start.record()
    for _ in range(loss_steps):
        engine.step(embeddings, scalars=trainer.loss._scalars)
    stop.record()
    fence()
    loss_ms = start.elapsed_time(stop) / loss_steps
    trainer.check()

    def reduce_max(value: float) -> float:
        if world == 1:
            return value
        tensor = torch.tensor([value], dtype=torch.float64, device=device)
        dist.all_reduce(tensor, op=dist.ReduceOp.MAX)
        return float(tensor.item())

    elapsed_ms = reduce_max(elapsed_ms)
    loss_ms = reduce_max(loss_ms)
    if e2e_ms is not None:
        e2e_ms = reduce_max(e2e_ms)
    every_clock = gather_objects(clocks)
    cells_per_step_job = world * trainer.cells_per_step()
    value = cells_per_step_job * steps / (elapsed_ms * 1e-3) / 1e9
    uses_multicast = bool(getattr(trainer.domain, "uses_multicast", False))
    multicast_kernels = ext.last_collective_path() == 1  # what the collective launcher of this process actually used
    if rank == 0:
        reasons = sorted({reason for record in every_clock for reason in record.get("reasons", [])})
        medians = [record.get("sm_mhz") for record in every_clock]
        known = [m for m in medians if m is not None]
        clock_line = dict(clocks)
        clock_line.update({"reasons": reasons, "sm_mhz": min(known) if known else None, "sm_mhz_per_rank": medians,
                           "samples_per_rank": [record.get("samples", 0) for record in every_clock]})
        ms_per_step = elapsed_ms / steps
        line = {
            "metric": "scored_cells_per_second", "value": round(value, 2), "unit": "Gcells/s", "n_gpus": world,
            "steps": steps, "warmup": warmup, "ms_per_step": round(ms_per_step, 4), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": round(value / (PUBLISHED_GCELLS_PER_GPU * world), 3), "dtype": "bf16",
            "data": "synthetic N(0,1) inputs, random-init (Xavier) weights",
            "impl": "ours",
            "config": {
                "model": f"MLP projector {arguments.in_features}->{arguments.mid_features}->{arguments.hidden} (bf16) + "
                         f"K={arguments.prefixes} Matryoshka sigmoid loss + AdamW",
                "rows_per_gpu": rows, "global_batch": rows * world, "seq_len": 1, "hidden": arguments.hidden,
                "prefixes": list(trainer.ladder.ends), "parallelism": f"dp{world}",
                "cells_per_step_per_gpu": trainer.cells_per_step(),
                "collectives": "multimem (NVLS)" if uses_multicast else "peer-to-peer",
                "l2": "inputs rotate over 4 batches (134 MB > 126 MB L2); the step's working set is ~3 GB",
                "baseline_note": "vs_baseline divides by the reference's published 275 Gcells/s per GPU (8xB300, H=1024, "
                                 "loss step only) times n_gpus",
                "final_loss": final_loss,
                "idle_before_e2e_region_s": IDLE_BEFORE_E2E_S,
            },
            "gpu_launches": int(launches),
            "clocks": clock_line,
            # evidence beside the number: correctness of these ranks, which collective kernels ran, where the time goes
            "oracle": oracle_block,
            "ranks_disagreeing_on_loss": ranks_disagreeing_on_loss,
            "multicast_kernels": multicast_kernels,
            "loss_step_ms": round(loss_ms, 4),
            "loss_ms_per_block": round(loss_ms / world, 4),
            "non_loss_ms": round(ms_per_step - loss_ms, 4),
            "ms_times_sm_mhz": round(ms_per_step * clock_line["sm_mhz"], 1) if clock_line["sm_mhz"] else None,
        }
        if e2e_ms is not None:
            line["e2e"] = {"value": round(cells_per_step_job * steps / (e2e_ms * 1e-3) / 1e9, 2), "unit": "Gcells/s",
                           "ms_per_step": round(e2e_ms / steps, 4),
                           "h2d_bytes_per_step": trainer.h2d_bytes_per_step(), "d2h_bytes_per_step": trainer.d2h_bytes_per_step(),
                           # rank 0's median SM clock in each timed region: the end-to-end loop runs second, on a GPU that
                           # has been at its power limit for longer
                           "sm_mhz": e2e_clock, "sm_mhz_device_region": device_clock}
        print(json.dumps(line), flush=True)
    trainer.close()
    if world > 1:
        dist.destroy_process_group()
    return 0


def small_oracle(rank: int, world: int, device, hidden: int, prefixes: int) -> dict:
    """One box step of 128 rows per rank with pair positives, checked on rank 0 against the float64 evaluation of the
    whole world: relative loss error, relative L2 error of all ranks' gradients, and how many ranks hold loss bits that
    differ from rank 0's. Runs before the timed regions, on a domain of its own."""
    import torch
    import torch.distributed as dist

    from scalingcontrasts_b200 import LossSpec, Matryoshka
    from scalingcontrasts_b200.cpu import oracle, relative_l2
    from scalingcontrasts_b200.parallel.box import BoxLoss
    from scalingcontrasts_b200.parallel.domain import Domain
    from scalingcontrasts_b200.utils.keyed import normal_embeddings

    rows, spec = 128, LossSpec("pairs")
    ladder = Matryoshka.halvings(hidden, prefixes)
    domain = Domain.create(payload_scalars=16, heap_bytes=BoxLoss.heap_bytes(rows, hidden, ladder.count), device=device)
    engine = BoxLoss(rows, hidden, ladder, spec, domain)
    block = normal_embeddings(rows, hidden, seed=1, rank=rank).to(device)
    gradient, summands = engine.step(block, 10.0, -10.0)
    torch.cuda.synchronize(device)
    engine.check()
    gradient, summands = gradient.clone(), summands.clone()
    if world > 1:
        blocks = [torch.empty_like(block) for _ in range(world)]
        gradients = [torch.empty_like(gradient) for _ in range(world)]
        losses = [torch.empty_like(summands) for _ in range(world)]
        dist.all_gather(blocks, block)
        dist.all_gather(gradients, gradient)
        dist.all_gather(losses, summands)
    else:
        blocks, gradients, losses = [block], [gradient], [summands]
    path = domain.collective_path()
    domain.close()
    if rank != 0:
        return {}
    expected = oracle(torch.cat([b.cpu() for b in blocks]), ladder, 10.0, -10.0, spec)
    first = int(losses[0][0].view(torch.int32).item())
    return {"rows_per_rank": rows, "hidden": hidden, "prefixes": list(ladder.ends), "positives": "pairs", "ranks": world,
            "rel_loss": abs(float(losses[0][0]) - expected.loss) / abs(expected.loss),
            "rel_grad": float(relative_l2(torch.cat([g.float().cpu() for g in gradients]), expected.gradient)),
            "ranks_disagreeing": sum(1 for other in losses if int(other[0].view(torch.int32).item()) != first),
            "collectives": path}


if __name__ == "__main__":
    sys.exit(main())
