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

``--impl reference`` is the reference arm. The reference is a C++/CUDA/Mojo tree without a Python package, so it cannot
be installed into ``baseline/_ref``; the arm prints its ``unavailable`` line.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys

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

    rows, steps, warmup = arguments.rows, arguments.steps, max(arguments.warmup, 3)
    trainer = ContrastiveTrainer(rows, arguments.in_features, arguments.mid_features, arguments.hidden, arguments.prefixes,
                                 device=device, seed=0)
    generator = torch.Generator(device="cpu").manual_seed(1234 + rank)
    rotation = 4  # 4 x 33.5 MB of inputs > 126 MB of L2, on top of a ~3 GB working set per step
    host_batches = [torch.randn(rows, arguments.in_features, generator=generator).to(torch.bfloat16).pin_memory()
                    for _ in range(rotation)]
    device_batches = [batch.to(device) for batch in host_batches]

    def fence() -> None:
        torch.cuda.synchronize(device)
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize(device)

    # ---- device-timed steps on resident batches ---------------------------------------------------------------
    for step in range(warmup):
        trainer.step_on_device(device_batches[step % rotation])
    fence()
    trainer.check()
    sampler = ClockSampler(local_rank).start() if rank == 0 else None
    launches_before = ext.launch_count()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for step in range(steps):
        trainer.step_on_device(device_batches[step % rotation])
    stop.record()
    fence()
    elapsed_ms = start.elapsed_time(stop)
    launches = ext.launch_count() - launches_before
    clocks = sampler.stop() if sampler is not None else None
    trainer.check()
    final_loss = float(trainer.loss.last_summands[0])

    # ---- end to end through the public step(): pinned host batches in, loss out, every step --------------------
    e2e_ms = None
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

    def reduce_max(value: float) -> float:
        if world == 1:
            return value
        tensor = torch.tensor([value], dtype=torch.float64, device=device)
        dist.all_reduce(tensor, op=dist.ReduceOp.MAX)
        return float(tensor.item())

    elapsed_ms = reduce_max(elapsed_ms)
    if e2e_ms is not None:
        e2e_ms = reduce_max(e2e_ms)
    cells_per_step_job = world * trainer.cells_per_step()
    value = cells_per_step_job * steps / (elapsed_ms * 1e-3) / 1e9
    uses_multicast = bool(getattr(trainer.domain, "uses_multicast", False))
    if rank == 0:
        line = {
            "metric": "scored_cells_per_second", "value": round(value, 2), "unit": "Gcells/s", "n_gpus": world,
            "steps": steps, "warmup": warmup, "ms_per_step": round(elapsed_ms / steps, 4), "higher_is_better": True,
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
            },
            "gpu_launches": int(launches),
            "clocks": clocks,
        }
        if e2e_ms is not None:
            line["e2e"] = {"value": round(cells_per_step_job * steps / (e2e_ms * 1e-3) / 1e9, 2), "unit": "Gcells/s",
                           "ms_per_step": round(e2e_ms / steps, 4),
                           "h2d_bytes_per_step": trainer.h2d_bytes_per_step(), "d2h_bytes_per_step": trainer.d2h_bytes_per_step()}
        print(json.dumps(line), flush=True)
    trainer.close()
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
