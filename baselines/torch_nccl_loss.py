"""torch + NCCL baseline of the Matryoshka sigmoid loss in the all_gather style of big_vision / open_clip ``gather``:
every rank gathers the other ranks' embeddings (gradients flow back through a reduce-scatter), then per prefix
``normalize -> matmul -> * t + b -> logsigmoid`` under autograd. Timed and measured like the library's own modes.

    torchrun --nproc-per-node 8 --master-addr 127.0.0.1 baselines/torch_nccl_loss.py --pairs 4096 --hidden 768 --prefixes 5
    python baselines/torch_nccl_loss.py --pairs 4096 --hidden 768 --prefixes 5 --simulate 72

``--impl oneset`` scores one set of rows against itself (the cells this library scores: R x N R x K per rank);
``--impl twotower`` is the image/text form (2 x as many matrix products per cell pair). One CSV row:

    pairs,hidden,prefixes,world,impl,dtype,saved_bytes,peak_bytes,min_ms,median_ms,gcells_per_s_per_gpu

Stands in for the reference's ``baseline_torch.py`` (open_clip) and ``baseline_jax.py`` (big_vision), whose packages
are not on this image; same columns as ``baseline_torch.py:128``.
"""
from __future__ import annotations

import argparse
import os

import torch
import torch.distributed as dist
import torch.nn.functional as F


class GatherWithGradient(torch.autograd.Function):
    """all_gather whose backward reduce-scatters the gradient back to the owners."""

    @staticmethod
    def forward(ctx, block):
        world = dist.get_world_size()
        gathered = torch.empty(world * block.shape[0], block.shape[1], dtype=block.dtype, device=block.device)
        dist.all_gather_into_tensor(gathered, block.contiguous())
        return gathered

    @staticmethod
    def backward(ctx, grad):
        world = dist.get_world_size()
        out = torch.empty(grad.shape[0] // world, grad.shape[1], dtype=grad.dtype, device=grad.device)
        dist.reduce_scatter_tensor(out, grad.contiguous())
        return out


def prefix_widths(hidden: int, prefixes: int):
    return [hidden >> (prefixes - 1 - p) for p in range(prefixes)]


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--pairs", type=int, default=1024)
    parser.add_argument("--hidden", type=int, default=1024)
    parser.add_argument("--prefixes", type=int, default=1)
    parser.add_argument("--impl", choices=["oneset", "twotower"], default="oneset")
    parser.add_argument("--simulate", type=int, default=0, help="one rank of this many GPUs, on one GPU")
    parser.add_argument("--dtype", choices=["bf16", "fp32"], default="bf16")
    parser.add_argument("--windows", type=int, default=10)
    parser.add_argument("--calls-per-window", type=int, default=3)
    parser.add_argument("--header", action="store_true")
    arguments = parser.parse_args()

    distributed = "WORLD_SIZE" in os.environ and arguments.simulate == 0 and int(os.environ["WORLD_SIZE"]) > 1
    rank = int(os.environ.get("RANK", 0)) if distributed else 0
    world = int(os.environ["WORLD_SIZE"]) if distributed else max(arguments.simulate, 1)
    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0)))
    torch.cuda.set_device(device)
    if distributed:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)
    dtype = torch.bfloat16 if arguments.dtype == "bf16" else torch.float32
    generator = torch.Generator(device=device).manual_seed(rank)
    shape = (arguments.pairs, arguments.hidden)
    first = F.normalize(torch.randn(shape, device=device, generator=generator), dim=-1).to(dtype).requires_grad_(True)
    second = F.normalize(torch.randn(shape, device=device, generator=generator), dim=-1).to(dtype).requires_grad_(True)
    scale = torch.tensor(10.0, device=device, requires_grad=True)
    bias = torch.tensor(-10.0, device=device, requires_grad=True)
    widths = prefix_widths(arguments.hidden, arguments.prefixes)
    rows = arguments.pairs

    def others(block):
        if distributed:
            return GatherWithGradient.apply(block)
        if world == 1:
            return block
        # one rank of a simulated world: the own block, then detached stand-ins for the received ones
        return torch.cat([block] + [block.detach().clone().requires_grad_(True) for _ in range(world - 1)])

    def forward():
        queries = first
        candidates = others(first if arguments.impl == "oneset" else second)
        labels = -torch.ones(rows, candidates.shape[0], device=device, dtype=torch.float32)
        offset = rank * rows
        labels[torch.arange(rows, device=device), offset + torch.arange(rows, device=device)] = 1.0
        total = 0.0
        for width in widths:
            q = F.normalize(queries[:, :width].float(), dim=-1).to(dtype)
            c = F.normalize(candidates[:, :width].float(), dim=-1).to(dtype)
            logits = (q @ c.T).float() * scale + bias
            total = total + F.softplus(-labels * logits).sum() / candidates.shape[0]
        return total

    def step():
        first.grad = second.grad = scale.grad = bias.grad = None
        forward().backward()

    step()
    torch.cuda.synchronize()
    first.grad = second.grad = scale.grad = bias.grad = None
    torch.cuda.empty_cache()
    baseline = torch.cuda.memory_allocated()
    torch.cuda.reset_peak_memory_stats()
    total = forward()
    saved = torch.cuda.memory_allocated() - baseline
    total.backward()
    torch.cuda.synchronize()
    peak = torch.cuda.max_memory_allocated() - baseline

    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    per_call = []
    for _ in range(arguments.windows):
        if distributed:
            dist.barrier()
        torch.cuda.synchronize()
        start.record()
        for _ in range(arguments.calls_per_window):
            step()
        stop.record()
        stop.synchronize()
        elapsed = torch.tensor([start.elapsed_time(stop) / arguments.calls_per_window], device=device, dtype=torch.float64)
        if distributed:
            dist.all_reduce(elapsed, op=dist.ReduceOp.MAX)
        per_call.append(float(elapsed))
    per_call.sort()
    if rank == 0:
        if arguments.header:
            print("pairs,hidden,prefixes,world,impl,dtype,saved_bytes,peak_bytes,min_ms,median_ms,gcells_per_s_per_gpu")
        impl = arguments.impl if distributed or world == 1 else f"{arguments.impl}-simulated"
        cells = rows * rows * world * arguments.prefixes
        print(f"{rows},{arguments.hidden},{arguments.prefixes},{world},torch-nccl-{impl},{arguments.dtype},{saved},{peak},"
              f"{per_call[0]:.4f},{per_call[len(per_call) // 2]:.4f},{cells / per_call[0] / 1e6:.1f}", flush=True)
    if distributed:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
