"""A second, independent comparator in plain torch: the one-set Matryoshka sigmoid loss with a neighbour exchange (ring)
instead of an all_gather, in the style of open_clip's ``bidir`` / ``shift`` modes. Blocks travel around the ring with
``batch_isend_irecv``; every rank scores its own rows against the block in hand, per prefix
``normalize -> matmul -> * t + b -> softplus`` under autograd, and keeps the gradient of its own rows only: a cell and its
mirror are the same number, so the owner applies both (twice the off-block gradient) and nothing flows back around the
ring. That is this library's row-owned algorithm without its kernels, which makes it the like-for-like framework
baseline; the all_gather form is ``baselines/torch_nccl_loss.py``.

    torchrun --nproc-per-node 8 --master-addr 127.0.0.1 baselines/torch_ring_loss.py --pairs 4096 --hidden 768 --prefixes 5
    torchrun --nproc-per-node 2 --master-addr 127.0.0.1 baselines/torch_ring_loss.py --device cpu --pairs 128 --hidden 256 --prefixes 3

One CSV row, the columns of the reference's baselines (baseline_torch.py:128) plus the cell rate:

    pairs,hidden,prefixes,world,impl,dtype,saved_bytes,peak_bytes,min_ms,median_ms,gcells_per_s_per_gpu

Stands in for the reference's ``baseline_jax.py`` (big_vision under JAX), whose package is not on this image.
"""
from __future__ import annotations

import argparse
import os
import time
from typing import List, Sequence, Tuple

import torch
import torch.distributed as dist
import torch.nn.functional as F


def prefix_widths(hidden: int, prefixes: int) -> List[int]:
    return [hidden >> (prefixes - 1 - p) for p in range(prefixes)]


def block_loss(queries: torch.Tensor, candidates: torch.Tensor, widths: Sequence[int], scale: torch.Tensor, bias: torch.Tensor,
               own: bool, live: int) -> torch.Tensor:
    """Sum over prefixes of the sigmoid loss of ``queries`` against ``candidates`` (weight 1 / live per cell). In the own
    block the diagonal cell is the positive with its cosine taken as exactly 1, as in the reference's oracle
    (scalingcontrasts.cu:155-159)."""
    total = queries.new_zeros((), dtype=torch.float32)
    for width in widths:
        q = F.normalize(queries[:, :width].float(), dim=-1)
        c = F.normalize(candidates[:, :width].float(), dim=-1)
        logits = (q.to(queries.dtype) @ c.to(queries.dtype).T).float() * scale + bias
        signs = -torch.ones_like(logits)
        if own:
            index = torch.arange(logits.shape[0], device=logits.device)
            logits = logits.clone()
            logits[index, index] = scale * 1.0 + bias
            signs[index, index] = 1.0
        total = total + F.softplus(-signs * logits).sum() / live
    return total


def ring_step(block: torch.Tensor, widths: Sequence[int], scale: torch.Tensor, bias: torch.Tensor,
              group=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """One step on this rank: returns (this rank's share of the loss, gradient of the whole world's loss with respect to
    this rank's rows). ``block`` is ``[rows, hidden]``; ranks hold equally sized blocks."""
    distributed = dist.is_available() and dist.is_initialized()
    world = dist.get_world_size(group) if distributed else 1
    rank = dist.get_rank(group) if distributed else 0
    live = world * block.shape[0]
    queries = block.detach().clone().requires_grad_(True)
    in_hand = block.detach().clone()
    loss_share = torch.zeros((), dtype=torch.float32, device=block.device)
    for hop in range(world):
        pending, received = [], None
        if hop + 1 < world:  # pass the block in hand on while it is being scored
            received = torch.empty_like(in_hand)
            right = dist.get_global_rank(group, (rank + 1) % world) if group is not None else (rank + 1) % world
            left = dist.get_global_rank(group, (rank - 1) % world) if group is not None else (rank - 1) % world
            pending = dist.batch_isend_irecv([dist.P2POp(dist.isend, in_hand, right, group),
                                              dist.P2POp(dist.irecv, received, left, group)])
        if hop == 0:
            loss = block_loss(queries, queries, widths, scale, bias, True, live)  # both sides attached: the mirror is inside
            loss.backward()
        else:
            loss = block_loss(queries, in_hand, widths, scale, bias, False, live)
            (2.0 * loss).backward()  # the owner applies the cell and its mirror
        loss_share = loss_share + loss.detach()
        for request in pending:
            request.wait()
        if received is not None:
            in_hand = received
    return loss_share, queries.grad


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--pairs", type=int, default=1024)
    parser.add_argument("--hidden", type=int, default=1024)
    parser.add_argument("--prefixes", type=int, default=1)
    parser.add_argument("--dtype", choices=["bf16", "fp32"], default="bf16")
    parser.add_argument("--device", choices=["cuda", "cpu"], default="cuda")
    parser.add_argument("--windows", type=int, default=10)
    parser.add_argument("--calls-per-window", type=int, default=3)
    parser.add_argument("--header", action="store_true")
    arguments = parser.parse_args()

    distributed = int(os.environ.get("WORLD_SIZE", "1")) > 1
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    cuda = arguments.device == "cuda"
    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0))) if cuda else torch.device("cpu")
    if cuda:
        torch.cuda.set_device(device)
    if distributed:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device) if cuda else dist.init_process_group("gloo")
    dtype = torch.bfloat16 if arguments.dtype == "bf16" else torch.float32
    generator = torch.Generator().manual_seed(rank)
    block = torch.randn(arguments.pairs, arguments.hidden, generator=generator).to(device=device, dtype=dtype)
    scale = torch.tensor(10.0, device=device)
    bias = torch.tensor(-10.0, device=device)
    widths = prefix_widths(arguments.hidden, arguments.prefixes)

    def step() -> None:
        ring_step(block, widths, scale, bias)

    def drain() -> None:
        if cuda:
            torch.cuda.synchronize()

    step()
    drain()
    saved = peak = 0
    if cuda:
        torch.cuda.empty_cache()
        baseline = torch.cuda.memory_allocated()
        torch.cuda.reset_peak_memory_stats()
        step()
        drain()
        peak = torch.cuda.max_memory_allocated() - baseline
    per_call = []
    for _ in range(arguments.windows):
        if distributed:
            dist.barrier()
        drain()
        if cuda:
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
        begin = time.perf_counter()
        for _ in range(arguments.calls_per_window):
            step()
        if cuda:
            stop.record()
            stop.synchronize()
            elapsed_ms = start.elapsed_time(stop) / arguments.calls_per_window
        else:
            elapsed_ms = (time.perf_counter() - begin) * 1e3 / arguments.calls_per_window
        elapsed = torch.tensor([elapsed_ms], device=device, dtype=torch.float64)
        if distributed:
            dist.all_reduce(elapsed, op=dist.ReduceOp.MAX)
        per_call.append(float(elapsed))
    per_call.sort()
    if rank == 0:
        if arguments.header:
            print("pairs,hidden,prefixes,world,impl,dtype,saved_bytes,peak_bytes,min_ms,median_ms,gcells_per_s_per_gpu")
        cells = arguments.pairs * arguments.pairs * world * arguments.prefixes
        print(f"{arguments.pairs},{arguments.hidden},{arguments.prefixes},{world},torch-ring-oneset,{arguments.dtype},{saved},{peak},"
              f"{per_call[0]:.4f},{per_call[len(per_call) // 2]:.4f},{cells / per_call[0] / 1e6:.1f}", flush=True)
    if distributed:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
