"""NCCL all-reduce and reduce-scatter sweep, the comparator of the library's ``collectives`` mode: float32, in place,
1 KiB to 128 MiB, 20 calls per window after 5 warm-up calls, CUDA-event timed, maximum over ranks, nccl-tests bus
bandwidth (all-reduce ``bytes/t * 2(n-1)/n``, reduce-scatter ``bytes/t * (n-1)/n`` with ``bytes`` the whole per-GPU
payload). Run it twice, with ``NCCL_NVLS_ENABLE=1`` and ``NCCL_NVLS_ENABLE=0``:

    NCCL_NVLS_ENABLE=1 torchrun --nproc-per-node 8 --master-addr 127.0.0.1 baselines/nccl_collectives.py
    NCCL_NVLS_ENABLE=0 torchrun --nproc-per-node 8 --master-addr 127.0.0.1 baselines/nccl_collectives.py

Rows: ``nccl_all_reduce|nccl_reduce_scatter,count,bytes,min_us,median_us,algbw,busbw,nvls``.
Stands in for nccl-tests (``all_reduce_perf`` / ``reduce_scatter_perf -g 8 -n 20 -w 5 -c 0``), which is not installed.
"""
from __future__ import annotations

import argparse
import os

import torch
import torch.distributed as dist


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--min-kib", type=int, default=1)
    parser.add_argument("--max-mib", type=int, default=128)
    parser.add_argument("--windows", type=int, default=5)
    parser.add_argument("--calls", type=int, default=20)
    parser.add_argument("--warm", type=int, default=5)
    arguments = parser.parse_args()
    local_rank = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", device_id=device)
    rank, count = dist.get_rank(), dist.get_world_size()
    nvls = os.environ.get("NCCL_NVLS_ENABLE", "default")
    max_scalars = arguments.max_mib * (1 << 20) // 4
    payload = torch.rand(max_scalars, device=device) * 2 - 1
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def timed(call):
        for _ in range(arguments.warm):
            call()
        samples = []
        for _ in range(arguments.windows):
            torch.cuda.synchronize()
            dist.barrier()
            torch.cuda.synchronize()
            start.record()
            for _ in range(arguments.calls):
                call()
            stop.record()
            stop.synchronize()
            elapsed = torch.tensor([start.elapsed_time(stop) / arguments.calls], device=device, dtype=torch.float64)
            dist.all_reduce(elapsed, op=dist.ReduceOp.MAX)
            samples.append(float(elapsed))
        samples.sort()
        return samples[0], samples[len(samples) // 2]

    if rank == 0:
        print("op,count,bytes,min_us,median_us,algbw,busbw,nvls", flush=True)
    scalars = max(arguments.min_kib * 1024 // 4, 4 * count)
    while scalars <= max_scalars:
        shard = scalars // count // 4 * 4
        total = shard * count
        view = payload[:total]
        own = view[rank * shard:(rank + 1) * shard]
        for name, call, factor in (("nccl_reduce_scatter", lambda: dist.reduce_scatter_tensor(own, view), (count - 1) / count),
                                   ("nccl_all_reduce", lambda: dist.all_reduce(view), 2 * (count - 1) / count)):
            low, middle = timed(call)
            algbw = total * 4 / (low * 1e6)
            if rank == 0:
                print(f"{name},{count},{total * 4},{low * 1e3:.2f},{middle * 1e3:.2f},{algbw:.2f},{algbw * factor:.2f},{nvls}",
                      flush=True)
            payload.uniform_(-1, 1)
        scalars *= 2
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
