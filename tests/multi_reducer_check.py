"""Run under torchrun by test_gpu_multi.py: the overlapped gradient reducer must give every rank the NCCL sum."""
import os

import torch
import torch.distributed as dist


def main() -> None:
    from scalingcontrasts_b200.models.projector import Projector
    from scalingcontrasts_b200.parallel.domain import Domain
    from scalingcontrasts_b200.parallel.reducer import GradientReducer

    local_rank = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    dist.init_process_group("nccl", device_id=device)
    rank = dist.get_rank()
    model = Projector(64, 128, 64, torch.bfloat16, device, seed=0)
    domain = Domain.create(payload_scalars=16, heap_bytes=GradientReducer.heap_bytes(model.parameters()), device=device)
    reducer = GradientReducer(model.parameters(), domain, bucket_bytes=16 << 10)
    for step in range(3):
        x = torch.randn(256, 64, generator=torch.Generator().manual_seed(100 * step + rank)).to(device, torch.bfloat16)
        model.zero_grad(set_to_none=True)
        # odd steps: the tower's backward writes its gradients straight into the reducer's bucket slots (no copy in the hook)
        model.gradient_landing = reducer.landing_buffers(model) if step % 2 else None
        model(x).float().square().sum().backward()
        if step % 2:
            assert all(p.grad.data_ptr() == reducer.landing_buffers(model)[n].data_ptr() for n, p in model.named_parameters())
        reducer.wait()
        torch.cuda.synchronize()
        # the same backward without hooks, summed by NCCL in float32
        reference = Projector(64, 128, 64, torch.bfloat16, device, seed=0)
        reference(x).float().square().sum().backward()
        for mine, theirs in zip(model.parameters(), reference.parameters()):
            expected = theirs.grad.float()
            dist.all_reduce(expected)
            error = (mine.grad.float() - expected).norm() / expected.norm().clamp_min(1e-12)
            assert float(error) < 1e-2, float(error)  # bfloat16 storage of the reduced value
    domain.check()
    dist.barrier()
    if rank == 0:
        print("reducer ok", flush=True)
    domain.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
