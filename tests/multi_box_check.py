"""Run under torchrun on two or more GPUs (tests/test_gpu_multi.py starts it): box steps that close with a barrier
instead of the summands all-reduce, back to back on changing inputs, and steps replayed as CUDA graphs, all against the
float64 evaluation of the world."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from scalingcontrasts_b200 import LossSpec, Matryoshka  # noqa: E402
from scalingcontrasts_b200.cpu import oracle, relative_l2  # noqa: E402
from scalingcontrasts_b200.config import SUMMAND_SLOTS  # noqa: E402
from scalingcontrasts_b200.parallel.box import BoxLoss  # noqa: E402
from scalingcontrasts_b200.parallel.domain import Domain  # noqa: E402
from scalingcontrasts_b200.utils.keyed import normal_embeddings  # noqa: E402


def main() -> None:
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    device = torch.device("cuda", torch.cuda.current_device())
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    dist.init_process_group("nccl", device_id=device)
    rows, hidden, spec = 256, 768, LossSpec("pairs")
    ladder = Matryoshka.halvings(hidden, 5)
    domain = Domain.create(payload_scalars=16, heap_bytes=BoxLoss.heap_bytes(rows, hidden, ladder.count), device=device)
    engine = BoxLoss(rows, hidden, ladder, spec, domain)

    def check(step_index: int, gradient: torch.Tensor, summands: torch.Tensor, block: torch.Tensor, reduced: bool) -> None:
        blocks = [torch.empty_like(block) for _ in range(world)]
        gradients = [torch.empty_like(gradient) for _ in range(world)]
        dist.all_gather(blocks, block)
        dist.all_gather(gradients, gradient)
        total = summands.clone()
        if not reduced:
            dist.all_reduce(total)
        expected = oracle(torch.cat([b.cpu() for b in blocks]), ladder, 10.0, -10.0, spec)
        error = relative_l2(torch.cat([g.float().cpu() for g in gradients]), expected.gradient)
        assert abs(float(total[0]) - expected.loss) <= 2e-6 * abs(expected.loss), (step_index, float(total[0]), expected.loss)
        assert error < 4e-3, (step_index, error)

    # 1. steps without the closing all-reduce, back to back, every step on new rows: the barrier that replaces the
    #    all-reduce must keep a fast rank's next publish from overwriting a block a slower peer still reads
    inputs = [normal_embeddings(rows, hidden, seed=40 + step, rank=rank).to(device) for step in range(4)]
    outcomes = []
    for block in inputs:
        gradient, summands = engine.step(block, 10.0, -10.0, reduce=False)
        outcomes.append((gradient.clone(), summands.clone()))
    torch.cuda.synchronize()
    engine.check()
    for index, (gradient, summands) in enumerate(outcomes):
        check(index, gradient, summands, inputs[index], reduced=False)

    # 2. the same steps with the all-reduce, eagerly and as CUDA graphs (first call eager, second captures, then replays):
    #    the bits must not depend on how the step was enqueued
    eager = []
    for block in inputs:
        gradient, summands = engine.step(block, 10.0, -10.0, graph=False)
        eager.append((gradient.clone(), summands[:SUMMAND_SLOTS].clone()))
    for index, block in enumerate(inputs):
        gradient, summands = engine.step(block, 10.0, -10.0, graph=True)
        torch.cuda.synchronize()
        assert torch.equal(gradient, eager[index][0]) and torch.equal(summands[:SUMMAND_SLOTS], eager[index][1]), index
        check(10 + index, gradient.clone(), summands.clone(), block, reduced=True)
    engine.check()
    dist.barrier()
    domain.close()
    if rank == 0:
        print("box steps ok", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
