"""Host-side logic of the multi-process paths, run as gloo ranks on the CPU: descriptor exchange, host domain, the loss
module's CPU path across ranks, and failure detection when a rank never joins."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port() -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as probe:
        probe.bind(("127.0.0.1", 0))
        return probe.getsockname()[1]


def _launch(worker, world: int, *arguments) -> None:
    mp.start_processes(worker, args=(world, _free_port()) + arguments, nprocs=world, join=True, start_method="spawn")


def _init(rank: int, world: int, port: int) -> None:
    os.environ.update({"MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port), "RANK": str(rank), "WORLD_SIZE": str(world)})
    dist.init_process_group("gloo", rank=rank, world_size=world)


def _exchange_worker(rank: int, world: int, port: int) -> None:
    from scalingcontrasts_b200.parallel.domain import StoreRendezvous, _exchange_descriptors

    _init(rank, world, port)
    rendezvous = StoreRendezvous()
    own = os.memfd_create(f"rank{rank}")
    os.write(own, f"hello from {rank}".encode())
    shared = os.memfd_create("shared")
    os.write(shared, b"shared object")
    descriptors, extra = _exchange_descriptors(rendezvous, own, (lambda: shared) if rank == 0 else None)
    assert len(descriptors) == world and extra >= 0
    assert os.pread(extra, 64, 0) == b"shared object"
    for peer, descriptor in enumerate(descriptors):
        assert os.pread(descriptor, 64, 0) == f"hello from {peer}".encode()  # the peer's file, through SCM_RIGHTS
    rendezvous.barrier("after-read")
    assert rendezvous.all_agree("all-true", True) is True
    assert rendezvous.all_agree("one-false", rank != 1) is False
    dist.destroy_process_group()


def test_descriptor_exchange_over_unix_socket():
    _launch(_exchange_worker, 3)


def _loss_worker(rank: int, world: int, port: int) -> None:
    from scalingcontrasts_b200 import LossSpec, Matryoshka
    from scalingcontrasts_b200.cpu import oracle, relative_l2
    from scalingcontrasts_b200.models.loss import MatryoshkaSigmoidLoss
    from scalingcontrasts_b200.parallel.domain import Domain
    from scalingcontrasts_b200.utils.keyed import normal_embeddings

    _init(rank, world, port)
    domain = Domain.create(payload_scalars=16, device="cpu")
    assert type(domain).__name__ == "HostDomain" and domain.members == world
    domain.payload()[:4] = torch.arange(4, dtype=torch.float32) + rank
    domain.all_reduce(4)
    assert torch.equal(domain.payload()[:4], torch.tensor([1.0, 3.0, 5.0, 7.0]))
    spec = LossSpec("pairs")
    ladder = Matryoshka.halvings(256, 3)
    blocks = [normal_embeddings(128, 256, 0, r, torch.float32) for r in range(world)]
    module = MatryoshkaSigmoidLoss(128, 256, 3, spec=spec, device="cpu")
    mine = blocks[rank].clone().requires_grad_(True)
    loss = module(mine)
    loss.backward()
    expected = oracle(torch.cat(blocks), ladder, 10.0, -10.0, spec)
    assert float(loss) == pytest.approx(expected.loss, rel=1e-6)
    assert relative_l2(mine.grad, expected.gradient[rank * 128:(rank + 1) * 128]) < 1e-5
    assert float(module.logit_bias.grad) == pytest.approx(expected.bias_grad, rel=1e-5)
    assert float(module.logit_scale.grad) == pytest.approx(expected.log_beta_grad, rel=1e-4, abs=1e-6)
    dist.destroy_process_group()


def test_config_one_on_two_gloo_ranks():
    _launch(_loss_worker, 2)


def _missing_rank_worker(rank: int, world: int, port: int) -> None:
    from scalingcontrasts_b200.parallel.domain import DomainError, StoreRendezvous

    _init(rank, world, port)
    rendezvous = StoreRendezvous(timeout_s=0.5)
    rendezvous.barrier("everyone")
    if rank == 1:
        # this rank never joins the next barrier: it leaves between steps, with nothing in flight
        dist.destroy_process_group()
        return
    with pytest.raises(DomainError):
        rendezvous.barrier("one-missing")
    dist.destroy_process_group()


def test_a_rank_that_never_joins_is_detected_on_the_host():
    _launch(_missing_rank_worker, 2)


def _ring_worker(rank: int, world: int, port: int) -> None:
    import importlib.util

    from scalingcontrasts_b200 import LossSpec, Matryoshka
    from scalingcontrasts_b200.cpu import oracle, relative_l2
    from scalingcontrasts_b200.utils.keyed import normal_embeddings

    _init(rank, world, port)
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "baselines", "torch_ring_loss.py")
    spec = importlib.util.spec_from_file_location("torch_ring_loss", path)
    ring = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ring)
    rows, hidden, prefixes = 64, 128, 3
    block = normal_embeddings(rows, hidden, seed=3, rank=rank).float()
    loss_share, gradient = ring.ring_step(block, ring.prefix_widths(hidden, prefixes), torch.tensor(10.0), torch.tensor(-10.0))
    blocks = [torch.empty_like(block) for _ in range(world)]
    gradients = [torch.empty_like(gradient) for _ in range(world)]
    dist.all_gather(blocks, block)
    dist.all_gather(gradients, gradient)
    total = loss_share.clone()
    dist.all_reduce(total)
    expected = oracle(torch.cat(blocks), Matryoshka.halvings(hidden, prefixes), 10.0, -10.0, LossSpec("self"))
    assert abs(float(total) - expected.loss) <= 1e-5 * abs(expected.loss)
    assert relative_l2(torch.cat(gradients), expected.gradient) < 1e-4
    dist.destroy_process_group()


def test_ring_exchange_baseline_agrees_with_the_oracle():
    """The plain-torch neighbour-exchange comparator (baselines/torch_ring_loss.py) computes the same loss and row-owned
    gradient as the float64 oracle: a baseline that is wrong would flatter whatever is compared with it."""
    _launch(_ring_worker, 3)
