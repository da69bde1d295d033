"""Single-GPU checks of the symmetric domain and its collectives: a world of one still runs every kernel, and the
bounded wait is exercised with arrivals that nobody makes."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def domains():
    from scalingcontrasts_b200.parallel.domain import Domain

    made = {}
    for multicast in (True, False):
        made[multicast] = Domain.create(payload_scalars=1 << 16, heap_bytes=1 << 20, device="cuda", multicast=multicast, budget_s=0.2)
    yield made
    for domain in made.values():
        domain.close()


@pytest.mark.parametrize("multicast", [True, False])
def test_world_of_one_collectives(domains, ext, multicast):
    from scalingcontrasts_b200.utils.keyed import keyed_fractions

    domain = domains[multicast]
    payload = domain.payload()
    values = keyed_fractions(1 << 16, 1, 0).cuda()
    payload.copy_(values)
    domain.barrier()
    domain.all_reduce()
    domain.reduce_scatter(1 << 16)
    domain.barrier()
    torch.cuda.synchronize()
    domain.check()
    assert torch.equal(payload, values)  # a sum over one member changes nothing
    payload.copy_(values)
    domain.all_reduce(scale=0.5)
    torch.cuda.synchronize()
    assert torch.equal(payload, values * 0.5)
    out = torch.empty(1 << 16, device="cuda")
    domain.reduce_scatter(1 << 16, out=out, scale=2.0)
    torch.cuda.synchronize()
    assert torch.equal(out, values)
    # bfloat16 payload in the heap, reduced in float32
    offset = domain.alloc(4096 * 2)
    region = domain.tensor(offset, (4096,), torch.bfloat16)
    region.copy_(values[:4096].to(torch.bfloat16))
    domain.all_reduce(4096, offset=offset, dtype=torch.bfloat16, scale=2.0)
    torch.cuda.synchronize()
    assert torch.equal(region, (values[:4096].to(torch.bfloat16).float() * 2.0).to(torch.bfloat16))
    domain.check()


@pytest.mark.parametrize("multicast", [True, False])
def test_one_round_and_two_round_all_reduce_agree(domains, multicast):
    """Payloads of up to 64 KiB take the one-round latency form by default; forced through the two-round form they must
    give the same bits, at the largest such size and at a few vectors, in float32 and in bfloat16 with a scale."""
    from scalingcontrasts_b200.utils.keyed import keyed_fractions

    domain = domains[multicast]
    payload = domain.payload()
    values = keyed_fractions(1 << 14, 1, 3).cuda()
    for scalars in (1 << 14, 12 * 4, 4):
        outcomes = []
        for latency in (None, False, None):  # one-round twice in a row: both sets of staging slots get used
            payload[:1 << 14].copy_(values)
            domain.all_reduce(scalars, scale=0.25, latency=latency)
            torch.cuda.synchronize()
            outcomes.append(payload[:1 << 14].clone())
        assert torch.equal(outcomes[0], outcomes[1]) and torch.equal(outcomes[0], outcomes[2])
        assert torch.equal(outcomes[0][:scalars], values[:scalars] * 0.25) and torch.equal(outcomes[0][scalars:], values[scalars:])
    domain.check()
    assert domain.collective_path() in ("multimem", "peer")


def test_bounded_wait_reports_and_recovers(domains):
    from scalingcontrasts_b200.parallel.domain import DomainError

    domain = domains[False]
    domain.set_budget(0.05)
    domain.expect_arrivals(1)  # nobody makes this arrival: the wait must run out, not hang
    torch.cuda.synchronize()
    with pytest.raises(DomainError):
        domain.check()
    words = domain.status_words()
    assert words[0] == 1 and words[1] == 3
    domain.barrier()  # poisoned: returns at once
    torch.cuda.synchronize()
    domain.reset()
    domain.set_budget(0.2)
    domain.barrier()
    domain.all_reduce(16)
    torch.cuda.synchronize()
    domain.check()


def test_channels_are_independent(domains):
    domain = domains[True]
    side = torch.cuda.Stream()
    domain.payload().fill_(1.0)
    torch.cuda.synchronize()
    domain.all_reduce(64, channel=0)
    domain.all_reduce(64, side, offset=domain.alloc(1024), channel=1)
    torch.cuda.synchronize()
    domain.check()
