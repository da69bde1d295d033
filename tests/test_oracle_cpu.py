import math

import pytest
import torch

from scalingcontrasts_b200 import LossSpec, Matryoshka
from scalingcontrasts_b200.cpu import CpuStreamedLoss, oracle, oracle_loops, relative_l2, simulate_world
from scalingcontrasts_b200.utils.keyed import normal_embeddings

SPECS = [LossSpec("self"), LossSpec("pairs"), LossSpec("pairs", "skip"), LossSpec("pairs", "own")]


def autograd_reference(world, ladder, beta, bias, spec):
    """An independent statement of the loss through torch autograd (float64)."""
    v = world.clone().double().requires_grad_(True)
    t = torch.tensor(math.log(beta), dtype=torch.float64, requires_grad=True)
    b = torch.tensor(bias, dtype=torch.float64, requires_grad=True)
    n = v.shape[0]
    index = torch.arange(n)
    own = index[:, None] == index[None, :]
    z = -torch.ones(n, n, dtype=torch.float64)
    if spec.pairs:
        z[(index[:, None] ^ 1) == index[None, :]] = 1.0
    weight = torch.ones(n, n, dtype=torch.float64)
    if spec.diagonal == "own":
        z[own] = 1.0
    elif spec.diagonal == "skip":
        weight[own] = 0.0
    total = 0.0
    for width in ladder.ends:
        p = torch.nn.functional.normalize(v[:, :width], dim=-1)
        cosine = p @ p.T
        cosine = torch.where(own, torch.ones_like(cosine), cosine)
        total = total + (weight * torch.nn.functional.softplus(-z * (t.exp() * cosine + b))).sum() / n
    total.backward()
    return float(total), v.grad, float(b.grad), float(t.grad)


@pytest.mark.parametrize("spec", SPECS, ids=lambda s: f"{s.positives}-{s.diagonal}")
def test_vectorised_oracle_matches_loops_and_autograd(spec):
    torch.manual_seed(1)
    ladder = Matryoshka.halvings(64, 3)
    world = torch.randn(20, 64, dtype=torch.float64)
    fast, slow = oracle(world, ladder, 10.0, -10.0, spec), oracle_loops(world, ladder, 10.0, -10.0, spec)
    assert fast.loss == pytest.approx(slow.loss, rel=1e-12)
    assert relative_l2(fast.gradient, slow.gradient) < 1e-12
    loss, gradient, bias_grad, scale_grad = autograd_reference(world, ladder, 10.0, -10.0, spec)
    assert fast.loss == pytest.approx(loss, rel=1e-12)
    assert relative_l2(fast.gradient, gradient) < 1e-10
    assert fast.bias_grad == pytest.approx(bias_grad, rel=1e-10)
    assert fast.log_beta_grad == pytest.approx(scale_grad, rel=1e-10)


def test_native_oracle_twin(ext):
    torch.manual_seed(2)
    ladder = Matryoshka.halvings(64, 3)
    world = torch.randn(24, 64, dtype=torch.float64)
    for spec in SPECS:
        expected = oracle(world, ladder, 10.0, -10.0, spec)
        gradient, out = ext.oracle_loops(world, list(ladder.ends), 10.0, -10.0, spec.code())
        assert float(out[0]) == pytest.approx(expected.loss, rel=1e-12)
        assert float(out[1]) == pytest.approx(expected.bias_grad, rel=1e-10)
        assert float(out[2]) == pytest.approx(expected.log_beta_grad, rel=1e-10)
        assert relative_l2(gradient, expected.gradient) < 1e-12
        assert torch.allclose(out[4:7], expected.band_losses, rtol=1e-12)


def test_config_one_world_of_two_fp32_against_float64():
    """R=128 rows per rank, H=256, K=3 (64/128/256), N(0,1) seed 0 normalised, pairs positives, two ranks."""
    ladder = Matryoshka.halvings(256, 3)
    spec = LossSpec("pairs")
    blocks = [normal_embeddings(128, 256, 0, rank, torch.float32) for rank in range(2)]
    expected = oracle(torch.cat(blocks), ladder, 10.0, -10.0, spec)
    gradients, summands = simulate_world(blocks, ladder, 10.0, -10.0, spec, torch.float32)
    assert float(summands[0]) == pytest.approx(expected.loss, rel=1e-6)
    assert relative_l2(torch.cat(gradients), expected.gradient) < 1e-5
    assert float(summands[1]) == pytest.approx(expected.bias_grad, rel=1e-5)
    assert float(summands[2]) == pytest.approx(expected.log_beta_grad, rel=1e-4, abs=1e-6)
    assert torch.allclose(summands[4:7].double(), expected.band_losses, rtol=1e-6)


def test_block_order_does_not_matter():
    ladder = Matryoshka.halvings(128, 2)
    blocks = [normal_embeddings(32, 128, 3, rank, torch.float64) for rank in range(4)]
    forward, total_forward = simulate_world(blocks, ladder, 10.0, -10.0, dtype=torch.float64)
    backward, total_backward = simulate_world(blocks, ladder, 10.0, -10.0, dtype=torch.float64,
                                              order=lambda rank: reversed(range(4)))
    assert relative_l2(torch.cat(forward), torch.cat(backward)) < 1e-13
    assert torch.allclose(total_forward, total_backward, rtol=1e-13)


@pytest.mark.parametrize("hidden,prefixes", [(64, 1), (256, 3)])
def test_collinear_rows_have_exactly_zero_gradient(hidden, prefixes):
    """Rows e0 scaled by 1, 1/16, 1/256 and 0: every cosine is 1, floored or undefined, so nothing may move."""
    ladder = Matryoshka.halvings(hidden, prefixes)
    rows = torch.zeros(128, hidden, dtype=torch.float32)
    scales = [1.0, 1.0 / 16, 1.0 / 256, 0.0]
    for i in range(128):
        rows[i, 0] = scales[i % 4]
    loss = CpuStreamedLoss(128, hidden, ladder)
    loss.begin(rows)
    loss.score(rows, rows, 0, 0, 10.0, -10.0, 128)
    gradient, _ = loss.finish(rows, torch.empty(128, hidden))
    assert torch.count_nonzero(gradient) == 0


def test_memory_is_independent_of_world_size():
    ladder = Matryoshka.halvings(64, 2)
    loss = CpuStreamedLoss(16, 64, ladder)
    before = loss.bytes()
    block = torch.randn(16, 64)
    loss.begin(block)
    for peer in range(9):
        loss.score(block, block, 0, peer * 16, 10.0, -10.0, 9 * 16)
    loss.finish(block, torch.empty(16, 64))
    assert loss.bytes() == before
