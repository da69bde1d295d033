"""``FusedAdamW`` (csrc/optim.cu) against AdamW written out in float32 torch operations."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _reference_step(p32, g32, m, v, step, lr, b1, b2, eps, decay):
    p32 = p32 * (1.0 - lr * decay)
    m = b1 * m + (1.0 - b1) * g32
    v = b2 * v + (1.0 - b2) * g32 * g32
    c1, c2 = 1.0 - b1 ** step, 1.0 - b2 ** step
    p32 = p32 - (lr / c1) * m / (v.sqrt() / (c2 ** 0.5) + eps)
    return p32, m, v


@pytest.mark.parametrize("decay", [0.0, 0.1])
def test_five_steps_match_the_float32_statement(decay):
    from scalingcontrasts_b200.optim import FusedAdamW

    torch.manual_seed(0)
    shapes = [((3072, 1024), torch.bfloat16), ((768,), torch.bfloat16), ((13, 5), torch.bfloat16), ((), torch.float32),
              ((1000,), torch.float32)]
    params = [torch.randn(shape, device="cuda").to(dtype).requires_grad_(True) for shape, dtype in shapes]
    lr, betas, eps = 1e-2, (0.9, 0.95), 1e-8
    optimizer = FusedAdamW(params, lr=lr, betas=betas, eps=eps, weight_decay=decay)
    shadow = [p.detach().float().clone() for p in params]
    moments = [(torch.zeros_like(s), torch.zeros_like(s)) for s in shadow]
    for step in range(1, 6):
        for index, p in enumerate(params):
            p.grad = (torch.randn(p.shape, device="cuda") * (10.0 ** (index - 2))).to(p.dtype)
        optimizer.step()
        torch.cuda.synchronize()
        for index, p in enumerate(params):
            # the reference restarts from the parameter as the kernel rounded it, so that one step is compared at a time
            updated, m, v = _reference_step(shadow[index], p.grad.float(), *moments[index], step, lr, *betas, eps, decay)
            moments[index] = (m, v)
            expected = updated.to(p.dtype)
            difference = (p.detach().float() - expected.float()).abs()
            tolerance = 2.0 ** -7 * expected.float().abs() + 1e-6 if p.dtype == torch.bfloat16 else 1e-5 * expected.abs() + 1e-7
            assert bool((difference <= tolerance).all()), (step, index, float(difference.max()))
            assert torch.allclose(optimizer.exp_avg[index], m, rtol=1e-5, atol=1e-7 * float(m.abs().max() + 1))
            assert torch.allclose(optimizer.exp_avg_sq[index], v, rtol=1e-5, atol=1e-7 * float(v.abs().max() + 1))
            shadow[index] = p.detach().float().clone()


def test_checkpoint_restores_the_moments_bit_for_bit():
    from scalingcontrasts_b200.optim import FusedAdamW

    torch.manual_seed(1)

    def fresh():
        return [torch.full((256, 64), 0.5, device="cuda", dtype=torch.bfloat16).requires_grad_(True),
                torch.tensor(2.0, device="cuda").requires_grad_(True)]

    gradients = [[torch.randn(256, 64, device="cuda").to(torch.bfloat16), torch.randn((), device="cuda")] for _ in range(4)]

    def run(optimizer, params, which):
        for index in which:
            for p, g in zip(params, gradients[index]):
                p.grad = g.clone()
            optimizer.step()

    params = fresh()
    straight = FusedAdamW(params, lr=1e-2)
    run(straight, params, range(4))
    first = fresh()
    before = FusedAdamW(first, lr=1e-2)
    run(before, first, range(2))
    state = before.state_dict()
    second = [p.detach().clone().requires_grad_(True) for p in first]
    after = FusedAdamW(second, lr=1e-3)  # everything comes from the checkpoint, the learning rate too
    after.load_state_dict(state)
    run(after, second, range(2, 4))
    torch.cuda.synchronize()
    for a, b in zip(params, second):
        assert torch.equal(a, b)
    for a, b in zip(straight.exp_avg_sq, after.exp_avg_sq):
        assert torch.equal(a, b)
