"""The projector's fused elementwise kernels (GELU forward; GELU backward with the bias gradient; column sums) against
the plain torch composition of the same tower, in float32 arithmetic on the same bfloat16 parameters."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rows,features", [(256, (128, 256, 64)), (1000, (64, 3072, 768)), (4096, (1024, 3072, 768))])
def test_fused_tower_matches_the_plain_modules(rows, features):
    from scalingcontrasts_b200.models.projector import Projector

    torch.backends.cuda.matmul.allow_tf32 = False
    fused = Projector(*features, device="cuda", seed=3, fused=True)
    plain = Projector(*features, device="cuda", seed=3, fused=False)
    with torch.no_grad():  # non-zero biases, so that their gradients and the epilogues are exercised
        for module in (fused, plain):
            module.fc1.bias.copy_(torch.linspace(-0.5, 0.5, features[1]).to(torch.bfloat16))
            module.fc2.bias.copy_(torch.linspace(0.25, -0.25, features[2]).to(torch.bfloat16))
    x = torch.randn(rows, features[0], device="cuda", generator=torch.Generator(device="cuda").manual_seed(1)).to(torch.bfloat16)
    upstream = torch.randn(rows, features[2], device="cuda", generator=torch.Generator(device="cuda").manual_seed(2)).to(torch.bfloat16)
    outputs = []
    for module in (fused, plain):
        y = module(x)
        y.backward(upstream)
        outputs.append((y.float(), [p.grad.float() for p in module.parameters()]))
    # float32 statement of the same tower on the same bfloat16 parameters
    w1, b1, w2, b2 = (p.detach().float().requires_grad_(True) for p in plain.parameters())
    reference = torch.nn.functional.gelu(x.float() @ w1.t() + b1) @ w2.t() + b2
    reference.backward(upstream.float())
    exact = [w1.grad, b1.grad, w2.grad, b2.grad]

    def error(a, b):
        return float((a - b).norm() / b.norm().clamp_min(1e-12))

    assert error(outputs[0][0], reference.detach()) < 1e-2 and error(outputs[1][0], reference.detach()) < 1e-2
    for mine, theirs, truth in zip(outputs[0][1], outputs[1][1], exact):
        assert error(mine, truth) < 2e-2, "fused gradient against float32"
        assert error(mine, truth) <= 1.5 * error(theirs, truth) + 2e-3, "the fused tower is no less accurate than the plain one"


def test_fused_tower_is_bit_reproducible():
    from scalingcontrasts_b200.models.projector import Projector

    tower = Projector(64, 3072, 768, device="cuda", seed=5)
    x = torch.randn(2048, 64, device="cuda").to(torch.bfloat16)
    upstream = torch.randn(2048, 768, device="cuda").to(torch.bfloat16)
    runs = []
    for _ in range(3):
        tower.zero_grad(set_to_none=True)
        y = tower(x)
        y.backward(upstream)
        runs.append([y.clone()] + [p.grad.clone() for p in tower.parameters()])
    for later in runs[1:]:
        assert all(torch.equal(a, b) for a, b in zip(runs[0], later))


def test_gradients_land_in_named_buffers_without_a_copy():
    """With ``gradient_landing`` set (a gradient reducer's bucket slots), the tower's backward produces each parameter's
    gradient in that buffer and autograd adopts it: same values as without, and `.grad` points into the buffer."""
    from scalingcontrasts_b200.models.projector import Projector

    tower = Projector(64, 256, 128, device="cuda", seed=7)
    x = torch.randn(512, 64, device="cuda").to(torch.bfloat16)
    upstream = torch.randn(512, 128, device="cuda").to(torch.bfloat16)
    tower(x).backward(upstream)
    expected = {name: parameter.grad.clone() for name, parameter in tower.named_parameters()}
    buffers = {name: torch.full_like(parameter, float("nan")) for name, parameter in tower.named_parameters()}
    tower.gradient_landing = buffers
    for _ in range(2):  # the second step rewrites the same buffers
        tower.zero_grad(set_to_none=True)
        tower(x).backward(upstream)
        for name, parameter in tower.named_parameters():
            assert parameter.grad.data_ptr() == buffers[name].data_ptr(), name
            assert torch.equal(parameter.grad, expected[name]), name
