"""The loss module on the CPU: autograd wiring checked against finite differences, and the state_dict layout."""
import math

import torch

from scalingcontrasts_b200 import LossSpec
from scalingcontrasts_b200.models.loss import MatryoshkaSigmoidLoss


def test_gradcheck_of_the_cpu_twin_in_float64():
    torch.manual_seed(0)
    module = MatryoshkaSigmoidLoss(8, 32, prefixes=2, spec=LossSpec("pairs"), device="cpu")
    module.logit_scale.data = module.logit_scale.data.double()
    module.logit_bias.data = module.logit_bias.data.double()
    embeddings = torch.randn(8, 32, dtype=torch.float64, requires_grad=True)

    def evaluate(x, scale, bias):
        module.logit_scale.data.copy_(scale.detach())
        module.logit_bias.data.copy_(bias.detach())
        from scalingcontrasts_b200.models.loss import _HostLoss

        return _HostLoss.apply(x, scale, bias, module)

    scale = torch.tensor(math.log(10.0), dtype=torch.float64, requires_grad=True)
    bias = torch.tensor(-10.0, dtype=torch.float64, requires_grad=True)
    assert torch.autograd.gradcheck(evaluate, (embeddings, scale, bias), eps=1e-6, atol=1e-6, rtol=1e-4)


def test_state_dict_keeps_the_siglip_layout_and_initial_values():
    module = MatryoshkaSigmoidLoss(8, 32, prefixes=2, device="cpu")
    state = module.state_dict()
    assert list(state) == ["logit_scale", "logit_bias"]
    assert state["logit_scale"].shape == () and state["logit_bias"].shape == ()
    assert float(state["logit_scale"]) == float(torch.tensor(math.log(10.0), dtype=torch.float32)) and float(state["logit_bias"]) == -10.0
    other = MatryoshkaSigmoidLoss(8, 32, prefixes=2, device="cpu", init_logit_scale=0.0, init_logit_bias=0.0)
    other.load_state_dict(state)
    assert float(other.logit_bias) == -10.0


def test_roofline_columns_use_the_measured_file_or_say_fallback():
    from scalingcontrasts_b200.utils.roofline import load_peaks, loss_step_roofline_ms

    peaks = load_peaks()
    assert peaks.source in ("measured", "fallback") and peaks.bf16_tflops > 0
    # R = 16384, 8 GPUs, H = 768: 9.69 TFLOP of tensor work per rank
    bound = loss_step_roofline_ms(16384, 8, 768, peaks)
    assert abs(bound - 2.0 * 1536 * 16384 * 131072 / (peaks.bf16_tflops * 1e12) * 1e3) < 1e-9
