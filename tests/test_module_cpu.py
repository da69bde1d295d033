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


def test_roofline_columns_use_the_measured_file_or_say_fallback(tmp_path, monkeypatch):
    import json

    from scalingcontrasts_b200.utils.roofline import FALLBACK_BF16_TFLOPS, load_peaks, loss_step_roofline_ms

    # no file named, none in the working directory: the fallback figures, labelled as such
    monkeypatch.chdir(tmp_path)
    monkeypatch.delenv("SC_MEASURED_PEAKS", raising=False)
    fallback = load_peaks()
    assert fallback.source == "fallback" and fallback.bf16_tflops == FALLBACK_BF16_TFLOPS
    # a file named by the environment variable, or explicitly
    path = tmp_path / "peaks.json"
    path.write_text(json.dumps({"hbm_gbs": 6000.0, "bf16_tflops": 1600.0, "bf16_tflops_sustained": 1400.0}))
    monkeypatch.setenv("SC_MEASURED_PEAKS", str(path))
    peaks = load_peaks()
    assert peaks.source == "measured" and peaks.bf16_tflops == 1600.0 and load_peaks(str(path)) == peaks
    # R = 16384, 8 GPUs, H = 768: 9.69 TFLOP of tensor work per rank; a step row uses the sustained peak, a kernel row the burst
    flops = 2.0 * 1536 * 16384 * 131072
    assert abs(loss_step_roofline_ms(16384, 8, 768, peaks) - flops / (1400.0 * 1e12) * 1e3) < 1e-9
    assert abs(loss_step_roofline_ms(16384, 8, 768, peaks, sustained=False) - flops / (1600.0 * 1e12) * 1e3) < 1e-9


def test_fused_adamw_refuses_what_its_kernel_cannot_take():
    import pytest
    import torch

    from scalingcontrasts_b200.optim import FusedAdamW

    with pytest.raises(ValueError, match="at least one"):
        FusedAdamW([])
    with pytest.raises(ValueError, match="contiguous CUDA parameters"):
        FusedAdamW([torch.zeros(4, requires_grad=True)])  # a CPU tensor
