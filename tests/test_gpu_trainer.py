import pytest
import torch

pytestmark = pytest.mark.gpu


def test_training_steps_reduce_the_loss_and_checkpoints_resume_bitwise(tmp_path):
    from scalingcontrasts_b200.trainer import ContrastiveTrainer

    def make():
        return ContrastiveTrainer(rows=256, in_features=128, mid_features=256, hidden=256, prefixes=3, lr=1e-3, device="cuda", seed=3)

    generator = torch.Generator().manual_seed(0)
    batches = [torch.randn(256, 128, generator=generator).to(torch.bfloat16).pin_memory() for _ in range(4)]
    trainer = make()
    losses = []
    for step in range(24):
        trainer.step(batches[step % 4])
        losses.append(trainer.last_loss())
    trainer.check()
    assert all(value == value for value in losses)
    assert sum(losses[-4:]) < sum(losses[:4])
    path = tmp_path / "checkpoint.pt"
    torch.save(trainer.state_dict(), path)
    trainer.step(batches[0])
    expected = trainer.last_loss()
    trainer.close()
    resumed = make()
    resumed.load_state_dict(torch.load(path, weights_only=False))
    assert resumed.steps_done == 24
    resumed.step(batches[0])
    assert resumed.last_loss() == expected
    state = resumed.loss.state_dict()
    assert set(state) == {"logit_scale", "logit_bias"} and state["logit_scale"].dim() == 0
    resumed.close()


def test_smoke_entry_point():
    import __graft_entry__

    __graft_entry__.smoke()


def test_a_recorded_timeout_surfaces_with_the_next_loss():
    """The status words ride along with every loss; a wait that ran out is reported without any extra synchronisation.
    The failure is made on the host: the word is written the way a tile kernel would record it."""
    from scalingcontrasts_b200.trainer import ContrastiveTrainer

    trainer = ContrastiveTrainer(rows=256, in_features=128, mid_features=256, hidden=256, prefixes=3, device="cuda", seed=1)
    batch = torch.randn(256, 128).to(torch.bfloat16).pin_memory()
    trainer.step(batch)
    assert trainer.last_loss() is not None
    trainer.loss.engine.loss.status[0] = 2
    trainer.step(batch)
    with pytest.raises(RuntimeError, match="bounded device wait"):
        trainer.last_loss()
    trainer.close()


def test_unit_upstream_hands_the_same_gradients_on():
    """``unit_upstream`` skips the multiplication of the row gradients by the upstream gradient of ``loss.backward()``,
    which is one: parameter and input gradients are the same bits with and without it."""
    from scalingcontrasts_b200 import MatryoshkaSigmoidLoss

    rows, hidden = 256, 256
    outcomes = []
    for unit in (False, True):
        torch.manual_seed(3)
        criterion = MatryoshkaSigmoidLoss(rows, hidden, prefixes=3, device="cuda")
        criterion.unit_upstream = unit
        embeddings = torch.randn(rows, hidden, device="cuda").to(torch.bfloat16).requires_grad_(True)
        loss = criterion(embeddings)
        loss.backward()
        torch.cuda.synchronize()
        outcomes.append((embeddings.grad.clone(), criterion.logit_scale.grad.clone(), criterion.logit_bias.grad.clone(), loss.detach().clone()))
    for a, b in zip(*outcomes):
        assert torch.equal(a, b)
