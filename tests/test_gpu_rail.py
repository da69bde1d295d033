"""The rail's loopback transport on one GPU: both ends live in this process."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _pair(rows=256, hidden=128):
    from scalingcontrasts_b200.parallel.rail import RdmaRail

    blocks = [torch.randn(rows, hidden, device="cuda").to(torch.bfloat16) for _ in range(2)]
    landings = [torch.zeros(2, rows, hidden, dtype=torch.bfloat16, device="cuda") for _ in range(2)]
    rails = [RdmaRail(blocks[i], landings[i], hosts=2, host=i) for i in range(2)]
    rails[0].connect(rails[1].local)
    rails[1].connect(rails[0].local)
    return blocks, landings, rails


def test_blocks_land_in_the_parity_buffer_and_summands_cross():
    blocks, landings, rails = _pair()
    for step in range(4):
        parity = step % 2
        blocks[0].add_(1.0)
        blocks[1].sub_(1.0)
        rails[0].post_embeddings(parity)
        rails[1].post_embeddings(parity)
        assert rails[0].await_landed(5.0) == blocks[0].numel() * 2
        assert rails[1].await_landed(5.0) == blocks[1].numel() * 2
        torch.cuda.synchronize()
        assert torch.equal(landings[1][parity], blocks[0]) and torch.equal(landings[0][parity], blocks[1])
    rails[0].post_summands(0, [1.0, 2.0, 3.0, 4.0])
    assert rails[1].await_landed(5.0) == 16
    assert rails[1].read_summands(0, 4) == [1.0, 2.0, 3.0, 4.0]
    for rail in rails:
        rail.close()


def test_injected_completion_error_and_missing_completion_raise():
    from scalingcontrasts_b200.parallel.rail import RailError

    blocks, landings, rails = _pair(128, 64)
    rails[0].inject_completion_error(12)
    rails[0].post_embeddings(0)
    with pytest.raises(RailError, match="status 12"):
        rails[1].await_landed(5.0)
    with pytest.raises(RailError, match="timed out"):
        rails[1].await_landed(0.05)  # nothing was posted: the host-side wait is bounded
    rails[0].post_embeddings(1)
    assert rails[1].await_landed(5.0) == blocks[0].numel() * 2  # the rail still works afterwards
    for rail in rails:
        rail.close()
