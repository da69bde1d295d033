"""Device kernels of the streamed loss against plain float32 / float64 torch statements of the same operations."""
import pytest
import torch

from scalingcontrasts_b200 import LossSpec, Matryoshka
from scalingcontrasts_b200.cpu import CpuStreamedLoss, oracle, relative_l2
from scalingcontrasts_b200.utils.keyed import keyed_embeddings, normal_embeddings

pytestmark = pytest.mark.gpu


def _loss(rows, hidden, ladder, spec=LossSpec("self"), fused=None):
    from scalingcontrasts_b200.ops.streamed_loss import StreamedLoss

    return StreamedLoss(rows, hidden, ladder, spec, "cuda", fused=fused)


def _float32_matmul_exact():
    torch.backends.cuda.matmul.allow_tf32 = False


def test_prefix_norms_transpose_and_keyed_generator(ext):
    from scalingcontrasts_b200.cpu.streamed import prefix_inverse_norms
    from scalingcontrasts_b200.ops.streamed_loss import BlockNorms, compute_block_norms, keyed_embeddings_device

    ladder = Matryoshka.halvings(768, 5)
    block = keyed_embeddings_device(256, 768, salt=3, scale=1.0)
    assert torch.equal(block.cpu(), keyed_embeddings(256, 768, 3, 1.0))
    norms = BlockNorms(5, 256, device="cuda")
    copy = torch.empty_like(block)
    compute_block_norms(block, ladder, norms, copy_to=copy)
    expected = prefix_inverse_norms(block, ladder)
    assert torch.equal(copy, block)
    assert torch.allclose(norms.inverse, expected, rtol=2e-6)
    assert torch.allclose(norms.tile_max, expected.view(5, 4, 64).amax(dim=2), rtol=2e-6)
    out = torch.empty(768, 256, dtype=torch.bfloat16, device="cuda")
    ext.transpose(block.data_ptr(), out.data_ptr(), 256, 768, torch.cuda.current_stream().cuda_stream)
    assert torch.equal(out, block.T.contiguous())


@pytest.mark.parametrize("rows,hidden,prefixes", [(128, 64, 1), (128, 128, 2), (128, 256, 3), (256, 1024, 4), (256, 768, 5),
                                                  (128, 1024, 6), (128, 1024, 7), (128, 2048, 8)])
def test_forward_cube_and_backward_fold_against_float32(ext, rows, hidden, prefixes):
    """The forward kernel's per-band gradient cubes and the backward kernel's fold, each checked on its own."""
    _float32_matmul_exact()
    ladder = Matryoshka.halvings(hidden, prefixes)
    queries = normal_embeddings(rows, hidden, seed=1, rank=0).cuda()
    candidates = normal_embeddings(rows, hidden, seed=1, rank=1).cuda()
    loss = _loss(rows, hidden, ladder, fused=False)
    loss.begin(queries)
    loss.score(queries, candidates, 0, rows, 10.0, -10.0, 2 * rows)
    torch.cuda.synchronize()
    loss.check()
    reference = CpuStreamedLoss(rows, hidden, ladder, LossSpec("self"), torch.float32, "cuda", keep_cubes=True)
    reference.begin(queries)
    reference.score(queries, candidates, 0, rows, 10.0, -10.0, 2 * rows)
    # the cube is stored without the loss's factor 2 / live; the backward kernel applies it
    cube = loss.similarity_gradients.float() * (2.0 / (2 * rows))
    for band in range(prefixes):
        assert relative_l2(cube[band], reference.last_cubes[band]) < 6e-3, f"cube of band {band}"
    # backward alone: fold the kernel's own bfloat16 cube with a float32 matmul and compare
    expected = torch.zeros(rows, hidden, device="cuda")
    for band in range(prefixes):
        begin, end = ladder.begin(band), ladder.end(band)
        expected[:, begin:end] = cube[band] @ candidates.float()[:, begin:end]
    assert relative_l2(loss.query_gradient, expected) < 1e-5
    # row accumulators: bias-grad, log-beta-grad, prefix losses, coefficients
    accumulators = loss.row_accumulators
    assert torch.allclose(accumulators[0], reference.row_bias_grad, rtol=2e-4, atol=1e-9)
    assert torch.allclose(accumulators[2:2 + prefixes], reference.row_loss, rtol=2e-5, atol=1e-9)
    assert relative_l2(accumulators[2 + prefixes:], reference.self_coefficients) < 2e-4


@pytest.mark.parametrize("spec", [LossSpec("self"), LossSpec("pairs"), LossSpec("pairs", "skip")],
                         ids=lambda s: f"{s.positives}-{s.diagonal}")
@pytest.mark.parametrize("rows,hidden,prefixes,kind", [(128, 256, 3, "normal"), (128, 768, 5, "normal"), (256, 768, 5, "keyed")])
@pytest.mark.parametrize("fused", [False, True], ids=["two-kernel", "fused"])
def test_world_of_two_blocks_against_the_float64_oracle(spec, rows, hidden, prefixes, kind, fused):
    """One GPU plays both ranks of a two-rank world in turn; loss, per-prefix losses, gradients and the two scalar
    gradients are compared with the float64 evaluation of the whole world. Both forms of the tile kernels are held to
    the same tolerances: the forward kernel with a gradient cube and a backward kernel, and the fused kernel that folds
    the gradient itself."""
    ladder = Matryoshka.halvings(hidden, prefixes)
    if kind == "normal":
        blocks = [normal_embeddings(rows, hidden, seed=1, rank=r).cuda() for r in range(2)]
    else:
        blocks = [keyed_embeddings(rows, hidden, r, 1.0).cuda() for r in range(2)]
    expected = oracle(torch.cat(blocks).cpu(), ladder, 10.0, -10.0, spec)
    loss = _loss(rows, hidden, ladder, spec, fused=fused)
    total = torch.zeros(12, dtype=torch.float64)
    gradients = []
    for rank in range(2):
        loss.begin(blocks[rank])
        for peer in (rank, 1 - rank):
            loss.score(blocks[rank], blocks[peer], rank * rows, peer * rows, 10.0, -10.0, 2 * rows)
        gradient, summands = loss.finish(blocks[rank])
        torch.cuda.synchronize()
        loss.check()
        gradients.append(gradient.float().cpu())
        total += summands.double().cpu()
    assert float(total[0]) == pytest.approx(expected.loss, rel=2e-6)
    assert torch.allclose(total[4:4 + prefixes], expected.band_losses, rtol=2e-6)
    assert relative_l2(torch.cat(gradients), expected.gradient) < 4e-3
    assert float(total[1]) == pytest.approx(expected.bias_grad, rel=1e-4)
    assert float(total[2]) == pytest.approx(expected.log_beta_grad, rel=1e-3, abs=1e-6)


@pytest.mark.parametrize("hidden,prefixes,spec", [(128, 2, LossSpec("pairs")), (256, 3, LossSpec("self")), (256, 5, LossSpec("pairs")),
                                                  (768, 5, LossSpec("pairs")), (384, 6, LossSpec("self"))],
                         ids=["K2-pairs", "K3-self", "K5-pairs", "H768-K5-pairs", "K6-self"])
@pytest.mark.parametrize("fused", [False, True], ids=["two-kernel", "fused"])
def test_many_tiles_per_cta_wrap_the_slot_and_barrier_rings(hidden, prefixes, spec, fused):
    """4096 rows against themselves: every CTA walks about fourteen tiles, so the eight tensor-memory slots and the eight
    release barriers wrap several times (with the tile's slot count both dividing eight and not), runs end inside a
    CTA's walk, and the diagonal crosses 96 tiles. Compared with the float32 statement of the same step."""
    _float32_matmul_exact()
    rows = 4096
    ladder = (Matryoshka.halvings(hidden, prefixes) if hidden == 768 else
              Matryoshka(tuple(hidden * (k + 1) // prefixes // 16 * 16 for k in range(prefixes))))
    queries = normal_embeddings(rows, hidden, seed=7, rank=0).cuda()
    loss = _loss(rows, hidden, ladder, spec, fused=fused)
    assert loss.fused == fused
    reference = CpuStreamedLoss(rows, hidden, ladder, spec, torch.float32, "cuda")
    outcomes = []
    for engine in (loss, reference):
        engine.begin(queries)
        engine.score(queries, queries, 0, 0, 10.0, -10.0, rows)
        gradient, summands = engine.finish(queries)
        outcomes.append((gradient.float(), summands.double()))
    torch.cuda.synchronize()
    loss.check()
    assert relative_l2(outcomes[0][0], outcomes[1][0]) < 4e-3
    assert torch.allclose(outcomes[0][1][:3], outcomes[1][1][:3], rtol=2e-4, atol=1e-7)
    assert torch.allclose(outcomes[0][1][4:4 + prefixes], outcomes[1][1][4:4 + prefixes], rtol=2e-5)


@pytest.mark.parametrize("fused", [False, True], ids=["two-kernel", "fused"])
def test_runs_of_one_tile_and_of_several_agree(fused):
    """A CTA's work item is a run of candidate tiles whose per-row sums leave as one record. Runs of four tiles and runs
    of one tile must give the same step (the fold over records is a float32 sum, so: to rounding)."""
    from scalingcontrasts_b200.ops.streamed_loss import StreamedLoss

    rows, hidden = 2048, 256
    ladder = Matryoshka.halvings(hidden, 3)
    queries = normal_embeddings(rows, hidden, seed=11, rank=0).cuda()
    outcomes = []
    for forced in (4, 1):
        loss = StreamedLoss(rows, hidden, ladder, LossSpec("pairs"), "cuda", fused=fused, tiles_per_run=forced)
        assert loss.tiles_per_run == forced
        loss.begin(queries)
        loss.score(queries, queries, 0, 0, 10.0, -10.0, rows)
        gradient, summands = loss.finish(queries)
        torch.cuda.synchronize()
        loss.check()
        outcomes.append((gradient.float(), summands.double()))
    assert relative_l2(outcomes[0][0], outcomes[1][0]) < 1e-3
    assert torch.allclose(outcomes[0][1], outcomes[1][1], rtol=1e-5, atol=1e-9)


def test_block_order_invariance_and_bitwise_repeat():
    ladder = Matryoshka.halvings(256, 3)
    blocks = [normal_embeddings(128, 256, seed=5, rank=r).cuda() for r in range(3)]
    loss = _loss(128, 256, ladder)
    results = []
    for order in ((0, 1, 2), (2, 1, 0), (0, 1, 2)):
        loss.begin(blocks[0])
        for peer in order:
            loss.score(blocks[0], blocks[peer], 0, peer * 128, 10.0, -10.0, 3 * 128)
        gradient, summands = loss.finish(blocks[0])
        torch.cuda.synchronize()
        results.append((gradient.clone(), summands.clone()))
    assert torch.equal(results[0][0], results[2][0]) and torch.equal(results[0][1], results[2][1])  # bit for bit
    assert relative_l2(results[1][0].float(), results[0][0].float()) < 2e-3
    assert torch.allclose(results[1][1], results[0][1], rtol=1e-5)


@pytest.mark.parametrize("hidden,prefixes", [(64, 1), (256, 3)])
def test_collinear_rows_have_exactly_zero_gradient(hidden, prefixes):
    ladder = Matryoshka.halvings(hidden, prefixes)
    rows = torch.zeros(128, hidden, dtype=torch.float32)
    for i in range(128):
        rows[i, 0] = [1.0, 1.0 / 16, 1.0 / 256, 0.0][i % 4]
    block = rows.to(torch.bfloat16).cuda()
    loss = _loss(128, hidden, ladder)
    loss.begin(block)
    loss.score(block, block, 0, 0, 10.0, -10.0, 128)
    gradient, _ = loss.finish(block)
    torch.cuda.synchronize()
    loss.check()
    assert torch.count_nonzero(gradient) == 0


def test_scratch_does_not_grow_and_device_scalars_override():
    ladder = Matryoshka.halvings(256, 3)
    block = normal_embeddings(128, 256, seed=7).cuda()
    loss = _loss(128, 256, ladder)
    before = loss.bytes()
    scalars = torch.tensor([10.0, -10.0], device="cuda")
    outputs = []
    for use_scalars in (False, True):
        loss.begin(block)
        for peer in range(4):
            loss.score(block, block, 0, peer * 128, 1.0 if use_scalars else 10.0, 0.0 if use_scalars else -10.0, 4 * 128,
                       scalars=scalars if use_scalars else None)
        outputs.append(tuple(t.clone() for t in loss.finish(block)))
    torch.cuda.synchronize()
    assert loss.bytes() == before
    assert torch.equal(outputs[0][0], outputs[1][0]) and torch.equal(outputs[0][1], outputs[1][1])


@pytest.mark.parametrize("beta,bias", [(5.0, 0.0), (20.0, -3.0), (1.0, 2.0)])
@pytest.mark.parametrize("spec", [LossSpec("self"), LossSpec("pairs")], ids=lambda s: s.positives)
@pytest.mark.parametrize("through_device", [False, True], ids=["host-scalars", "device-scalars"])
def test_learned_scale_and_bias_against_the_float64_oracle(beta, bias, spec, through_device):
    """Away from beta = 10, bias = -10 most cells leave the easy-negative series path: logits near and above zero take
    the general form (decay of the absolute value, reciprocal, full log1p polynomial, hinge), and a warp's patch may mix
    both. Checked against the float64 evaluation with the scalars given as host floats and through the device pointer a
    trainer uses."""
    rows, hidden, prefixes = 256, 256, 3
    ladder = Matryoshka.halvings(hidden, prefixes)
    blocks = [normal_embeddings(rows, hidden, seed=3, rank=r).cuda() for r in range(2)]
    expected = oracle(torch.cat(blocks).cpu(), ladder, beta, bias, spec)
    loss = _loss(rows, hidden, ladder, spec)
    scalars = torch.tensor([beta, bias], device="cuda") if through_device else None
    total = torch.zeros(12, dtype=torch.float64)
    gradients = []
    for rank in range(2):
        loss.begin(blocks[rank])
        for peer in (rank, 1 - rank):
            loss.score(blocks[rank], blocks[peer], rank * rows, peer * rows, 0.0 if through_device else beta,
                       0.0 if through_device else bias, 2 * rows, scalars=scalars)
        gradient, summands = loss.finish(blocks[rank])
        torch.cuda.synchronize()
        loss.check()
        gradients.append(gradient.float().cpu())
        total += summands.double().cpu()
    assert float(total[0]) == pytest.approx(expected.loss, rel=2e-6)
    assert torch.allclose(total[4:4 + prefixes], expected.band_losses, rtol=2e-6)
    assert relative_l2(torch.cat(gradients), expected.gradient) < 4e-3
    assert float(total[1]) == pytest.approx(expected.bias_grad, rel=1e-4)
    assert float(total[2]) == pytest.approx(expected.log_beta_grad, rel=1e-3, abs=1e-6)


def test_pull_inside_the_forward_launch_copies_the_bytes_and_changes_nothing():
    """``simulate`` with ``pull=True`` scores blocks 1.. from the staging buffers that the forward launch of the block
    before filled with its pull warp; with ``pull=False`` every block is scored from the source. Same bits either way,
    and the staged bytes (embeddings and norms) equal the source."""
    from scalingcontrasts_b200.parallel.box import BoxLoss

    rows, hidden = 512, 768
    ladder = Matryoshka.halvings(hidden, 5)
    engine = BoxLoss(rows, hidden, ladder, LossSpec("pairs"), None, "cuda")
    block = normal_embeddings(rows, hidden, seed=9, rank=0).cuda()
    outcomes = []
    for pull in (True, False):
        for staged in engine.staged:
            staged.zero_()
        gradient, summands = engine.simulate(block, 4, pull=pull)
        torch.cuda.synchronize()
        engine.check()
        outcomes.append((gradient.clone(), summands.clone()))
        if pull:
            for slot in range(2):
                assert torch.equal(engine.staged[slot], block)
                assert torch.equal(engine.staged_norms[slot].storage, engine.norms.storage)
    assert torch.equal(outcomes[0][0], outcomes[1][0]) and torch.equal(outcomes[0][1], outcomes[1][1])


@pytest.mark.parametrize("world", [1, 2, 5])
def test_backward_beside_the_next_forward_gives_the_same_bits(world):
    """With ``overlap_backward`` a block's gradient GEMM runs on a second stream beside the next block's forward kernel,
    from a second gradient cube and a third staging buffer. Every gradient element still receives its blocks' terms in
    block order, so gradient and summands equal the in-line run bit for bit, step after step."""
    from scalingcontrasts_b200.parallel.box import BoxLoss

    rows, hidden = 512, 768
    ladder = Matryoshka.halvings(hidden, 5)
    block = normal_embeddings(rows, hidden, seed=11, rank=0).cuda()
    outcomes = []
    for overlap in (False, True):
        engine = BoxLoss(rows, hidden, ladder, LossSpec("pairs"), None, "cuda", overlap_backward=overlap)
        assert engine.loss.overlap_backward == overlap
        for _ in range(3):
            gradient, summands = engine.simulate(block, world)
        torch.cuda.synchronize()
        engine.check()
        outcomes.append((gradient.clone(), summands.clone()))
    assert torch.equal(outcomes[0][0], outcomes[1][0]) and torch.equal(outcomes[0][1], outcomes[1][1])


def test_overlapped_step_replays_as_a_cuda_graph():
    """The overlapped step forks onto the plan's two streams and joins them again before it ends, so it can be captured
    whole; replays give the bits of the eager run."""
    from scalingcontrasts_b200.parallel.box import BoxLoss

    rows, hidden, world = 512, 768, 4
    ladder = Matryoshka.halvings(hidden, 5)
    block = normal_embeddings(rows, hidden, seed=12, rank=0).cuda()
    engine = BoxLoss(rows, hidden, ladder, LossSpec("pairs"), None, "cuda", overlap_backward=True)
    gradient, summands = engine.simulate(block, world)
    torch.cuda.synchronize()
    expected = (gradient.clone(), summands.clone())
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        engine.simulate(block, world)  # warm-up on the capture stream
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            engine.simulate(block, world)
    torch.cuda.current_stream().wait_stream(stream)
    for _ in range(3):
        engine.gradient.zero_()
        graph.replay()
        torch.cuda.synchronize()
        engine.check()
        assert torch.equal(engine.gradient, expected[0]) and torch.equal(engine.summands, expected[1])


def test_backward_split_over_candidates_matches_the_single_pass():
    """``backward_split`` divides the candidate range between CTAs that add with float32 reductions in no fixed order:
    the same gradient as the single pass to float32 rounding (and the summands, which do not pass through it, to the bit)."""
    from scalingcontrasts_b200.ops.streamed_loss import StreamedLoss

    rows, hidden = 512, 256
    ladder = Matryoshka.halvings(hidden, 3)
    queries = normal_embeddings(rows, hidden, seed=13, rank=0).cuda()
    outcomes = []
    for split in (1, 4):
        loss = StreamedLoss(rows, hidden, ladder, LossSpec("self"), "cuda", backward_split=split, fused=False)
        loss.begin(queries)
        loss.score(queries, queries, 0, 0, 10.0, -10.0, rows)
        torch.cuda.synchronize()
        loss.check()
        outcomes.append((loss.query_gradient.clone(), loss.row_accumulators.clone()))
    assert relative_l2(outcomes[1][0], outcomes[0][0]) < 1e-5
    assert torch.equal(outcomes[0][1], outcomes[1][1])


@pytest.mark.parametrize("fused", [False, True], ids=["two-kernel", "fused"])
def test_twenty_repeats_of_a_many_tile_step_and_poisoned_scratch(fused):
    """4096 rows against themselves, the real ladder, twenty times: every CTA walks many tiles and the rings wrap, and
    every repeat must reproduce the first one's loss summands bit for bit (per-row sums are folded in a fixed order). The
    two-kernel form also reproduces the gradient bit for bit; the fused form adds one partial gradient per run of tiles
    with float32 reductions whose order is not fixed, so its gradient repeats to rounding only. Before every repeat the
    scratch buffers are filled with NaN bit patterns: nothing may be read before it is written."""
    rows, hidden = 4096, 768
    ladder = Matryoshka.halvings(hidden, 5)
    queries = normal_embeddings(rows, hidden, seed=21, rank=0).cuda()
    loss = _loss(rows, hidden, ladder, LossSpec("pairs"), fused=fused)
    first = None
    for repeat in range(20):
        for scratch in (loss.partials, loss.similarity_gradients, loss.transposed_candidates, loss.candidate_norms.storage,
                        loss.query_gradient, loss.row_accumulators):
            scratch.view(torch.int16 if scratch.dtype == torch.bfloat16 else torch.int32).fill_(-1)  # all ones: a NaN
        loss.begin(queries)
        loss.score(queries, queries, 0, 0, 10.0, -10.0, rows)
        gradient, summands = loss.finish(queries)
        torch.cuda.synchronize()
        loss.check()
        assert bool(torch.isfinite(summands).all()) and bool(torch.isfinite(gradient.float()).all())
        if first is None:
            first = (gradient.clone(), summands.clone())
            continue
        assert torch.equal(summands, first[1]), f"repeat {repeat}: the loss summands changed bits"
        if fused:
            assert relative_l2(gradient.float(), first[0].float()) < 1e-3
        else:
            assert torch.equal(gradient, first[0]), f"repeat {repeat}: the gradient changed bits"


@pytest.mark.parametrize("rows,hidden,ends", [(256, 768, (48, 96, 192, 384, 768)), (128, 1024, (64, 128, 256, 512, 1024)),
                                              (128, 256, (16, 80, 256)), (256, 64, (64,))])
def test_backward_reads_row_major_candidates_like_transposed_ones(ext, rows, hidden, ends):
    """The backward kernel takes the candidates either transposed ([H, R], a K-major operand) or as they lie in memory
    ([R, H], handed to the tensor cores as an MN-major operand, no copy). Same cube, same candidates: the same gradient
    to float32 rounding of the accumulation order, and both equal to the float32 matmul."""
    _float32_matmul_exact()
    stream = torch.cuda.current_stream().cuda_stream
    generator = torch.Generator(device="cuda").manual_seed(5)
    cube = (torch.randn(len(ends), rows, rows, device="cuda", generator=generator) * 0.1).to(torch.bfloat16)
    candidates = torch.randn(rows, hidden, device="cuda", generator=generator).to(torch.bfloat16)
    transposed = candidates.T.contiguous()
    status = torch.zeros(8, dtype=torch.int32, device="cuda")
    outcomes = []
    for row_major in (0, candidates.data_ptr()):
        gradient = torch.zeros(rows, hidden, device="cuda")
        ext.backward(cube.data_ptr(), transposed.data_ptr() if row_major == 0 else 0, gradient.data_ptr(), status.data_ptr(), rows,
                     rows, hidden, list(ends), 1, 0.5, 2_000_000_000, stream, row_major=row_major)
        torch.cuda.synchronize()
        assert status.tolist()[0] == 0
        outcomes.append(gradient)
    reference = 0.5 * torch.cat([cube[b].float() @ candidates.float()[:, (0 if b == 0 else ends[b - 1]):ends[b]]
                                 for b in range(len(ends))], dim=1)
    assert relative_l2(outcomes[0], reference) < 1e-5
    assert relative_l2(outcomes[1], reference) < 1e-5
    assert relative_l2(outcomes[1], outcomes[0]) < 1e-6


@pytest.mark.parametrize("hidden,ends", [(768, (48, 96, 192, 384, 768)), (1024, (64, 128, 256, 512, 1024)),
                                         (1104, (16, 32, 336, 1104))])
def test_backward_of_a_large_launch_with_an_odd_number_of_row_blocks(ext, hidden, ends):
    """12928 query rows are 101 row blocks: enough for the large-launch tiling (two row blocks per CTA, a band of 257 to
    384 channels in one-block CTAs that take it whole, the tiles of a wider band side by side in the grid) and an odd
    count, so the last two-block CTA of every tile owns a single block. Few candidates keep the cube small. Both operand
    layouts against the float32 matmul."""
    _float32_matmul_exact()
    rows_q, rows_c = 12928, 128
    tiles, ctas = ext.backward_plan(rows_q, list(ends), 1, torch.cuda.get_device_properties(0).multi_processor_count)
    assert any(tile[3] == 2 for tile in tiles)  # the large-launch tiling is what runs
    stream = torch.cuda.current_stream().cuda_stream
    generator = torch.Generator(device="cuda").manual_seed(6)
    cube = (torch.randn(len(ends), rows_q, rows_c, device="cuda", generator=generator) * 0.1).to(torch.bfloat16)
    candidates = torch.randn(rows_c, hidden, device="cuda", generator=generator).to(torch.bfloat16)
    transposed = candidates.T.contiguous()
    status = torch.zeros(8, dtype=torch.int32, device="cuda")
    reference = 0.5 * torch.cat([cube[b].float() @ candidates.float()[:, (0 if b == 0 else ends[b - 1]):ends[b]]
                                 for b in range(len(ends))], dim=1)
    for row_major in (0, candidates.data_ptr()):
        gradient = torch.zeros(rows_q, hidden, device="cuda")
        ext.backward(cube.data_ptr(), transposed.data_ptr() if row_major == 0 else 0, gradient.data_ptr(), status.data_ptr(),
                     rows_q, rows_c, hidden, list(ends), 1, 0.5, 2_000_000_000, stream, row_major=row_major)
        torch.cuda.synchronize()
        assert status.tolist()[0] == 0
        assert relative_l2(gradient, reference) < 1e-5
        assert relative_l2(gradient[-128:], reference[-128:]) < 1e-5  # the odd last row block
