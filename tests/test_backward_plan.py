"""The backward launch's tile table (``csrc/loss_bwd.cu``: ``plan_tiles``) and the kernel's way of finding a CTA's tile
in it, replayed on the CPU: over many shapes every (channel, row block) of the gradient is owned by exactly one CTA, no
CTA reaches past the matrix, and the shapes stay inside what a CTA's tensor memory and stage hold."""
from __future__ import annotations

import itertools

import pytest

from scalingcontrasts_b200._ext import available, native

pytestmark = pytest.mark.skipif(not available(), reason="the native extension is not built")

LADDERS = [
    [48, 96, 192, 384, 768],        # the benchmark's ladder: widest band 384 channels
    [64, 128, 256, 512, 1024],      # widest band 512: two tiles of 256 that share their cube rows
    [256], [1024], [16], [768],     # one band; 768 = three tiles in one group
    [16, 32, 336, 1104],            # irregular: bands of 16, 16, 304 (whole-band tile) and 768
    [320, 640, 1280],               # three bands of 320
    [64, 128, 192, 256, 320, 384, 448, 512],
]


def _cta_to_work(tiles, cta):
    """What ``backward_kernel`` computes from ``blockIdx.x``: the tile and the first row block."""
    index = 0
    while index + tiles[index][5] < len(tiles) and cta >= tiles[index + tiles[index][5]][4]:
        index += tiles[index][5]
    within, group = cta - tiles[index][4], tiles[index][5]
    index += within % group
    band, channel0, width, blocks, _, _ = tiles[index]
    return index, within // group * blocks


@pytest.mark.parametrize("ends,rows,multiprocessors", list(itertools.product(LADDERS, [128, 384, 1024, 4096, 16384], [4, 148])))
def test_every_gradient_element_has_exactly_one_cta(ends, rows, multiprocessors):
    ext = native()
    tiles, ctas = ext.backward_plan(rows, ends, 1, multiprocessors)
    tiles = [tuple(t) for t in tiles]
    row_blocks = rows // 128
    owners = {}
    starts = [0] + ends[:-1]
    for cta in range(ctas):
        index, first_block = _cta_to_work(tiles, cta)
        band, channel0, width, blocks, _, _ = tiles[index]
        assert blocks in (1, 2) and width % 16 == 0 and 16 <= width
        assert starts[band] <= channel0 and channel0 + width <= ends[band]      # a tile never crosses a band edge
        assert blocks * 256 <= 512 if width <= 256 else (blocks == 1 and width <= 384)  # tensor-memory columns and stage
        assert first_block < row_blocks                                           # every CTA of the grid has work
        for block in range(first_block, min(first_block + blocks, row_blocks)):
            for chunk in range(channel0 // 16, (channel0 + width) // 16):
                assert (block, chunk) not in owners, (cta, owners[(block, chunk)])
                owners[(block, chunk)] = cta
    assert len(owners) == row_blocks * ends[-1] // 16
    # the tiles of a group belong to one band and have one shape of CTA
    for index, tile in enumerate(tiles):
        first = index
        while first > 0 and tiles[first - 1][4] == tile[4]:
            first -= 1
        members = [t for t in tiles if t[4] == tile[4]]
        assert len(members) == tile[5] and len({(t[0], t[3]) for t in members}) == 1


def test_a_wide_band_gets_whole_band_ctas_only_in_a_large_launch():
    ext = native()
    large, _ = ext.backward_plan(16384, [48, 96, 192, 384, 768], 1, 148)
    small, _ = ext.backward_plan(4096, [48, 96, 192, 384, 768], 1, 148)
    assert [tuple(t)[:4] for t in large][-1] == (4, 384, 384, 1)           # one-block CTAs of the whole band, last in the grid
    assert all(t[3] == 2 for t in large[:-1])
    assert all(t[3] == 1 and t[2] <= 256 for t in small)


def test_bad_ladders_are_refused():
    ext = native()
    for ends in ([48, 40, 768], [24, 768], [64, 64]):
        with pytest.raises(RuntimeError):
            ext.backward_plan(1024, ends, 1, 148)


@pytest.mark.parametrize("rows_q,rows_c", [(128, 128), (1024, 1024), (4096, 4096), (16384, 16384), (16384, 128), (128, 16384),
                                           (12928, 4096)])
def test_forward_run_length_divides_the_tiles_and_sizes_the_partial_records(rows_q, rows_c):
    """The forward kernel's work items are (strip of 128 rows, run of consecutive 64-candidate tiles). The chosen run
    length must divide a strip's tiles, and one partial record exists per (run, column group of the epilogue)."""
    ext = native()
    column_tiles = rows_c // 64
    for multiprocessors in (4, 148):
        run = ext.forward_choose_tiles_per_run(rows_q, rows_c, multiprocessors)
        assert run >= 1 and column_tiles % run == 0
        slots = ext.forward_partial_slots(rows_c, run)
        assert slots % (column_tiles // run) == 0 and slots // (column_tiles // run) in (2, 4)  # 8 or 16 epilogue warps
        fused_run = ext.forward_choose_tiles_per_run_fused(rows_q, rows_c, multiprocessors)
        assert 1 <= fused_run <= 16 and column_tiles % fused_run == 0
    assert ext.forward_quantities(5) == 12
