"""The native launchers refuse malformed shapes on the host, before anything is enqueued: these checks need no GPU (the
calls below raise before they reach a CUDA call), so bad input is never what a GPU test feeds a kernel."""
import pytest


def _forward(ext, **changes):
    arguments = dict(queries=256, candidates=256, q_inv=256, c_inv=256, c_tile_max=256, cube=256, partials=256, status=0,
                     rows_q=128, rows_c=128, hidden=256, ends=[64, 128, 256], tiles_per_run=1, beta=10.0, bias=-10.0,
                     weight=1.0 / 128, scalars=0, query_base=0, candidate_base=0, spec_code=0, budget_ns=10 ** 9, pull_src0=0,
                     pull_dst0=0, pull_bytes0=0, pull_src1=0, pull_dst1=0, pull_bytes1=0, sms=148, stream=0)
    arguments.update(changes)
    return ext.forward(**arguments)


@pytest.mark.parametrize("changes,message", [
    (dict(rows_q=100), "multiples of 128"),
    (dict(rows_c=96), "multiples of 128"),
    (dict(hidden=8192, ends=[8192]), "up to 4096"),
    (dict(ends=[64, 128]), "widest prefix must equal hidden"),
    (dict(ends=[128, 64, 256]), "ascend"),
    (dict(ends=[64, 64, 256]), "ascend"),
    (dict(ends=[24, 128, 256]), "multiples of 16"),
    (dict(tiles_per_run=3), "tiles_per_run must divide"),
    (dict(pull_bytes0=24), "multiples of 16"),
    (dict(sms=0), "multiprocessor count"),
    (dict(fused=True, ends=[32, 64, 96, 128, 160, 192, 256]), "at most six prefixes"),
    (dict(fused=True, rows_c=128 * 32, tiles_per_run=32), "at most 16 tiles"),
    (dict(fused=True), "scratch is too small"),
])
def test_forward_refuses_bad_shapes(ext, changes, message):
    with pytest.raises(RuntimeError, match=message):
        _forward(ext, **changes)


def test_backward_and_small_launchers_refuse_bad_shapes(ext):
    with pytest.raises(RuntimeError, match="multiples of 128"):
        ext.backward(256, 256, 256, 0, 100, 128, 256, [256], 1, 1.0, 10 ** 9, 0)
    with pytest.raises(RuntimeError, match="split must be at least 1"):
        ext.backward(256, 256, 256, 0, 128, 128, 256, [256], 0, 1.0, 10 ** 9, 0)
    with pytest.raises(RuntimeError, match="ascend"):
        ext.backward(256, 256, 256, 0, 128, 128, 256, [128, 64, 256], 1, 1.0, 10 ** 9, 0)
    with pytest.raises(RuntimeError, match="no candidates"):
        ext.backward(256, 0, 256, 0, 128, 128, 256, [256], 1, 1.0, 10 ** 9, 0)
    with pytest.raises(RuntimeError, match="multiple of 8"):
        ext.prefix_norms(256, 0, 256, 0, 128, 100, [100], 0)
    with pytest.raises(RuntimeError, match="multiples of 16"):
        ext.pull(256, 256, 24, 0, 0, 0, 4, 0)
    with pytest.raises(RuntimeError, match="1..8 prefixes"):
        ext.prefix_norms(256, 0, 256, 0, 128, 64, [], 0)


def test_the_ordinary_build_is_not_the_bounds_checked_one(ext):
    import os

    assert bool(ext.BOUNDS_BUILD) == (os.environ.get("SC_NATIVE_VARIANT", "") == "bounds")
    assert all(word == 0 for record in ext.bounds_records() for word in record) or bool(ext.BOUNDS_BUILD)


@pytest.mark.parametrize("entries,step,betas,message", [
    ([(256, 256, 256, 256, 8, True)], 0, (0.9, 0.999), "starts at 1"),
    ([(256, 256, 256, 256, 8, True)], 1, (1.0, 0.999), "betas"),
    ([(0, 256, 256, 256, 8, True)], 1, (0.9, 0.999), "null pointer"),
    ([(256, 256, 256, 256, 0, False)], 1, (0.9, 0.999), "empty tensor"),
])
def test_adamw_refuses_bad_arguments(ext, entries, step, betas, message):
    with pytest.raises(RuntimeError, match=message):
        ext.adamw_step(entries, 1e-3, betas[0], betas[1], 1e-8, 0.0, step, 0)
