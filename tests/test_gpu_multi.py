"""Multi-GPU checks, one process per GPU, driven through the command line modes (which is also how a user runs them).
They need at least two visible GPUs and are skipped otherwise."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _gpus() -> int:
    return min(torch.cuda.device_count(), 8) if torch.cuda.is_available() else 0


def _run(*arguments: str, timeout: int = 600) -> list:
    environment = dict(os.environ, PYTHONPATH=ROOT, NCCL_NVLS_ENABLE="0")
    result = subprocess.run([sys.executable, "-m", "scalingcontrasts_b200.cli", *arguments], cwd=ROOT, env=environment,
                            capture_output=True, text=True, timeout=timeout)
    assert result.returncode == 0, result.stdout[-3000:] + result.stderr[-3000:]
    return [line.split(",") for line in result.stdout.strip().splitlines() if "," in line]


needs_two = pytest.mark.skipif(_gpus() < 2, reason="needs at least two GPUs")


@needs_two
@pytest.mark.parametrize("flags", [(), ("--no-multicast",)], ids=["multimem", "peer"])
def test_collectives_are_exact_and_repeat_bit_for_bit(flags):
    rows = _run("collectives", "--gpus", str(_gpus()), "--min-kib", "1", "--max-mib", "4", "--repeats", "5", "--windows", "2", *flags)
    path = "peer" if flags else "multimem"
    for name in ("validation", "validation_one_round"):  # the two-round form at the largest size, the one-round form at 64 KiB
        validation = [row for row in rows if row[0] == name][0]
        assert int(validation[1]) == _gpus()
        assert (int(validation[3]), int(validation[4]), int(validation[6])) == (0, 0, 0)
        assert validation[7] == path  # the kernels that ran are the ones the row claims
    assert all(row[7] == path for row in rows if row[0] in ("all_reduce", "all_reduce_two_round", "reduce_scatter"))
    assert any(row[0] == "all_reduce_two_round" for row in rows)
    assert any(row[0] == "barrier" for row in rows) and any(row[0] == "all_reduce" for row in rows)
    assert all(float(row[3]) > 0 for row in rows if row[0] in ("all_reduce", "reduce_scatter"))


@needs_two
@pytest.mark.parametrize("positives", ["self", "pairs"])
def test_box_oracle_against_float64(positives):
    row = _run("oracle", "--gpus", str(_gpus()), "--rows", "128", "--hidden", "768", "--prefixes", "5", "--inputs", "normal",
               "--seed", "1", "--positives", positives)[-1]
    exact, measured, error, disagreeing = float(row[5]), float(row[6]), float(row[7]), int(row[8])
    assert int(row[4]) == _gpus()
    assert abs(measured - exact) <= 2e-6 * abs(exact)
    assert error < 4e-3
    assert disagreeing == 0  # every rank holds the same loss, bit for bit


@needs_two
def test_box_and_train_modes_run():
    box = _run("box", "--gpus", str(_gpus()), "--rows", "512", "--hidden", "256", "--prefixes", "3", "--windows", "2")[-1]
    assert box[0] == "box" and int(box[4]) == _gpus() and float(box[6]) > 0
    train = _run("train", "--gpus", str(_gpus()), "--rows", "512", "--hidden", "256", "--prefixes", "3", "--warm", "3", "--steps", "10")[-1]
    assert train[0] == "train" and float(train[5]) > 0


@needs_two
def test_gradient_reducer_matches_nccl_sum():
    script = os.path.join(ROOT, "tests", "multi_reducer_check.py")
    environment = dict(os.environ, PYTHONPATH=ROOT, NCCL_NVLS_ENABLE="0")
    result = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={min(_gpus(), 4)}",
                             "--master-addr", "127.0.0.1", "--master-port", "29631", script], cwd=ROOT, env=environment,
                            capture_output=True, text=True, timeout=600)
    assert result.returncode == 0, result.stdout[-3000:] + result.stderr[-3000:]
    assert "reducer ok" in result.stdout


@needs_two
def test_box_steps_without_the_closing_all_reduce_and_as_cuda_graphs():
    script = os.path.join(ROOT, "tests", "multi_box_check.py")
    environment = dict(os.environ, PYTHONPATH=ROOT, NCCL_NVLS_ENABLE="0")
    result = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={min(_gpus(), 4)}",
                             "--master-addr", "127.0.0.1", "--master-port", "29633", script], cwd=ROOT, env=environment,
                            capture_output=True, text=True, timeout=600)
    assert result.returncode == 0, result.stdout[-3000:] + result.stderr[-3000:]
    assert "box steps ok" in result.stdout


@needs_two
def test_hosts_mode_over_loopback_rails_against_float64():
    """Two logical hosts on this box, their blocks crossing the rails, checked like the box oracle."""
    gpus = _gpus() - _gpus() % 2
    row = _run("hosts", "--hosts", "2", "--gpus", str(gpus), "--rows", "128", "--hidden", "256", "--prefixes", "3", "--inputs",
               "normal", "--seed", "2", "--windows", "0")[-1]
    exact, measured, error, disagreeing = float(row[5]), float(row[6]), float(row[7]), int(row[8])
    assert row[0] == "oracle" and int(row[4]) == gpus
    assert abs(measured - exact) <= 2e-6 * abs(exact) and error < 4e-3 and disagreeing == 0
    timed = _run("hosts", "--hosts", "2", "--gpus", str(gpus), "--rows", "256", "--hidden", "256", "--prefixes", "3", "--windows", "2")[-1]
    assert timed[0] == "hosts" and float(timed[6]) > 0
