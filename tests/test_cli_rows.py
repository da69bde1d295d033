"""Row formats and flag handling of the command line, on the CPU."""
import subprocess
import sys

import pytest

from scalingcontrasts_b200 import cli


def _run(*arguments):
    return subprocess.run([sys.executable, "-m", "scalingcontrasts_b200.cli", *arguments], capture_output=True, text=True, timeout=300)


def test_unknown_flag_exits_with_status_two():
    result = _run("box", "--no-such-flag", "1")
    assert result.returncode == 2 and "unrecognized arguments" in result.stderr


def test_invalid_values_are_rejected():
    assert _run("box", "--rows", "0", "--device", "cpu").returncode != 0
    assert _run("hosts", "--hosts", "2", "--host", "2", "--device", "cpu").returncode != 0


def test_cpu_oracle_row_has_the_reference_columns():
    result = _run("oracle", "--device", "cpu", "--rows", "64", "--hidden", "128", "--prefixes", "3", "--gpus", "1", "--header",
                  "--positives", "pairs", "--inputs", "normal")
    assert result.returncode == 0, result.stderr
    header, row = result.stdout.strip().splitlines()[-2:]
    assert header == cli.HEADERS["oracle"]
    fields = row.split(",")
    assert fields[0] == "oracle" and fields[1:5] == ["64", "128", "3", "1"] and len(fields) == 9
    exact, measured, error, disagreeing = float(fields[5]), float(fields[6]), float(fields[7]), int(fields[8])
    assert abs(exact - measured) < 1e-5 * abs(exact) and error < 1e-4 and disagreeing == 0


def test_defaults_match_the_reference_binary():
    arguments = cli.build_parser().parse_args(["collectives"])
    assert (arguments.rows, arguments.hidden, arguments.prefixes, arguments.windows, arguments.max_mib, arguments.repeats) == (
        1024, 1024, 5, 10, 128, 1000)
    settings = cli.settings_from(cli.build_parser().parse_args(["box", "--ends", "64,256,768", "--hidden", "768"]))
    assert settings.ladder().ends == (64, 256, 768)
    with pytest.raises(SystemExit):
        cli.build_parser().parse_args(["fly"])
