import errno
import threading

import pytest

from scalingcontrasts_b200.parallel.rail import exchange_endpoint


def test_endpoint_files_cross_and_are_atomic(tmp_path):
    results = {}

    def side(own, remote, record):
        results[own] = exchange_endpoint(str(tmp_path), own, remote, 3, record, deadline_s=10.0)

    threads = [threading.Thread(target=side, args=(0, 1, b"A" * 208)), threading.Thread(target=side, args=(1, 0, b"B" * 208))]
    for thread in threads:
        thread.start()
    for thread in threads:
        thread.join()
    assert results[0] == b"B" * 208 and results[1] == b"A" * 208
    names = sorted(p.name for p in tmp_path.iterdir())
    assert names == ["endpoint-0-1-3", "endpoint-1-0-3"]  # no .partial left behind


def test_a_missing_counterpart_times_out(tmp_path):
    with pytest.raises(TimeoutError) as caught:
        exchange_endpoint(str(tmp_path), 0, 1, 0, b"x" * 16, deadline_s=0.05)
    assert caught.value.errno == errno.ETIMEDOUT
