import numpy as np
import torch

from scalingcontrasts_b200.utils import keyed


def test_splitmix64_known_values():
    # First outputs of the splitmix64 finalizer for keys 0, 1, 2 computed with Python integers.
    def reference(v):
        mask = (1 << 64) - 1
        v = ((v ^ (v >> 30)) * 0xBF58476D1CE4E5B9) & mask
        v = ((v ^ (v >> 27)) * 0x94D049BB133111EB) & mask
        return v ^ (v >> 31)

    keys = np.array([0, 1, 2, 12345678901234567, (1 << 64) - 1], dtype=np.uint64)
    assert [int(x) for x in keyed.splitmix64(keys)] == [reference(int(k)) for k in keys]


def test_embeddings_range_and_determinism():
    a = keyed.keyed_embeddings(64, 128, salt=3, scale=0.1)
    b = keyed.keyed_embeddings(64, 128, salt=3, scale=0.1)
    c = keyed.keyed_embeddings(64, 128, salt=4, scale=0.1)
    assert a.dtype == torch.bfloat16 and torch.equal(a, b) and not torch.equal(a, c)
    assert float(a.float().abs().max()) <= 0.05 + 1e-3


def test_integers_sum_exactly_in_any_order():
    members, scalars = 8, 4096
    values = [keyed.keyed_integers(scalars, members, m) for m in range(members)]
    assert all(float(v.max()) < 4096 and float(v.min()) >= 0 for v in values)
    forward = sum(values)
    backward = sum(reversed(values))
    assert torch.equal(forward, backward) and torch.equal(forward, keyed.keyed_integer_sums(scalars, members))


def test_fractions_are_order_sensitive_material():
    values = [keyed.keyed_fractions(1 << 12, 8, m) for m in range(8)]
    assert all(float(v.min()) >= -0.5 and float(v.max()) < 0.5 for v in values)
    assert not torch.equal(values[0], values[1])
