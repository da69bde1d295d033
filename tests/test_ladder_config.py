import pytest

from scalingcontrasts_b200 import LossSpec, Matryoshka, Settings


def test_halvings_match_the_reference_rule():
    assert Matryoshka.halvings(1024, 5).ends == (64, 128, 256, 512, 1024)
    assert Matryoshka.halvings(768, 5).ends == (48, 96, 192, 384, 768)
    assert Matryoshka.halvings(256, 3).ends == (64, 128, 256)


def test_bands():
    ladder = Matryoshka.halvings(768, 5)
    assert [ladder.begin(b) for b in range(5)] == [0, 48, 96, 192, 384]
    assert [ladder.width(b) for b in range(5)] == [48, 48, 96, 192, 384]
    assert ladder.band_of(0) == 0 and ladder.band_of(47) == 0 and ladder.band_of(48) == 1 and ladder.band_of(767) == 4
    assert ladder.padded() == [48, 96, 192, 384, 768, 0, 0, 0]
    assert ladder.mma_depth_per_cell() == 1536


def test_validation():
    with pytest.raises(ValueError):
        Matryoshka((64, 64))
    with pytest.raises(ValueError):
        Matryoshka(tuple(range(16, 16 * 10, 16)))
    with pytest.raises(ValueError):
        Matryoshka.halvings(768, 5).check_device_shape(100, 768)
    with pytest.raises(ValueError):
        Matryoshka((40, 768)).check_device_shape(128, 768)
    Matryoshka.halvings(768, 5).check_device_shape(128, 768)  # edges at multiples of 16 are fine


def test_spec_codes_and_defaults():
    assert LossSpec("self").diagonal == "own" and LossSpec("self").code() == 0
    assert LossSpec("pairs").diagonal == "negative" and LossSpec("pairs").code() == 1 | (1 << 1)
    assert LossSpec("pairs", "skip").code() == 1 | (2 << 1)
    with pytest.raises(ValueError):
        LossSpec("triples")


def test_settings_defaults_are_the_reference_flags():
    s = Settings()
    assert (s.rows, s.hidden, s.prefixes, s.windows, s.max_mib, s.repeats, s.host, s.hosts) == (1024, 1024, 5, 10, 128, 1000, 0, 1)
    s.validate()
    with pytest.raises(ValueError):
        Settings(rows=0).validate()
    with pytest.raises(ValueError):
        Settings(host=2, hosts=2).validate()
