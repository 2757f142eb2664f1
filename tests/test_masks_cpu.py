"""CPU tests of the counter-based draw restatement (oracle/philox.py): the published known-answer vectors of
Philox4x32-10 pin the generator; the derived masks have the probabilities the reference asks its generators for."""
import numpy as np

from oracle import philox


def test_philox4x32_10_known_answers():
    kat = [
        ((0x00000000, 0x00000000, 0x00000000, 0x00000000), (0x00000000, 0x00000000), (0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8)),
        ((0xffffffff, 0xffffffff, 0xffffffff, 0xffffffff), (0xffffffff, 0xffffffff), (0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd)),
        ((0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344), (0xa4093822, 0x299f31d0), (0xd16cfe09, 0x94fdcceb, 0x5001e420, 0x24126ea1)),
    ]
    for ctr, key, want in kat:
        got = philox.philox4x32_10(np.array([ctr], np.uint32), key)[0]
        assert [int(x) for x in got] == list(want)


def test_uniform_range_and_moments():
    u = philox.uniform(seed=7, step=3, layer=2, kind=0, n=1 << 18)
    assert u.dtype == np.float32 and u.min() >= 0.0 and u.max() < 1.0
    assert abs(float(u.mean()) - 0.5) < 4 * (1 / 12 ** 0.5) / (1 << 9)
    assert abs(float(np.corrcoef(u[:-1], u[1:])[0, 1])) < 0.01


def test_streams_differ_by_every_coordinate():
    base = philox.uniform(1, 0, 1, 0, 4096)
    for other in (philox.uniform(2, 0, 1, 0, 4096), philox.uniform(1, 1, 0 + 1, 0, 4096), philox.uniform(1, 0, 2, 0, 4096),
                  philox.uniform(1, 0, 1, 1, 4096), philox.uniform(1 + (1 << 32), 0, 1, 0, 4096), philox.uniform(1, 1 << 32, 1, 0, 4096)):
        assert (base != other).mean() > 0.99
    assert np.array_equal(base, philox.uniform(1, 0, 1, 0, 4096))
    assert np.array_equal(base[:1000], philox.uniform(1, 0, 1, 0, 1000))   # a prefix does not depend on the length asked for


def test_mask_probabilities():
    n = 1 << 17
    keep = philox.bernoulli_mask(5, 0, 1, n, 0.6)
    assert abs(keep.mean() - 0.6) < 4 * (0.24 / n) ** 0.5
    zs, zo = philox.zoneout_masks(5, 0, 1, n, 0.1, 0.3)
    assert abs(zs.mean() - 0.9) < 4 * (0.09 / n) ** 0.5 and abs(zo.mean() - 0.7) < 4 * (0.21 / n) ** 0.5
    m, a, b = philox.shakedrop(5, 0, 1, 4096, 32, 0.5)
    assert abs(m.mean() - 0.5) < 4 * (0.25 / 4096) ** 0.5
    assert a.min() >= -1.0 and a.max() < 1.0 and abs(a.mean()) < 0.01
    assert b.min() >= 0.0 and b.max() < 1.0 and abs(b.mean() - 0.5) < 0.01
