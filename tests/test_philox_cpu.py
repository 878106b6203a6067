"""Known-answer vectors of Philox-4x32-10 (Random123 distribution, kat_vectors) for the numpy
restatement that the GPU tests use to check the dropout kernels' keep-bits."""
import numpy as np

from util import dropout_keep_bits, philox4x32_10


def test_philox_known_answers():
    z = np.zeros((1, 4), dtype=np.uint32)
    assert [hex(v) for v in philox4x32_10(z, (0, 0))[0]] == ["0x6627e8d5", "0xe169c58d", "0xbc57ac4c", "0x9b00dbd8"]
    f = np.full((1, 4), 0xFFFFFFFF, dtype=np.uint32)
    assert [hex(v) for v in philox4x32_10(f, (0xFFFFFFFF, 0xFFFFFFFF))[0]] == ["0x408f276d", "0x41c83b0e", "0xa20bc7c6",
                                                                              "0x6d5451fd"]
    pi = np.array([[0x243F6A88, 0x85A308D3, 0x13198A2E, 0x03707344]], dtype=np.uint32)
    assert [hex(v) for v in philox4x32_10(pi, (0xA4093822, 0x299F31D0))[0]] == ["0xd16cfe09", "0x94fdcceb", "0x5001e420",
                                                                               "0x24126ea1"]


def test_keep_bits_rate_and_determinism():
    a = dropout_keep_bits(64, 64, 1234567890123, 0.5)
    b = dropout_keep_bits(64, 64, 1234567890123, 0.5)
    assert np.array_equal(a, b) and a.max() <= 15
    rate = np.unpackbits(a[..., None], axis=-1)[..., 4:].mean()
    assert abs(rate - 0.5) < 0.03
    assert np.array_equal(dropout_keep_bits(4, 4, 7, 0.0), np.full((4, 4), 15, dtype=np.uint8))
