"""Host side of the trellis converter: sign draws, tile order, butterflies, rates (no GPU)."""
import numpy as np
import pytest
import torch

from euhedral_b200 import trellis_convert as T
from oracle import oracle_np as O


def test_tile_order_is_the_decoders():
    row, col = O.trellis_position_rc(np.arange(256))
    assert np.array_equal(T.tile_order(), row * 16 + col)
    assert sorted(T.tile_order().tolist()) == list(range(256))


def test_hadamard_is_the_sylvester_matrix():
    i = np.arange(128)
    h = np.where(np.bitwise_count(i[:, None] & i[None, :]) & 1, -1.0, 1.0) / np.sqrt(128.0)
    rng = np.random.default_rng(5)
    x = rng.standard_normal((256, 384)).astype(np.float32)
    along_n = T.hadamard128(torch.from_numpy(x), 1).numpy()
    want = (x.reshape(256, 3, 128).astype(np.float64) @ h).reshape(256, 384)
    assert np.allclose(along_n, want, atol=2e-6)
    along_k = T.hadamard128(torch.from_numpy(x), 0).numpy()
    want = np.einsum("ij,bjc->bic", h, x.reshape(2, 128, 384).astype(np.float64)).reshape(256, 384)
    assert np.allclose(along_k, want, atol=2e-6)
    # its own inverse
    assert np.allclose(T.hadamard128(torch.from_numpy(along_k), 0).numpy(), x, atol=2e-6)


def test_sign_draws_follow_splitmix64():
    # SplitMix64 step by step in Python integers, against the vectorised draw
    def draws(seed, count):
        mask, state, out = (1 << 64) - 1, seed & ((1 << 64) - 1), []
        for _ in range(count):
            state = (state + 0x9E3779B97F4A7C15) & mask
            z = ((state ^ (state >> 33)) * 0x62A9D9ED799705F5) & mask
            z = ((z ^ (z >> 28)) * 0xCB24D0A5C88C35B3) & mask
            value = z >> 32
            out.append(1.0 if value >= 1 << 31 else -1.0)     # the int is negative
        return np.array(out, dtype=np.float32)

    for seed in (0, 1, -7, 1234567890123):
        su, sv = T.java_signs(seed, 128, 256)
        want = draws(seed, 384)
        assert np.array_equal(su, want[:128]) and np.array_equal(sv, want[128:])
        assert 0.3 < (su > 0).mean() < 0.7


def test_rates():
    assert [T.words_per_tile(b) for b in (2, 2.5, 3, 3.5, 4, 5, 6)] == [32, 40, 48, 56, 64, 80, 96]
    with pytest.raises(ValueError):
        T.words_per_tile(4.5)
    assert T.drift(2) == 1.018 and T.drift(3) == 1.004 and T.drift(4) == 1.0
