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


def test_regularize_is_undone_by_the_decoders_formula(monkeypatch):
    """W = diag(su) H_K Q H_N diag(sv) for the rotated Q the tile search sees (with the global scale inside su): the
    algebra of TrellisQuantizer.java:242-263 and of the decoder, on the CPU (the search itself needs the GPU)."""
    converter = T.TrellisConverter("cpu")
    monkeypatch.setattr(converter, "global_scale", lambda w, bits: 0.875)
    rng = np.random.default_rng(9)
    k, n = 256, 384
    w = (rng.standard_normal((k, n)) * 0.02 * rng.uniform(0.3, 3.0, size=(1, n))).astype(np.float32)
    w[:, 5] = 0.0                                            # an output channel without energy
    su_signs, sv_signs = [torch.from_numpy(v) for v in T.java_signs(4, k, n)]
    for apply in (True, False):
        q, su, sv, g = converter.regularize(torch.from_numpy(w.copy()), su_signs, sv_signs, apply, 3.0)
        assert g == 0.875 and sv[5] == 0.0
        back = T.hadamard128(T.hadamard128(q, 0) * su[:, None], 1) * sv[None, :]
        keep = np.arange(n) != 5
        assert np.allclose(back.numpy()[:, keep], w[:, keep], rtol=0, atol=2e-7 + 1e-5 * np.abs(w[:, keep]).max())
        # rows of the rotated weight sit at the codebook's scale times g
        rms = q.double().square().mean().sqrt().item()
        assert abs(rms / (T.CODEBOOK_SCALE * 0.875) - 1.0) < 0.05
        # signs: su carries -sign (the codebook scale is negated), sv carries +sign
        assert torch.equal(torch.sign(su), -su_signs) and torch.equal(torch.sign(sv)[keep], sv_signs[keep])
        if not apply:
            assert torch.equal(sv[keep].abs(), torch.ones(n - 1))


def test_tiles_of_follows_the_tile_order():
    converter = T.TrellisConverter("cpu")
    k, n = 32, 48
    w = torch.arange(k * n, dtype=torch.float32).view(k, n)
    tiles = converter.tiles_of(w)
    assert tiles.shape == (6, 256)
    row, col = O.trellis_position_rc(np.arange(256))
    for tile, (kt, nt) in enumerate((a, b) for a in range(2) for b in range(3)):
        assert np.array_equal(tiles[tile].numpy(), w.numpy()[kt * 16 + row, nt * 16 + col])


def test_shapes_must_be_multiples_of_128():
    converter = T.TrellisConverter("cpu")
    with pytest.raises(ValueError):
        converter.quantize(torch.zeros(128, 192), 3.0, seed=1)
    with pytest.raises(ValueError):
        converter.quantize(torch.zeros(128, 128), 4.5, seed=1)
