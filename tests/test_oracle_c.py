"""The plain-C checker (oracle/oracle.c) against the NumPy oracle and the golden vectors."""

import numpy as np
import pytest

from oracle import oracle_c as OC
from oracle import oracle_np as O


@pytest.mark.parametrize("case", ["gauss", "spread", "padded", "edge"])
def test_c_nvfp4_bytes(golden, case):
    g = golden("nvfp4")
    weights = g[f"{case}_weights"]
    n, k = weights.shape
    blob = OC.nvfp4_quantize(weights, threads=3)
    assert blob.tobytes() == g[f"{case}_blob"].tobytes()
    dense = OC.nvfp4_dense(blob, n, k)
    assert np.array_equal(dense.view(np.uint32), g[f"{case}_dense"][:, :k].view(np.uint32))


@pytest.mark.parametrize("case", ["gauss", "spread", "padded", "edge"])
def test_c_q3_bytes(golden, case):
    g = golden("q3")
    weights = g[f"{case}_weights"]
    n, k = weights.shape
    blob = OC.q3_quantize(weights, threads=2)
    assert blob.tobytes() == g[f"{case}_blob"].tobytes()
    assert np.array_equal(OC.q3_dense(blob, n, k), O.q3_dense(blob.tobytes(), n, k))


def test_c_linears_match_float64():
    rng = np.random.default_rng(11)
    n, k, rows = 48, 1024, 3
    weights = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    x = O.bf16_bits(rng.standard_normal((rows, k)).astype(np.float32))
    for pack, linear, dense in ((OC.nvfp4_quantize, OC.nvfp4_linear, O.nvfp4_dense), (OC.q3_quantize, OC.q3_linear, O.q3_dense)):
        blob = pack(weights)
        y = linear(x, blob, n, k)
        ref = O.linear_f64(x, dense(blob.tobytes(), n, k))
        assert np.max(np.abs(y - ref)) <= 2e-5 * np.max(np.abs(ref))


@pytest.mark.parametrize("w", [16, 40, 48, 56, 64, 96, 128])
def test_c_trellis_tiles(golden, w):
    g = golden("trellis")
    words = g[f"random_{w}_words"]
    assert np.array_equal(OC.trellis_decode_tiles(words, w).view(np.uint16), g[f"random_{w}_values"].view(np.uint16))


def test_c_trellis_linear(golden):
    g = golden("trellis")
    for prefix, ends in (("linear", [256]), ("seg", list(g["seg_ends"]))):
        y = OC.trellis_linear(g[f"{prefix}_x"], g[f"{prefix}_payload"], g[f"{prefix}_suh"], g[f"{prefix}_svh"], ends)
        ref = g[f"{prefix}_y_f64"]
        assert np.max(np.abs(y - ref)) <= 1e-4 * np.max(np.abs(ref))
