"""The CPU oracle against golden vectors produced by the reference itself (tests/golden/make_golden.py) and against the
reference's own golden files (GPTQ decode fixtures, trellis tile fixtures)."""

import numpy as np
import pytest

from oracle import oracle_np as O


def test_e4m3_table_and_rounding(golden):
    g = golden("nvfp4")
    assert np.array_equal(O.e4m3_value(np.arange(127)), g["e4m3_table"])
    assert np.array_equal(O.e4m3_encode(g["e4m3_probe"]), g["e4m3_codes"])
    assert np.array_equal(O.e2m1_encode_magnitude(g["e2m1_probe"]), g["e2m1_codes"])


def test_nvfp4_offsets(golden):
    g = golden("nvfp4")
    for (n, k), expect in zip(g["offset_shapes"], g["offsets"]):
        assert O.nvfp4_offsets(int(n), int(k)) == tuple(int(v) for v in expect)
    # core/src/test/.../artifact/Nvfp4LayoutTest.java:18-30
    assert O.nvfp4_offsets(3, 1024) == (1536, 1792, 1796)
    assert O.nvfp4_sd4_offsets(3, 1024)[2] == 1812   # Nvfp4LayoutTest.java:60-79


@pytest.mark.parametrize("case", ["gauss", "spread", "padded", "edge"])
def test_nvfp4_quantize_bytes_and_dequant(golden, case):
    g = golden("nvfp4")
    weights, blob, dense = g[f"{case}_weights"], g[f"{case}_blob"].tobytes(), g[f"{case}_dense"]
    assert O.nvfp4_pack(weights) == blob
    n, k = weights.shape
    codes, scales, gs = O.nvfp4_unpack(blob, n, k)
    mine = O.nvfp4_dequantize(codes, scales, gs)
    assert np.array_equal(mine.view(np.uint32), dense.view(np.uint32))


def test_nvfp4_gptq_fixture_decode(golden):
    g = golden("gptq_decode")
    stem = "NVFP4-row-split-k128-v1-seq"
    codes, scales, decoded = g[f"{stem}-codes"], g[f"{stem}-scales"], g[f"{stem}-decoded"]
    mine = O.nvfp4_dequantize(codes, scales, np.float32(g["nvfp4_global_scale"]))
    assert np.array_equal(mine.view(np.uint32), decoded.view(np.uint32))


def test_q3_sizes_and_pack_order(golden):
    g = golden("q3")
    for (n, k), size in zip(g["size_shapes"], g["sizes"]):
        assert O.q3_offsets(int(n), int(k))[1] == int(size)
    assert np.array_equal(O.q3_pack_codes(np.repeat(g["pack_codes"], 1, axis=0)), g["pack_bytes"])


@pytest.mark.parametrize("case", ["gauss", "spread", "padded", "edge"])
def test_q3_quantize_bytes(golden, case):
    g = golden("q3")
    weights, blob = g[f"{case}_weights"], g[f"{case}_blob"].tobytes()
    assert O.q3_pack(weights) == blob
    n, k = weights.shape
    codes, scales = O.q3_unpack(blob, n, k)
    requantized_codes, requantized_scales = O.q3_quantize(weights)
    assert np.array_equal(codes, requantized_codes)
    assert np.array_equal(scales.view(np.uint16), requantized_scales.view(np.uint16))


@pytest.mark.parametrize("stem", ["Q3G64_F16S-row-split-k128-v1-seq", "Q3G64_F16S-row-split-k128-v1-act"])
def test_q3_gptq_fixture_decode(golden, stem):
    g = golden("gptq_decode")
    codes, scales, decoded = g[f"{stem}-codes"], g[f"{stem}-scales"], g[f"{stem}-decoded"]
    n, k = codes.shape
    blob = O.q3_assemble(codes, scales, n, k)
    mine = O.q3_dense(blob, n, k)
    # The fixture keeps the sign of the value a zero code came from (-0.0); code * scale gives the scale's sign.
    nonzero = decoded != 0
    assert np.array_equal(mine[nonzero].view(np.uint32), decoded[nonzero].view(np.uint32))
    assert not mine[~nonzero].any()


@pytest.mark.parametrize("w", [32, 40, 48, 56, 64, 80, 96])
def test_trellis_golden_tiles(golden, w):
    g = golden("trellis")
    mine = O.trellis_decode_tiles(g[f"tiles_{w}_packed"], w)
    assert np.array_equal(mine.view(np.uint16), g[f"tiles_{w}_out"].view(np.uint16))


@pytest.mark.parametrize("w", list(range(16, 129, 8)))
def test_trellis_random_words_every_width(golden, w):
    g = golden("trellis")
    mine = O.trellis_decode_tiles(g[f"random_{w}_words"], w)
    assert np.array_equal(mine.view(np.uint16), g[f"random_{w}_values"].view(np.uint16))


def test_trellis_linear_and_helpers(golden):
    g = golden("trellis")
    q = O.trellis_rotated_weight(g["linear_payload"])
    assert np.array_equal(q[:48, :48].view(np.uint16), g["linear_q_corner"].view(np.uint16))
    y = O.trellis_linear_f64(g["linear_x"], g["linear_payload"], g["linear_suh"], g["linear_svh"], [256])
    assert np.allclose(y, g["linear_y_f64"], rtol=1e-12, atol=1e-12)
    y2 = O.trellis_linear_f64(g["seg_x"], g["seg_payload"], g["seg_suh"], g["seg_svh"], list(g["seg_ends"]))
    assert np.allclose(y2, g["seg_y_f64"], rtol=1e-12, atol=1e-12)
    assert np.array_equal(O.hadamard128(g["hadamard_in"]).view(np.uint32), g["hadamard_out"].view(np.uint32))
    assert np.array_equal(O.trellis_fragment_order(g["fragment_in"]), g["fragment_out"])
    for (k, n, t), s in zip(g["splits_cases"], g["splits"]):
        assert O.trellis_splits(int(k), int(n), int(t)) == int(s)
    # The float32 production-route model agrees with float64 within the reference's kernel tolerance
    # (native/tests/test_trellis.py:157-165: 0.004 |y| + 0.004 rms).
    model = O.trellis_linear_kernel_model(g["linear_x"], g["linear_payload"], g["linear_suh"], g["linear_svh"], [256])
    rms = float(np.sqrt(np.mean(y ** 2)))
    assert np.all(np.abs(model - y) <= 0.004 * np.abs(y) + 0.004 * rms)


def test_bf16_rounding():
    values = np.array([1.0, 1.00390625, 1.005859375, -3.1415926, 1e-30, 65504.0], dtype=np.float32)
    bits = O.bf16_bits(values)
    assert bits[0] == 0x3F80 and bits[1] == 0x3F80 and bits[2] == 0x3F81  # tie to even, then above the tie
    assert np.array_equal(O.bf16_to_f32(bits), O.round_bf16(values))


def test_activation_quantizer_properties():
    """Two NVFP4 terms reconstruct BF16 activations to about 1% (native/tests/test_nvfp4_native.py:108-117 asserts
    < 1.2% for the device quantizer); one term to about 10%."""
    rng = np.random.default_rng(7)
    x = O.bf16_bits(rng.standard_normal((4, 512)).astype(np.float32))
    xf = O.bf16_to_f32(x).astype(np.float64)
    for terms, bound in ((1, 0.13), (2, 0.012)):
        codes, scales, g = O.quantize_activations(x, terms)
        err = np.linalg.norm(O.activations_dense(codes, scales, g) - xf) / np.linalg.norm(xf)
        assert err < bound, (terms, err)
    zero = np.zeros((1, 128), dtype=np.uint16)
    codes, scales, g = O.quantize_activations(zero)
    assert g[0] == 1.0 and not codes.any() and not scales.any()
    assert O.activation_layout(4096, 5120)[2] == O.activation_layout(4096, 5120)[1] + 4 * 4096


@pytest.mark.parametrize("case", ["gauss", "spread", "padded"])
def test_nvfp4_sd4_layout_and_values(golden, case):
    """Table-indexed NVFP4 (row-split-k128-sd4-v1) as the reference's converter writes it: geometry, and the dense values
    through the oracle's table lookup, bit for bit."""
    g = golden("nvfp4_sd4")
    w = g[f"{case}_weights"]
    n, k = w.shape
    blob = g[f"{case}_blob"].tobytes()
    assert len(blob) == O.nvfp4_sd4_offsets(n, k)[2]
    dense = O.nvfp4_sd4_dense(blob, n, k)
    assert np.array_equal(dense.view(np.uint32), g[f"{case}_dense"][:, :k].astype(np.float32).view(np.uint32))
    for (rows, cols), expect in zip(g["offset_shapes"], g["offsets"]):
        assert O.nvfp4_sd4_offsets(int(rows), int(cols)) == tuple(int(v) for v in expect)
    # the stand-in generator of the kernel tests gives a well-formed tensor whose values use table entries only
    plain = O.nvfp4_pack(w)
    again = O.nvfp4_sd4_from_plain(plain, n, k, np.random.default_rng(1))
    assert len(again) == len(blob)
    codes, scales, _ = O.nvfp4_unpack(O.nvfp4_sd4_to_plain(again, n, k), n, k)
    table = np.frombuffer(again, dtype=np.uint8)[O.nvfp4_sd4_offsets(n, k)[1]:][:16]
    assert np.all(np.isin(scales, table)) and np.array_equal(codes, O.nvfp4_unpack(plain, n, k)[0])


@pytest.mark.parametrize("w,ka,mask", [(32, 2, 0), (40, 2, 0xAAAA), (48, 3, 0), (56, 3, 0xAAAA), (64, 4, 0), (80, 5, 0), (96, 6, 0)])
def test_trellis_tile_encoder_reproduces_the_golden_tiles(golden, w, ka, mask):
    """The restated tail-biting Viterbi (FP16 costs, lowest predecessor on ties, two passes) gives the reference encoder's
    own states, decoded values and packed words on its golden tiles, bit for bit, at all seven rates."""
    from oracle import oracle_c as OC
    g = golden("trellis")
    states, decoded = OC.trellis_encode_tiles(g["tiles_in"], ka, mask)
    assert np.array_equal(states, g[f"tiles_{w}_idx"])
    assert np.array_equal(decoded.astype(np.float16).view(np.uint16), g[f"tiles_{w}_out"].view(np.uint16))
    packed = O.trellis_pack_states(states, ka, mask)
    assert packed.shape[1] == w and np.array_equal(packed, g[f"tiles_{w}_packed"])
    # and the decoder reads the packed words back to the same values
    assert np.array_equal(O.trellis_decode_tiles(packed, w).view(np.uint16), g[f"tiles_{w}_out"].view(np.uint16))


def test_q3_weights_are_two_bf16_terms_exactly():
    """The Q3 prefill's claim, for EVERY finite FP16 scale and every code: code * f32(scale) = hi + lo with hi = bf16(code *
    scale) and lo = bf16(code * scale - hi), both roundings to nearest even, and nothing is lost (the residual after hi has at
    most six significant bits)."""
    scales = np.arange(65536, dtype=np.uint16).view(np.float16)
    scales = scales[np.isfinite(scales)].astype(np.float32)
    for code in range(-4, 4):
        value = np.float32(code) * scales                       # exact: 3 bits times 11 bits
        assert np.array_equal(value.astype(np.float64), np.float64(code) * scales.astype(np.float64))
        hi = O.bf16_to_f32(O.bf16_bits(value))
        rest = value - hi                                        # exact in float32 (Sterbenz-like: same binade or below)
        assert np.array_equal(rest.astype(np.float64), value.astype(np.float64) - hi.astype(np.float64))
        lo = O.bf16_to_f32(O.bf16_bits(rest))
        assert np.array_equal(lo, rest)                          # the residual is a BF16 value: no second rounding error
        assert np.array_equal(hi.astype(np.float64) + lo.astype(np.float64), value.astype(np.float64))


def test_trellis_prefill_model_is_the_linear_up_to_its_bf16_roundings():
    """The model of the reference's prefill plan (BF16 activations, BF16 decoded weight, BF16 products, BF16 output) against the
    unrounded float64 linear of the same object: they differ by those roundings only."""
    rng = np.random.default_rng(17)
    k, n, w, ends = 256, 384, 48, [128, 384]
    payload = rng.integers(-32768, 32768, size=(k // 16, n // 16, w), dtype=np.int16)
    suh = (rng.choice([-1.0, 1.0], size=(2, k)) * rng.uniform(0.5, 2.0, size=(2, k))).astype(np.float16)
    svh = rng.uniform(0.01, 1.0, size=n).astype(np.float16)
    x = O.bf16_bits(rng.standard_normal((7, k)).astype(np.float32))
    model = O.trellis_prefill_model(x, payload, suh, svh, ends).astype(np.float64)
    exact = O.trellis_linear_f64(x, payload, suh, svh, ends)
    rms = float(np.sqrt(np.mean(exact ** 2)))
    assert np.all(np.abs(model - exact) <= 0.02 * np.abs(exact) + 0.02 * rms)
    assert np.sqrt(np.mean((model - exact) ** 2)) < 0.006 * rms
    assert np.array_equal(O.bf16_to_f32(O.bf16_bits(model.astype(np.float32))), model.astype(np.float32))   # BF16 values
