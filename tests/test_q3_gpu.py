"""Q3G64_F16S decode GEMV through the C ABI against the oracle (modelled on native/tests/test_q3_kernels.py)."""

import numpy as np
import pytest

from euhedral_b200 import library, sharding
from oracle import oracle_c as OC
from oracle import oracle_np as O
from tests.gpu_util import Device, max_relative_error, random_x

pytestmark = pytest.mark.gpu

SHAPES = [(1024, 16), (1024, 64), (5120, 96), (17408, 32), (5120, 1024), (128, 16), (2560, 192)]  # (K, N)


@pytest.fixture(scope="module")
def dev():
    device = Device()
    yield device
    assert device.gpu.take_device_error() == 0
    device.release()


def random_tensor(rng, n, k):
    """Random codes and edge FP16 scales (zero, subnormal, large, negative), as the reference's kernel test does
    (native/tests/test_q3_kernels.py:25,121-133)."""
    codes = rng.integers(-4, 4, size=(n, k)).astype(np.int8)
    groups = k // 64
    scales = (rng.standard_normal((n, groups)) * 0.01).astype(np.float16)
    scales[0, 0] = 0.0
    scales[-1, -1] = np.float16(6.0e-8)
    scales[n // 2, groups // 2] = np.float16(-3.5)
    scales[1 % n, 0] = np.float16(1000.0)
    blob = np.frombuffer(O.q3_assemble(codes, scales, n, k), dtype=np.uint8).copy()
    return blob, O.q3_dense(blob.tobytes(), n, k)


def run(dev, x_bits, blob, n, k, reference=False, **select):
    rows = x_bits.shape[0]
    d_x, d_w, d_y = dev.put(x_bits), dev.put(blob), dev.empty(rows * n * 2)
    with dev.submit(**select) as gpu:
        call = gpu.linear_q3_reference_bf16 if reference else gpu.linear_q3_bf16
        call(d_x.data_ptr(), d_w.data_ptr(), d_y.data_ptr(), rows, k, n, blob.size)
    return dev.get(d_y, np.uint16, (rows, n))


def close_to(got_bits, expect):
    got = O.bf16_to_f32(got_bits).astype(np.float64)
    bound = np.abs(expect) * 2.0 ** -7 + np.max(np.abs(expect)) * 1e-3
    return np.all(np.abs(got - expect) <= bound) and max_relative_error(got, expect) <= 2e-3 + 2.0 ** -8


@pytest.mark.parametrize("k,n", SHAPES)
def test_decode_matches_float64(dev, k, n):
    rng = np.random.default_rng(k * 17 + n)
    blob, dense = random_tensor(rng, n, k)
    for rows in (1, 2, 3, 4, 5, 8):
        x = random_x(rng, rows, k)
        assert close_to(run(dev, x, blob, n, k), O.linear_f64(x, dense)), (rows, k, n)


def test_quantized_gaussian_weights(dev):
    rng = np.random.default_rng(0xE1)
    k, n = 5120, 256
    weights = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    blob = OC.q3_quantize(weights)
    x = random_x(rng, 3, k)
    assert close_to(run(dev, x, blob, n, k), O.linear_f64(x, O.q3_dense(blob.tobytes(), n, k)))


@pytest.mark.parametrize("k,n", SHAPES)
def test_rows_are_bitwise_the_one_row_call(dev, k, n):
    rng = np.random.default_rng(k + 3 * n)
    blob, _ = random_tensor(rng, n, k)
    x = random_x(rng, 8, k)
    single = np.concatenate([run(dev, x[r:r + 1], blob, n, k) for r in range(8)])
    for rows in (3, 8):
        assert np.array_equal(run(dev, x[:rows], blob, n, k), single[:rows])
    many = random_x(rng, 32, k)
    grouped = run(dev, many, blob, n, k, row_exact=True)   # without it, more than 8 rows take the prefill route
    for r in (0, 7, 8, 31):
        assert np.array_equal(grouped[r], run(dev, many[r:r + 1], blob, n, k)[0])


def test_scalar_kernel_and_exact_numerics(dev):
    rng = np.random.default_rng(12)
    k, n = 1024, 32
    blob, dense = random_tensor(rng, n, k)
    x = random_x(rng, 2, k)
    reference = run(dev, x, blob, n, k, reference=True)
    assert np.array_equal(reference, O.q3_linear_scalar_kernel(x, blob.tobytes(), n, k))
    dev.gpu.select_exact_numerics(True)
    try:
        assert np.array_equal(run(dev, x, blob, n, k), reference)
    finally:
        dev.gpu.select_exact_numerics(False)
    # K % 128 != 0: no decode kernel, the scalar kernel runs (K is padded to 128 in the layout)
    k2, n2 = 200, 16
    weights = (rng.standard_normal((n2, k2)) * 0.02).astype(np.float32)
    blob2 = OC.q3_quantize(weights)
    x2 = random_x(rng, 2, k2)
    assert np.array_equal(run(dev, x2, blob2, n2, k2), O.q3_linear_scalar_kernel(x2, blob2.tobytes(), n2, k2))


def test_status_codes(dev):
    lib = library.load()
    k, n = 1024, 16
    blob, _ = random_tensor(np.random.default_rng(2), n, k)
    d_x, d_w, d_y = dev.put(random_x(np.random.default_rng(3), 1, k)), dev.put(blob), dev.empty(n * 2)
    call = lib.euhedral_cuda_linear_q3_bf16
    assert call(None, d_w.data_ptr(), d_y.data_ptr(), 1, k, n, blob.size) == library.INVALID_ARGUMENT
    assert call(d_x.data_ptr(), d_w.data_ptr(), d_y.data_ptr(), 1, k, n, 0) == library.INVALID_ARGUMENT
    assert call(d_x.data_ptr(), d_w.data_ptr(), d_y.data_ptr(), 1, k, n, blob.size + 2) == library.FORMAT_MISMATCH
    assert call(d_x.data_ptr(), d_w.data_ptr(), d_y.data_ptr(), 1, k, n, blob.size) == library.SUCCESS


def test_row_shards_equal_the_whole(dev):
    rng = np.random.default_rng(8)
    k, n = 5120, 1024
    blob, _ = random_tensor(rng, n, k)
    x = random_x(rng, 3, k)
    whole = run(dev, x, blob, n, k)
    for shards in (2, 8):
        parts = [run(dev, x, sharding.q3_rows(blob, n, k, s * n // shards, n // shards), n // shards, k) for s in range(shards)]
        assert np.array_equal(np.concatenate(parts, axis=1), whole)


# The last two are the fused objects the reference's converter emits and its host calls as one tensor: query_key_value
# (5120 + 1024 + 1024 rows) and gate_up (2 x 17408 rows), tools/euhedral_artifacts/trellis.py:128-146.
@pytest.mark.parametrize("n,k", [(17408, 5120), (5120, 17408), (1024, 5120), (5120, 5120), (7168, 5120), (34816, 5120)])
def test_model_shapes(dev, n, k):
    rng = np.random.default_rng(0xE1)
    weights = (rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.02))
    blob = OC.q3_quantize(weights)
    for rows in (1, 3, 4, 5):
        x = random_x(np.random.default_rng(0xA0 + rows), rows, k)
        got = O.bf16_to_f32(run(dev, x, blob, n, k)).astype(np.float64)
        expect = OC.q3_linear(x, blob, n, k).astype(np.float64)
        assert max_relative_error(got, expect) <= 2e-3 + 2.0 ** -8


# Shapes that take every launch geometry of the decode kernel: tall tensors on the persistent grid (several tiles per warp
# in turn, a last cluster with a short share, an odd tile count), one K slice (no cluster) on the persistent grid, two K
# slices, an odd number of chunks per slice, few rows of tiles.
GRID_SHAPES = [(17424, 5120), (40000, 1024), (3088, 2048), (2000, 1536), (5120, 17408), (48, 4352), (9232, 8192)]  # (N, K)


@pytest.mark.parametrize("n,k", GRID_SHAPES)
def test_launch_geometries(dev, n, k):
    plan = library.decode_plan("q3", 5, k, n)
    assert plan["ctas"] % plan["k_slices"] == 0
    rng = np.random.default_rng(n * 31 + k)
    weights = rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.02)
    blob = OC.q3_quantize(weights)
    for rows in (1, 2, 5, 8):
        x = random_x(np.random.default_rng(0xB0 + rows), rows, k)
        got_bits = run(dev, x, blob, n, k)
        got = O.bf16_to_f32(got_bits).astype(np.float64)
        expect = OC.q3_linear(x, blob, n, k).astype(np.float64)
        assert max_relative_error(got, expect) <= 2e-3 + 2.0 ** -8, (rows, n, k)
        if rows == 5:   # every row of the call is the one-row call, bit for bit
            for r in (0, 4):
                assert np.array_equal(run(dev, x[r:r + 1], blob, n, k)[0], got_bits[r])



def test_every_fp16_scale_pattern(dev):
    """The FP16 group scale reaches the sum as its exact FP32 value for every finite bit pattern, subnormals and both
    zeros included (the reference pins its conversion over all 65,536 patterns, native/tests/test_q3_conversion.py:18-41;
    NaN payloads are the scalar oracle's business only, native/src/q3/contiguous.cuh:16-20). One row per pattern: a single
    code 1 under that scale against x = 1, so the output is bf16(f32(scale)) - on the decode kernel and on the scalar one
    (the scale -0 gives +0: every sum starts at +0)."""
    n, k = 65536, 128
    patterns = np.arange(n, dtype=np.uint16)
    finite = ((patterns >> 10) & 31) != 31
    codes = np.zeros((n, k), dtype=np.int8)
    codes[:, 0] = 1
    scales = np.zeros((n, 2), dtype=np.float16)
    scales[:, 0] = np.where(finite, patterns, 0).astype(np.uint16).view(np.float16)
    blob = np.frombuffer(O.q3_assemble(codes, scales, n, k), dtype=np.uint8).copy()
    x = np.zeros((1, k), dtype=np.uint16)
    x[0, 0] = 0x3F80   # 1.0
    expect = O.bf16_bits(scales[:, 0].astype(np.float32))
    expect[0x8000] = 0   # a sum that starts at +0 stays +0 when -0 is added
    for reference in (False, True):
        got = run(dev, x, blob, n, k, reference=reference)[0]
        wrong = np.flatnonzero(finite & (got != expect))
        assert wrong.size == 0, (reference, wrong.size, [(hex(int(i)), hex(int(got[i])), hex(int(expect[i]))) for i in wrong[:12]])
