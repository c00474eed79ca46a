"""NVFP4 tensors with table-indexed block scales (layout row-split-k128-sd4-v1; the reference's `_sd4` twin kernels,
native/src/nvfp4/scale_table.cuh:4-15, native/src/host/nvfp4_linear.c:17-19) through the C ABI. A block's scale IS its
table entry, so such a tensor and the plain tensor with every entry written out hold the same values and the kernels sum
them in the same order: every route must give the plain twin's bits."""

import ctypes as C

import numpy as np
import pytest

from euhedral_b200 import layouts, library, sharding
from oracle import oracle_c as OC
from oracle import oracle_np as O
from tests.gpu_util import Device, max_relative_error, random_x

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    device = Device()
    yield device
    assert device.gpu.take_device_error() == 0
    device.release()


def twins(rng, n, k):
    """(table-indexed tensor, its plain twin) as byte arrays."""
    plain = OC.nvfp4_quantize((rng.standard_normal((n, k)) * rng.uniform(0.01, 1.0, (n, 1))).astype(np.float32))
    indexed = O.nvfp4_sd4_from_plain(plain.tobytes(), n, k, rng)
    twin = O.nvfp4_sd4_to_plain(indexed, n, k)
    return np.frombuffer(indexed, dtype=np.uint8).copy(), np.frombuffer(twin, dtype=np.uint8).copy()


def run(dev, x_bits, blob, n, k, **select):
    rows = x_bits.shape[0]
    d_x, d_w, d_y = dev.put(x_bits), dev.put(blob), dev.empty(rows * n * 2)
    with dev.submit(**select) as gpu:
        gpu.linear_nvfp4_bf16(d_x.data_ptr(), d_w.data_ptr(), d_y.data_ptr(), rows, k, n, blob.size)
    return dev.get(d_y, np.uint16, (rows, n))


@pytest.mark.parametrize("n,k", [(1024, 5120), (640, 17408), (48, 1024), (5120, 5120), (2176, 640)])
def test_decode_gives_the_plain_twin_bits(dev, n, k):
    rng = np.random.default_rng(n + k)
    indexed, twin = twins(rng, n, k)
    assert indexed.size == O.nvfp4_sd4_offsets(n, k)[2] != twin.size
    for rows in (1, 3, 5, 8, 11):
        x = random_x(rng, rows, k)
        got = run(dev, x, indexed, n, k, row_exact=True)
        assert np.array_equal(got, run(dev, x, twin, n, k, row_exact=True)), (n, k, rows)
    x = random_x(rng, 4, k)
    expect = OC.nvfp4_linear(x, twin, n, k).astype(np.float64)
    assert max_relative_error(O.bf16_to_f32(run(dev, x, indexed, n, k)).astype(np.float64), expect) <= 2e-3 + 2.0 ** -8


def test_scalar_kernel_and_odd_shapes(dev):
    rng = np.random.default_rng(8)
    for n, k in ((40, 96), (64, 1024)):          # K not a multiple of 128: scalar kernel; then exact numerics on a decode shape
        indexed, twin = twins(rng, n, k)
        x = random_x(rng, 3, k)
        dev.gpu.select_exact_numerics(True)
        try:
            exact = run(dev, x, indexed, n, k)
            assert np.array_equal(exact, run(dev, x, twin, n, k))
        finally:
            dev.gpu.select_exact_numerics(False)
        assert np.array_equal(exact, O.nvfp4_linear_scalar_kernel(x, twin.tobytes(), n, k))


def test_group_and_native_route(dev):
    rng = np.random.default_rng(9)
    k, ns, rows = 5120, (640, 128, 2176), 5
    pairs = [twins(rng, n, k) for n in ns]
    x = random_x(rng, rows, k)
    d_x = dev.put(x)
    d_w = [dev.put(indexed) for indexed, _ in pairs]
    d_y = [dev.empty(rows * n * 2) for n in ns]
    with dev.submit(pdl=True) as gpu:
        assert gpu.linear_group_bf16("nvfp4", [d_x.data_ptr()] * len(ns), [w.data_ptr() for w in d_w], [y.data_ptr() for y in d_y], rows, k,
                                     list(ns), [indexed.size for indexed, _ in pairs])
    for i, n in enumerate(ns):
        assert np.array_equal(dev.get(d_y[i], np.uint16, (rows, n)), run(dev, x, pairs[i][1], n, k, row_exact=True))
    # the tcgen05 route: the scale repack looks the indices up, the GEMM is the same
    lib = dev.gpu.lib
    n, k, rows = 1280, 1024, 300
    indexed, twin = twins(rng, n, k)
    x = random_x(rng, rows, k)
    need = lib.euhedral_cuda_nvfp4_native_scratch_bytes(rows, k, n)
    outputs = []
    for blob in (indexed, twin):
        d_x, d_w, d_y, d_s = dev.put(x), dev.put(blob), dev.empty(rows * n * 2), dev.empty(need)
        with dev.submit(pdl=True):
            assert lib.euhedral_cuda_linear_nvfp4_native_bf16(d_x.data_ptr(), d_w.data_ptr(), d_y.data_ptr(), d_s.data_ptr(), rows, k, n,
                                                              blob.size, need) == 0
        outputs.append(dev.get(d_y, np.uint16, (rows, n)))
    assert np.array_equal(outputs[0], outputs[1]) and outputs[0].any()
    # a size that is neither layout is refused
    d_x, d_w, d_y = dev.put(x), dev.put(indexed), dev.empty(rows * n * 2)
    with dev.submit():
        assert lib.euhedral_cuda_linear_nvfp4_bf16(d_x.data_ptr(), d_w.data_ptr(), d_y.data_ptr(), 2, k, n, indexed.size + 4) == library.FORMAT_MISMATCH


def test_row_shards_equal_the_whole(dev):
    rng = np.random.default_rng(10)
    n, k = 1024, 5120
    indexed, _ = twins(rng, n, k)
    assert indexed.size == layouts.nvfp4_sd4_byte_size(n, k)
    x = random_x(rng, 5, k)
    whole = run(dev, x, indexed, n, k)
    parts = [run(dev, x, sharding.nvfp4_sd4_rows(indexed, n, k, s * n // 4, n // 4), n // 4, k) for s in range(4)]
    assert np.array_equal(np.concatenate(parts, axis=1), whole)
