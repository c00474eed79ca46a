"""Decode GEMV behaviour that spans both formats, through the C ABI: the grouped entry points against the single-tensor
ones (bitwise), the kernel's own error separated from the BF16 rounding of the output (one unit in the last place
against the rounded float64 result), a decode launch chained into a scalar-kernel launch under programmatic dependent
launch, and weights outside device memory."""

import ctypes as C

import numpy as np
import pytest

from euhedral_b200 import library
from oracle import oracle_c as OC
from oracle import oracle_np as O
from tests.gpu_util import Device, random_x

pytestmark = pytest.mark.gpu

QUANTIZE = {"q3": OC.q3_quantize, "nvfp4": OC.nvfp4_quantize}
DENSE = {"q3": OC.q3_dense, "nvfp4": OC.nvfp4_dense}


@pytest.fixture(scope="module")
def dev():
    device = Device()
    yield device
    assert device.gpu.take_device_error() == 0
    device.release()


def single(dev, fmt, d_x, d_w, size, rows, k, n, **select):
    select.setdefault("row_exact", True)   # 9 rows and more stay on the decode kernel (no native FP4 route)
    d_y = dev.empty(rows * n * 2)
    with dev.submit(**select) as gpu:
        call = gpu.linear_q3_bf16 if fmt == "q3" else gpu.linear_nvfp4_bf16
        call(d_x.data_ptr(), d_w.data_ptr(), d_y.data_ptr(), rows, k, n, size)
    return dev.get(d_y, np.uint16, (rows, n))


@pytest.mark.parametrize("fmt", ["q3", "nvfp4"])
@pytest.mark.parametrize("k,ns", [(5120, (640, 128, 128, 2176, 16)), (17408, (640, 272)), (1024, (48, 16, 4000)), (640, (32, 64))])
def test_group_is_bitwise_the_single_calls(dev, fmt, k, ns):
    rng = np.random.default_rng(k + len(ns))
    blobs = [QUANTIZE[fmt]((rng.standard_normal((n, k)) * 0.02).astype(np.float32)) for n in ns]
    d_w = [dev.put(blob) for blob in blobs]
    for rows in (1, 3, 5, 8, 11):
        xs = [random_x(rng, rows, k) for _ in range(2)]
        d_x = [dev.put(x) for x in xs]
        which = [i % 2 if i else 0 for i in range(len(ns))]     # the first two tensors share their input, then alternate
        d_y = [dev.empty(rows * n * 2) for n in ns]
        with dev.submit(pdl=True) as gpu:
            assert gpu.linear_group_bf16(fmt, [d_x[w].data_ptr() for w in which], [w.data_ptr() for w in d_w], [y.data_ptr() for y in d_y],
                                         rows, k, list(ns), [blob.size for blob in blobs])
        for i, n in enumerate(ns):
            grouped = dev.get(d_y[i], np.uint16, (rows, n))
            assert np.array_equal(grouped, single(dev, fmt, d_x[which[i]], d_w[i], blobs[i].size, rows, k, n)), (fmt, k, n, rows)


def test_group_of_more_than_eight_tensors_and_status_codes(dev):
    rng = np.random.default_rng(77)
    k, n, rows, count = 1024, 64, 2, 11
    blobs = [OC.q3_quantize((rng.standard_normal((n, k)) * 0.02).astype(np.float32)) for _ in range(count)]
    d_w = [dev.put(blob) for blob in blobs]
    d_x = dev.put(random_x(rng, rows, k))
    d_y = [dev.empty(rows * n * 2) for _ in range(count)]
    with dev.submit() as gpu:
        assert gpu.linear_group_bf16("q3", [d_x.data_ptr()] * count, [w.data_ptr() for w in d_w], [y.data_ptr() for y in d_y], rows, k,
                                     [n] * count, [blob.size for blob in blobs])
    for i in range(count):
        assert np.array_equal(dev.get(d_y[i], np.uint16, (rows, n)), single(dev, "q3", d_x, d_w[i], blobs[i].size, rows, k, n))
    lib = library.load()
    one = (C.c_void_p * 1)
    args = (one(d_x.data_ptr()), one(d_w[0].data_ptr()), one(d_y[0].data_ptr()))
    sizes = (C.c_uint64 * 1)(blobs[0].size)
    assert lib.euhedral_b200_linear_group_q3_bf16(0, *args, rows, k, (C.c_uint32 * 1)(n), sizes) == library.INVALID_ARGUMENT
    assert lib.euhedral_b200_linear_group_q3_bf16(1, *args, rows, k, (C.c_uint32 * 1)(n), (C.c_uint64 * 1)(5)) == library.FORMAT_MISMATCH
    assert lib.euhedral_b200_linear_group_q3_bf16(1, *args, 40, k, (C.c_uint32 * 1)(n), sizes) == library.ROUTE_UNAVAILABLE
    assert lib.euhedral_b200_linear_group_nvfp4_bf16(1, one(d_x.data_ptr() + 2), args[1], args[2], rows, k, (C.c_uint32 * 1)(n),
                                                     (C.c_uint64 * 1)(O.nvfp4_offsets(n, k)[2])) == library.INVALID_ARGUMENT


@pytest.mark.parametrize("fmt", ["q3", "nvfp4"])
@pytest.mark.parametrize("n,k", [(1024, 5120), (640, 17408)])
def test_output_is_within_one_ulp_of_the_rounded_float64_result(dev, fmt, n, k):
    """The output is BF16: where |y| is not tiny, the kernel's bits are those of bf16(float64 reference) or a neighbour,
    so the kernel's own error (FP32 accumulation) stays far inside the 2e-3 bound."""
    rng = np.random.default_rng(n + k)
    blob = QUANTIZE[fmt]((rng.standard_normal((n, k)) * 0.02).astype(np.float32))
    dense = DENSE[fmt](blob, n, k)
    d_w = dev.put(blob)
    for rows in (1, 4):
        x = random_x(rng, rows, k)
        got = single(dev, fmt, dev.put(x), d_w, blob.size, rows, k, n)
        expect = O.linear_f64(x, dense)
        rounded = O.bf16_bits(expect.astype(np.float32))
        large = np.abs(expect) >= 1e-2 * np.max(np.abs(expect))
        distance = np.abs(got.astype(np.int32) - rounded.astype(np.int32))
        assert np.all(distance[large] <= 1), (fmt, rows, int(distance[large].max()))
        # ... and almost always the very same bits: what is left of the 2e-3 bound after the output rounding (2^-9 at the
        # largest output) belongs to the kernel, whose own error is orders of magnitude below it
        assert np.mean(distance[large] == 0) >= 0.97, (fmt, rows, float(np.mean(distance[large] == 0)))
        kernel_error = np.max(np.abs(O.bf16_to_f32(got).astype(np.float64) - O.bf16_to_f32(rounded).astype(np.float64))[large]
                              / np.abs(expect[large]))
        assert kernel_error <= 2.0 ** -7   # one unit in the last place at most


def test_decode_then_scalar_kernel_under_dependent_launch(dev):
    """A scalar-kernel launch that reads what the decode launch before it wrote: with programmatic dependent launch
    selected the result is the same as without (the scalar kernels never start early)."""
    rng = np.random.default_rng(12)
    k, n, rows = 5120, 5120, 3
    first = OC.q3_quantize((rng.standard_normal((n, k)) * 0.02).astype(np.float32))
    second = OC.q3_quantize((rng.standard_normal((48, n)) * 0.02).astype(np.float32))
    d_a, d_b, d_x = dev.put(first), dev.put(second), dev.put(random_x(rng, rows, k))
    results = []
    for pdl in (False, True):
        d_mid, d_y = dev.empty(rows * n * 2, fill=0), dev.empty(rows * 48 * 2, fill=0)
        with dev.submit(pdl=pdl) as gpu:
            for _ in range(3):
                gpu.linear_q3_bf16(d_x.data_ptr(), d_a.data_ptr(), d_mid.data_ptr(), rows, k, n, first.size)
                gpu.linear_q3_reference_bf16(d_mid.data_ptr(), d_b.data_ptr(), d_y.data_ptr(), rows, n, 48, second.size)
        results.append(dev.get(d_y, np.uint16, (rows, 48)))
    assert np.array_equal(results[0], results[1])
    assert results[0].any()


@pytest.mark.parametrize("fmt", ["q3", "nvfp4"])
def test_host_mapped_weights_take_the_scalar_kernel(dev, fmt):
    """Weights in pinned host memory (the reference maps small tensors zero-copy for calls of up to 64 rows) are never
    given to a tensor map: the call runs the plain-load scalar kernel and gives its bits."""
    rng = np.random.default_rng(31)
    k, n, rows = 1024, 64, 2
    blob = QUANTIZE[fmt]((rng.standard_normal((n, k)) * 0.02).astype(np.float32))
    lib = library.load()
    host = lib.euhedral_cuda_host_malloc(blob.size)
    assert host
    try:
        C.memmove(host, blob.ctypes.data, blob.size)
        x = random_x(rng, rows, k)
        d_x, d_y = dev.put(x), dev.empty(rows * n * 2)
        with dev.submit() as gpu:
            call = gpu.linear_q3_bf16 if fmt == "q3" else gpu.linear_nvfp4_bf16
            call(d_x.data_ptr(), host, d_y.data_ptr(), rows, k, n, blob.size)
        got = dev.get(d_y, np.uint16, (rows, n))
        dev.gpu.select_exact_numerics(True)
        try:
            exact = single(dev, fmt, d_x, dev.put(blob), blob.size, rows, k, n)
        finally:
            dev.gpu.select_exact_numerics(False)
        assert np.array_equal(got, exact)
        one = C.c_void_p * 1
        with dev.submit():
            group = lib.euhedral_b200_linear_group_q3_bf16 if fmt == "q3" else lib.euhedral_b200_linear_group_nvfp4_bf16
            assert group(1, one(d_x.data_ptr()), one(host), one(d_y.data_ptr()), rows, k, (C.c_uint32 * 1)(n), (C.c_uint64 * 1)(blob.size)) \
                == library.ROUTE_UNAVAILABLE
    finally:
        dev.torch.cuda.synchronize()
        lib.euhedral_cuda_host_free(host)
