"""Q3 prefill (two exact BF16 terms per weight through the tcgen05 BF16 GEMM) behind the reference's Q3 MX entry points,
against float64 on exact products (the reference's own criterion, native/tests/test_q3_mx.py: the route agrees with
FP64 to the BF16 output rounding)."""

import numpy as np
import pytest

from oracle import oracle_np as O
from tests.gpu_util import Device, random_x
from tests.test_q3_gpu import random_tensor

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    device = Device()
    yield device
    assert device.gpu.take_device_error() == 0
    device.release()


def prefill(dev, x_bits, blob, n, k, paired=False, **select):
    lib = dev.gpu.lib
    rows = x_bits.shape[0]
    need = lib.euhedral_cuda_q3_mx_scratch_bytes(rows, k, n)
    width = n // 2 if paired else n
    d_x, d_w, d_y, d_s = dev.put(x_bits), dev.put(blob), dev.empty(rows * width * 2), dev.empty(need, fill=0x3C)
    entry = lib.euhedral_cuda_q3_mx_gate_up_swiglu_bf16 if paired else lib.euhedral_cuda_linear_q3_mx_bf16
    with dev.submit(**select):
        status = entry(d_x.data_ptr(), d_w.data_ptr(), d_y.data_ptr(), d_s.data_ptr(), rows, k, n, blob.size, need)
    if status != 0:
        return status
    return dev.get(d_y, np.uint16, (rows, width))


@pytest.mark.parametrize("rows,k,n", [(33, 128, 128), (200, 512, 384), (130, 1024, 1152), (1030, 256, 640)])
def test_against_float64(dev, rows, k, n):
    rng = np.random.default_rng(rows + k)
    blob, dense = random_tensor(rng, n, k)
    x = random_x(rng, rows, k)
    assert dev.gpu.lib.euhedral_cuda_q3_mx_available() == 1
    got = prefill(dev, x, blob, n, k)
    exact = O.linear_f64(x, dense)
    # sums of exact products in FP32, one rounding to BF16: equal to the rounded float64 result, or a BF16 step away where
    # the FP32 sum and the float64 sum fall on different sides of a rounding boundary
    same = got == O.bf16_bits(exact.astype(np.float32))
    assert same.mean() > 0.99, same.mean()
    scale = np.abs(exact).max(axis=1, keepdims=True)
    assert np.all(np.abs(O.bf16_to_f32(got).astype(np.float64) - exact) <= 2.0 ** -8 * np.abs(exact) + 1e-5 * scale)


def test_rows_do_not_depend_on_their_neighbours(dev):
    rng = np.random.default_rng(3)
    k, n = 512, 256
    blob, _ = random_tensor(rng, n, k)
    x = random_x(rng, 140, k)
    whole = prefill(dev, x, blob, n, k)
    assert np.array_equal(prefill(dev, x[100:139], blob, n, k), whole[100:139])
    # a chunk of the output rows of the tensor gives the whole tensor's bits (select_split_rows has nothing to fix)
    dev.gpu.lib.euhedral_cuda_q3_mx_select_split_rows(n)
    half_blob, _ = slice_rows(blob, n, k, 128, 128)
    assert np.array_equal(prefill(dev, x, half_blob, 128, k), whole[:, 128:])
    dev.gpu.lib.euhedral_cuda_q3_mx_select_split_rows(0)


def slice_rows(blob, n, k, first, count):
    codes, scales = O.q3_unpack(blob.tobytes(), n, k)
    part = np.frombuffer(O.q3_assemble(codes[first:first + count], scales[first:first + count], count, k), dtype=np.uint8).copy()
    return part, O.q3_dense(part.tobytes(), count, k)


def test_gate_up_swiglu(dev):
    rng = np.random.default_rng(8)
    rows, k, outputs = 150, 384, 768                     # 384 SwiGLU columns: three paired tiles
    blob, dense = random_tensor(rng, outputs, k)
    dense = dense * 0.05                                  # keep the gate in the range where SiLU bends
    codes, scales = O.q3_unpack(blob.tobytes(), outputs, k)
    blob = np.frombuffer(O.q3_assemble(codes, (scales.astype(np.float32) * 0.05).astype(np.float16), outputs, k), dtype=np.uint8).copy()
    dense = O.q3_dense(blob.tobytes(), outputs, k)
    x = random_x(rng, rows, k)
    got = prefill(dev, x, blob, outputs, k, paired=True)
    plain = prefill(dev, x, blob, outputs, k)
    gate, up = O.bf16_to_f32(plain[:, :outputs // 2]), O.bf16_to_f32(plain[:, outputs // 2:])
    with np.errstate(over="ignore"):                                           # a gate of -3500 (the crafted scale): exp overflows to inf, SiLU to -0
        expect = (gate / (1.0 + np.exp(-gate.astype(np.float64)))) * up      # on the plain route's own BF16 gate and up
    same = got == O.bf16_bits(expect.astype(np.float32))
    assert same.mean() > 0.99
    assert np.all(np.abs(O.bf16_to_f32(got).astype(np.float64) - expect) <= 2.0 ** -7 * np.abs(expect) + 1e-30)


def test_statuses(dev):
    lib = dev.gpu.lib
    rng = np.random.default_rng(1)
    blob, _ = random_tensor(rng, 128, 128)
    x = random_x(rng, 40, 128)
    assert prefill(dev, x, blob, 128, 128, row_exact=True) == -5          # row-exact execution declines the route
    assert prefill(dev, x[:32], blob, 128, 128) == -5                     # 32 rows and fewer belong to the decode kernels
    assert not isinstance(prefill(dev, x[:33], blob, 128, 128), int)
    d = dev.empty(1 << 20)
    p = d.data_ptr()
    assert lib.euhedral_cuda_linear_q3_mx_bf16(p, p, p, p, 40, 128, 128, blob.size - 1, 1 << 20) == -3      # not the tensor's size
    assert lib.euhedral_cuda_linear_q3_mx_bf16(p, p, p, p, 40, 128, 128, blob.size, 1024) == -2             # scratch too small
    assert lib.euhedral_cuda_q3_mx_scratch_bytes(9, 128, 128) == 128 * 128 * 4
    small, _ = random_tensor(rng, 64, 128)
    assert lib.euhedral_cuda_linear_q3_mx_bf16(p, p, p, p, 40, 128, 64, small.size, 1 << 20) == -5          # weight rows not a multiple of 128
    previous = lib.euhedral_cuda_select_exact_numerics(1)
    try:
        assert prefill(dev, x, blob, 128, 128) == -5
    finally:
        lib.euhedral_cuda_select_exact_numerics(previous)


def test_operator_routes_by_row_count(dev):
    """GroupedLinearFormat.linear / CudaGpuMemory.linear_q3_bf16: more than 8 rows try the prefill route; it takes 33 rows and
    more, and leaves fewer rows, row-exact launches and shapes it declines to the decode kernels."""
    from euhedral_b200.formats import GroupedLinearFormat, LinearLaunch, TensorHandle
    rng = np.random.default_rng(41)
    rows, k, n = 40, 256, 256
    blob, _ = random_tensor(rng, n, k)
    x = random_x(rng, rows, k)
    d_x, d_w, d_y = dev.put(x), dev.put(blob), dev.empty(rows * n * 2)
    handle = TensorHandle("w", (n, k), d_w.data_ptr(), blob.size)
    with dev.submit() as gpu:
        GroupedLinearFormat().linear(gpu, LinearLaunch(d_x.data_ptr(), d_y.data_ptr(), [handle], rows, k, n))
    assert np.array_equal(dev.get(d_y, np.uint16, (rows, n)), prefill(dev, x, blob, n, k))
    # 24 rows: the prefill entry declines, the decode kernels run them as groups of 8, each row bitwise its one-row call
    for select in ({}, {"row_exact": True}):
        with dev.submit(**select) as gpu:
            GroupedLinearFormat().linear(gpu, LinearLaunch(d_x.data_ptr(), d_y.data_ptr(), [handle], 24, k, n))
        many = dev.get(d_y, np.uint16, (rows, n))[:24].copy()
        with dev.submit() as gpu:
            gpu.linear_q3_bf16(d_x.data_ptr() + 7 * k * 2, d_w.data_ptr(), d_y.data_ptr(), 1, k, n, blob.size)
        assert np.array_equal(dev.get(d_y, np.uint16, (rows, n))[0], many[7])


@pytest.mark.parametrize("n,k", [(17408, 5120), (5120, 17408)])
def test_model_shapes_at_4096_rows(dev, n, k):
    """Full size (gate and down at 4096 tokens): sampled rows against the FP32-accumulated C oracle, and against the decode
    kernel on the same rows - two independent sums of the same exact products, a BF16 step apart at most."""
    from oracle import oracle_c as OC
    from tests.test_q3_gpu import run
    rng = np.random.default_rng(0xE2)
    weights = (rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.02))
    blob = OC.q3_quantize(weights)
    x = random_x(np.random.default_rng(0xA9), 4096, k)
    got = prefill(dev, x, blob, n, k)
    sample = np.array([0, 1, 127, 128, 2049, 3000, 4094, 4095])
    expect = OC.q3_linear(x[sample], blob, n, k).astype(np.float64)
    g = O.bf16_to_f32(got[sample]).astype(np.float64)
    scale = np.abs(expect).max(axis=1, keepdims=True)
    assert np.all(np.abs(g - expect) <= 2.0 ** -8 * np.abs(expect) + 2e-5 * scale)
    decode = O.bf16_to_f32(run(dev, x[sample], blob, n, k)).astype(np.float64)
    assert np.all(np.abs(g - decode) <= 2.0 ** -7 * np.abs(decode) + 2e-5 * scale)
    assert (got[sample] == run(dev, x[sample], blob, n, k)).mean() > 0.97


def test_cta_pairs_give_the_single_cta_bits(dev):
    lib = dev.gpu.lib
    rng = np.random.default_rng(52)
    rows, k, n = 700, 384, 768
    blob, _ = random_tensor(rng, n, k)
    x = random_x(rng, rows, k)
    pairs, pairs_swiglu = prefill(dev, x, blob, n, k), prefill(dev, x, blob, n, k, paired=True)
    lib.euhedral_b200_select_bf16_pairs(0)
    try:
        assert np.array_equal(prefill(dev, x, blob, n, k), pairs)
        assert np.array_equal(prefill(dev, x, blob, n, k, paired=True), pairs_swiglu)
    finally:
        lib.euhedral_b200_select_bf16_pairs(1)
