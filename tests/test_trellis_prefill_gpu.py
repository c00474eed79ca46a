"""Trellis prefill (rotate, decode to BF16, tcgen05 BF16 linear per segment, rotate back) as one call, and the BF16 epilogue
table entry, against the oracle's model of the reference's prefill plan."""

import ctypes as C

import numpy as np
import pytest

from euhedral_b200.gpu import KernelArguments
from oracle import oracle_np as O
from tests.gpu_util import Device, random_x
from tests.test_trellis_gpu import random_object

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    device = Device()
    yield device
    assert device.gpu.take_device_error() == 0
    device.release()


def prefill(dev, x_bits, payload, suh, svh, ends):
    lib = dev.gpu.lib
    rows, (kt, nt, w) = x_bits.shape[0], payload.shape
    k, n, s = kt * 16, nt * 16, len(ends)
    need = lib.euhedral_b200_prefill_trellis_scratch_bytes(rows, k, n, s)
    host_ends = (C.c_int32 * s)(*ends)
    d = [dev.put(x_bits), dev.put(payload.astype("<i2")), dev.put(suh.astype("<f2")), dev.put(svh.astype("<f2")),
         dev.put(np.array(ends, dtype="<i4"))]
    d_y, d_s = dev.empty(rows * n * 2), dev.empty(need, fill=0x5A)
    with dev.submit():
        status = lib.euhedral_b200_prefill_trellis_bf16(*[t.data_ptr() for t in d], C.cast(host_ends, C.c_void_p), d_y.data_ptr(), d_s.data_ptr(),
                                                        need, rows, k, n, w, s)
    assert status == 0, status
    return dev.get(d_y, np.uint16, (rows, n))


def close(got_bits, expect):
    """Both sides are rounded to BF16: where the kernel's FP32 sums and the model's float64 sums fall on different sides of a
    rounding boundary they differ by one BF16 step (2^-7 of the value at most); beyond that, the reference's own bound."""
    got = O.bf16_to_f32(got_bits).astype(np.float64)
    rms = float(np.sqrt(np.mean(expect.astype(np.float64) ** 2)))
    return np.all(np.abs(got - expect) <= 2.0 ** -7 * np.abs(expect) + 0.004 * rms)


@pytest.mark.parametrize("rows,k,n,w,ends", [
    (128, 256, 256, 48, [256]),              # one tile
    (300, 384, 640, 48, [640]),              # a ragged last row tile, a half-wide last column tile, six K steps
    (77, 256, 896, 40, [256, 384, 896]),     # three segments of 256, 128 and 512 columns, half-step rate
    (1100, 1024, 512, 64, [256, 512]),       # more tiles than one wave of a few SMs' worth, two segments
])
def test_against_the_plan_model(dev, rows, k, n, w, ends):
    rng = np.random.default_rng(rows + n)
    payload, suh, svh = random_object(rng, k, n, w, segments=len(ends))
    x = random_x(rng, rows, k)
    got = prefill(dev, x, payload, suh, svh, ends)
    expect = O.trellis_prefill_model(x, payload, suh, svh, ends)
    assert close(got, expect)
    # and, more loosely, the unrounded float64 linear (the BF16 roundings of the plan are what separates them)
    exact = O.trellis_linear_f64(x, payload, suh, svh, ends)
    rms = float(np.sqrt(np.mean(exact ** 2)))
    assert np.all(np.abs(O.bf16_to_f32(got).astype(np.float64) - exact) <= 0.02 * np.abs(exact) + 0.02 * rms)


def test_rows_do_not_depend_on_their_neighbours(dev):
    rng = np.random.default_rng(5)
    k, n, w = 256, 384, 48
    payload, suh, svh = random_object(rng, k, n, w)
    x = random_x(rng, 200, k)
    whole = prefill(dev, x, payload, suh, svh, [n])
    assert np.array_equal(prefill(dev, x[130:131], payload, suh, svh, [n]), whole[130:131])
    assert np.array_equal(prefill(dev, x[:9], payload, suh, svh, [n]), whole[:9])
    assert np.array_equal(prefill(dev, x, payload, suh, svh, [n]), whole)      # and twice the same bits


def test_epilogue_bf16_table_entry(dev):
    rng = np.random.default_rng(6)
    rows, n, ends = 5, 640, [128, 384, 640]
    svh = rng.uniform(0.01, 1.0, size=n).astype(np.float16)
    blocks = [O.bf16_bits(rng.standard_normal((rows, b - a)).astype(np.float32)) for a, b in zip([0] + ends[:-1], ends)]
    rotated = np.concatenate([b.reshape(-1) for b in blocks])                  # segment g at rows * start_g, row stride width_g
    d_r, d_e, d_v, d_y = dev.put(rotated), dev.put(np.array(ends, dtype="<i4")), dev.put(svh.view(np.uint16)), dev.empty(rows * n * 2)
    assert dev.gpu.table_kernel_available("TRELLIS_EPILOGUE_BF16")
    with dev.submit() as gpu:
        gpu.launch_table_kernel("TRELLIS_EPILOGUE_BF16", n // 128, rows, 1, 128, 1, 1, 0,
                                KernelArguments().pointer(d_r.data_ptr()).pointer(d_e.data_ptr()).int32(len(ends)).pointer(d_v.data_ptr())
                                .pointer(d_y.data_ptr()).int32(rows).int32(n))
    z = np.concatenate([O.bf16_to_f32(b) for b in blocks], axis=1)
    expect = O.bf16_bits(O.hadamard128(z) * svh.astype(np.float32))
    assert np.array_equal(dev.get(d_y, np.uint16, (rows, n)), expect)


def test_status_codes(dev):
    lib = dev.gpu.lib
    x, t = dev.empty(4096), dev.empty(1 << 20)
    ends = (C.c_int32 * 1)(256)
    ok = (x.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(), C.cast(ends, C.c_void_p), t.data_ptr(), t.data_ptr())
    assert lib.euhedral_b200_prefill_trellis_bf16(*ok, 1 << 20, 4, 256, 200, 48, 1) == -5        # out features not a multiple of 128
    assert lib.euhedral_b200_prefill_trellis_bf16(*ok, 1024, 4, 256, 256, 48, 1) == -2           # scratch too small
    bad = (C.c_int32 * 1)(128)
    assert lib.euhedral_b200_prefill_trellis_bf16(*ok[:5], C.cast(bad, C.c_void_p), *ok[6:], 1 << 20, 4, 256, 256, 48, 1) == -1   # ends stop short
    assert lib.euhedral_b200_prefill_trellis_scratch_bytes(4, 256, 256, 1) == 2048 + 131072


def test_bf16_linear_alone(dev):
    """The plan's BF16 linear by itself: FP32 sums of exact products, rounded once."""
    lib = dev.gpu.lib
    rng = np.random.default_rng(12)
    for rows, k, n in ((1, 64, 128), (130, 192, 384), (257, 512, 1152)):
        a, b = O.bf16_bits(rng.standard_normal((rows, k)).astype(np.float32)), O.bf16_bits(rng.standard_normal((n, k)).astype(np.float32))
        d_a, d_b, d_y = dev.put(a), dev.put(b), dev.empty(rows * n * 2)
        with dev.submit():
            assert lib.euhedral_b200_linear_bf16(d_a.data_ptr(), d_b.data_ptr(), d_y.data_ptr(), rows, k, n) == 0
        exact = O.bf16_to_f32(a).astype(np.float64) @ O.bf16_to_f32(b).astype(np.float64).T
        got = dev.get(d_y, np.uint16, (rows, n))
        same = got == O.bf16_bits(exact.astype(np.float32))
        assert same.mean() > 0.995                                   # FP32 accumulation against float64: a rounding boundary now and then
        assert np.all(np.abs(O.bf16_to_f32(got).astype(np.float64) - exact) <= 2.0 ** -8 * np.abs(exact) + 1e-4 * np.abs(exact).max())
    d = dev.empty(1 << 16)
    assert lib.euhedral_b200_linear_bf16(d.data_ptr(), d.data_ptr(), d.data_ptr(), 4, 96, 128) == -5
    assert lib.euhedral_b200_linear_bf16(d.data_ptr() + 2, d.data_ptr(), d.data_ptr(), 4, 64, 128) == -1


def test_operator_routes_many_rows_to_the_prefill(dev):
    """TrellisFormat.linear: beyond the tensor-core route's row limit and not row-exact, the operator runs the prefill plan."""
    from euhedral_b200.formats import LinearLaunch, TensorHandle, TrellisFormat, TrellisSettings
    rng = np.random.default_rng(31)
    rows, k, n, w, ends = 600, 256, 384, 48, [128, 384]
    payload, suh, svh = random_object(rng, k, n, w, segments=2)
    x = random_x(rng, rows, k)
    fmt = TrellisFormat(TrellisSettings(target_ctas=148))
    tensors = [dev.put(payload.astype("<i2")), dev.put(suh.astype("<f2")), dev.put(svh.astype("<f2")), dev.put(np.array(ends, dtype="<i4"))]
    shapes = [payload.shape, (2, k), (n,), (2,)]
    handles = [TensorHandle(f"t{i}", tuple(shape), t.data_ptr(), t.numel()) for i, (t, shape) in enumerate(zip(tensors, shapes))]
    need = fmt.scratch_bytes(dev.gpu, rows, k, n, 2, row_exact=False)
    assert need == dev.gpu.lib.euhedral_b200_prefill_trellis_scratch_bytes(rows, k, n, 2)
    d_x, d_y, d_s = dev.put(x), dev.empty(rows * n * 2), dev.empty(need)
    with dev.submit() as gpu:
        fmt.linear(gpu, LinearLaunch(d_x.data_ptr(), d_y.data_ptr(), handles, rows, k, n, scratch=d_s.data_ptr(), scratch_bytes=need, segment_ends=ends))
    assert np.array_equal(dev.get(d_y, np.uint16, (rows, n)), prefill(dev, x, payload, suh, svh, ends))
    with pytest.raises(ValueError):      # two segments: the plan needs their ends on the host
        with dev.submit() as gpu:
            fmt.linear(gpu, LinearLaunch(d_x.data_ptr(), d_y.data_ptr(), handles, rows, k, n, scratch=d_s.data_ptr(), scratch_bytes=need))
    # 64 rows and more that need not be row-exact run the plan too (the whole-K kernels of the reference are not carried);
    # fewer rows, and row-exact launches, stay on the tensor-core decode route
    whole = prefill(dev, x, payload, suh, svh, ends)
    for count, expect_plan in ((64, True), (63, False)):
        need = fmt.scratch_bytes(dev.gpu, count, k, n, 2, row_exact=False)
        d_s = dev.empty(need)
        with dev.submit() as gpu:
            fmt.linear(gpu, LinearLaunch(d_x.data_ptr(), d_y.data_ptr(), handles, count, k, n, scratch=d_s.data_ptr(), scratch_bytes=need, segment_ends=ends))
        got = dev.get(d_y, np.uint16, (rows, n))[:count]
        assert np.array_equal(got, whole[:count]) == expect_plan
        assert close(got, O.trellis_prefill_model(x[:count], payload, suh, svh, ends)) or not expect_plan


def test_gate_up_at_4096_rows_against_the_decode_route(dev):
    """Full size (the fused gate_up object, two segments, 4096 tokens): sampled rows of the prefill against the one-launch
    trellis linear on the same rows. The two routes round differently on the way (BF16 against FP16 activations and
    weights, BF16 products against FP32), so they agree to the reference's bound with the BF16 steps added, not to the bit."""
    import torch
    from euhedral_b200 import synthetic
    lib = dev.gpu.lib
    rows, k, n, w, ends = 4096, 5120, 34816, 48, [17408, 34816]
    payload, suh, svh, d_ends = synthetic.trellis_object(n, k, w, 77, 2, device="cuda")
    x = synthetic.bf16_rows(rows, k, 78, device="cuda")
    need = lib.euhedral_b200_prefill_trellis_scratch_bytes(rows, k, n, 2)
    scratch, y = torch.empty(need, dtype=torch.uint8, device="cuda"), torch.empty((rows, n), dtype=torch.int16, device="cuda")
    host_ends = (C.c_int32 * 2)(*ends)
    with dev.submit():
        assert lib.euhedral_b200_prefill_trellis_bf16(x.data_ptr(), payload.data_ptr(), suh.data_ptr(), svh.data_ptr(), d_ends.data_ptr(),
                                                      C.cast(host_ends, C.c_void_p), y.data_ptr(), scratch.data_ptr(), need, rows, k, n, w, 2) == 0
    sample = torch.tensor([0, 127, 128, 2500, 4095], device="cuda")
    xs = x[sample].contiguous()
    need2 = lib.euhedral_b200_linear_trellis_scratch_bytes(5, k, n, 2, 0)
    scratch2, y2 = torch.empty(max(need2, 256), dtype=torch.uint8, device="cuda"), torch.empty((5, n), dtype=torch.int16, device="cuda")
    with dev.submit():
        assert lib.euhedral_b200_linear_trellis_bf16(xs.data_ptr(), payload.data_ptr(), suh.data_ptr(), svh.data_ptr(), d_ends.data_ptr(), y2.data_ptr(),
                                                     scratch2.data_ptr(), need2, 5, k, n, w, 2, 0) == 0
    torch.cuda.synchronize()
    got = O.bf16_to_f32(y[sample].cpu().numpy().view(np.uint16)).astype(np.float64)
    decode = O.bf16_to_f32(y2.cpu().numpy().view(np.uint16)).astype(np.float64)
    rms = float(np.sqrt(np.mean(decode ** 2)))
    # BF16 weights and activations carry 2^-9 relative rounding each: about 0.002 rms of independent error per output, so the
    # largest of 174,080 differences sits near five of those; the root mean square is the sharper statement
    assert np.all(np.abs(got - decode) <= 2.0 ** -6 * np.abs(decode) + 0.02 * rms)
    assert np.sqrt(np.mean((got - decode) ** 2)) < 0.004 * rms


def test_cta_pairs_give_the_single_cta_bits(dev):
    """Calls of 512 rows and more run the BF16 linear on CTA pairs; the K order and the accumulation are the same."""
    lib = dev.gpu.lib
    rng = np.random.default_rng(51)
    for rows, k, n, w, ends in ((600, 256, 640, 48, [640]), (1100, 512, 896, 48, [256, 384, 896])):
        payload, suh, svh = random_object(rng, k, n, w, segments=len(ends))
        x = random_x(rng, rows, k)
        pairs = prefill(dev, x, payload, suh, svh, ends)
        lib.euhedral_b200_select_bf16_pairs(0)
        try:
            single = prefill(dev, x, payload, suh, svh, ends)
        finally:
            lib.euhedral_b200_select_bf16_pairs(1)
        assert np.array_equal(pairs, single)
        assert close(pairs, O.trellis_prefill_model(x, payload, suh, svh, ends))


def test_column_shards_equal_the_whole(dev):
    """N-sharding for several GPUs: a shard of the object's output columns (the reference's rows() operator cuts on segment
    boundaries) run as a self-contained object gives the whole object's columns bit for bit - every 128-column block is one
    FP32 sum over K per row, whatever stands beside it."""
    from euhedral_b200 import sharding
    rng = np.random.default_rng(61)
    rows, k, n, w, ends = 530, 384, 1024, 48, [256, 512, 768, 1024]
    payload, suh, svh = random_object(rng, k, n, w, segments=4)
    x = random_x(rng, rows, k)
    whole = prefill(dev, x, payload, suh, svh, ends)
    parts = []
    for first, count in ((0, 256), (256, 512), (768, 256)):      # one segment, two segments, the last segment
        p, s, v, e = sharding.trellis_rows(payload, suh, svh, ends, first, count)
        parts.append(prefill(dev, x, p, s, v, [int(end) for end in e]))
    assert np.array_equal(np.concatenate(parts, axis=1), whole)
