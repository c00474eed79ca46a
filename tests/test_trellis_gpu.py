"""Trellis linear (prepass, tensor-core GEMM, epilogue, decode, scalar kernel) through the kernel-table ABI against
the oracle (modelled on native/tests/test_trellis.py)."""

import numpy as np
import pytest

from euhedral_b200 import layouts, sharding
from euhedral_b200.formats import LinearLaunch, TensorHandle, TrellisFormat, TrellisSettings
from euhedral_b200.gpu import KernelArguments
from oracle import oracle_c as OC
from oracle import oracle_np as O
from tests.gpu_util import Device, random_x

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    device = Device()
    yield device
    assert device.gpu.take_device_error() == 0
    device.release()


def random_object(rng, k, n, w, segments=1, scale=1.0):
    payload = rng.integers(-32768, 32768, size=(k // 16, n // 16, w), dtype=np.int16)
    suh = (rng.choice([-1.0, 1.0], size=(segments, k)) * rng.uniform(0.5, 2.0, size=(segments, k))).astype(np.float16)
    svh = (rng.uniform(0.01, 1.0, size=n) * scale).astype(np.float16)
    return payload, suh, svh


class DeviceLinear:
    def __init__(self, dev, payload, suh, svh, ends, target_ctas):
        self.dev = dev
        self.kt, self.nt, self.w = payload.shape
        self.k, self.n, self.ends = self.kt * 16, self.nt * 16, list(ends)
        layouts.trellis_validate_segments(self.ends, self.n)
        self.format = TrellisFormat(TrellisSettings(target_ctas=target_ctas))
        self.tensors = [dev.put(payload.astype("<i2")), dev.put(suh.astype("<f2")), dev.put(svh.astype("<f2")),
                        dev.put(np.array(self.ends, dtype="<i4"))]
        shapes = [payload.shape, (len(self.ends), self.k), (self.n,), (len(self.ends),)]
        self.handles = [TensorHandle(f"t{i}", tuple(shape), t.data_ptr(), t.numel()) for i, (t, shape) in enumerate(zip(self.tensors, shapes))]

    def linear(self, x_bits, **select):
        rows = x_bits.shape[0]
        need = self.format.scratch_bytes(self.dev.gpu, rows, self.k, self.n, len(self.ends))
        d_x, d_y, d_s = self.dev.put(x_bits), self.dev.empty(rows * self.n * 2), self.dev.empty(need)
        launch = LinearLaunch(d_x.data_ptr(), d_y.data_ptr(), self.handles, rows, self.k, self.n, scratch=d_s.data_ptr(),
                              scratch_bytes=need, row_exact=True)
        with self.dev.submit(**select) as gpu:
            self.format.linear(gpu, launch)
        return self.dev.get(d_y, np.uint16, (rows, self.n))

    def one_call(self, x_bits, splits, **select):
        """The same linear as ONE launch (euhedral_b200_linear_trellis_bf16) with the split count given."""
        rows = x_bits.shape[0]
        need = self.dev.gpu.lib.euhedral_b200_linear_trellis_scratch_bytes(rows, self.k, self.n, len(self.ends), splits)
        d_x, d_y, d_s = self.dev.put(x_bits), self.dev.empty(rows * self.n * 2), self.dev.empty(max(need, 256), fill=0xA5)
        with self.dev.submit(**select) as gpu:
            gpu.linear_trellis_bf16(d_x.data_ptr(), *[t.data_ptr() for t in self.tensors[:3]], self.tensors[3].data_ptr(), d_y.data_ptr(),
                                    d_s.data_ptr(), need, rows, self.k, self.n, self.w, len(self.ends), splits)
        return self.dev.get(d_y, np.uint16, (rows, self.n))


def within_kernel_tolerance(got_bits, expect):
    """native/tests/test_trellis.py:157-165."""
    got = O.bf16_to_f32(got_bits).astype(np.float64)
    rms = float(np.sqrt(np.mean(expect ** 2)))
    return np.all(np.abs(got - expect) <= 0.004 * np.abs(expect) + 0.004 * rms)


@pytest.mark.parametrize("w", [16, 24, 32, 40, 48, 56, 64, 72, 80, 88, 96, 104, 112, 120, 128])
def test_decode_bf16_bitwise(dev, w):
    rng = np.random.default_rng(w)
    k, n = 128, 256
    payload, _, _ = random_object(rng, k, n, w)
    d_words, d_out = dev.put(payload.astype("<i2")), dev.empty(n * k * 2)
    with dev.submit() as gpu:
        gpu.launch_table_kernel("TRELLIS_DECODE_BF16", (k // 16) * (n // 16), 1, 1, 256, 1, 1, 0,
                                KernelArguments().pointer(d_words.data_ptr()).pointer(d_out.data_ptr()).int32(k).int32(n).int32(w))
    got = dev.get(d_out, np.uint16, (n, k))
    assert np.array_equal(got, O.bf16_bits(O.trellis_rotated_weight(payload).astype(np.float32).T))


@pytest.mark.parametrize("rows,k,s", [(3, 1024, 2), (203, 384, 3)])     # few rows: a warp per block; many: a thread per block
def test_prepass_bitwise(dev, rows, k, s):
    rng = np.random.default_rng(3)
    x = random_x(rng, rows, k)
    suh = (rng.choice([-1.0, 1.0], size=(s, k)) * rng.uniform(0.5, 2.0, size=(s, k))).astype(np.float16)
    d_x, d_suh, d_out = dev.put(x), dev.put(suh), dev.empty(s * rows * k * 2)
    for layout in (0, 1):
        with dev.submit() as gpu:
            gpu.launch_table_kernel("TRELLIS_PREPASS", (k + 511) // 512, rows, s, 128, 1, 1, 0,
                                    KernelArguments().pointer(d_x.data_ptr()).pointer(d_suh.data_ptr()).pointer(d_out.data_ptr())
                                    .int32(rows).int32(k).int32(s).int32(layout))
        got = dev.get(d_out, np.uint16, (s, rows, k))
        if layout == 0:
            expect = O.trellis_fragment_order(O.trellis_prepass(x, suh).view(np.uint16))
        else:
            rotated = O.hadamard128((O.bf16_to_f32(x)[None] * suh.astype(np.float32)[:, None, :]).astype(np.float32))
            expect = O.bf16_bits(rotated)
        assert np.array_equal(got, expect), layout


@pytest.mark.parametrize("w", [16, 24, 32, 40, 48, 56, 64, 72, 80, 88, 96, 104, 112, 120, 128])   # every stored width: every lane decoder
@pytest.mark.parametrize("target", [8, 140])
def test_tensor_core_route_matches_float64(dev, w, target):
    rng = np.random.default_rng(w + target)
    k, n = 1024, 512
    payload, suh, svh = random_object(rng, k, n, w, segments=2)
    linear = DeviceLinear(dev, payload, suh, svh, [256, 512], target)
    splits = TrellisFormat.splits(k, n, target)
    for rows in (1, 5, 8, 13, 40):
        x = random_x(rng, rows, k)
        expect = O.trellis_linear_f64(x, payload, suh, svh, [256, 512])
        got = linear.linear(x)
        assert within_kernel_tolerance(got, expect), (w, target, rows)
        if rows in (5, 13):
            assert np.array_equal(linear.one_call(x, splits), got), (w, target, rows)   # one launch: the same bits


# The layer's projection shapes (N x K) at the model's stored widths, one and two segments, through the operator's own
# launch plan for this device (K splits of 20, 20, 9 and 30 at 148 SMs: a split's tile rows are not a multiple of the 16
# the streaming stage holds, so stages reach past their split), against the plain-C restatement of the reference's
# linear (native/src/reference/trellis.cuh:14-55) within the reference's kernel tolerance.
@pytest.mark.parametrize("n,k", [(5120, 5120), (1024, 5120), (17408, 5120), (5120, 17408)])
@pytest.mark.parametrize("w", [40, 48, 56, 64])
def test_layer_shapes(dev, n, k, w):
    rng = np.random.default_rng(n + k + w)
    segments = 1 + (w // 8) % 2                       # 40, 56: two segments; 48, 64: one
    ends = [n] if segments == 1 else [n // 2, n]
    payload, suh, svh = random_object(rng, k, n, w, segments=segments)
    linear = DeviceLinear(dev, payload, suh, svh, ends, 8 * dev.gpu.multiprocessor_count())
    splits = TrellisFormat.splits(k, n, 8 * dev.gpu.multiprocessor_count())
    for rows in (1, 5):
        x = random_x(rng, rows, k)
        expect = OC.trellis_linear(x, payload, suh, svh, ends).astype(np.float64)
        got = linear.linear(x)
        assert within_kernel_tolerance(got, expect), (n, k, w, rows)
        assert np.array_equal(linear.one_call(x, splits, pdl=True), got), (n, k, w, rows)   # one launch, the same bits


def test_one_call_linear_is_bitwise_the_table_launches(dev):
    """The one-launch linear (activations rotated inside the kernel, splits joined by whoever finishes last) against the
    three table launches a host plans one by one."""
    rng = np.random.default_rng(44)
    k, n, w = 2048, 512, 48
    payload, suh, svh = random_object(rng, k, n, w, segments=2)
    ends = [256, 512]
    lib = dev.gpu.lib
    for target, rows in ((8, 3), (140, 5), (140, 1), (1, 7), (1, 20), (30, 13), (64, 40)):
        table = DeviceLinear(dev, payload, suh, svh, ends, target)
        x = random_x(rng, rows, k)
        expect = table.linear(x)
        splits = TrellisFormat.splits(k, n, target)
        assert np.array_equal(table.one_call(x, splits), expect), (target, rows)
        need = lib.euhedral_b200_linear_trellis_scratch_bytes(rows, k, n, 2, splits)
        # a flag per block and split, then the partials; nothing with one split
        assert need == (((n // 128 * splits * 8 + 255) & ~255) + splits * rows * n * 4 if splits > 1 else 0)
        d_x, d_y, d_s = dev.put(x), dev.empty(rows * n * 2), dev.empty(need)
        with dev.submit(pdl=True) as gpu:
            gpu.linear_trellis_bf16(d_x.data_ptr(), *[t.data_ptr() for t in table.tensors[:3]], table.tensors[3].data_ptr(), d_y.data_ptr(),
                                    d_s.data_ptr(), need, rows, k, n, w, 2, splits)
        assert np.array_equal(dev.get(d_y, np.uint16, (rows, n)), expect)
    # splits = 0 takes the device's default split count; a scratch that is too small is refused
    need = lib.euhedral_b200_linear_trellis_scratch_bytes(2, k, n, 2, 0)
    d_x, d_y, d_s = dev.put(random_x(rng, 2, k)), dev.empty(2 * n * 2), dev.empty(need)
    t = [h.data_ptr() for h in table.tensors]
    with dev.submit():
        assert lib.euhedral_b200_linear_trellis_bf16(d_x.data_ptr(), t[0], t[1], t[2], t[3], d_y.data_ptr(), d_s.data_ptr(), need, 2, k, n, w, 2, 0) == 0
        assert lib.euhedral_b200_linear_trellis_bf16(d_x.data_ptr(), t[0], t[1], t[2], t[3], d_y.data_ptr(), d_s.data_ptr(), 1024, 2, k, n, w, 2, 0) == -2


def test_golden_linear_fixture(dev, golden):
    g = golden("trellis")
    linear = DeviceLinear(dev, g["linear_payload"], g["linear_suh"], g["linear_svh"], [256], 140)
    assert within_kernel_tolerance(linear.linear(g["linear_x"]), g["linear_y_f64"])
    two = DeviceLinear(dev, g["seg_payload"], g["seg_suh"], g["seg_svh"], list(g["seg_ends"]), 8)
    assert within_kernel_tolerance(two.linear(g["seg_x"]), g["seg_y_f64"])


def test_rows_are_bitwise_independent(dev):
    rng = np.random.default_rng(21)
    k, n, w = 1024, 256, 48
    payload, suh, svh = random_object(rng, k, n, w)
    for target in (2, 64):
        linear = DeviceLinear(dev, payload, suh, svh, [n], target)
        x = random_x(rng, 33, k)
        single = np.concatenate([linear.linear(x[r:r + 1]) for r in (0, 1, 7, 8, 32)])
        for rows in (2, 8, 9, 33):
            got = linear.linear(x[:rows])
            for at, r in enumerate((0, 1, 7, 8, 32)):
                if r < rows:
                    assert np.array_equal(got[r], single[at]), (target, rows, r)
        assert np.array_equal(linear.linear(x[:5], pdl=True), linear.linear(x[:5]))


def test_scalar_kernel_matches_float64(dev):
    rng = np.random.default_rng(22)
    k, n, w = 256, 256, 40
    payload, suh, svh = random_object(rng, k, n, w, segments=2)
    linear = DeviceLinear(dev, payload, suh, svh, [128, 256], 8)
    x = random_x(rng, 2, k)
    dev.gpu.select_exact_numerics(True)
    try:
        got = O.bf16_to_f32(linear.linear(x)).astype(np.float64)
    finally:
        dev.gpu.select_exact_numerics(False)
    expect = O.trellis_linear_f64(x, payload, suh, svh, [128, 256])
    assert np.all(np.abs(got - expect) <= np.abs(expect) * 2.0 ** -7 + np.max(np.abs(expect)) * 1e-3)


def test_column_shards_equal_the_whole(dev):
    """Cut at a segment boundary, with the K split fixed from the whole object's shape, a shard's columns are bitwise
    the whole object's."""
    rng = np.random.default_rng(23)
    k, n, w = 1024, 512, 48
    payload, suh, svh = random_object(rng, k, n, w, segments=2)
    ends = [256, 512]
    x = random_x(rng, 5, k)
    whole_splits = TrellisFormat.splits(k, n, 64)
    whole = DeviceLinear(dev, payload, suh, svh, ends, 64).linear(x)
    parts = []
    for first in (0, 256):
        p, s, v, e = sharding.trellis_rows(payload, suh, svh, ends, first, 256)
        # target chosen so that the shard's split count equals the whole object's
        shard = DeviceLinear(dev, p, s, v, e, whole_splits * (256 // 128))
        assert TrellisFormat.splits(k, 256, whole_splits * 2) == whole_splits
        parts.append(shard.linear(x))
    assert np.array_equal(np.concatenate(parts, axis=1), whole)


def test_table_abi(dev):
    lib = dev.gpu.lib
    names = [lib.euhedral_cuda_linear_kernel_name(i).decode() for i in range(lib.euhedral_cuda_linear_kernel_count())]
    assert names[:2] == ["euhedral_trellis_prepass", "euhedral_trellis_mma"] and names[4] == "euhedral_trellis_epilogue"
    assert dev.gpu.table_kernel_available("TRELLIS_MMA") and not dev.gpu.table_kernel_available("TRELLIS_MMA_ROWS_FP8")
    from euhedral_b200.gpu import GpuMemoryException
    with pytest.raises(GpuMemoryException) as wrong_count:
        dev.gpu.launch_table_kernel("TRELLIS_EPILOGUE", 1, 1, 1, 128, 1, 1, 0, KernelArguments().pointer(0).int32(1))
    assert wrong_count.value.status == -1
    with pytest.raises(GpuMemoryException) as wrong_width:
        dev.gpu.launch_table_kernel("TRELLIS_EPILOGUE", 1, 1, 1, 128, 1, 1, 0,
                                    KernelArguments().pointer(0).pointer(1).pointer(0).pointer(0).int32(1).int32(128))
    assert wrong_width.value.status == -1
    with pytest.raises(GpuMemoryException) as unavailable:
        dev.gpu.launch_table_kernel("TRELLIS_MMA_ROWS", 1, 1, 1, 256, 1, 1, 0, KernelArguments())
    assert unavailable.value.status == -5


def test_one_launch_linear_replayed_from_a_graph(dev):
    """A captured one-launch linear carries the same flag tag on every replay: each replay must still wait for its own
    partial sums (the CTA that finishes a column block unsets the block's flags)."""
    torch = dev.torch
    rng = np.random.default_rng(45)
    k, n, w, rows = 2048, 512, 48, 5
    payload, suh, svh = random_object(rng, k, n, w)
    linear = DeviceLinear(dev, payload, suh, svh, [n], 140)
    splits = TrellisFormat.splits(k, n, 140)
    assert splits > 1
    lib = dev.gpu.lib
    need = lib.euhedral_b200_linear_trellis_scratch_bytes(rows, k, n, 1, splits)
    xs = [random_x(rng, rows, k) for _ in range(4)]
    d_x, d_y, d_s = dev.put(xs[0]), dev.empty(rows * n * 2), dev.empty(need)
    t = [h.data_ptr() for h in linear.tensors]
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream), dev.gpu.submit(stream.cuda_stream, pdl=True):
        args = (d_x.data_ptr(), t[0], t[1], t[2], t[3], d_y.data_ptr(), d_s.data_ptr(), need, rows, k, n, w, 1, splits)
        assert lib.euhedral_b200_linear_trellis_bf16(*args) == 0          # warm: plans and maps are made before the capture
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            assert lib.euhedral_b200_linear_trellis_bf16(*args) == 0
        for x in xs:
            d_x.copy_(torch.from_numpy(x.view(np.uint8).reshape(-1).copy()))
            torch.cuda.synchronize()
            graph.replay()
            torch.cuda.synchronize()
            assert np.array_equal(dev.get(d_y, np.uint16, (rows, n)), linear.one_call(x, splits))
