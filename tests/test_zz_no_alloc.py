"""The trellis linear that brings its own scratch (a static device array inside the library), for callers that cannot
allocate device memory when they call: two calls in a row through the C ABI must equal, bit for bit, the regular
three-launch route with caller scratch. Collected last on purpose."""

import numpy as np
import pytest

from euhedral_b200 import library
from euhedral_b200.formats import TrellisFormat
from tests.gpu_util import Device, random_x
from tests.test_trellis_gpu import DeviceLinear, random_object

pytestmark = pytest.mark.gpu


def test_static_scratch_linear_matches_caller_scratch_twice():
    dev = Device()
    try:
        lib = dev.gpu.lib
        assert lib.euhedral_b200_static_scratch_bytes() == 8 << 20
        rng = np.random.default_rng(77)
        k, n, w = 1024, 512, 48
        ends = [256, 512]
        payload, suh, svh = random_object(rng, k, n, w, segments=2)
        regular = DeviceLinear(dev, payload, suh, svh, ends, target_ctas=64)
        splits = TrellisFormat.splits(k, n, 64)
        assert splits > 1
        d_words, d_suh, d_svh, d_ends = regular.tensors
        for call, rows in enumerate((5, 8)):        # two calls in a row share the array; the second reuses its bytes
            x = random_x(rng, rows, k)
            expect = regular.linear(x)
            d_x, d_y = dev.put(x), dev.empty(rows * n * 2)
            with dev.submit():
                status = lib.euhedral_b200_linear_trellis_bf16_static(d_x.data_ptr(), d_words.data_ptr(), d_suh.data_ptr(), d_svh.data_ptr(),
                                                                      d_ends.data_ptr(), d_y.data_ptr(), rows, k, n, w, 2, splits)
            assert status == 0, (call, status)
            assert np.array_equal(dev.get(d_y, np.uint16, (rows, n)), expect), call
        # a single split finishes inside the GEMM kernel
        one = DeviceLinear(dev, payload, suh, svh, ends, target_ctas=1)
        x = random_x(rng, 3, k)
        d_x, d_y = dev.put(x), dev.empty(3 * n * 2)
        with dev.submit():
            assert lib.euhedral_b200_linear_trellis_bf16_static(d_x.data_ptr(), d_words.data_ptr(), d_suh.data_ptr(), d_svh.data_ptr(),
                                                                d_ends.data_ptr(), d_y.data_ptr(), 3, k, n, w, 2, 1) == 0
        assert np.array_equal(dev.get(d_y, np.uint16, (3, n)), one.linear(x))
        # too large for the static array: refused before anything is launched
        assert lib.euhedral_b200_linear_trellis_bf16_static(d_x.data_ptr(), d_words.data_ptr(), d_suh.data_ptr(), d_svh.data_ptr(),
                                                            d_ends.data_ptr(), d_y.data_ptr(), 4096, k, n, w, 2, splits) == library.SIZE_OVERFLOW
        assert dev.gpu.take_device_error() == 0
    finally:
        dev.release()
