"""The converter's trellis tile encoder on the GPU (euhedral_b200_trellis_encode_tiles) against the reference encoder's
golden tiles and against the CPU restatement that those tiles pin."""

import numpy as np
import pytest

from euhedral_b200 import library
from oracle import oracle_c as OC
from oracle import oracle_np as O
from tests.gpu_util import Device

pytestmark = pytest.mark.gpu

RATES = [(32, 2, 0), (40, 2, 0xAAAA), (48, 3, 0), (56, 3, 0xAAAA), (64, 4, 0), (80, 5, 0), (96, 6, 0)]


@pytest.fixture(scope="module")
def dev():
    device = Device()
    yield device
    assert device.gpu.take_device_error() == 0
    device.release()


def encode(dev, tiles, w):
    lib = dev.gpu.lib
    count = tiles.shape[0]
    need = lib.euhedral_b200_trellis_encode_scratch_bytes(count, w)
    d_t, d_s, d_h = dev.put(np.ascontiguousarray(tiles, dtype=np.float32)), dev.empty(count * 512), dev.empty(need)
    d_v, d_w = dev.empty(count * 1024), dev.empty(count * w * 2)
    with dev.submit():
        assert lib.euhedral_b200_trellis_encode_tiles(d_t.data_ptr(), count, w, d_s.data_ptr(), d_v.data_ptr(), d_w.data_ptr(), d_h.data_ptr(), need) == 0
    encode.decoded, encode.words = dev.get(d_v, np.float32, (count, 256)), dev.get(d_w, np.int16, (count, w))
    return dev.get(d_s, np.uint16, (count, 256))


@pytest.mark.parametrize("w,ka,mask", RATES)
def test_golden_tiles(dev, golden, w, ka, mask):
    g = golden("trellis")
    states = encode(dev, g["tiles_in"], w)
    assert np.array_equal(states, g[f"tiles_{w}_idx"])
    packed = O.trellis_pack_states(states, ka, mask)
    assert np.array_equal(packed, g[f"tiles_{w}_packed"])
    assert np.array_equal(encode.words, packed)       # the library's own packing and values
    assert np.array_equal(encode.decoded.astype(np.float16).view(np.uint16), g[f"tiles_{w}_out"].view(np.uint16))
    assert np.array_equal(O.trellis_decode_tiles(packed, w).view(np.uint16), g[f"tiles_{w}_out"].view(np.uint16))


@pytest.mark.parametrize("w,ka,mask", [(48, 3, 0), (40, 2, 0xAAAA)])
def test_more_tiles_than_ctas_against_the_cpu_restatement(dev, w, ka, mask):
    """Every CTA encodes several tiles in turn (its history slab and cost rows are reused); scaled and shifted inputs."""
    rng = np.random.default_rng(w)
    count = 4 * dev.gpu.multiprocessor_count() + 3
    tiles = (rng.standard_normal((count, 256)) * rng.uniform(0.2, 1.5, (count, 1))).astype(np.float32)
    tiles[0] = 0.0
    tiles[1, ::7] = 4.0
    expect, _ = OC.trellis_encode_tiles(tiles[:24], ka, mask)
    states = encode(dev, tiles, w)
    assert np.array_equal(states[:24], expect)
    again = encode(dev, tiles[count - 8:], w)     # the same tiles at other places of the list: the same states
    assert np.array_equal(again, states[count - 8:])


def test_status_codes(dev):
    lib = dev.gpu.lib
    tiles = dev.put(np.zeros((2, 256), dtype=np.float32))
    out, scratch = dev.empty(1024), dev.empty(1 << 20)
    with dev.submit():
        assert lib.euhedral_b200_trellis_encode_tiles(tiles.data_ptr(), 2, 72, out.data_ptr(), 0, 0, scratch.data_ptr(), 1 << 20) == library.ROUTE_UNAVAILABLE
        assert lib.euhedral_b200_trellis_encode_tiles(tiles.data_ptr(), 2, 48, out.data_ptr(), 0, 0, scratch.data_ptr(), 1024) == library.SIZE_OVERFLOW
        assert lib.euhedral_b200_trellis_encode_tiles(0, 2, 48, out.data_ptr(), 0, 0, scratch.data_ptr(), 1 << 20) == library.INVALID_ARGUMENT
    assert lib.euhedral_b200_trellis_encode_scratch_bytes(2, 48) == 2 * 256 * 8192
