"""The prefill activation quantizer against the reference's own kernel: oracle/_ref/libref_quantize.so is the
reference's quantize_rows<2> (native/src/nvfp4_native/native.cuh:66-168) compiled for sm_100a by
oracle/make_ref_quantize.py. Codes, block scales and row scales of this library's quantizer, and of the NumPy
restatement the other tests check against, must equal it bit for bit."""

import ctypes as C
from pathlib import Path

import numpy as np
import pytest

from euhedral_b200 import layouts
from oracle import oracle_np as O
from tests.gpu_util import Device

pytestmark = pytest.mark.gpu

LIBRARY = Path(__file__).resolve().parents[1] / "oracle" / "_ref" / "libref_quantize.so"


@pytest.fixture(scope="module")
def reference():
    if not LIBRARY.exists():
        pytest.skip("oracle/_ref/libref_quantize.so has not been built (python oracle/make_ref_quantize.py needs the reference tree)")
    lib = C.CDLL(str(LIBRARY))
    for name in ("ref_quantize_bytes", "ref_quantize_scale_offset", "ref_quantize_global_offset"):
        getattr(lib, name).restype = C.c_uint64
        getattr(lib, name).argtypes = [C.c_uint32, C.c_uint32]
    lib.ref_quantize.restype = C.c_int
    lib.ref_quantize.argtypes = [C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32]
    return lib


@pytest.fixture(scope="module")
def dev():
    device = Device()
    yield device
    assert device.gpu.take_device_error() == 0
    device.release()


def seeded_rows(rows, k, seed):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((rows, k)).astype(np.float32)
    x[1] = 0.0                                   # a zero row: row scale 1, every code and scale 0
    x[2, 16:32] = 0.0                            # a zero block inside a row
    x[3] *= 1e-30                                # tiny magnitudes (the row scale is tiny too)
    x[4, 5] = 1000.0                             # an outlier: its block saturates the E4M3 scale at 448, the others go subnormal
    x[5] = np.repeat(np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0], dtype=np.float32), k // 8)   # E2M1 rounding ties once scaled
    x[6] = -x[5]
    x[7] *= 1e4
    return O.bf16_bits(x)


def reference_quantize(reference, dev, x_bits):
    rows, k = x_bits.shape
    need = reference.ref_quantize_bytes(rows, k)
    d_x, d_out = dev.put(x_bits), dev.empty(need, fill=0)
    dev.torch.cuda.synchronize()
    assert reference.ref_quantize(d_x.data_ptr(), d_out.data_ptr(), rows, k) == 0
    raw = dev.get(d_out, np.uint8, (need,))
    half, pad = k // 2, -(-rows // 128) * 128
    planes = raw[:2 * rows * half].reshape(2, rows, half)
    codes = np.empty((2, rows, k), dtype=np.uint8)
    codes[:, :, 0::2] = planes & 15
    codes[:, :, 1::2] = planes >> 4
    scale_offset, global_offset = reference.ref_quantize_scale_offset(rows, k), reference.ref_quantize_global_offset(rows, k)
    # the 8 scale bytes of a row for K tile j (128 values) of term t sit at ((j * terms + t) * pad + row) * 8
    tiles = raw[scale_offset:scale_offset + (k // 128) * 2 * pad * 8].reshape(k // 128, 2, pad, 8)
    scales = np.ascontiguousarray(tiles[:, :, :rows].transpose(1, 2, 0, 3)).reshape(2, rows, k // 16)
    g = raw[global_offset:global_offset + 4 * rows].view(np.float32).copy()
    return codes, scales, g


def library_quantize(dev, x_bits):
    rows, k = x_bits.shape
    lib = dev.gpu.lib
    need = lib.euhedral_cuda_nvfp4_native_scratch_bytes(rows, k, 128)
    d_x, d_s = dev.put(x_bits), dev.empty(need, fill=0)
    with dev.submit():
        assert lib.euhedral_b200_nvfp4_native_quantize(d_x.data_ptr(), d_s.data_ptr(), rows, k, need) == 0
    raw = dev.get(d_s, np.uint8, (need,))
    half = k // 2
    planes = raw[:2 * rows * half].reshape(2, rows, half)
    codes = np.empty((2, rows, k), dtype=np.uint8)
    codes[:, :, 0::2] = planes & 15
    codes[:, :, 1::2] = planes >> 4
    sfa_offset = layouts.align_up(2 * rows * half, 256)
    row_tiles, k_blocks = -(-rows // 128), k // 64
    # atoms [row tile][K block of 64][term][512]: byte (r % 32) * 16 + (r / 32) * 4 + s of the atom holds scale s of row r
    atoms = raw[sfa_offset:sfa_offset + row_tiles * k_blocks * 2 * 512].reshape(row_tiles, k_blocks, 2, 32, 4, 4)
    by_row = atoms.transpose(2, 0, 4, 3, 1, 5).reshape(2, row_tiles * 128, k // 16)   # [term][tile, r / 32, r % 32][K block, s]
    scales = np.ascontiguousarray(by_row[:, :rows])
    global_offset = layouts.align_up(sfa_offset + row_tiles * k_blocks * 2 * 512, 256)
    g = raw[global_offset:global_offset + 4 * rows].view(np.float32).copy()
    return codes, scales, g


@pytest.mark.parametrize("rows,k", [(8, 256), (130, 1024), (300, 5120)])
def test_quantizer_equals_the_reference_kernel_bitwise(reference, dev, rows, k):
    x = seeded_rows(rows, k, rows + k)
    ref_codes, ref_scales, ref_g = reference_quantize(reference, dev, x)
    codes, scales, g = library_quantize(dev, x)
    assert np.array_equal(g.view(np.uint32), ref_g.view(np.uint32))
    assert np.array_equal(scales, ref_scales)
    assert np.array_equal(codes, ref_codes)
    assert ref_scales.max() == 0x7E and (ref_scales[0] == 0).any()        # a saturated scale and zero scales are both present
    # ... and so does the NumPy restatement that the GEMM tests build their expected operands from
    np_codes, np_scales, np_g = O.quantize_activations(x, 2)
    assert np.array_equal(np_g.view(np.uint32), ref_g.view(np.uint32))
    assert np.array_equal(np_scales, ref_scales)
    assert np.array_equal(np_codes, ref_codes)
