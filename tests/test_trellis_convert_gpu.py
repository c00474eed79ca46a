"""The trellis converter end to end on the GPU: a dense weight in, an object out that the trellis linear and the oracle's
decoder both read back as the weight, to the rounding error of the rate."""

import numpy as np
import pytest
import torch

from euhedral_b200 import trellis_convert as T
from oracle import oracle_np as O
from tests.gpu_util import Device, random_x
from tests.test_trellis_gpu import DeviceLinear

pytestmark = pytest.mark.gpu

# relative squared error of a unit Gaussian under the bitshift trellis by rate, with room (the published figures of
# the code family are about 0.07, 0.02 and 0.005 at 2, 3 and 4 bits)
BOUND = {2.0: 0.10, 2.5: 0.06, 3.0: 0.035, 3.5: 0.02, 4.0: 0.012}


@pytest.fixture(scope="module")
def dev():
    device = Device()
    yield device
    assert device.gpu.take_device_error() == 0
    device.release()


@pytest.fixture(scope="module")
def converter(dev):
    return T.TrellisConverter("cuda", chunk_tiles=512)


def gaussian(n, k, seed, sigma=0.02):
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal((n, k)) * sigma).astype(np.float32)
    w *= rng.uniform(0.5, 2.0, size=(n, 1)).astype(np.float32)        # output channels of different energy
    return w


def rebuilt(obj):
    """W' [n, k] float64 of an object: diag(su) H_K Q H_N diag(sv), transposed."""
    q = O.trellis_rotated_weight(obj.payload.cpu().numpy()).astype(np.float64)      # [k, n]
    su, sv = obj.suh.cpu().numpy().astype(np.float64), obj.svh.cpu().numpy().astype(np.float64)
    i = np.arange(128)
    h = np.where(np.bitwise_count(i[:, None] & i[None, :]) & 1, -1.0, 1.0) / np.sqrt(128.0)
    k, n = q.shape
    q = np.einsum("ij,bjc->bic", h, q.reshape(k // 128, 128, n)).reshape(k, n)
    q = (q.reshape(k, n // 128, 128) @ h).reshape(k, n)
    return (su[:, None] * q * sv[None, :]).T


@pytest.mark.parametrize("bits", [2.0, 2.5, 3.0, 3.5, 4.0])
def test_object_reads_back_as_the_weight(converter, bits):
    n, k = 384, 256
    w = gaussian(n, k, int(bits * 10))
    obj = converter.quantize(torch.from_numpy(w).cuda(), bits, seed=7)
    assert obj.payload.shape == (k // 16, n // 16, T.words_per_tile(bits)) and obj.payload.dtype == torch.int16
    assert obj.suh.shape == (k,) and obj.svh.shape == (n,) and obj.suh.dtype == torch.float16
    error = np.sum((rebuilt(obj) - w) ** 2) / np.sum(w.astype(np.float64) ** 2)
    assert error < BOUND[bits], error
    assert 0.5 < obj.scale < 1.5
    # the sign vectors are the seed's
    su, sv = T.java_signs(7, k, n)
    assert np.array_equal(np.sign(obj.suh.cpu().numpy().astype(np.float32)), -su)      # su = sign * rms / -scale
    assert np.array_equal(np.sign(obj.svh.cpu().numpy().astype(np.float32)), sv)


def test_same_seed_same_object(converter):
    w = torch.from_numpy(gaussian(256, 256, 3)).cuda()
    a, b = converter.quantize(w, 3.0, seed=11), converter.quantize(w, 3.0, seed=11)
    assert torch.equal(a.payload, b.payload) and torch.equal(a.suh, b.suh) and torch.equal(a.svh, b.svh)
    c = converter.quantize(w, 3.0, seed=12)
    assert not torch.equal(a.suh, c.suh)


def test_rate_lowers_the_error(converter):
    w = torch.from_numpy(gaussian(256, 256, 5)).cuda()
    errors = [converter.quantize(w, bits, seed=1).proxy for bits in (2.0, 3.0, 4.0, 5.0, 6.0)]
    assert all(a > b for a, b in zip(errors, errors[1:])), errors


def test_linear_on_a_converted_weight(dev, converter):
    n, k, bits = 512, 384, 3.0
    w = gaussian(n, k, 21)
    obj = converter.quantize(torch.from_numpy(w).cuda(), bits, seed=3)
    payload, suh, svh, ends = T.TrellisConverter.fuse([obj])
    linear = DeviceLinear(dev, payload.cpu().numpy(), suh.cpu().numpy(), svh.cpu().numpy(), ends.cpu().numpy(), 148)
    x = random_x(np.random.default_rng(4), 3, k)
    got = O.bf16_to_f32(linear.one_call(x, 0)).astype(np.float64)
    xf = O.bf16_to_f32(x).astype(np.float64)
    # against the object's own weight: the kernel's tolerance; against the dense weight: the rate's rounding error
    own = xf @ rebuilt(obj).T
    assert np.all(np.abs(got - own) <= 0.01 * np.abs(own) + 0.01 * np.sqrt(np.mean(own ** 2)))
    dense = xf @ w.astype(np.float64).T
    assert np.sum((got - dense) ** 2) / np.sum(dense ** 2) < BOUND[bits] * 1.5


def test_fused_object_is_its_members_side_by_side(dev, converter):
    k = 256
    parts = [converter.quantize(torch.from_numpy(gaussian(n, k, 30 + i)).cuda(), 3.0, seed=30 + i) for i, n in enumerate((256, 128, 128))]
    payload, suh, svh, ends = T.TrellisConverter.fuse(parts)
    assert ends.tolist() == [256, 384, 512] and suh.shape == (3, k) and payload.shape == (16, 32, 48)
    x = random_x(np.random.default_rng(8), 2, k)
    fused = DeviceLinear(dev, payload.cpu().numpy(), suh.cpu().numpy(), svh.cpu().numpy(), ends.cpu().numpy(), 148).one_call(x, 2)
    first = 0
    for part in parts:
        p, s, v, e = T.TrellisConverter.fuse([part])
        alone = DeviceLinear(dev, p.cpu().numpy(), s.cpu().numpy(), v.cpu().numpy(), e.cpu().numpy(), 148).one_call(x, 2)
        assert np.array_equal(fused[:, first:first + alone.shape[1]], alone)
        first += alone.shape[1]


def test_degenerate_weights_convert(converter):
    # all zeros: every RMS takes the 0.1 stand-in, the stored output scales are 0, the object decodes to zeros
    obj = converter.quantize(torch.zeros(128, 128, device="cuda"), 3.0, seed=2)
    assert torch.count_nonzero(obj.svh) == 0 and torch.isfinite(obj.suh.float()).all()
    assert np.all(rebuilt(obj) == 0.0)
    # one live output channel among dead ones, and BF16 input
    w = torch.zeros(256, 128, device="cuda")
    w[17] = torch.randn(128, generator=torch.Generator(device="cuda").manual_seed(1), device="cuda") * 0.05
    obj = converter.quantize(w.bfloat16(), 4.0, seed=2)
    back = rebuilt(obj)
    dense = w.bfloat16().float().cpu().numpy().astype(np.float64)
    assert np.sum((back - dense) ** 2) / np.sum(dense ** 2) < 0.05
    assert np.all(np.isfinite(back))


def test_without_output_scales(converter):
    w = gaussian(256, 256, 44)
    obj = converter.quantize(torch.from_numpy(w).cuda(), 3.0, seed=5, apply_out_scales=False)
    assert torch.equal(obj.svh.float().abs(), torch.ones(256, device="cuda"))
    # channels of different energy share one scale now: the error is larger than with output scales, but bounded
    error = np.sum((rebuilt(obj) - w) ** 2) / np.sum(w.astype(np.float64) ** 2)
    assert error < 0.08, error
