"""Seeded synthetic tensors in the three weight layouts, built with torch on whatever device is asked for (the GPU in
the benchmark, the CPU in tests). These stand in for the model's weights: N(0, sigma^2) values rounded the way the
reference's converter rounds them (tools/euhedral_artifacts/nvfp4.py:85-105, grouped.py:39-66,129-135), and for trellis
objects random words with the scale distributions of the reference's kernel tests (native/tests/test_trellis.py:64-68).
The arithmetic is float32/float64 IEEE in the converter's order, so the bytes equal the converter's for the same values.
"""

from __future__ import annotations

import torch

from euhedral_b200 import layouts


def gaussian(n: int, k: int, seed: int, sigma: float = 0.02, device="cpu") -> torch.Tensor:
    generator = torch.Generator(device=device)
    generator.manual_seed(seed)
    return torch.randn((n, k), generator=generator, device=device, dtype=torch.float32) * sigma


def bf16_rows(rows: int, k: int, seed: int, device="cpu") -> torch.Tensor:
    """N(0, 1) activations as BF16 bit patterns (int16), rounded to nearest even."""
    generator = torch.Generator(device=device)
    generator.manual_seed(seed)
    values = torch.randn((rows, k), generator=generator, device=device, dtype=torch.float32)
    return values.to(torch.bfloat16).view(torch.int16)


def _nearest(values: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """Index of the nearest entry of the ascending `table`, ties to the even index, saturating."""
    upper = torch.searchsorted(table, values.contiguous()).clamp(1, table.numel() - 1)
    lower = upper - 1
    below, above = values - table[lower], table[upper] - values
    index = torch.where((above < below) | ((above == below) & (upper % 2 == 0)), upper, lower)
    index = torch.where(values >= table[-1], torch.full_like(index, table.numel() - 1), index)
    return torch.where(values <= table[0], torch.zeros_like(index), index)


def _e4m3_table(device) -> torch.Tensor:
    code = torch.arange(127, device=device)
    exponent, mantissa = code >> 3, (code & 7).double()
    normal = (1 + mantissa / 8) * torch.pow(torch.tensor(2.0, dtype=torch.float64, device=device), (exponent - 7).double())
    subnormal = mantissa / 8 * 2.0 ** -6
    return torch.where(exponent == 0, subnormal, normal).float()


def nvfp4_tensor(weights: torch.Tensor) -> torch.Tensor:
    """uint8 tensor holding a whole NVFP4 row-split-k128-v1 object of float32 `weights` [n, k] (k a multiple of 128)."""
    n, k = weights.shape
    if k % 128:
        raise ValueError("k must be a multiple of 128")
    device = weights.device
    e4m3 = _e4m3_table(device)
    e2m1 = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], device=device)
    global_scale = weights.abs().max() / torch.tensor(2688.0, device=device)
    out = torch.zeros(layouts.nvfp4_byte_size(n, k), dtype=torch.uint8, device=device)
    scale_offset, trailer = layouts.nvfp4_scale_offset(n, k), layouts.nvfp4_trailer_offset(n, k)
    step_rows = max(1, (1 << 24) // k)
    for begin in range(0, n, step_rows):
        blocks = weights[begin:begin + step_rows].reshape(-1, k // 16, 16)
        rows = blocks.shape[0]
        if float(global_scale) > 0:
            ratio = blocks.abs().amax(dim=2) / 6.0 / global_scale
        else:
            ratio = torch.zeros(blocks.shape[:2], device=device)
        scale_codes = _nearest(ratio, e4m3)
        decode = e4m3[scale_codes] * global_scale
        scaled = torch.where(decode[..., None] > 0, blocks.abs() / decode[..., None], torch.zeros_like(blocks))
        magnitude = _nearest(scaled, e2m1)
        codes = (magnitude | (((blocks < 0) & (magnitude > 0)).long() << 3)).reshape(rows, k)
        packed = (codes[:, 0::2] | (codes[:, 1::2] << 4)).to(torch.uint8)
        out[begin * (k // 2):(begin + rows) * (k // 2)] = packed.reshape(-1)
        out[scale_offset + begin * (k // 16):scale_offset + (begin + rows) * (k // 16)] = scale_codes.to(torch.uint8).reshape(-1)
    out[trailer:trailer + 4] = global_scale.reshape(1).float().view(torch.uint8)
    return out


def q3_tensor(weights: torch.Tensor) -> torch.Tensor:
    """uint8 tensor holding a whole Q3G64_F16S row-split-k128-v1 object of float32 `weights` [n, k] (k % 128 == 0)."""
    n, k = weights.shape
    if k % 128:
        raise ValueError("k must be a multiple of 128")
    device = weights.device
    groups = k // 64
    out = torch.zeros(layouts.q3_byte_size(n, k), dtype=torch.uint8, device=device)
    scale_offset = layouts.q3_scale_offset(n, k)
    shifts = (3 * torch.arange(8, device=device)).long()
    step_rows = max(1, (1 << 24) // k)
    for begin in range(0, n, step_rows):
        grouped = weights[begin:begin + step_rows].reshape(-1, groups, 64)
        rows = grouped.shape[0]
        amax = grouped.abs().amax(dim=2)
        scales = (amax.double() / 3.0).float().half()
        scales = torch.where((scales == 0) & (amax > 0), torch.full_like(scales, 2.0 ** -24), scales)
        inverse = torch.where(scales > 0, (1.0 / scales.double()).float(), torch.zeros_like(amax))
        codes = torch.round(grouped * inverse[..., None]).clamp(-4, 3).long() & 7
        # 8 codes -> 24 bits -> 3 bytes, little-endian bit stream
        word = (codes.reshape(rows, groups, 8, 8) << shifts).sum(dim=3)
        triple = torch.stack([word & 255, (word >> 8) & 255, (word >> 16) & 255], dim=3).to(torch.uint8)
        out[begin * groups * 24:(begin + rows) * groups * 24] = triple.reshape(-1)
        out[scale_offset + begin * groups * 2:scale_offset + (begin + rows) * groups * 2] = scales.reshape(-1).view(torch.uint8)
    return out


def trellis_object(n: int, k: int, w: int, seed: int, segments: int = 1, device="cpu"):
    """(payload int16 [k/16, n/16, w], suh f16 [s, k], svh f16 [n], ends i32 [s]) with uniformly random words."""
    generator = torch.Generator(device=device)
    generator.manual_seed(seed)
    kt, nt, w = layouts.trellis_payload_shape(n, k, w)
    payload = torch.randint(-32768, 32768, (kt, nt, w), generator=generator, device=device, dtype=torch.int32).to(torch.int16)
    sign = torch.randint(0, 2, (segments, k), generator=generator, device=device).float() * 2 - 1
    suh = (sign * (0.5 + 1.5 * torch.rand((segments, k), generator=generator, device=device))).half()
    svh = (0.01 + 0.99 * torch.rand((n,), generator=generator, device=device)).half()
    width = n // segments // 128 * 128
    ends = [width * (i + 1) for i in range(segments - 1)] + [n]
    return payload, suh, svh, torch.tensor(ends, dtype=torch.int32, device=device)
