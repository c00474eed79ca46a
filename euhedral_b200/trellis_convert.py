"""Converter of a dense linear weight to a trellis-tile16-v1 object, uncalibrated path.

Mirrors the reference's `TrellisQuantizer.quantize` with no Hessian (quantization/src/main/java/.../trellis/
TrellisQuantizer.java:103-180, `count == 0`): sign vectors from the seed, `regularize` (:242-263: output scales from
the column RMS, `W / sv`, Hadamard along n, input scales from the row RMS, `W / su`, Hadamard along k, the searched
global scale), then every 16 x 16 tile rounded by the tail-biting Viterbi search and packed. The per-value work
(RMS, scales, butterflies, the tile gather) is elementwise torch on the device; the search - all the time of a
conversion - is the library's `euhedral_b200_trellis_encode_tiles` (csrc/trellis_encode.cuh), which also packs the
words the linears read.

What is fixed by the format's golden tiles is the tile search and the packing (bit for bit). The steps before it follow
the reference's arithmetic (double-precision sums where it uses them, the same butterfly order, the same sampling and
grids for the global scale) but have no golden vectors: an object made here decodes with the reference's kernels and
its scales agree with the reference's to rounding, not necessarily to the bit.
"""

from __future__ import annotations

import dataclasses

import numpy as np
import torch

from euhedral_b200 import library

CODEBOOK_SCALE = 1.24371088          # trellis.cu:873-879 (input_scales)
_INV_SQRT_128 = float(np.float32(0.08838834764831845))
_MASK64 = (1 << 64) - 1


def words_per_tile(bits: float) -> int:
    """16-bit words of a tile at `bits` per weight (TrellisKernels.wordsPerTile): 16 bits."""
    words = int(round(bits * 16))
    if words not in (32, 40, 48, 56, 64, 80, 96):
        raise ValueError(f"no trellis rate of {bits} bits")
    return words


def java_signs(seed: int, count_k: int, count_n: int) -> tuple[np.ndarray, np.ndarray]:
    """The two sign vectors (+-1 as float32) `new SplittableRandom(seed)` gives through `nextBoolean()`, k first
    (TrellisQuantizer.java:111-112,444-448). SplitMix64 as java.util.SplittableRandom publishes it: the state advances
    by the golden gamma, a draw is the sign of the 32-bit mix of the state."""
    total = count_k + count_n
    state = (np.uint64(seed & _MASK64) + np.uint64(0x9E3779B97F4A7C15) * np.arange(1, total + 1, dtype=np.uint64))
    z = (state ^ (state >> np.uint64(33))) * np.uint64(0x62A9D9ED799705F5)
    z = (z ^ (z >> np.uint64(28))) * np.uint64(0xCB24D0A5C88C35B3)
    negative = (z >> np.uint64(63)).astype(bool)        # top bit of the upper 32 bits: nextInt() < 0
    signs = np.where(negative, 1.0, -1.0).astype(np.float32)
    return signs[:count_k], signs[count_k:]


def tile_order() -> np.ndarray:
    """element (row * 16 + column of the 16 x 16 tile of W [k, n]) of tensor-core position 0..255
    (native/src/trellis/codebook.cuh:65-71)."""
    pos = np.arange(256)
    t, j = pos >> 3, pos & 7
    row = (t & 3) * 2 + ((j >> 1) & 1) * 8 + (j & 1)
    col = (t >> 2) + (j >> 2) * 8
    return (row * 16 + col).astype(np.int64)


def hadamard128(x: torch.Tensor, axis: int) -> torch.Tensor:
    """Sylvester-order Walsh-Hadamard over every block of 128 along `axis`, divided by sqrt(128), by the same butterflies
    as trellis.cu:584-613 (stage h pairs i with i + h)."""
    x = x.movedim(axis, -1).contiguous()
    shape = x.shape
    x = x.view(-1, 128)
    h = 1
    while h < 128:
        y = x.view(-1, 128 // (2 * h), 2, h)
        a, b = y[:, :, 0, :], y[:, :, 1, :]
        x = torch.stack((a + b, a - b), dim=2).view(-1, 128)
        h *= 2
    return (x * _INV_SQRT_128).view(shape).movedim(-1, axis).contiguous()


def drift(bits: float) -> float:
    """The allowance for the growth of the weights by rate (TrellisQuantizer.java:266-271)."""
    return {2.0: 1.018, 2.5: 1.009, 3.0: 1.004}.get(float(bits), 1.0)


@dataclasses.dataclass
class TrellisObject:
    payload: torch.Tensor      # int16 [k/16, n/16, w]
    suh: torch.Tensor          # float16 [k]
    svh: torch.Tensor          # float16 [n]
    scale: float               # the searched global scale
    proxy: float               # mean squared rounding error in the rotated basis


class TrellisConverter:
    """Holds the search's scratch; `quantize` converts one weight, `fuse` concatenates converted weights along n."""

    def __init__(self, device="cuda", chunk_tiles: int = 1 << 16):
        self.lib = library.load()
        self.device = torch.device(device)
        self.chunk = chunk_tiles
        self.order = torch.from_numpy(tile_order()).to(self.device)
        self._scratch = None

    # ---- the tile search ---------------------------------------------------------------------------------------------
    def encode(self, tiles: torch.Tensor, bits: float, want_words: bool = True):
        """tiles float32 [count, 256] in tensor-core order -> (values float32 [count, 256], words int16 [count, w] or None)."""
        lib, w = self.lib, words_per_tile(bits)
        count = tiles.shape[0]
        tiles = tiles.contiguous()
        values = torch.empty((count, 256), dtype=torch.float32, device=self.device)
        words = torch.empty((count, w), dtype=torch.int16, device=self.device) if want_words else None
        states = torch.empty((min(count, self.chunk), 256), dtype=torch.int16, device=self.device)
        need = lib.euhedral_b200_trellis_encode_scratch_bytes(min(count, self.chunk), w)
        if self._scratch is None or self._scratch.numel() < need:
            self._scratch = torch.empty(need, dtype=torch.uint8, device=self.device)
        # The search runs on torch's current stream so that it is ordered with the tensor work around it. The thread's stream
        # selection in the library is put back afterwards (a caller may be inside a submission of its own).
        stream = torch.cuda.current_stream(self.device).cuda_stream
        before = lib.euhedral_cuda_submission_stream() or 0
        if stream != before:
            if stream == 0:
                lib.euhedral_cuda_stream_clear()
            elif lib.euhedral_cuda_stream_select(stream) != 0:
                raise RuntimeError("stream select failed")
        try:
            for first in range(0, count, self.chunk):
                part = min(self.chunk, count - first)
                status = lib.euhedral_b200_trellis_encode_tiles(
                    tiles[first:].data_ptr(), part, w, states.data_ptr(), values[first:].data_ptr(),
                    words[first:].data_ptr() if want_words else 0, self._scratch.data_ptr(), self._scratch.numel())
                if status != 0:
                    raise RuntimeError(f"trellis_encode_tiles failed with status {status}")
        finally:
            if stream != before:
                if before == 0:
                    lib.euhedral_cuda_stream_clear()
                else:
                    lib.euhedral_cuda_stream_select(before)
        return values, words

    # ---- regularize (TrellisQuantizer.java:242-263) -------------------------------------------------------------------
    def regularize(self, w: torch.Tensor, su_signs: torch.Tensor, sv_signs: torch.Tensor, apply_out_scales: bool, bits: float):
        """w float32 [k, n] -> (rotated and scaled w, su [k], sv [n], global scale)."""
        k, n = w.shape
        rms = torch.sqrt(w.double().square().sum(0) / k).float()                       # column_rms, trellis.cu:823-841
        mean = (rms.double().sum() / n).float()
        normalised = bool(mean > 1e-30)                                                # output_scales, trellis.cu:856-870
        s = rms / mean if normalised else rms.clone()
        zero = s.abs() < 1e-30
        if apply_out_scales or not normalised:
            s = torch.where(zero, torch.full_like(s, 0.1), s)
            divisor = sv_signs * s + 1e-10
        else:
            divisor = sv_signs.clone()
        sv = torch.where(zero, torch.zeros_like(divisor), divisor)
        w = hadamard128(w / divisor[None, :], 1)
        rms = torch.sqrt(w.double().square().sum(1) / n).float()                       # row_rms, input_scales
        rms = torch.where(rms.abs() < 1e-30, torch.full_like(rms, 0.1), rms)
        su = su_signs * rms / (-CODEBOOK_SCALE) + 1e-10
        w = hadamard128(w / su[:, None], 0)
        g = self.global_scale(w, bits)
        return w * g, su / g, sv, g

    def tiles_of(self, w: torch.Tensor) -> torch.Tensor:
        """w [k, n] -> [k/16 * n/16, 256] in tensor-core order, tile (kt, nt) at kt * n/16 + nt."""
        k, n = w.shape
        return w.view(k // 16, 16, n // 16, 16).permute(0, 2, 1, 3).reshape(-1, 256)[:, self.order].contiguous()

    # ---- the global scale (TrellisQuantizer.java:276-334) -------------------------------------------------------------
    def global_scale(self, w: torch.Tensor, bits: float) -> float:
        k, n = w.shape
        tiles_k, tiles_n, width = k // 16, n // 16, 3
        diagonal, total = max(tiles_k, tiles_n), (k // 16) * (n // 16)
        energy = (w.view(tiles_k, 16, tiles_n, 16).double().square().sum((1, 3)) / 256.0).float().reshape(-1)
        extreme = min(max(8, diagonal * width // 16), (total + 1) // 2)
        order = torch.sort(energy, stable=True).indices                                # ties by tile index
        i = torch.arange(diagonal, device=self.device)[:, None]
        j = torch.arange(width, device=self.device)[None, :]
        sample = ((i % tiles_k) * tiles_n + (i + j) % tiles_n).reshape(-1)
        sample = torch.cat((sample, order[-extreme:].flip(0), order[:extreme]))
        all_tiles = w.view(tiles_k, 16, tiles_n, 16).permute(0, 2, 1, 3).reshape(total, 256)
        sampled = (all_tiles[sample][:, self.order] * np.float32(drift(bits))).contiguous()    # gather_tiles

        coarse = [0.1 + 0.2 * c for c in range(10)]
        errors = self.candidate_errors(sampled, 3, coarse, bits)
        center = int(np.argmin(errors))                                                # first of equal minima
        step = 0.075
        fine = [coarse[center] + step * (c - 2) for c in range(5)]
        errors = self.candidate_errors(sampled, 1, fine, bits)
        best = int(np.argmin(errors))
        offset = 0.0
        if 0 < best < len(fine) - 1:
            y0, y1, y2 = (float(errors[best - 1]), float(errors[best]), float(errors[best + 1]))
            denominator = y0 - 2 * y1 + y2
            offset = 0.5 * (y0 - y2) / denominator if denominator > 0 else 0.0
            offset = max(-0.5, min(0.5, offset))
        return float(np.float32(max(fine[best] + offset * step, 0.01)))

    def candidate_errors(self, sampled: torch.Tensor, stride: int, scales, bits: float) -> np.ndarray:
        """Mean squared error of rounding every `stride`th sample at each scale (TrellisQuantizer.java:337-362)."""
        picked = sampled[::stride]
        s = torch.tensor([np.float32(v) for v in scales], dtype=torch.float32, device=self.device)
        scaled = (picked[None, :, :] * s[:, None, None]).reshape(-1, 256)
        values, _ = self.encode(scaled, bits, want_words=False)
        d = values.view(len(scales), -1, 256) / s[:, None, None] - picked[None, :, :]
        return d.double().square().mean((1, 2)).float().cpu().numpy()

    # ---- a whole weight ------------------------------------------------------------------------------------------------
    def quantize(self, weight: torch.Tensor, bits: float, seed: int, apply_out_scales: bool = True) -> TrellisObject:
        """weight [n, k] (any float type, on the device) -> its trellis object at `bits` per weight."""
        n, k = weight.shape
        if n <= 0 or k <= 0 or n % 128 or k % 128:
            raise ValueError(f"shape [{n}, {k}] not a multiple of 128")
        w = words_per_tile(bits)
        signs_k, signs_n = java_signs(seed, k, n)
        su_signs, sv_signs = torch.from_numpy(signs_k).to(self.device), torch.from_numpy(signs_n).to(self.device)
        original = weight.to(self.device).float().t().contiguous()                     # [k, n]
        regular, su, sv, g = self.regularize(original, su_signs, sv_signs, apply_out_scales, bits)
        del original
        values, words = self.encode(self.tiles_of(regular), bits)
        proxy = float((values - self.tiles_of(regular)).double().square().mean())
        return TrellisObject(words.view(k // 16, n // 16, w), su.half(), sv.half(), g, proxy)

    @staticmethod
    def fuse(parts) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
        """Objects that share k, side by side along n: (payload, suh [s, k], svh, ends int32 [s]) - how the artifact
        writer lays out query_key_value and gate_up (tools/euhedral_artifacts/trellis.py:128-146)."""
        payload = torch.cat([p.payload for p in parts], dim=1).contiguous()
        suh = torch.stack([p.suh for p in parts]).contiguous()
        svh = torch.cat([p.svh for p in parts]).contiguous()
        ends = torch.tensor(np.cumsum([p.svh.numel() for p in parts]), dtype=torch.int32, device=payload.device)
        return payload, suh, svh, ends
