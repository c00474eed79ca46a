"""Column (N) sharding of quantized tensors across the GPUs of one node, and the all-gather that joins the output
slices. The slicing follows the reference's `rows` operators (core/.../artifact/format/Nvfp4Format.java:109-130,
core/.../artifact/format/TrellisFormat.java:199-282): rows [first, first + rows) become a self-contained tensor in
the same layout, so the same kernels run on a shard. The reference itself is single-GPU; the collective is new here.

Host-side functions work on NumPy byte arrays; `ShardedLinear` is the torch.distributed wrapper (NCCL on GPUs, gloo
in CPU tests of the plumbing)."""

from __future__ import annotations

import numpy as np

from euhedral_b200 import layouts


def shard_range(n: int, world_size: int, rank: int, unit: int) -> tuple[int, int]:
    """(first row, rows) of `rank`: n / world_size rows each, which must be a multiple of `unit`."""
    if n % world_size or (n // world_size) % unit:
        raise ValueError(f"{n} rows do not split into {world_size} shards of whole {unit}-row units")
    rows = n // world_size
    return rank * rows, rows


def nvfp4_rows(blob: np.ndarray, n: int, k: int, first: int, rows: int) -> np.ndarray:
    """Rows [first, first + rows) of an NVFP4 tensor: code rows, scale rows and the shared FP32 scale."""
    blob = np.ascontiguousarray(blob, dtype=np.uint8)
    kp = layouts.padded_k(k)
    row_bytes, row_scales = kp // 2, kp // 16
    out = np.zeros(layouts.nvfp4_byte_size(rows, k), dtype=np.uint8)
    out[:rows * row_bytes] = blob[first * row_bytes:(first + rows) * row_bytes]
    src, dst = layouts.nvfp4_scale_offset(n, k), layouts.nvfp4_scale_offset(rows, k)
    out[dst:dst + rows * row_scales] = blob[src + first * row_scales:src + (first + rows) * row_scales]
    src, dst = layouts.nvfp4_trailer_offset(n, k), layouts.nvfp4_trailer_offset(rows, k)
    out[dst:dst + 4] = blob[src:src + 4]
    return out


def nvfp4_sd4_rows(blob: np.ndarray, n: int, k: int, first: int, rows: int) -> np.ndarray:
    """The same for the table-indexed layout: code rows, index rows, and the tensor's table and FP32 scale."""
    blob = np.ascontiguousarray(blob, dtype=np.uint8)
    kp = layouts.padded_k(k)
    row_bytes, row_indices = kp // 2, kp // 32
    out = np.zeros(layouts.nvfp4_sd4_byte_size(rows, k), dtype=np.uint8)
    out[:rows * row_bytes] = blob[first * row_bytes:(first + rows) * row_bytes]
    src, dst = layouts.nvfp4_scale_offset(n, k), layouts.nvfp4_scale_offset(rows, k)
    out[dst:dst + rows * row_indices] = blob[src + first * row_indices:src + (first + rows) * row_indices]
    src, dst = layouts.nvfp4_sd4_table_offset(n, k), layouts.nvfp4_sd4_table_offset(rows, k)
    out[dst:dst + 20] = blob[src:src + 20]
    return out


def q3_rows(blob: np.ndarray, n: int, k: int, first: int, rows: int) -> np.ndarray:
    blob = np.ascontiguousarray(blob, dtype=np.uint8)
    groups = layouts.q3_groups(k)
    row_bytes, row_scales = groups * 24, groups * 2
    out = np.zeros(layouts.q3_byte_size(rows, k), dtype=np.uint8)
    out[:rows * row_bytes] = blob[first * row_bytes:(first + rows) * row_bytes]
    src, dst = layouts.q3_scale_offset(n, k), layouts.q3_scale_offset(rows, k)
    out[dst:dst + rows * row_scales] = blob[src + first * row_scales:src + (first + rows) * row_scales]
    return out


def trellis_rows(payload: np.ndarray, suh: np.ndarray, svh: np.ndarray, ends, first: int, rows: int):
    """(payload, suh, svh, ends) of output columns [first, first + rows): tile columns cut per k-tile row, svh cut,
    the suh rows of the segments touched and their ends rebased. Both ends must be segment boundaries (or 0 and n)."""
    kt, nt, w = payload.shape
    n, last = nt * 16, first + rows
    ends = [int(e) for e in ends]
    if first < 0 or rows <= 0 or last > n or first % 16 or rows % 16:
        raise ValueError(f"rows {first}..{last} are outside the object")
    bounds = [0] + ends
    if first not in bounds or last not in bounds:
        raise ValueError(f"rows {first}..{last} do not start and end on segment boundaries {ends}")
    lo, hi = bounds.index(first), bounds.index(last)
    cut = [e - first for e in ends[lo:hi]]
    suh = np.asarray(suh).reshape(len(ends), -1)
    return (np.ascontiguousarray(payload[:, first // 16:last // 16, :]), np.ascontiguousarray(suh[lo:hi]),
            np.ascontiguousarray(np.asarray(svh)[first:last]), cut)


def gather_columns(local, world_size: int, group=None):
    """All-gather of the [rows, n / world_size] output slices into [rows, n] (column concatenation). `local` is a torch
    tensor; with world_size 1 it is returned as it is."""
    if world_size == 1:
        return local
    import torch
    import torch.distributed as dist
    rows, width = local.shape
    # Gathered as raw bytes: the slices are BF16 bit patterns, and every backend moves uint8.
    flat = local.contiguous().view(torch.uint8).reshape(rows, -1)
    gathered = torch.empty((world_size * rows, flat.shape[1]), dtype=torch.uint8, device=local.device)
    dist.all_gather_into_tensor(gathered, flat, group=group)
    joined = gathered.reshape(world_size, rows, -1).permute(1, 0, 2).reshape(rows, -1).contiguous()
    return joined.view(local.dtype).reshape(rows, world_size * width)


def gather_packed(packed, gathered, group=None):
    """One all-gather of a rank's packed output slices (1-D) into `gathered` (world_size times as long, rank-major): the
    decode-sized slices of a whole step travel in one collective, because at a few KB each the collective's latency,
    not its bandwidth, is the cost. Rank r's slice of output j is at r * len(packed) + offset_j."""
    import torch
    import torch.distributed as dist
    dist.all_gather_into_tensor(gathered.view(torch.uint8), packed.view(torch.uint8), group=group)
    return gathered
