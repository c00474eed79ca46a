"""Helpers of the GPU parity tests: device buffers through torch, calls through the C ABI mirror."""

from __future__ import annotations

import numpy as np

from oracle import oracle_np as O


def torch_cuda():
    import torch
    if not torch.cuda.is_available():
        raise RuntimeError("these tests need a CUDA device")
    return torch


class Device:
    """A CudaGpuMemory with torch-owned buffers; every call is queued on a side stream of its own."""

    def __init__(self):
        from euhedral_b200.gpu import CudaGpuMemory
        self.torch = torch_cuda()
        self.gpu = CudaGpuMemory()
        self.side = self.torch.cuda.Stream()   # the library takes a real stream handle, not the default stream's 0
        self.keep = []

    def put(self, array: np.ndarray):
        array = np.ascontiguousarray(array)
        tensor = self.torch.from_numpy(array.view(np.uint8).reshape(-1).copy()).cuda()
        self.keep.append(tensor)
        return tensor

    def empty(self, byte_size: int, fill: int = 0xA5):
        tensor = self.torch.full((max(byte_size, 1),), fill, dtype=self.torch.uint8, device="cuda")
        self.keep.append(tensor)
        return tensor

    def get(self, tensor, dtype, shape) -> np.ndarray:
        self.torch.cuda.synchronize()
        count = int(np.prod(shape)) * np.dtype(dtype).itemsize
        return tensor[:count].cpu().numpy().view(dtype).reshape(shape).copy()

    def stream(self) -> int:
        return self.side.cuda_stream

    def submit(self, pdl: bool = False, row_exact: bool = False):
        self.torch.cuda.current_stream().synchronize()   # uploads ran on torch's stream
        return self.gpu.submit(self.stream(), pdl=pdl, row_exact=row_exact)

    def release(self):
        self.torch.cuda.synchronize()
        self.keep.clear()


def random_x(rng, rows: int, k: int) -> np.ndarray:
    return O.bf16_bits(rng.standard_normal((rows, k)).astype(np.float32))


def elementwise_bound(y: np.ndarray) -> np.ndarray:
    """The reference's decode tolerance (native/tests/test_nvfp4.py:102-105): |y| 2^-7 + max|y| 1e-3."""
    return np.abs(y) * 2.0 ** -7 + np.max(np.abs(y)) * 1e-3


def max_relative_error(got: np.ndarray, expect: np.ndarray) -> float:
    return float(np.max(np.abs(got - expect)) / np.max(np.abs(expect)))
