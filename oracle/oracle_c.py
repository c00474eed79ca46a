"""ctypes view of liboracle.so (oracle/oracle.c), the plain-C CPU checker. TEST INFRASTRUCTURE ONLY: imported by
tests, the smoke check and the benchmark's CPU-baseline leg, never by the product package."""

from __future__ import annotations

import ctypes as C
import os
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
_LIB = None


def build() -> Path:
    subprocess.run(["make", "-C", str(HERE), "liboracle.so"], check=True, capture_output=True)
    return HERE / "liboracle.so"


def lib() -> C.CDLL:
    global _LIB
    if _LIB is None:
        path = HERE / "liboracle.so"
        if not path.exists() or path.stat().st_mtime < (HERE / "oracle.c").stat().st_mtime:
            build()
        _LIB = C.CDLL(str(path))
    return _LIB


def default_threads() -> int:
    return max(1, len(os.sched_getaffinity(0)))


def _p(array):
    return array.ctypes.data_as(C.c_void_p)


def nvfp4_size(n: int, k: int):
    a, b, c = C.c_uint64(), C.c_uint64(), C.c_uint64()
    lib().oracle_nvfp4_offsets(C.c_uint32(n), C.c_uint32(k), C.byref(a), C.byref(b), C.byref(c))
    return a.value, b.value, c.value


def nvfp4_quantize(weights: np.ndarray, threads: int | None = None) -> np.ndarray:
    weights = np.ascontiguousarray(weights, dtype=np.float32)
    n, k = weights.shape
    blob = np.zeros(nvfp4_size(n, k)[2], dtype=np.uint8)
    lib().oracle_nvfp4_quantize(_p(weights), C.c_uint32(n), C.c_uint32(k), _p(blob), C.c_int(threads or default_threads()))
    return blob


def nvfp4_dense(blob: np.ndarray, n: int, k: int, threads: int | None = None) -> np.ndarray:
    blob = np.ascontiguousarray(blob, dtype=np.uint8)
    dense = np.empty((n, k), dtype=np.float32)
    lib().oracle_nvfp4_dense(_p(blob), C.c_uint32(n), C.c_uint32(k), _p(dense), C.c_int(threads or default_threads()))
    return dense


def nvfp4_linear(x_bits: np.ndarray, blob: np.ndarray, n: int, k: int, threads: int | None = None) -> np.ndarray:
    x_bits = np.ascontiguousarray(x_bits, dtype=np.uint16)
    blob = np.ascontiguousarray(blob, dtype=np.uint8)
    rows = x_bits.shape[0]
    y = np.empty((rows, n), dtype=np.float32)
    lib().oracle_nvfp4_linear(_p(x_bits), _p(blob), _p(y), C.c_uint32(rows), C.c_uint32(k), C.c_uint32(n),
                              C.c_int(threads or default_threads()))
    return y


def q3_size(n: int, k: int):
    a, b = C.c_uint64(), C.c_uint64()
    lib().oracle_q3_offsets(C.c_uint32(n), C.c_uint32(k), C.byref(a), C.byref(b))
    return a.value, b.value


def q3_quantize(weights: np.ndarray, threads: int | None = None) -> np.ndarray:
    weights = np.ascontiguousarray(weights, dtype=np.float32)
    n, k = weights.shape
    blob = np.zeros(q3_size(n, k)[1], dtype=np.uint8)
    lib().oracle_q3_quantize(_p(weights), C.c_uint32(n), C.c_uint32(k), _p(blob), C.c_int(threads or default_threads()))
    return blob


def q3_dense(blob: np.ndarray, n: int, k: int, threads: int | None = None) -> np.ndarray:
    blob = np.ascontiguousarray(blob, dtype=np.uint8)
    dense = np.empty((n, k), dtype=np.float32)
    lib().oracle_q3_dense(_p(blob), C.c_uint32(n), C.c_uint32(k), _p(dense), C.c_int(threads or default_threads()))
    return dense


def q3_linear(x_bits: np.ndarray, blob: np.ndarray, n: int, k: int, threads: int | None = None) -> np.ndarray:
    x_bits = np.ascontiguousarray(x_bits, dtype=np.uint16)
    blob = np.ascontiguousarray(blob, dtype=np.uint8)
    rows = x_bits.shape[0]
    y = np.empty((rows, n), dtype=np.float32)
    lib().oracle_q3_linear(_p(x_bits), _p(blob), _p(y), C.c_uint32(rows), C.c_uint32(k), C.c_uint32(n),
                           C.c_int(threads or default_threads()))
    return y


def trellis_decode_tiles(words: np.ndarray, w: int) -> np.ndarray:
    words = np.ascontiguousarray(words, dtype="<i2").reshape(-1, w).view(np.uint16)
    out = np.empty((words.shape[0], 256), dtype=np.uint16)
    for i in range(words.shape[0]):
        lib().oracle_trellis_decode_tile(_p(words[i]), C.c_int(w), _p(out[i]))
    return out.view(np.float16)


def trellis_linear(x_bits, payload, suh, svh, ends, threads: int | None = None) -> np.ndarray:
    payload = np.ascontiguousarray(payload, dtype="<i2")
    kt, nt, w = payload.shape
    k, n = kt * 16, nt * 16
    x_bits = np.ascontiguousarray(x_bits, dtype=np.uint16)
    suh = np.ascontiguousarray(np.asarray(suh, dtype=np.float16).reshape(len(ends), k))
    svh = np.ascontiguousarray(svh, dtype=np.float16)
    ends = np.ascontiguousarray(ends, dtype=np.int32)
    rows = x_bits.shape[0]
    y = np.empty((rows, n), dtype=np.float32)
    lib().oracle_trellis_linear(_p(x_bits), _p(payload), _p(suh), _p(svh), _p(ends), C.c_int(len(ends)), _p(y),
                                C.c_int(rows), C.c_int(k), C.c_int(n), C.c_int(w), C.c_int(threads or default_threads()))
    return y


def trellis_encode_tiles(tiles: np.ndarray, ka: int, mask: int = 0, threads: int | None = None):
    """float32 [count, 256] tiles (kernel element order) -> (states uint16 [count, 256], decoded float32 [count, 256]):
    the reference's tail-biting Viterbi tile encoder restated (quantization/src/main/resources/cuda/trellis.cu:34-399).
    ka bits per position plus one where bit (position mod 16) of mask is set (0xAAAA: the half-step rates)."""
    tiles = np.ascontiguousarray(tiles, dtype=np.float32)
    count = tiles.shape[0]
    states = np.empty((count, 256), dtype=np.uint16)
    decoded = np.empty((count, 256), dtype=np.float32)
    lib().oracle_trellis_encode_tiles(_p(tiles), C.c_uint32(count), C.c_int(ka), C.c_uint32(mask), _p(states), _p(decoded),
                                      C.c_int(threads or default_threads()))
    return states, decoded
