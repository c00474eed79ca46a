"""N-sharding on CPU: the shard cutters produce self-contained tensors (checked with the oracle) and the all-gather of
output slices reassembles [rows, N] on two gloo ranks."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from euhedral_b200 import layouts, sharding
from oracle import oracle_c as OC
from oracle import oracle_np as O


def test_shard_range_and_errors():
    assert sharding.shard_range(17408, 8, 3, 128) == (3 * 2176, 2176)
    with pytest.raises(ValueError):
        sharding.shard_range(1000, 3, 0, 16)
    with pytest.raises(ValueError):
        sharding.shard_range(1024, 8, 0, 256)       # 128 rows per shard is not a whole 256-row unit


@pytest.mark.parametrize("fmt", ["nvfp4", "q3"])
def test_row_shards_are_self_contained_tensors(fmt):
    rng = np.random.default_rng(5)
    n, k = 96, 384
    weights = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    quantize, cut, dense, size = ((OC.nvfp4_quantize, sharding.nvfp4_rows, O.nvfp4_dense, layouts.nvfp4_byte_size) if fmt == "nvfp4"
                                  else (OC.q3_quantize, sharding.q3_rows, O.q3_dense, layouts.q3_byte_size))
    blob = quantize(weights)
    whole = dense(blob.tobytes(), n, k)
    for first, rows in ((0, 32), (32, 32), (64, 32), (16, 48)):
        part = cut(blob, n, k, first, rows)
        assert part.size == size(rows, k)
        assert np.array_equal(dense(part.tobytes(), rows, k), whole[first:first + rows])


def test_trellis_column_shards():
    rng = np.random.default_rng(6)
    k, n, w = 128, 512, 40
    payload = rng.integers(-32768, 32768, size=(k // 16, n // 16, w), dtype=np.int16)
    suh = rng.uniform(0.5, 2.0, size=(2, k)).astype(np.float16)
    svh = rng.uniform(0.01, 1.0, size=n).astype(np.float16)
    ends = [256, 512]
    x = O.bf16_bits(rng.standard_normal((2, k)).astype(np.float32))
    whole = O.trellis_linear_f64(x, payload, suh, svh, ends)
    for first in (0, 256):
        p, s, v, e = sharding.trellis_rows(payload, suh, svh, ends, first, 256)
        assert e == [256] and s.shape == (1, k)
        assert np.allclose(O.trellis_linear_f64(x, p, s, v, e), whole[:, first:first + 256], rtol=0, atol=0)
    with pytest.raises(ValueError):
        sharding.trellis_rows(payload, suh, svh, ends, 128, 256)      # not on a segment boundary


def _rank(rank, world, port, results):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    rows, n = 3, 64
    full = torch.arange(rows * n, dtype=torch.int16).reshape(rows, n)
    first, width = sharding.shard_range(n, world, rank, 16)
    gathered = sharding.gather_columns(full[:, first:first + width].contiguous(), world)
    results[rank] = bool(torch.equal(gathered, full))
    dist.destroy_process_group()


def test_all_gather_of_output_slices_on_two_gloo_ranks():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_rank, args=(2, port, results), nprocs=2, join=True)
    assert dict(results) == {0: True, 1: True}
