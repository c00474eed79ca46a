"""The torch builders of synthetic tensors produce the converter's bytes (checked against the oracle)."""

import numpy as np
import torch

from euhedral_b200 import layouts, synthetic
from oracle import oracle_np as O


def test_nvfp4_bytes_equal_the_oracle():
    weights = synthetic.gaussian(48, 384, seed=3)
    weights[5] *= 40.0
    weights[7, :16] = 0.0
    blob = synthetic.nvfp4_tensor(weights).numpy()
    assert blob.tobytes() == O.nvfp4_pack(weights.numpy())


def test_q3_bytes_equal_the_oracle():
    weights = synthetic.gaussian(40, 256, seed=4)
    weights[3] = 0.0
    weights[9] *= 1e-9
    blob = synthetic.q3_tensor(weights).numpy()
    assert blob.tobytes() == O.q3_pack(weights.numpy())


def test_activations_and_trellis_shapes():
    bits = synthetic.bf16_rows(3, 256, seed=1).numpy().view(np.uint16)
    generator = torch.Generator().manual_seed(1)
    values = torch.randn((3, 256), generator=generator).numpy()
    assert np.array_equal(bits, O.bf16_bits(values))
    payload, suh, svh, ends = synthetic.trellis_object(512, 256, 48, seed=2, segments=2)
    assert payload.shape == (16, 32, 48) and suh.shape == (2, 256) and svh.shape == (512,)
    layouts.trellis_validate_segments(ends.tolist(), 512)
    assert float(suh.abs().min()) >= 0.5 and float(svh.min()) >= 0.01
