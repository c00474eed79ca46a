"""Generates the golden vectors under tests/golden from the reference itself.

Run where the reference checkout is mounted (argument 1 or $EUHEDRAL_REFERENCE name its root):

    python tests/golden/make_golden.py [reference_root]

It imports the reference's Python converter (tools/euhedral_artifacts/{nvfp4,grouped}.py) and its NumPy trellis
decoder (native/tests/trellis_reference.py) unchanged, runs them on seeded inputs, and stores inputs and outputs as
small .npz files. It also stores subsets of the reference's own golden files (GPTQ decode fixtures, trellis tile
fixtures). The tests then check the CPU oracle against these files without needing the reference checkout.
"""

from __future__ import annotations

import io
import os
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
ROOT = Path(sys.argv[1] if len(sys.argv) > 1 else os.environ.get("EUHEDRAL_REFERENCE", "/root/reference"))
sys.path.insert(0, str(ROOT / "tools"))
sys.path.insert(0, str(ROOT / "native" / "tests"))

from euhedral_artifacts import grouped, nvfp4  # noqa: E402
from euhedral_artifacts.sources import MatrixSource  # noqa: E402
import trellis_reference as tref  # noqa: E402


def matrix_source(weights: np.ndarray):
    try:
        return MatrixSource(weights.shape, lambda a, b: weights[a:b])
    except TypeError:
        return MatrixSource(shape=weights.shape, read_rows=lambda a, b: weights[a:b])


def nvfp4_cases():
    rng = np.random.default_rng(0xE0)
    out = {}
    # (rows, K): K a multiple of 128; one K that needs padding.
    weights = {
        "gauss": (rng.standard_normal((24, 256)) * 0.02).astype(np.float32),
        "spread": (rng.standard_normal((16, 384)) * np.exp(rng.uniform(-6.0, 1.0, (16, 1)))).astype(np.float32),
        "padded": (rng.standard_normal((8, 200)) * 0.02).astype(np.float32),
    }
    # Edge rows: zeros, a lone outlier, exact ties of the E2M1 grid, tiny blocks that hit E4M3 subnormals.
    edge = np.zeros((8, 128), dtype=np.float32)
    edge[1, 5] = 3.0
    edge[2, :16] = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, -0.25, -0.75, -1.25, -1.75, -2.5, -3.5, -5.0,
                             -6.0], dtype=np.float32) * 0.5
    edge[3, :] = 1e-6
    edge[4, :] = np.linspace(-1.0, 1.0, 128, dtype=np.float32) * 1e-4
    edge[5, 16:32] = 6.0
    edge[6, :] = rng.standard_normal(128).astype(np.float32) * 1e-3
    edge[7, ::2] = -0.0
    weights["edge"] = edge
    for name, w in weights.items():
        buffer = io.BytesIO()
        nvfp4.quantize_nvfp4_matrix(buffer, 0, matrix_source(w))
        blob = buffer.getvalue()
        n, k = w.shape
        kp = (k + 127) // 128 * 128
        scale_off, global_off, size = nvfp4.nvfp4_offsets((n, k))
        blob = blob.ljust(size, b"\0")
        raw = np.frombuffer(blob, dtype=np.uint8)
        packed = raw[:n * kp // 2].reshape(n, kp // 2)
        scales = raw[scale_off:scale_off + n * kp // 16].reshape(n, kp // 16)
        g = np.frombuffer(blob[global_off:global_off + 4], dtype="<f4")[0]
        dense = nvfp4.dequantize_nvfp4_rows(packed, scales, np.float32(g))
        out[f"{name}_weights"] = w
        out[f"{name}_blob"] = raw.copy()
        out[f"{name}_dense"] = dense
    # Table rounding, including every tie.
    probe = np.concatenate([nvfp4.E4M3_VALUES, (nvfp4.E4M3_VALUES[:-1] + nvfp4.E4M3_VALUES[1:]) / 2,
                            rng.uniform(0, 500, 512).astype(np.float32),
                            np.exp(rng.uniform(-12, 7, 512)).astype(np.float32)]).astype(np.float32)
    out["e4m3_probe"] = probe
    out["e4m3_codes"] = nvfp4.round_to_table(probe, nvfp4.E4M3_VALUES)
    probe2 = np.concatenate([nvfp4.E2M1_VALUES, (nvfp4.E2M1_VALUES[:-1] + nvfp4.E2M1_VALUES[1:]) / 2,
                             rng.uniform(0, 8, 512).astype(np.float32)]).astype(np.float32)
    out["e2m1_probe"] = probe2
    out["e2m1_codes"] = nvfp4.round_to_table(probe2, nvfp4.E2M1_VALUES)
    out["e4m3_table"] = nvfp4.E4M3_VALUES
    shapes = np.array([(3, 1024), (17408, 5120), (5120, 17408), (1024, 5120), (5120, 5120), (32, 640), (7, 200)])
    out["offset_shapes"] = shapes
    out["offsets"] = np.array([nvfp4.nvfp4_offsets((int(n), int(k))) for n, k in shapes], dtype=np.int64)
    np.savez_compressed(HERE / "nvfp4.npz", **out)


def sd4_cases():
    """NVFP4 with table-indexed scales, written by the reference's converter (table search included), and its values."""
    rng = np.random.default_rng(0xD4)
    out = {}
    weights = {
        "gauss": (rng.standard_normal((24, 256)) * 0.02).astype(np.float32),
        "spread": (rng.standard_normal((16, 384)) * np.exp(rng.uniform(-6.0, 1.0, (16, 1)))).astype(np.float32),
        "padded": (rng.standard_normal((8, 200)) * 0.02).astype(np.float32),
    }
    for name, w in weights.items():
        buffer = io.BytesIO()
        nvfp4.quantize_nvfp4_sd4_matrix(buffer, 0, matrix_source(w))
        n, k = w.shape
        kp = (k + 127) // 128 * 128
        index_off, table_off, size = nvfp4.nvfp4_sd4_offsets((n, k))
        blob = buffer.getvalue().ljust(size, b"\0")
        raw = np.frombuffer(blob, dtype=np.uint8)
        packed = raw[:n * kp // 2].reshape(n, kp // 2)
        indices = raw[index_off:index_off + n * kp // 32].reshape(n, kp // 32)
        table = raw[table_off:table_off + 16]
        g = np.frombuffer(blob[table_off + 16:table_off + 20], dtype="<f4")[0]
        out[f"{name}_weights"] = w
        out[f"{name}_blob"] = raw.copy()
        out[f"{name}_dense"] = nvfp4.dequantize_nvfp4_rows(packed, nvfp4.expand_nvfp4_sd4(indices, table), np.float32(g))
    shapes = np.array([(3, 1024), (17408, 5120), (5120, 17408), (1024, 5120), (32, 640), (7, 200)])
    out["offset_shapes"] = shapes
    out["offsets"] = np.array([nvfp4.nvfp4_sd4_offsets((int(n), int(k))) for n, k in shapes], dtype=np.int64)
    np.savez_compressed(HERE / "nvfp4_sd4.npz", **out)


def q3_cases():
    rng = np.random.default_rng(0xE1)
    out = {}
    weights = {
        "gauss": (rng.standard_normal((24, 256)) * 0.02).astype(np.float32),
        "spread": (rng.standard_normal((16, 1024)) * np.exp(rng.uniform(-6.0, 1.0, (16, 1)))).astype(np.float32),
        "padded": (rng.standard_normal((8, 200)) * 0.02).astype(np.float32),
    }
    edge = np.zeros((6, 128), dtype=np.float32)
    edge[1, 3] = 1.0
    edge[2, :] = 1e-9  # scale underflows FP16 -> 2^-24
    edge[3, :64] = np.linspace(-3.5, 3.5, 64, dtype=np.float32)  # ties of rint
    edge[4, :] = rng.standard_normal(128).astype(np.float32) * 100.0
    edge[5, 64:] = -2.0
    weights["edge"] = edge
    for name, w in weights.items():
        buffer = io.BytesIO()
        grouped.quantize_matrix(buffer, 0, matrix_source(w), "Q3G64_F16S")
        n, k = w.shape
        size = grouped.row_split_size((n, k), "Q3G64_F16S")
        blob = buffer.getvalue().ljust(size, b"\0")
        out[f"{name}_weights"] = w
        out[f"{name}_blob"] = np.frombuffer(blob, dtype=np.uint8).copy()
    shapes = np.array([(3, 1024), (17408, 5120), (5120, 17408), (1024, 5120), (5120, 5120), (32, 640), (7, 200)])
    out["size_shapes"] = shapes
    out["sizes"] = np.array([grouped.row_split_size((int(n), int(k)), "Q3G64_F16S") for n, k in shapes], dtype=np.int64)
    # pack order
    codes = rng.integers(-4, 4, size=(5, 64)).astype(np.int8)
    out["pack_codes"] = codes
    out["pack_bytes"] = np.frombuffer(grouped.pack_codes(codes, 3)[0], dtype=np.uint8).reshape(5, 24)
    np.savez_compressed(HERE / "q3.npz", **out)


def gptq_fixture_subset():
    """The reference's GPTQ golden files pin the decode of stored codes to values (rows 0..15 kept)."""
    source = ROOT / "quantization/src/test/resources/gptq-fixture"
    out = {}
    for stem in ("NVFP4-row-split-k128-v1-seq", "Q3G64_F16S-row-split-k128-v1-seq", "Q3G64_F16S-row-split-k128-v1-act"):
        for part in ("codes", "scales", "decoded"):
            out[f"{stem}-{part}"] = np.load(source / f"{stem}-{part}.npy")[:16]
    out["nvfp4_global_scale"] = np.float64(0.01413690485060215)  # cases.json
    np.savez_compressed(HERE / "gptq_decode.npz", **out)


def trellis_cases():
    source = ROOT / "quantization/src/test/resources/trellis-fixture"
    rng = np.random.default_rng(0xE2)
    out = {}
    for rate, w in (("2", 32), ("2.5", 40), ("3", 48), ("3.5", 56), ("4", 64), ("5", 80), ("6", 96)):
        packed = np.load(source / f"tiles-{rate}-packed.npy")
        golden = np.load(source / f"tiles-{rate}-out.npy")
        assert np.array_equal(tref.decode_tiles(packed, w).view(np.uint16), golden.view(np.uint16))
        out[f"tiles_{w}_packed"] = packed[:12]
        out[f"tiles_{w}_out"] = golden[:12]
        out[f"tiles_{w}_idx"] = np.load(source / f"tiles-{rate}-idx.npy")[:12]    # the encoder's 16-bit states
    out["tiles_in"] = np.load(source / "tiles-in.npy")[:12]                         # what the encoder was given
    # Random words at every stored width, decoded by the reference's NumPy decoder.
    for w in range(16, 129, 8):
        words = rng.integers(-32768, 32768, size=(3, w), dtype=np.int16)
        out[f"random_{w}_words"] = words
        out[f"random_{w}_values"] = tref.decode_tiles(words, w)
    # A 256 x 256 slice of the reference's 1024 x 512 three-bit linear fixture, as an object of its own.
    payload = np.load(source / "linear-trellis.npy")[:16, :16].copy()
    suh = np.load(source / "linear-suh.npy")[:256].copy()
    svh = np.load(source / "linear-svh.npy")[:256].copy()
    x = tref.bf16_bits(rng.standard_normal((3, 256)).astype(np.float32))
    out["linear_payload"], out["linear_suh"], out["linear_svh"], out["linear_x"] = payload, suh, svh, x
    out["linear_y_f64"] = tref.linear_f64(tref.bf16_values(x), payload, suh, svh, [256])
    out["linear_q_corner"] = tref.rotated_weight(payload)[:48, :48]
    # Two segments, random object.
    payload2 = rng.integers(-32768, 32768, size=(8, 16, 40), dtype=np.int16)
    suh2 = (rng.choice([-1.0, 1.0], size=(2, 128)) * rng.uniform(0.5, 2.0, size=(2, 128))).astype(np.float16)
    svh2 = rng.uniform(0.01, 1.0, size=256).astype(np.float16)
    x2 = tref.bf16_bits(rng.standard_normal((2, 128)).astype(np.float32))
    out["seg_payload"], out["seg_suh"], out["seg_svh"], out["seg_x"] = payload2, suh2, svh2, x2
    out["seg_ends"] = np.array([128, 256], dtype=np.int32)
    out["seg_y_f64"] = tref.linear_f64(tref.bf16_values(x2), payload2, suh2, svh2, [128, 256])
    # Hadamard, fragment order, splits.
    h_in = rng.standard_normal((3, 256)).astype(np.float32)
    out["hadamard_in"], out["hadamard_out"] = h_in, tref.hadamard128_f32(h_in)
    frag = np.arange(64, dtype=np.int32)
    out["fragment_in"], out["fragment_out"] = frag, tref.fragment_order(frag)
    cases = np.array([(5120, 5120, 1184), (5120, 1024, 1184), (5120, 17408, 1184), (17408, 5120, 1184),
                      (5120, 5120, 560), (1024, 512, 140), (256, 128, 8)])
    out["splits_cases"] = cases
    out["splits"] = np.array([tref.splits(int(k), int(n), int(t)) for k, n, t in cases])
    np.savez_compressed(HERE / "trellis.npz", **out)


def edrl_fixture():
    """A small EDRL v2 container written with the reference's own table encoder and offset assignment
    (tools/euhedral_artifacts/edrl.py; the header is packed as tools/euhedral_artifacts/pipeline.py:90-91 packs it),
    holding an NVFP4 and a Q3 linear rounded by the reference's converter, a BF16 norm vector and an I32 vector."""
    import struct
    from euhedral_artifacts import edrl
    rng = np.random.default_rng(0xED)
    payloads, plans = {}, []

    def plan(name, shape, dtype, fmt, layout, blob):
        payloads[name] = blob
        plans.append(edrl.ObjectPlan(name=name, shape=tuple(shape), source_dtype=dtype, format_name=fmt, layout=layout,
                                     byte_size=len(blob), writer=None))

    w4 = (rng.standard_normal((64, 512)) * 0.02).astype(np.float32)
    buffer = io.BytesIO()
    nvfp4.quantize_nvfp4_matrix(buffer, 0, matrix_source(w4))
    plan("model.layers.0.mlp.down_proj.weight", w4.shape, "BF16", "NVFP4", "row-split-k128-v1",
         buffer.getvalue().ljust(nvfp4.nvfp4_offsets(w4.shape)[2], b"\0"))
    w3 = (rng.standard_normal((32, 1024)) * 0.02).astype(np.float32)
    buffer = io.BytesIO()
    grouped.quantize_matrix(buffer, 0, matrix_source(w3), "Q3G64_F16S")
    plan("model.layers.0.self_attn.k_proj.weight", w3.shape, "BF16", "Q3G64_F16S", "row-split-k128-v1",
         buffer.getvalue().ljust(grouped.row_split_size(w3.shape, "Q3G64_F16S"), b"\0"))
    norm = (rng.standard_normal(1024).astype(np.float32).view(np.uint32) >> 16).astype("<u2")
    plan("model.norm.weight", (1024,), "BF16", "BF16", "contiguous-le-v1", norm.tobytes())
    ids = rng.integers(0, 1000, 17).astype("<i4")
    plan("draft.token_ids", (17,), "INT32", "I32", "contiguous-le-v1", ids.tobytes())
    metadata = b'{"format":"edrl-fixture","layers":1}'
    table_size = len(edrl.encode_table(plans))
    data_base = edrl.HEADER_SIZE + len(metadata) + table_size
    file_size = edrl.assign_offsets(plans, data_base)
    table = edrl.encode_table(plans)
    header = struct.pack(edrl.HEADER_FORMAT, edrl.MAGIC, edrl.VERSION, edrl.HEADER_SIZE, len(metadata), edrl.HEADER_SIZE + len(metadata),
                         len(plans), 0, data_base)
    image = bytearray(file_size)
    image[:len(header)] = header
    image[edrl.HEADER_SIZE:edrl.HEADER_SIZE + len(metadata)] = metadata
    image[edrl.HEADER_SIZE + len(metadata):data_base] = table
    for item in plans:
        image[item.offset:item.offset + item.byte_size] = payloads[item.name]
    (HERE / "tiny.edrl").write_bytes(bytes(image))
    with (HERE / "tiny.edrl").open("rb") as handle:      # the reference's own reader accepts it
        _, _, objects = edrl.read_table(handle)
    out = {"nvfp4_weights": w4, "q3_weights": w3, "norm": norm, "ids": ids,
           "names": np.array([o["name"] for o in objects]), "offsets": np.array([o["offset"] for o in objects], dtype=np.int64),
           "sizes": np.array([o["bytes"] for o in objects], dtype=np.int64),
           "formats": np.array([o["format"] for o in objects], dtype=np.int64), "layouts": np.array([o["layout"] for o in objects], dtype=np.int64)}
    np.savez_compressed(HERE / "edrl.npz", **out)


if __name__ == "__main__":
    edrl_fixture()
    nvfp4_cases()
    sd4_cases()
    q3_cases()
    gptq_fixture_subset()
    trellis_cases()
    for f in sorted(HERE.glob("*.npz")):
        print(f.name, f.stat().st_size)
