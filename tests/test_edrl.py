"""The EDRL v2 reader against a small container written with the reference's own table encoder (tests/golden/tiny.edrl,
made by tests/golden/make_golden.py) and against damaged copies of it."""

import struct

import numpy as np
import pytest

from euhedral_b200 import edrl
from oracle import oracle_np as O


@pytest.fixture()
def fixture(golden):
    from tests.conftest import GOLDEN
    return GOLDEN / "tiny.edrl", golden("edrl")


def test_table_matches_the_reference_reader(fixture):
    path, g = fixture
    with edrl.open_artifact(path) as artifact:
        assert [e.name for e in artifact.entries] == list(g["names"])
        assert [e.offset for e in artifact.entries] == list(g["offsets"])
        assert [e.byte_size for e in artifact.entries] == list(g["sizes"])
        assert [edrl.FORMATS.index(e.format) for e in artifact.entries] == list(g["formats"])
        assert [edrl.LAYOUTS.index(e.layout) for e in artifact.entries] == list(g["layouts"])
        assert artifact.metadata == b'{"format":"edrl-fixture","layers":1}'
        assert [e.name for e in artifact.linears()] == ["model.layers.0.mlp.down_proj.weight", "model.layers.0.self_attn.k_proj.weight"]
        assert [e.format for e in artifact.linears("NVFP4")] == ["NVFP4"]
        assert all(e.offset % 4096 == 0 for e in artifact.entries)
        assert np.array_equal(artifact.payload("model.norm.weight").view("<u2"), g["norm"])
        assert np.array_equal(artifact.payload("draft.token_ids").view("<i4"), g["ids"])
        with pytest.raises(KeyError):
            artifact.entry("missing")


def test_payloads_are_the_converters_bytes(fixture):
    """The stored linears are byte for byte what the restated quantizers give for the same weights, and decode to them."""
    path, g = fixture
    with edrl.open_artifact(path) as artifact:
        entry = artifact.entry("model.layers.0.mlp.down_proj.weight")
        blob = artifact.payload(entry.name)
        n, k = entry.shape
        assert blob.tobytes() == O.nvfp4_pack(g["nvfp4_weights"])
        dense = O.nvfp4_dense(blob.tobytes(), n, k)
        assert np.max(np.abs(dense - g["nvfp4_weights"])) <= np.max(np.abs(g["nvfp4_weights"])) / 6
        entry = artifact.entry("model.layers.0.self_attn.k_proj.weight")
        blob = artifact.payload(entry.name)
        assert blob.tobytes() == O.q3_pack(g["q3_weights"])


def test_damaged_containers_are_refused(fixture, tmp_path):
    path, _ = fixture
    image = bytearray(path.read_bytes())

    def refuse(edit, match):
        broken = bytearray(image)
        edit(broken)
        target = tmp_path / "broken.edrl"
        target.write_bytes(bytes(broken))
        with pytest.raises(edrl.ArtifactError, match=match):
            edrl.open_artifact(target)

    refuse(lambda b: b.__setitem__(slice(0, 4), struct.pack(">i", 0x12345678)), "not an EDRL")
    refuse(lambda b: b.__setitem__(slice(4, 8), struct.pack(">i", 3)), "not an EDRL")
    refuse(lambda b: b.__setitem__(slice(36, 40), struct.pack(">i", 1)), "not an EDRL")            # reserved field
    data_offset = struct.unpack_from(">q", image, 40)[0]
    refuse(lambda b: b.__setitem__(slice(40, 48), struct.pack(">q", data_offset + 4)), "gap")
    refuse(lambda b: b.__setitem__(slice(28, 32), struct.pack(">i", 5)), "past the data offset|bad|gap")   # object count
    target = tmp_path / "short.edrl"
    target.write_bytes(bytes(image[:20]))
    with pytest.raises(edrl.ArtifactError):
        edrl.open_artifact(target)


@pytest.mark.gpu
def test_artifact_linears_run_through_the_operators(fixture):
    """The linears of an artifact, handed to the format operators as the reader returns them, give the oracle's result."""
    from euhedral_b200.formats import GroupedLinearFormat, LinearLaunch, Nvfp4Format
    from tests.gpu_util import Device, max_relative_error, random_x
    path, _ = fixture
    dev = Device()
    try:
        with edrl.open_artifact(path) as artifact:
            for entry in artifact.linears():
                n, k = entry.shape
                operator, dense = (Nvfp4Format(), O.nvfp4_dense) if entry.format == "NVFP4" else (GroupedLinearFormat(), O.q3_dense)
                assert operator.accepts_byte_size(entry.shape, entry.byte_size)
                handle, tensor = artifact.to_device(entry.name)
                x = random_x(np.random.default_rng(n), 3, k)
                d_x, d_y = dev.put(x), dev.empty(3 * n * 2)
                with dev.submit(row_exact=True) as gpu:
                    operator.linear(gpu, LinearLaunch(d_x.data_ptr(), d_y.data_ptr(), [handle], 3, k, n, row_exact=True))
                got = O.bf16_to_f32(dev.get(d_y, np.uint16, (3, n))).astype(np.float64)
                expect = O.linear_f64(x, dense(artifact.payload(entry.name).tobytes(), n, k))
                assert max_relative_error(got, expect) <= 2e-3 + 2.0 ** -8
                del tensor
        assert dev.gpu.take_device_error() == 0
    finally:
        dev.release()
