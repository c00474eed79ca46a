"""Reader of the EDRL v2 artifact container: header, metadata, tensor table and block-aligned payloads, as the
reference's converter writes it (tools/euhedral_artifacts/edrl.py:11-138: big-endian header `>iiqqqiiq` of 48 bytes -
magic 0x5157454E, version 2, metadata offset and size, table offset, object count, a reserved zero, data offset - then
per object: name, rank, dimensions, source dtype, format and layout ordinals, payload offset and byte size). The reader
gives the quantized linears of an artifact to the operators of this package: a payload is handed over as the bytes the
kernels consume, unchanged.
"""

from __future__ import annotations

import mmap
import struct
from dataclasses import dataclass
from pathlib import Path

import numpy as np

from euhedral_b200 import layouts

MAGIC = 0x5157454E
VERSION = 2
HEADER_SIZE = 48
HEADER_FORMAT = ">iiqqqiiq"
PAYLOAD_ALIGNMENT = 4096

DTYPES = ("BF16", "FP16", None, None, None, None, "INT32")                           # ordinals 0, 1 and 6 are in use
FORMATS = ("BF16", "FP16", "FP32", "I32", "Q3G64_F16S", "Q4G64_F16S", "Q5G64_F16S", "NVFP4", "TRELLIS")
LAYOUTS = ("contiguous-le-v1", "row-split-k128-v1", "row-split-p2e2-v1", "row-split-k128-sd4-v1", "row-interleaved-nvfp4-v1",
           "trellis-tile16-v1")
ELEMENT_BYTES = {"BF16": 2, "FP16": 2, "FP32": 4, "I32": 4}


class ArtifactError(ValueError):
    pass


@dataclass(frozen=True)
class TensorEntry:
    name: str
    shape: tuple[int, ...]
    dtype: str | None
    format: str
    layout: str
    offset: int
    byte_size: int

    def expected_byte_size(self) -> int | None:
        """The byte size the layout rules give for this entry, where this package knows the layout."""
        if self.layout == "contiguous-le-v1" and self.format in ELEMENT_BYTES:
            return int(np.prod(self.shape)) * ELEMENT_BYTES[self.format]
        if self.layout == "row-split-k128-v1" and len(self.shape) == 2:
            if self.format == "NVFP4":
                return layouts.nvfp4_byte_size(*self.shape)
            if self.format == "Q3G64_F16S":
                return layouts.q3_byte_size(*self.shape)
        if self.layout == "trellis-tile16-v1" and self.format == "TRELLIS" and len(self.shape) == 3:
            return int(np.prod(self.shape)) * 2
        return None


class Artifact:
    """An opened artifact: `entries` in table order, `metadata` bytes, payloads read through a read-only memory map."""

    def __init__(self, path):
        self.path = Path(path)
        self._file = self.path.open("rb")
        try:
            self._map = mmap.mmap(self._file.fileno(), 0, access=mmap.ACCESS_READ)
        except ValueError as error:
            self._file.close()
            raise ArtifactError("input is not an EDRL v2 artifact") from error
        try:
            self._parse()
        except Exception:
            self.close()
            raise

    def _parse(self) -> None:
        data = self._map
        if len(data) < HEADER_SIZE:
            raise ArtifactError("input is not an EDRL v2 artifact")
        magic, version, metadata_offset, metadata_size, table_offset, count, reserved, data_offset = struct.unpack_from(HEADER_FORMAT, data, 0)
        if magic != MAGIC or version != VERSION or reserved != 0:
            raise ArtifactError("input is not an EDRL v2 artifact")
        if not (0 <= metadata_offset <= metadata_offset + metadata_size <= len(data)) or not (0 <= table_offset <= data_offset <= len(data)) or count < 0:
            raise ArtifactError("EDRL header points outside the file")
        self.metadata = bytes(data[metadata_offset:metadata_offset + metadata_size])
        self.data_offset = data_offset
        cursor = table_offset
        entries = []

        def take(fmt):
            nonlocal cursor
            size = struct.calcsize(fmt)
            if cursor + size > data_offset:
                raise ArtifactError("the tensor table runs past the data offset")
            values = struct.unpack_from(fmt, data, cursor)
            cursor += size
            return values

        for _ in range(count):
            (name_size,) = take(">i")
            if name_size <= 0 or cursor + name_size > data_offset:
                raise ArtifactError("bad tensor name in the table")
            name = bytes(data[cursor:cursor + name_size]).decode("utf-8")
            cursor += name_size
            (rank,) = take(">i")
            if rank <= 0 or rank > 8:
                raise ArtifactError(f"bad rank for {name}")
            shape = take(f">{rank}q")
            dtype, fmt, layout, offset, size = take(">iiiqq")
            if not (0 <= fmt < len(FORMATS)) or not (0 <= layout < len(LAYOUTS)) or not (0 <= dtype < len(DTYPES)):
                raise ArtifactError(f"unknown ordinal in the entry of {name}")
            if any(d <= 0 for d in shape) or offset < data_offset or offset % PAYLOAD_ALIGNMENT or size < 0 or offset + size > len(data):
                raise ArtifactError(f"the payload of {name} is misplaced")
            entries.append(TensorEntry(name, tuple(int(d) for d in shape), DTYPES[dtype], FORMATS[fmt], LAYOUTS[layout], offset, size))
        if cursor != data_offset:
            raise ArtifactError("unexpected gap between the tensor table and the data")
        for entry in entries:
            expected = entry.expected_byte_size()
            if expected is not None and expected != entry.byte_size:
                raise ArtifactError(f"{entry.name}: {entry.byte_size} bytes stored, the layout gives {expected}")
        self.entries = entries
        self._by_name = {entry.name: entry for entry in entries}

    def close(self) -> None:
        try:
            self._map.close()
        finally:
            self._file.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def __contains__(self, name: str) -> bool:
        return name in self._by_name

    def entry(self, name: str) -> TensorEntry:
        try:
            return self._by_name[name]
        except KeyError:
            raise KeyError(f"{self.path.name} holds no object named {name}") from None

    def payload(self, name: str) -> np.ndarray:
        """A copy of the object's bytes as a uint8 array (exactly what a kernel of the object's format consumes)."""
        entry = self.entry(name)
        return np.frombuffer(self._map, dtype=np.uint8, count=entry.byte_size, offset=entry.offset).copy()

    def linears(self, fmt: str | None = None) -> list[TensorEntry]:
        """The two-dimensional quantized objects (optionally of one format), in table order."""
        return [e for e in self.entries if len(e.shape) == 2 and e.format in ("NVFP4", "Q3G64_F16S") and fmt in (None, e.format)]

    def to_device(self, name: str, device="cuda"):
        """(TensorHandle, device tensor) of an object for the operators in `formats`: the payload copied to `device`."""
        import torch

        from euhedral_b200.formats import TensorHandle
        entry = self.entry(name)
        tensor = torch.from_numpy(self.payload(name)).to(device)
        return TensorHandle(entry.name, entry.shape, tensor.data_ptr(), entry.byte_size), tensor


def open_artifact(path) -> Artifact:
    return Artifact(path)
