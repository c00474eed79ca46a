"""Weight-format operators of the quantized-linear path: the Python mirror of the reference's `LinearFormat`
implementations (core/.../artifact/format/{LinearFormat,Nvfp4Format,GroupedLinearFormat,TrellisFormat}.java), same
method names in snake case, same routing and the same launch plans. A format turns one `LinearLaunch` into calls on
the GPU binding (`gpu.CudaGpuMemory`)."""

from __future__ import annotations

from dataclasses import dataclass, field

from euhedral_b200 import layouts
from euhedral_b200.gpu import CudaGpuMemory, KernelArguments


@dataclass(frozen=True)
class TensorHandle:
    """A resident tensor (core/.../artifact/TensorHandle.java): shape, device address and byte size."""
    name: str
    shape: tuple[int, ...]
    device_address: int
    byte_size: int


@dataclass
class LinearLaunch:
    """One linear to queue (core/.../artifact/format/LinearLaunch.java): BF16 `input` [rows, in_features] and `output`
    [rows, out_features] device addresses, the weight tensors, caller scratch and whether rows must be row-exact."""
    input: int
    output: int
    weights: list[TensorHandle]
    rows: int
    in_features: int
    out_features: int
    scratch: int = 0
    scratch_bytes: int = 0
    row_exact: bool = False
    host_mapped: bool = False
    segment_ends: list[int] | None = None


@dataclass(frozen=True)
class TrellisSettings:
    """kernels.trellis.* (core/.../settings/TrellisSettings.java:29-62): K-split target blocks (auto = 8 per SM), the row
    counts from which the whole-K kernels and their wide variant take over, and the most rows of the tensor-core route."""
    target_ctas: int
    mma_max_rows: int = 512
    whole_k_rows: int = 64
    whole_k_wide_rows: int = 128

    @staticmethod
    def for_device(multiprocessors: int) -> "TrellisSettings":
        return TrellisSettings(target_ctas=8 * multiprocessors)


class Nvfp4Format:
    """NVFP4 in its plain layout (row-split-k128-v1) or with table-indexed block scales (row-split-k128-sd4-v1); the
    library tells them apart by the tensor's byte size (Nvfp4Format.java:20-60,160-202)."""

    def __init__(self, sd4: bool = False):
        self.sd4 = sd4

    def byte_size(self, shape) -> int:
        size = layouts.nvfp4_sd4_byte_size if self.sd4 else layouts.nvfp4_byte_size
        return size(shape[0], shape[1])

    def accepts_byte_size(self, shape, byte_size: int) -> bool:
        return byte_size == self.byte_size(shape)

    def row_exact(self, rows: int) -> bool:
        return rows <= 32

    def scratch_bytes(self, gpu: CudaGpuMemory, rows: int, in_features: int, out_features: int) -> int:
        if rows < 9:
            return 0
        return gpu.lib.euhedral_cuda_nvfp4_native_scratch_bytes(rows, in_features, out_features)

    def linear(self, gpu: CudaGpuMemory, launch: LinearLaunch) -> None:
        weight = launch.weights[0]
        gpu.linear_nvfp4_bf16(launch.input, weight.device_address, launch.output, launch.rows, launch.in_features,
                              launch.out_features, weight.byte_size)


class GroupedLinearFormat:
    """Q3G64_F16S / row-split-k128-v1 (GroupedLinearFormat.java:73-84)."""

    def byte_size(self, shape) -> int:
        return layouts.q3_byte_size(shape[0], shape[1])

    def accepts_byte_size(self, shape, byte_size: int) -> bool:
        return byte_size == self.byte_size(shape)

    def row_exact(self, rows: int) -> bool:
        return rows <= 32

    def scratch_bytes(self, gpu, rows, in_features, out_features) -> int:
        return 0

    def linear(self, gpu: CudaGpuMemory, launch: LinearLaunch) -> None:
        weight = launch.weights[0]
        gpu.linear_q3_bf16(launch.input, weight.device_address, launch.output, launch.rows, launch.in_features,
                           launch.out_features, weight.byte_size)


class TrellisFormat:
    """TRELLIS / trellis-tile16-v1 (TrellisFormat.java:299-303,369-417,484-567). An object is four tensors:
    [payload int16 [k/16, n/16, w], suh f16 [s, k], svh f16 [n], segments i32 [s]]."""

    PREPASS_BLOCK_COLUMNS = 512
    EPILOGUE_BLOCK_COLUMNS = 512
    FRAGMENT_FP16, COLUMN_BF16, BLOCK_FP8 = 0, 1, 2
    MAX_GRID_ROWS = 65535

    def __init__(self, settings: TrellisSettings):
        self.settings = settings

    @staticmethod
    def splits(k: int, n: int, target_ctas: int) -> int:
        blocks = n // layouts.TRELLIS_BLOCK
        wanted = (target_ctas + blocks - 1) // blocks
        return max(1, min(wanted, k // 256))

    def byte_size(self, shape) -> int:
        kt, nt, w = shape
        return kt * nt * w * 2

    def mma_bytes(self, rows: int, k: int, n: int, segments: int) -> int:
        activations = layouts.align_up(segments * rows * k * 2, layouts.SCRATCH_ALIGNMENT)
        splits = self.splits(k, n, self.settings.target_ctas)
        split_rows = min(rows, self.settings.whole_k_rows - 1)
        if splits == 1 or split_rows == 0:
            return activations
        return activations + splits * split_rows * n * 4

    def scratch_bytes(self, gpu, rows: int, in_features: int, out_features: int, segments: int = 1, row_exact: bool = True) -> int:
        """What a linear of `rows` rows needs: the tensor-core route's activations and partial sums, or - beyond its row
        limit and not row-exact - the prefill plan's rotated activations and decoded weight."""
        if not row_exact and rows >= self.settings.whole_k_rows:
            return gpu.lib.euhedral_b200_prefill_trellis_scratch_bytes(rows, in_features, out_features, segments)
        return self.mma_bytes(rows, in_features, out_features, segments)

    def row_exact(self, rows: int) -> bool:
        return True

    def linear(self, gpu: CudaGpuMemory, launch: LinearLaunch) -> None:
        if len(launch.weights) != 4:
            raise ValueError(f"a trellis linear takes [object, suh, svh, segments]: {len(launch.weights)} tensors")
        payload, suh, svh, ends = launch.weights
        rows, k, n = launch.rows, launch.in_features, launch.out_features
        kt, nt, w = payload.shape
        if (nt * 16, kt * 16) != (n, k):
            raise ValueError(f"trellis object {payload.name} is not {n} x {k}")
        if rows <= 0 or rows > self.MAX_GRID_ROWS:
            raise ValueError(f"a trellis launch takes 1..{self.MAX_GRID_ROWS} rows: {rows}")
        segments = suh.shape[0]
        run = _TrellisLaunch(gpu, launch, payload.device_address, suh.device_address, svh.device_address,
                             ends.device_address, rows, k, n, w, segments)
        if gpu.exact_numerics():
            run.reference()
        elif launch.row_exact or rows < self.settings.whole_k_rows:
            run.tensor_core(self.settings)
        else:
            # The reference keeps up to mma_max_rows rows on its whole-K tensor-core kernels; this build does not carry
            # those, and its prefill plan takes any row count: launches of whole_k_rows rows and more that need not be
            # row-exact run the plan. An object of one segment needs no host copy of its ends.
            bounds = launch.segment_ends if launch.segment_ends is not None or segments != 1 else [n]
            run.prefill(bounds)


@dataclass
class _TrellisLaunch:
    gpu: CudaGpuMemory
    launch: LinearLaunch
    words: int
    suh: int
    svh: int
    ends: int
    rows: int
    k: int
    n: int
    w: int
    segments: int
    launches: list = field(default_factory=list)

    def _require_scratch(self, byte_size: int) -> None:
        if self.launch.scratch == 0 or self.launch.scratch_bytes < byte_size:
            raise ValueError(f"trellis linear needs {byte_size} bytes of scratch, has {self.launch.scratch_bytes}")

    def reference(self) -> None:
        self.gpu.launch_table_kernel(
            "TRELLIS_REFERENCE", self.rows * self.n, 1, 1, 128, 1, 1, 4 * self.k,
            KernelArguments().pointer(self.launch.input).pointer(self.words).pointer(self.suh).pointer(self.svh)
            .pointer(self.ends).int32(self.segments).pointer(self.launch.output).int32(self.rows).int32(self.k)
            .int32(self.n).int32(self.w))

    def prefill(self, bounds) -> None:
        """TrellisFormat.Launch.prefill (java:569-625): the plan's launches - prepass in the BF16 column layout, the payload
        decoded to BF16, a row-exact BF16 linear per segment, the BF16 epilogue - run as one call of the library."""
        if bounds is None or len(bounds) != self.segments:
            raise ValueError("a trellis prefill launch needs the host segment ends of its object")
        layouts.trellis_validate_segments(list(bounds), self.n)
        self._require_scratch(self.gpu.lib.euhedral_b200_prefill_trellis_scratch_bytes(self.rows, self.k, self.n, self.segments))
        self.gpu.prefill_trellis_bf16(self.launch.input, self.words, self.suh, self.svh, self.ends, list(bounds), self.launch.output,
                                      self.launch.scratch, self.launch.scratch_bytes, self.rows, self.k, self.n, self.w)

    def prepass(self, activations: int, layout: int) -> None:
        self.gpu.launch_table_kernel(
            "TRELLIS_PREPASS", -(-self.k // TrellisFormat.PREPASS_BLOCK_COLUMNS), self.rows, self.segments, 128, 1, 1, 0,
            KernelArguments().pointer(self.launch.input).pointer(self.suh).pointer(activations).int32(self.rows)
            .int32(self.k).int32(self.segments).int32(layout))

    def tensor_core(self, settings: TrellisSettings) -> None:
        splits = TrellisFormat.splits(self.k, self.n, settings.target_ctas)
        activations = layouts.align_up(self.segments * self.rows * self.k * 2, layouts.SCRATCH_ALIGNMENT)
        if self.rows >= settings.whole_k_rows:
            raise NotImplementedError("the whole-K trellis kernels (64 rows and more) are not part of this build")
        partials = 0 if splits == 1 else splits * self.rows * self.n * 4
        self._require_scratch(activations + partials)
        scratch = self.launch.scratch
        self.prepass(scratch, TrellisFormat.FRAGMENT_FP16)
        self.gpu.launch_table_kernel(
            "TRELLIS_MMA", self.n // layouts.TRELLIS_BLOCK, splits, 1, 256, 1, 1, 0,
            KernelArguments().pointer(scratch).pointer(self.words).pointer(self.ends).pointer(self.svh)
            .pointer(scratch + activations).pointer(self.launch.output).int32(self.rows).int32(self.k).int32(self.n)
            .int32(self.w).int32(splits).int32(self.segments))
        if splits == 1:
            return
        self.gpu.launch_table_kernel(
            "TRELLIS_EPILOGUE", -(-self.n // TrellisFormat.EPILOGUE_BLOCK_COLUMNS), self.rows, 1, 128, 1, 1, 0,
            KernelArguments().pointer(scratch + activations).int32(splits).pointer(self.svh).pointer(self.launch.output)
            .int32(self.rows).int32(self.n))
