"""B200-native (sm_100a) quantized-weight matmul for Euhedral: the dequantisation-fused decode GEMV (NVFP4, Q3,
trellis) and the NVFP4 prefill GEMM, behind the reference's C ABI for linears (include/euhedral_cuda.h).

`library` binds the C ABI with ctypes (the role the reference's Java FFM layer plays), `layouts` holds the byte
geometry of the weight formats, `formats` mirrors the reference's weight-format operators (LinearFormat) and
`sharding` splits tensors along N for multi-GPU runs. There is no CPU fallback: without the built CUDA library, or
without a B200, every operator raises."""

from euhedral_b200 import layouts  # noqa: F401

__all__ = ["layouts"]
