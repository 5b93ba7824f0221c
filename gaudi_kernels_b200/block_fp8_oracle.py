"""Import-path alias: `from gaudi_kernels_b200.block_fp8_oracle import reference` mirrors
`from gaudi_kernels.block_fp8_oracle import reference` of tracycam/gaudi-kernels, but runs on the GPU."""

from .block_fp8_gemm import reference

__all__ = ["reference"]
