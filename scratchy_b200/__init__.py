"""scratchy_b200 — B200 (sm_100a) quantized `Linear` kernels behind Scratchy's operator API.

The product is the C-ABI shared library ``libscratchy_cuda.so`` (sources in ``csrc/``,
declarations in ``include/scratchy_cuda.h``).  This package is the host-side mirror of the
reference's layer/loader interface for the quantized-linear path, used by the tests and
the benchmark; PyTorch only supplies device memory, streams and ``torch.distributed``.
There is no CPU fallback: every call fails loudly if the CUDA library is missing.
"""
from ._lib import ScratchyCudaError, lib, lib_path, Context  # noqa: F401
from .layers import (  # noqa: F401
    AffineQuantEmbedding, AffineQuantLinear, AffineTape, Fp8Linear, Fp8ActPack, GpuWeights, LinearLayer,
    load_layered_linear_affine_quant, load_layered_linear_fp8_dynamic,
)
