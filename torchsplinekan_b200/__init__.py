"""B-spline KAN layers for PyTorch on NVIDIA B200 (sm_100a).

Drop-in for the ``spline_kan`` package of torch-spline-kan: same classes,
constructor arguments, state-dict keys and operator names; the native backend
is a C-ABI CUDA library (``lib/libkan_b200.so``) written for Blackwell.
Importing the package loads that library and fails if it has not been built
(``python torchsplinekan_b200/build.py``); there is no fallback implementation
of the native operators.
"""
from . import _C                      # noqa: F401  (loads the library, registers torch.ops.spline_kan.*)
from .kan_linear import KANLinear
from .kan import KAN
from .data_parallel import GradientBucket, HostBatchPrefetcher, shard_rows

__version__ = "0.1.0"

__all__ = ["KANLinear", "KAN", "GradientBucket", "HostBatchPrefetcher", "shard_rows", "__version__"]
