"""B-spline KAN layers for PyTorch on NVIDIA B200 (sm_100a).

Drop-in for the ``spline_kan`` package of torch-spline-kan: same classes,
constructor arguments, state-dict keys and operator names; the native backend
is a C-ABI CUDA library (``lib/libkan_b200.so``) written for Blackwell, reached
through a thin compiled PyTorch operator layer (``_C``: ``torch.ops.spline_kan.*``,
the autograd node, the reference's pybind names).
Importing the package loads both and fails if they have not been built
(``python torchsplinekan_b200/build.py``); there is no fallback implementation
of the native operators.
"""
import torch as _torch                # noqa: F401  (the compiled operator layer links libtorch)

try:
    from . import _C                  # noqa: F401  (compiled: loads lib/libkan_b200.so, registers torch.ops.spline_kan.*)
except ImportError as exc:            # no fallback: say how to build and stop
    raise ImportError(
        "torchsplinekan_b200: the compiled operator layer (_C) or lib/libkan_b200.so is missing or stale; "
        "build them with `python torchsplinekan_b200/build.py` (needs nvcc and g++).  "
        f"This package has no fallback implementation.  [{exc}]") from exc
from .kan_linear import KANLinear
from .kan import KAN
from .data_parallel import GradientBucket, HostBatchPrefetcher, global_edge_means, shard_rows
from .pruning import PruneResult, prune_nodes

__version__ = "0.1.0"

__all__ = ["KANLinear", "KAN", "PruneResult", "prune_nodes", "GradientBucket", "HostBatchPrefetcher", "shard_rows", "global_edge_means",
           "__version__"]
