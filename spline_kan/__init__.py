"""
``spline_kan``: the import name of torch-spline-kan, served by the B200-native
implementation in :mod:`torchsplinekan_b200`.

Code written against the reference package keeps working unchanged::

    from spline_kan import KANLinear, KAN, PruneResult, prune_nodes
    from spline_kan.reference_backend import compute_basis
    from spline_kan import kan_linear, fused

Every submodule name of the reference (spline_kan/__init__.py:5-11 and the
modules beside it) is an alias of the module that implements it here, so
``spline_kan.kan_linear is torchsplinekan_b200.kan_linear`` and the objects in
them are identical, not copies.
"""
import sys as _sys

import torchsplinekan_b200 as _impl
from torchsplinekan_b200 import _C, dense_backend, fused, kan, kan_linear, pruning
from torchsplinekan_b200 import KAN, KANLinear, __version__
from torchsplinekan_b200.pruning import PruneResult, prune_nodes

reference_backend = dense_backend

for _name, _mod in (("_C", _C), ("reference_backend", dense_backend), ("fused", fused), ("kan", kan),
                    ("kan_linear", kan_linear), ("pruning", pruning)):
    _sys.modules[f"{__name__}.{_name}"] = _mod
del _name, _mod

__all__ = ["KANLinear", "KAN", "PruneResult", "prune_nodes", "__version__"]
