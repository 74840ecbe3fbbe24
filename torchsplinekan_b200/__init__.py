"""B-spline KAN layers for PyTorch on NVIDIA B200 (sm_100a).

Drop-in for the ``spline_kan`` package of torch-spline-kan: same classes,
constructor arguments, state-dict keys and operator names; the native backend
is a C-ABI CUDA library (``lib/libkan_b200.so``) written for Blackwell.
"""

__version__ = "0.1.0"
