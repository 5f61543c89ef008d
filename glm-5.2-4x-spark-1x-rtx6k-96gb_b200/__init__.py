"""B200-native routed-MoE expert FFN path of GLMRT (sm_100a).

The package holds the CUDA sources of libglmrt_b200.so (``csrc/``), the script that
builds it in-tree (``build.py``) and the host-side mirror of the reference's FFI layer
(``native.py``, ``layer.py``).  Importing the package does not load the shared library;
``native.library()`` does, and raises if it has not been built -- there is no CPU fallback.
"""
from . import native  # noqa: F401

__all__ = ["native"]
