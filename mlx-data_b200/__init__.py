"""B200-native image-transform-and-batch path for mlx-data pipelines.

The directory name carries a hyphen, so the package is imported under the name
``mlx_data_b200`` by loading this file with importlib (see ``load_package`` in
the repository's ``__graft_entry__.py``).  ``_capi`` is the ctypes face of the
C ABI; the CUDA library it loads is the only implementation - nothing here
computes on the CPU.
"""
from . import _capi  # noqa: F401
from ._capi import Context, MlxdError, make_batch_desc, SAMPLE_DTYPE  # noqa: F401

__all__ = ["Context", "MlxdError", "make_batch_desc", "SAMPLE_DTYPE", "_capi"]
