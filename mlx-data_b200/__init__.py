"""B200-native image-transform-and-batch path with the mlx-data pipeline API.

``Buffer``, ``Stream``, ``buffer_from_vector`` and ``core`` come from the
compiled module ``_c`` (C++ pipeline over the CUDA library's C ABI) and take the
same method and keyword names as mlx-data, so
``buffer_from_vector(samples).to_stream().image_resize_smallest_side("image", 256)
.image_center_crop("image", 224, 224).batch(32)`` reads the same and yields the
same batches.  ``_capi`` is a ctypes face of the C ABI itself.

The directory name carries a hyphen, so import the package under the name
``mlx_data_b200`` with importlib (``load_package`` in ``__graft_entry__.py``).
Nothing here computes on the CPU: without the built libraries the import
fails, and without a CUDA device the first op raises.
"""
from . import _capi  # noqa: F401
from ._capi import Context, MlxdError, make_batch_desc, SAMPLE_DTYPE  # noqa: F401
from ._c import Buffer, Stream, buffer_from_vector, stream_python_iterable, core  # noqa: F401

__all__ = ["Buffer", "Stream", "buffer_from_vector", "stream_python_iterable", "core",
           "Context", "MlxdError", "make_batch_desc", "SAMPLE_DTYPE", "_capi"]
