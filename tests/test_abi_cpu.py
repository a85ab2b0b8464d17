"""CPU checks of the C ABI library: it loads without a GPU and exports every
entry point that include/mlxd_b200.h declares.  No compute call is made."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_entry_points():
    text = open(os.path.join(ROOT, "include", "mlxd_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = re.findall(r"MLXD_API\s+[\w\s\*]+?\b(mlxd_\w+)\s*\(", text)
    assert len(names) >= 19
    return names


def test_library_exports_every_declared_symbol(pkg):
    lib = pkg._capi.load()
    missing = [n for n in declared_entry_points() if not hasattr(lib, n)]
    assert not missing, missing
    assert sorted(declared_entry_points()) == sorted(pkg._capi.EXPORTS)


def test_struct_layouts_match_header(pkg):
    capi = pkg._capi
    assert ctypes.sizeof(capi.SampleDesc) == 96
    assert capi.SampleDesc.mx.offset == 48 and capi.SampleDesc.post_x.offset == 72
    assert capi.BatchDesc.pad_value.offset % 8 == 0
    assert ctypes.sizeof(capi.BatchDesc) == 104
    assert ctypes.sizeof(capi.Stats) == 104


def test_calls_without_a_gpu_fail_loudly(pkg):
    try:
        import torch
        if torch.cuda.is_available():
            pytest.skip("a GPU is present")
    except ImportError:
        pass
    with pytest.raises(pkg.MlxdError):
        pkg.Context(device=0, n_lanes=1)
    import numpy as np
    buf = pkg.buffer_from_vector([{"image": np.zeros((8, 8, 3), np.uint8)}])
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        buf.image_resize("image", 4, 4)[0]
