"""CPU-side checks of the drop-in boundary: the library loads, exports every declared symbol, and refuses to
compute without a GPU instead of falling back."""
import ctypes
import os

import pytest


def test_library_exports_every_declared_symbol():
    import __graft_entry__ as entry

    entry.build()
    from gradcraft_b200 import capi

    decl = capi.parse_header()
    assert len(decl) >= 55
    cdll = ctypes.CDLL(capi.LIB_PATH)
    missing = [name for name, _, _ in decl if not hasattr(cdll, name)]
    assert not missing, missing


def test_no_cpu_fallback():
    import torch

    if torch.cuda.is_available():
        pytest.skip("only meaningful on a machine without a GPU")
    from gradcraft_b200 import capi

    h = ctypes.c_void_p()
    with pytest.raises(capi.GcbError) as e:
        capi.lib().ctx_create(0, ctypes.byref(h))
    assert e.value.status == capi.CUDA_ERROR and "no CPU fallback" in str(e.value)
    with pytest.raises(capi.GcbError):
        capi.lib().fill_f32(None, None, 1.0, 4)


def test_product_does_not_import_the_oracle():
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for dirpath, _, files in os.walk(os.path.join(root, "gradcraft_b200")):
        if os.sep + "build" in dirpath:
            continue
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".cpp", ".hpp", ".h")):
                text = open(os.path.join(dirpath, f), errors="ignore").read()
                assert "oracle" not in text.lower(), os.path.join(dirpath, f)
