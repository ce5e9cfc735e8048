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


def test_reference_train_cpp_compiles_unchanged_against_the_host_api(tmp_path):
    """train.cpp of the reference, byte for byte, must build against gradcraft_b200/gradc (syntax + semantic check only)."""
    import shutil
    import subprocess

    from gradcraft_b200.build import reference_root

    src = os.path.join(reference_root() or "", "train.cpp")
    if not os.path.exists(src):
        pytest.skip("reference tree not present on this machine")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    shutil.copy(src, tmp_path / "train.cpp")  # a quoted include searches the including file's directory first
    r = subprocess.run(["g++", "-std=c++23", "-fsyntax-only", "-I", os.path.join(root, "gradcraft_b200"), "-I", "/usr/local/cuda/include", str(tmp_path / "train.cpp")],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-3000:]
