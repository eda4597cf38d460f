"""The C-ABI library loads and exports every symbol include/nn_b200.h declares (no GPU needed)."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    names = set()
    inc = os.path.join(ROOT, "include")
    for f in os.listdir(inc):
        if f.endswith(".h"):
            text = open(os.path.join(inc, f)).read()
            text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
            names |= set(re.findall(r"\b(nnb_[a-z0-9_]+)\s*\(", text))
    return names


def test_library_exports_every_declared_symbol(pkg):
    path = pkg.lib_path()
    assert os.path.exists(path), "libnn-b200.so not built (python neuralnet.cpp_b200/build.py)"
    handle = ctypes.CDLL(path)
    declared = _declared()
    assert len(declared) > 20
    missing = [n for n in sorted(declared) if not hasattr(handle, n)]
    assert not missing, f"declared in include/*.h but not exported: {missing}"


def test_python_binding_covers_header(pkg):
    from neuralnet_cpp_b200 import _lib

    declared = _declared()
    bound = set(_lib.exported_symbols())
    assert declared <= bound, f"header symbols without a ctypes signature: {sorted(declared - bound)}"
    pkg.lib()  # resolves every bound symbol


def test_engine_create_fails_loudly_without_gpu(pkg):
    import torch

    if torch.cuda.is_available():
        return
    h = ctypes.c_void_p()
    st = pkg.lib().nnb_engine_create(0, ctypes.byref(h))
    assert st != 0 and not h.value
    assert b"no CPU fallback" in pkg.lib().nnb_last_error() or b"CUDA" in pkg.lib().nnb_last_error()
