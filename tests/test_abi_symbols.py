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


def _compile_client(tmp_path, pkg):
    import subprocess

    libdir = os.path.dirname(pkg.lib_path())
    exe = str(tmp_path / "client")
    src = os.path.join(ROOT, "tests", "cabi", "client.c")
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", "-pedantic", "-I", os.path.join(ROOT, "include"), src, "-o", exe,
                    "-L", libdir, "-lnn-b200", f"-Wl,-rpath,{libdir}"], check=True)
    return exe


def test_header_is_plain_c_and_a_c_client_links(pkg, tmp_path):
    """include/nn_b200.h compiles as C99 and as C++17, and a C program links against the library; without a GPU
    it gets the library's error, not a fallback."""
    import subprocess

    import torch

    inc = os.path.join(ROOT, "include")
    for lang, std in (("c", "-std=c99"), ("c++", "-std=c++17")):
        subprocess.run(["gcc", "-x", lang, std, "-Wall", "-Werror", "-pedantic", "-fsyntax-only", "-I", inc,
                        os.path.join(inc, "nn_b200.h")], check=True)
    exe = _compile_client(tmp_path, pkg)
    if torch.cuda.is_available():
        return
    r = subprocess.run([exe], capture_output=True, text=True)
    assert r.returncode == 3 and "engine:" in r.stderr


def _compile_shim_test(tmp_path, pkg):
    import subprocess

    libdir = os.path.dirname(pkg.lib_path())
    exe = str(tmp_path / "shim_test")
    src = os.path.join(ROOT, "tests", "cabi", "shim_test.cpp")
    subprocess.run(["g++", "-std=c++17", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"), src, "-o", exe,
                    "-L", libdir, "-lnn-b200", f"-Wl,-rpath,{libdir}"], check=True)
    return exe


def test_cpp_engine_shim_compiles_and_links(pkg, tmp_path):
    """include/nn_b200.hpp (the ComputeEngine-shaped C++17 layer: tensors with write epochs, BitLinear, the RL pipeline
    classes) compiles warning-free and its test program links; without a GPU the program reports the engine's error."""
    import subprocess

    import torch

    exe = _compile_shim_test(tmp_path, pkg)
    if torch.cuda.is_available():
        return
    r = subprocess.run([exe], capture_output=True, text=True)
    assert r.returncode == 3 and "engine:" in r.stderr
