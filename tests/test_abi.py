"""The C-ABI library loads and exports every symbol include/mynah_b200.h declares.
No compute calls: runs without a GPU."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    src = open(os.path.join(ROOT, "include", "mynah_b200.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(mynah_b200_[a-z0-9_]+)\s*\(", src)))


def test_header_declares_the_boundary():
    syms = declared_symbols()
    for must in ("mynah_b200_available", "mynah_b200_gemm_wt", "mynah_b200_qmat_mul", "mynah_b200_log_mel",
                 "mynah_b200_subsampling_forward", "mynah_b200_encoder_forward_batch", "mynah_b200_ctc_decode",
                 "mynah_b200_greedy_decode", "mynah_b200_transcribe_batch"):
        assert must in syms


def test_library_exports_every_declared_symbol(pkg):
    if not os.path.exists(pkg.LIB_PATH):
        import importlib.util
        spec = importlib.util.spec_from_file_location("graft_entry", os.path.join(ROOT, "__graft_entry__.py"))
        ge = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(ge)
        ge.build()
    lib = ctypes.CDLL(pkg.LIB_PATH)
    missing = [s for s in declared_symbols() if not hasattr(lib, s)]
    assert not missing, missing


def test_error_reporting_without_device(pkg):
    """Without a GPU the library must say so instead of computing anything."""
    L = pkg.lib()
    if L.mynah_b200_available():
        pytest.skip("a device is present")
    assert pkg.lib().mynah_b200_model_new(None) is None
    assert b"device" in L.mynah_b200_last_error()
    with pytest.raises(pkg.BackendError):
        pkg.QMat(pkg.F32, __import__("numpy").zeros((4, 64), "float32"), 4, 64)


def test_header_is_plain_c_and_links_from_c(pkg, tmp_path):
    """gcc -std=c11 -pedantic -Werror compiles the reference-side shim against the header and the
    program runs against the built library."""
    import shutil
    import subprocess
    if not shutil.which("gcc"):
        pytest.skip("no gcc")
    if not os.path.exists(pkg.LIB_PATH):
        pytest.skip("library not built")
    exe = str(tmp_path / "shim")
    libdir = os.path.dirname(pkg.LIB_PATH)
    subprocess.run(["gcc", "-std=c11", "-Wall", "-Wextra", "-pedantic", "-Werror", "-I", os.path.join(ROOT, "include"),
                    os.path.join(ROOT, "tests", "c_abi_shim.c"), "-o", exe, "-L", libdir, "-l:" + os.path.basename(pkg.LIB_PATH),
                    "-Wl,-rpath," + libdir], check=True)
    r = subprocess.run([exe], capture_output=True, text=True)
    assert r.returncode == 0, (r.returncode, r.stdout, r.stderr)
