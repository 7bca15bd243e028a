"""The C-ABI library loads on a machine without a GPU and exports every symbol the header declares."""
import ctypes
import os
import re

import pytest

from flashck_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "flashck_b200.h")).read()
    return re.findall(r"^FLASHCK_API\s+[\w\s\*]+?\b(\w+)\(", text, flags=re.M)


def test_header_declares_the_reference_entry_points():
    names = set(_declared_symbols())
    for want in ("FmhaFwd", "FmhaFwdSplitKV", "FmhaFwdSplitKVCombine", "FmhaSplitKVCombine", "FmhaFwdAppendKV",
                 "FmhaFwdBatchPrefill", "FmhaFwdPagedKVPrefill"):
        assert want in names


def test_library_exports_every_declared_symbol():
    handle = ctypes.CDLL(_lib.LIB_PATH)
    names = _declared_symbols()
    assert len(names) >= 12
    for name in names:
        assert hasattr(handle, name), f"{name} is declared in include/flashck_b200.h but not exported"
        assert name in _lib.SIGNATURES, f"{name} has no ctypes signature in flashck_b200/_lib.py"


def test_version_and_argument_errors_without_gpu():
    lib = _lib.lib()
    assert b"sm_100a" in lib.FlashckVersion()
    # argument validation happens before any CUDA call
    rc = lib.FmhaFwd(None, None, None, None, None, None, None, None, 1, 1, 1, 3, 2, 64, 64, 1, 0.0, -1, -1, 0, None,
                     None, 4)
    assert rc == 1 and b"multiple" in lib.FlashckGetLastError()
    rc = lib.FmhaFwd(None, None, None, None, None, None, None, None, 1, 1, 1, 2, 2, 64, 64, 1, 0.0, -1, -1, 0, None,
                     None, 7)
    assert rc == 2 and b"dtype" in lib.FlashckGetLastError()
    rc = lib.FmhaFwdSplitKV(None, None, None, None, None, None, None, None, None, None, None, 1, 1, 1, 2, 2, 128, 128,
                            1, 1, 0, 0, 0.0, -1, -1, 0, None, 4)
    assert rc == 1 and b"null" in lib.FlashckGetLastError()
    with pytest.raises(RuntimeError, match="unknown"):
        _lib.set_instance_param(2, "no_such_key", 1)
    _lib.set_instance_param(2, "stages", 3)
    assert _lib.get_instance_param(2, "stages") == 3
    _lib.set_instance_param(2, "stages", 0)


def test_cpp_operator_api_compiles_links_and_throws(tmp_path):
    import shutil
    import subprocess
    gxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else shutil.which("g++")
    exe = str(tmp_path / "cpp_api_check")
    libdir = os.path.dirname(_lib.LIB_PATH)
    subprocess.run([gxx, "-std=c++17", "-I", os.path.join(ROOT, "include"), os.path.join(ROOT, "tests", "cpp_api_check.cpp"),
                    "-L", libdir, "-lflashck_b200", f"-Wl,-rpath,{libdir}", "-o", exe], check=True, capture_output=True)
    out = subprocess.run([exe], capture_output=True, text=True)
    assert out.returncode == 0 and "OK" in out.stdout, out.stdout + out.stderr
