"""The C-ABI shared library builds for sm_100a, loads without a GPU, and exports exactly the
entry points ``include/vrb.h`` declares.  No compute call is made here."""
import ctypes
import os
import re
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "vrb.h")


def declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(vrb_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_entry_points():
    names = declared_symbols()
    assert "vrb_layer_norm_modulate" in names and "vrb_group_norm" in names and len(names) >= 30


def test_library_exports_every_declared_symbol(cuda_lib):
    missing = [n for n in declared_symbols() if not hasattr(cuda_lib, n)]
    assert not missing, f"declared in vrb.h but not exported by libvrb.so: {missing}"


def test_binding_table_matches_header(cuda_lib):
    from vrhino_b200 import _lib
    assert sorted(_lib.SIGNATURES) == declared_symbols()


def test_sharded_library_exports_its_header(cuda_lib):
    """libvrb_sharded.so (the C++ multi-GPU host layer) exports what include/vrb_sharded.h declares, and its
    bounded wait works on the host: with a peer that never joins, vrbs_wait's loop gives up after the
    timeout, aborts the communicator once, and later calls are refused."""
    from vrhino_b200 import _lib, build
    if not os.path.exists(_lib.SHARDED_LIB_PATH):
        build.build_sharded()
    lib = _lib.load_sharded()
    text = re.sub(r"/\*.*?\*/", "", open(os.path.join(ROOT, "include", "vrb_sharded.h")).read(), flags=re.S)
    declared = sorted(set(re.findall(r"\b(vrbs_[a-z0-9_]+)\s*\(", text)))
    assert declared == sorted(_lib.SHARDED_SIGNATURES)
    assert not [n for n in declared if not hasattr(lib, n)]
    report = (ctypes.c_int64 * 4)()
    assert lib.vrbs_watchdog_selftest(120, report) == 0
    status, waited_ms, aborts, later = list(report)
    assert status == -6 and 120 <= waited_ms < 2000 and aborts == 1 and later == -7
    assert b"aborted" in lib.vrbs_last_error()


def test_exports_are_plain_c(cuda_lib):
    from vrhino_b200 import _lib
    out = subprocess.run(["nm", "-D", "--defined-only", _lib.LIB_PATH], capture_output=True, text=True, check=True).stdout
    exported = {line.split()[-1] for line in out.splitlines() if " T " in line}
    assert set(declared_symbols()) <= exported
    assert cuda_lib.vrb_abi_version() == 1
    assert cuda_lib.vrb_last_error() == b""


def test_header_compiles_as_c():
    """The header is C: plain pointers and sizes, no C++ or torch types."""
    src = '#include "vrb.h"\nint main(void) { return VRB_ABI_VERSION == 1 ? 0 : 1; }\n'
    proc = subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", "-pedantic", "-I", os.path.join(ROOT, "include"),
                           "-x", "c", "-", "-fsyntax-only"], input=src, capture_output=True, text=True)
    assert proc.returncode == 0, proc.stderr


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from vrhino_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "libvrb.so"))
    with pytest.raises(_lib.VrbError, match="no CPU or PyTorch fallback"):
        _lib.load()


def test_product_package_never_imports_the_oracle():
    pkg = os.path.join(ROOT, "vrhino_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".cpp", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text.lower() or f == "synth.py", f"{f} mentions the oracle"
