"""The reference's own C API test, compiled UNMODIFIED against this library.

``tests/test_c_api.cpp`` of the reference includes ``"../runtime/api/sparseflow_api.h"``; a shim header
at that relative path forwards to ``include/sparseflow_b200.h``.  The source is compiled where it
lies in a checkout of the reference (never copied); the test is skipped when no checkout is
present (``SPARSEFLOW_REFERENCE``, default: a ``reference`` folder beside this repository).  No GPU needed: with the inputs of that
test the dispatcher never launches a kernel."""
import os
import shutil
import subprocess

import pytest

from sparseflow_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.environ.get("SPARSEFLOW_REFERENCE", os.path.join(os.path.dirname(ROOT), "reference"))
SRC = os.path.join(REF, "tests", "test_c_api.cpp")


@pytest.mark.skipif(not os.path.exists(SRC), reason="no checkout of the reference")
@pytest.mark.skipif(shutil.which("g++") is None, reason="no g++")
def test_reference_test_c_api_compiles_and_passes(lib, tmp_path):
    shim = tmp_path / "shim"
    (shim / "tests").mkdir(parents=True)
    (shim / "runtime" / "api").mkdir(parents=True)
    (shim / "runtime" / "api" / "sparseflow_api.h").write_text('#include "sparseflow_b200.h"\n')
    exe = tmp_path / "test_c_api"
    libdir = os.path.dirname(_lib.LIB_PATH)
    subprocess.run(["g++", "-std=c++17", "-I", str(shim / "tests"), "-I", os.path.join(ROOT, "include"), SRC,
                    "-o", str(exe), "-L", libdir, "-lsparseflow_b200", f"-Wl,-rpath,{libdir}"], check=True)
    r = subprocess.run([str(exe)], cwd=tmp_path, capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "C API tests passed" in r.stdout
    assert "Cache hit working" in r.stdout and "Bucketing works correctly" in r.stdout
