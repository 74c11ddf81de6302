"""CPU checks of the boundary: the library loads, exports every symbol the header declares,
and refuses to run without a GPU (no CPU fallback).  No compute call is made here."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def built_lib():
    from mlfw_b200 import build
    return build.build()


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "b200q.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200q_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_symbols():
    names = declared_symbols()
    assert "b200q_create" in names and "b200q_int8_linear" in names and len(names) >= 30


def test_library_exports_every_declared_symbol(built_lib):
    lib = ctypes.CDLL(built_lib)
    missing = [n for n in declared_symbols() if not hasattr(lib, n)]
    assert not missing, f"declared in include/b200q.h but not exported: {missing}"


def test_binding_covers_every_declared_symbol(built_lib):
    from mlfw_b200 import _lib
    assert sorted(_lib.PROTOTYPES) == declared_symbols()
    _lib.load(built_lib)


def test_no_cpu_fallback(built_lib):
    import mlfw_b200
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(mlfw_b200.B200QError, match="no CUDA device"):
        mlfw_b200.Context(0)


def test_missing_library_fails_loudly(tmp_path):
    from mlfw_b200 import _lib
    with pytest.raises(_lib.B200QError, match="no CPU fallback"):
        _lib.load(str(tmp_path / "libb200q.so"))


def test_product_does_not_import_the_oracle():
    """Nothing shipped may import, link, open or execute the CPU oracle."""
    pkg = os.path.join(ROOT, "mlfw_b200")
    bad = re.compile(r"import\s+oracle|from\s+oracle|liboracle|oracle/|oracle\.(build|lib)|orc_[a-z]")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".ts", ".h")):
                src = open(os.path.join(dirpath, f)).read()
                assert not bad.search(src), f"{f} reaches into the oracle"
