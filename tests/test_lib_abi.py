"""The C-ABI library loads without a GPU and exports every symbol include/deepj_cuda.h declares."""
import ctypes
import os
import re

from deepj_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    hdr = open(os.path.join(ROOT, "include", "deepj_cuda.h")).read()
    hdr = re.sub(r"/\*.*?\*/", "", hdr, flags=re.S)
    return sorted(set(re.findall(r"\b(deepj_cuda_\w+)\s*\(", hdr)))


def test_header_declares_the_five_reference_natives():
    names = declared_symbols()
    for n in ("alloc_buffers", "upload_buffer", "download_buffer", "release_buffers", "flush_ops", "last_error"):
        assert f"deepj_cuda_{n}" in names


def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(_lib.LIB_PATH)
    for name in declared_symbols():
        assert hasattr(lib, name), name


def test_python_binding_covers_every_declared_symbol():
    assert sorted(_lib.SIGNATURES) == declared_symbols()
    _lib.load()


def test_oracle_is_not_imported_by_the_product_package():
    """The product path must never route through the oracle."""
    pkg = os.path.join(ROOT, "deepj_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cpp", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert "libdeepj_oracle" not in text or f == "build.py", f
                assert "import oracle" not in text and "oracle_" not in text, f
