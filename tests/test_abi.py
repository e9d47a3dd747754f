"""The C-ABI library loads without a GPU and exports every symbol the public header declares."""
import ctypes
import os
import re

from dyllm_b200 import _lib
from dyllm_b200.build import build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    names = set()
    inc = os.path.join(ROOT, "include")
    for f in os.listdir(inc):
        if f.endswith(".h"):
            text = open(os.path.join(inc, f)).read()
            text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
            names.update(re.findall(r"\b(dyllm_\w+)\s*\(", text))
    return names


def test_library_builds_and_exports_every_declared_symbol():
    path = build()
    lib = ctypes.CDLL(path)
    declared = _declared_symbols()
    assert len(declared) >= 10
    missing = [n for n in sorted(declared) if not hasattr(lib, n)]
    assert not missing, f"declared in include/*.h but not exported: {missing}"


def test_python_binding_covers_the_header():
    declared = _declared_symbols()
    assert declared == set(_lib.SIGNATURES), (declared ^ set(_lib.SIGNATURES))


def test_version_and_error_text_without_gpu():
    lib = _lib.load()
    assert lib.dyllm_version() >= 100
    # argument validation happens before any CUDA call
    rc = lib.dyllm_context_stats(None, None, None, 4, 7, 0, None)
    assert rc == -2
    assert b"multiple of 8" in lib.dyllm_last_error()
    rc = lib.dyllm_cache_get_seqs(None, None, None, None, None, 1, 4, 3, 2, None)
    assert rc == -2
