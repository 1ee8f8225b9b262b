"""The C-ABI library loads and exports every symbol include/qb200.h declares."""

import ctypes
import os
import re

from quabla_b200 import _build, _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "qb200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(qb200_[a-z0-9_]+)\s*\(", text)))


def test_header_and_binding_agree():
    assert declared_symbols() == sorted(_lib.SIGNATURES)


def test_library_exports_every_declared_symbol():
    path = _build.build()
    lib = ctypes.CDLL(path)
    for name in declared_symbols():
        assert hasattr(lib, name), name


def test_version_and_error_strings():
    lib = _lib.load()
    assert b"qb200" in lib.qb200_version()
    assert lib.qb200_plan_execute(None) == _lib.INVALID
    assert b"null plan" in lib.qb200_last_error()
