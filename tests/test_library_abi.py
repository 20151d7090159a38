"""The C-ABI library loads on a CPU-only host and exports what include/mie_b200.h declares."""

from __future__ import annotations

import ctypes
import re
from pathlib import Path

import pytest

from mini_inference_engine_b200 import _lib, build

HEADER = Path(__file__).resolve().parents[1] / "include" / "mie_b200.h"


def declared_functions() -> set[str]:
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return set(re.findall(r"\b(mie_[a-z0-9_]+)\s*\(", text))


@pytest.fixture(scope="module")
def library():
    build.build_library()
    return ctypes.CDLL(str(build.LIB_PATH))


def test_header_and_binding_agree():
    assert declared_functions() == set(_lib.exported_symbols())


def test_every_declared_symbol_is_exported(library):
    for name in declared_functions():
        assert hasattr(library, name), name


def test_host_only_calls_work_without_a_gpu(library):
    lib = _lib.load()
    assert lib.mie_version() >= 1
    assert lib.mie_decode_scratch_bytes(4, 32, 8, 128, 4 * 2048) > 0
    assert lib.mie_decode_scratch_bytes(-1, 32, 8, 128, 0) == 0


def test_argument_errors_are_reported_on_the_host(library):
    lib = _lib.load()
    empty_view = _lib.View4T(None, (ctypes.c_int64 * 4)(0, 0, 0, 0))
    empty_index = _lib.IndexT(None, 0, 0, 0)
    code = lib.mie_write_decode_kv(empty_view, empty_view, empty_index, empty_index, empty_index, empty_view,
                                   empty_view, 1, 1, 128, 16, 4, 1, 3, None, None)
    assert code == -1
    assert b"elem_bytes" in lib.mie_last_error()
    with pytest.raises(ValueError):
        _lib.check(code)


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", tmp_path / "libmie_b200.so")
    with pytest.raises(_lib.MieLibraryError, match="no CPU or PyTorch fallback"):
        _lib.load()


def test_library_path_override(monkeypatch, tmp_path):
    """``MIE_LIBRARY_PATH`` points the binding at a build kept elsewhere; a wrong path fails as loudly."""

    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setenv("MIE_LIBRARY_PATH", str(build.LIB_PATH))
    assert _lib.library_path() == build.LIB_PATH and _lib.load().mie_version() >= 1
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setenv("MIE_LIBRARY_PATH", str(tmp_path / "elsewhere.so"))
    with pytest.raises(_lib.MieLibraryError, match="elsewhere.so is missing"):
        _lib.load()
