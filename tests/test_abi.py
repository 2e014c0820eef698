"""The C-ABI library loads and exports every symbol include/ttq.h declares (no compute calls)."""
import ctypes
import os
import re

import pytest

from tattletale_b200 import _lib, formats

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_functions():
    text = open(os.path.join(ROOT, "include", "ttq.h")).read()
    return sorted(set(re.findall(r"TTQ_API[^;(]*?\b(ttq_\w+)\s*\(", text)))


def test_header_declares_functions():
    names = header_functions()
    assert "ttq_linear_forward" in names and "ttq_weight_create" in names and len(names) >= 15


def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(_lib.LIB_PATH)
    for name in header_functions():
        assert hasattr(lib, name), f"{name} is declared in ttq.h but not exported by libttq.so"


def test_binding_table_covers_header():
    assert sorted(_lib.SIGNATURES) == header_functions()


def test_nim_binding_covers_header():
    """The Nim side (uncompiled here: no Nim toolchain) imports every function the header declares."""
    nim = open(os.path.join(ROOT, "tattletale_b200", "nim", "quant_linear.nim")).read()
    bound = set(re.findall(r"proc (ttq_\w+)\(", nim))
    assert sorted(bound) == header_functions()


def test_new_entry_points_reject_null_handles():
    lib = _lib.load()
    assert lib.ttq_comm_local_buffer(None, None, None) == 1
    assert lib.ttq_comm_connect_pointers(None, None) == 1
    assert lib.ttq_comm_set_wait_limit(None, 10) == 1


def test_format_facts():
    lib = _lib.load()
    for fmt in (_lib.FMT_Q8_0, _lib.FMT_Q4_K, _lib.FMT_Q6_K):
        assert lib.ttq_block_elems(fmt) == formats.BLOCK_ELEMS[fmt]
        assert lib.ttq_block_bytes(fmt) == formats.BLOCK_BYTES[fmt]
    assert lib.ttq_packed_bytes(_lib.FMT_Q4_K, 4096, 4096) == 9437184
    assert lib.ttq_packed_bytes(_lib.FMT_Q8_0, 4096, 4096) == 17825792
    assert lib.ttq_packed_bytes(_lib.FMT_Q6_K, 128256, 4096) == 430940160
    assert lib.ttq_packed_bytes(_lib.FMT_Q4_K, 16, 100) == 0  # K not a multiple of 256
    assert lib.ttq_block_bytes(99) == 0
    assert formats.packed_bytes(_lib.FMT_Q4_K, 28672, 4096) == 66060288
    with pytest.raises(ValueError):
        formats.packed_bytes(_lib.FMT_Q6_K, 8, 100)


def test_status_strings_and_version():
    lib = _lib.load()
    assert lib.ttq_status_string(0) == b"ok"
    assert all(lib.ttq_status_string(s) for s in range(8))
    assert re.fullmatch(rb"\d+\.\d+\.\d+", lib.ttq_version())


def test_null_arguments_are_rejected_without_a_device():
    lib = _lib.load()
    assert lib.ttq_init(0, None) == 1
    assert lib.ttq_destroy(None) == 0
    assert lib.ttq_weight_destroy(None) == 0
    assert lib.ttq_weight_bytes(None) == 0
    assert lib.ttq_launch_count(None) == 0
    h = ctypes.c_void_p()
    assert lib.ttq_weight_create(None, 1, 16, 256, None, 0, None, ctypes.byref(h)) == 1
    assert lib.ttq_linear_forward(None, None, None, 0, 1, 1, None, 0, None, 0, 1, None) == 1
    assert lib.ttq_init(-1, ctypes.byref(h)) == 6  # TTQ_ERR_DEVICE: no such device


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "libttq.so"))
    with pytest.raises(ImportError, match="no non-CUDA implementation"):
        _lib.load()
