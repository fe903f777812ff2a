"""The C-ABI library loads and exports every symbol include/dilution_b200.h declares,
and rejects bad arguments before touching a device (no GPU needed)."""

from __future__ import annotations

import ctypes
import os
import re

import pytest

from conftest import ROOT, load_package


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "dilution_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(dilution_[a-z_0-9]+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    names = declared_symbols()
    for must in ("dilution_rowstats", "dilution_colsum_scan", "dilution_forward_main",
                 "dilution_backward", "dilution_decode", "dilution_version", "dilution_last_error"):
        assert must in names


def test_library_exports_every_declared_symbol():
    pkg = load_package()
    lib = ctypes.CDLL(pkg._lib.LIB_PATH)
    for name in declared_symbols():
        assert hasattr(lib, name), f"{name} declared in the header but not exported"
    assert set(pkg._lib.SIGNATURES) == set(declared_symbols())


def test_version_and_size_queries():
    lib = load_package()._lib.load()
    assert lib.dilution_version() == 5
    assert lib.dilution_backward_scratch_bytes(2, 100, 64) == 4 * (2 * 2 * 100 * 64 + 2 * 2 * 100) + 2 * 2 * 100 * 64
    assert lib.dilution_carry_rows(1, 2, 64, 1) == 32 and lib.dilution_carry_rows(1, 2, 64, 0) == 64
    assert lib.dilution_carry_rows(0, 0, 64, 1) == 32 and lib.dilution_carry_rows(1, 2, 128, 0) == 32
    a = lib.dilution_decode_scratch_bytes(4, 1000, 64)
    b = lib.dilution_decode_scratch_bytes(4, 2000, 64)
    assert 0 < a <= b


def test_argument_validation_happens_before_any_launch():
    pkg = load_package()
    lib = pkg._lib.load()
    one = ctypes.c_void_p(256)  # never dereferenced: validation fails first
    rc = lib.dilution_rowstats(one, one, 7, 0, 1, 8, 8, 0, 64, 0.125, one, one, None)
    assert rc == 1 and b"dtype" in lib.dilution_last_error()
    rc = lib.dilution_rowstats(one, one, 0, 0, 1, 8, 8, 0, 48, 0.125, one, one, None)
    assert rc == 2 and b"head_dim" in lib.dilution_last_error()
    rc = lib.dilution_rowstats(None, one, 0, 0, 1, 8, 8, 0, 64, 0.125, one, one, None)
    assert rc == 1 and b"null" in lib.dilution_last_error()
    rc = lib.dilution_decode(one, one, one, 1, 4, 16, 17, 64, 0.125, 1e-9, one, one, one, None)
    assert rc == 1 and b"capacity" in lib.dilution_last_error()
    with pytest.raises(ValueError):
        pkg._lib.check(rc, "dilution_decode")
    # the bid / share variants: bid codes and share steps that do not exist
    args = (one, one, one, 0, 0, 1, 8, 64, 0.125, 1e-9)
    rc = lib.dilution_variant_forward(*args, 8, 1, 1.0, one, one, one, one, one, one, None, None)
    assert rc == 1 and b"bid" in lib.dilution_last_error()
    rc = lib.dilution_variant_forward(*args, 3, 1, 1.0, None, None, one, one, one, one, None, None)
    assert rc == 1 and b"null" in lib.dilution_last_error()      # a bid with a row sum needs rmax / rden
    rc = lib.dilution_variant_forward(*args, 5, 3, 1.0, None, None, one, one, one, one, None, None)
    assert rc == 1 and b"share" in lib.dilution_last_error()
    rc = lib.dilution_variant_forward(*args, 0, 2, 1.0, None, None, one, one, one, one, None, None)
    assert rc == 1 and b"null" in lib.dilution_last_error()      # the softmax bid needs rmax / rden
    rc = lib.dilution_variant_forward(*args, 7, 1, 0.0, None, None, one, one, one, one, None, None)
    assert rc == 1 and b"shift" in lib.dilution_last_error()     # the shifted bids need a positive shift
