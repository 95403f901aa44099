"""The C-ABI library loads, exports every symbol the header declares, and rejects bad arguments
before touching a device (these checks need no GPU)."""

from __future__ import annotations

import ctypes
import re
from pathlib import Path

import pytest
from fast_kernels import capi

REPO = Path(__file__).resolve().parent.parent


def _declared_symbols() -> list[str]:
    names: list[str] = []
    for header in sorted((REPO / "include").glob("*.h")):
        names += re.findall(r"\b(fk_w4a16_\w+)\s*\(", header.read_text())
    return sorted(set(names))


def test_header_and_binding_table_agree() -> None:
    assert _declared_symbols() == sorted(capi.SIGNATURES)


def test_library_exports_every_declared_symbol() -> None:
    lib = ctypes.CDLL(str(capi.LIB_PATH))
    for name in _declared_symbols():
        assert hasattr(lib, name), f"{name} is declared in include/ but not exported"


def test_metadata_and_stride() -> None:
    lib = capi.load_library()
    assert lib.fk_w4a16_cuda_arch() == b"100a"
    assert lib.fk_w4a16_version().decode().count(".") == 2
    # stride = 128 * G / 2 + 512, the reference's expected_packet_stride_bytes (arc_w4a16.cu:23-26)
    assert capi.packet_stride_bytes(128) == 8704
    assert capi.packet_stride_bytes(64) == 4608
    assert capi.packet_stride_bytes(32) == 2560
    with pytest.raises(ValueError, match="group_size"):
        capi.packet_stride_bytes(16)


@pytest.mark.parametrize(
    ("batch", "n", "k", "group", "stride", "message"),
    [
        (0, 128, 256, 128, 8704, "batch and k must be positive"),
        (1, 128, 0, 128, 8704, "batch and k must be positive"),
        (1, 128, 256, 48, 8704, "group_size must be"),
        (1, 128, 200, 128, 8704, "k must be divisible by group_size"),
        (1, 0, 256, 128, 8704, "n must be positive"),
        (1, 130, 256, 128, 8704, "n must be a multiple of 128"),
        (1, 128, 256, 128, 4608, "packet_stride_bytes=4608 does not match expected 8704"),
    ],
)
def test_gemv_argument_errors_match_reference_wording(batch, n, k, group, stride, message) -> None:
    """Same rules and messages as validate_dimensions / validate_packet_stride
    (csrc/kernels/decode_quant_linear/arc_w4a16.cu:28-57 in the reference)."""
    lib = capi.load_library()
    code = lib.fk_w4a16_gemv(256, 256, 256, 256, 1 << 20, batch, n, k, group, stride, 0, None)
    assert code == capi.ERR_INVALID_ARGUMENT
    assert message in lib.fk_w4a16_last_error().decode()
    with pytest.raises(ValueError):
        capi.check(code)


def test_split_k_and_reduce_argument_errors() -> None:
    lib = capi.load_library()
    assert lib.fk_w4a16_gemv_split_k(256, 256, 256, 1, 128, 512, 128, 8704, 1, 0, None) == capi.ERR_INVALID_ARGUMENT
    assert "split_k_slices must be greater than 1" in lib.fk_w4a16_last_error().decode()
    assert lib.fk_w4a16_gemv_split_k(256, 256, 256, 1, 128, 512, 128, 8704, 5, 0, None) == capi.ERR_INVALID_ARGUMENT
    assert "must not exceed the number of groups" in lib.fk_w4a16_last_error().decode()
    assert lib.fk_w4a16_reduce_partials(256, 256, 1, 128, 1, 0, None) == capi.ERR_INVALID_ARGUMENT
    assert lib.fk_w4a16_gemv(256, 256, 256, 256, 1 << 20, 1, 128, 256, 128, 8704, 7, None) == capi.ERR_INVALID_ARGUMENT
    assert "dtype" in lib.fk_w4a16_last_error().decode()
    # misaligned and null pointers are refused before any launch
    assert lib.fk_w4a16_gemv(258, 256, 256, 256, 1 << 20, 1, 128, 256, 128, 8704, 0, None) == capi.ERR_INVALID_ARGUMENT
    assert "aligned" in lib.fk_w4a16_last_error().decode()
    assert lib.fk_w4a16_gemv(None, 256, 256, 256, 1 << 20, 1, 128, 256, 128, 8704, 0, None) == capi.ERR_INVALID_ARGUMENT
    assert "null" in lib.fk_w4a16_last_error().decode()
