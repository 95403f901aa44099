"""Python face of the CPU oracle (TEST INFRASTRUCTURE ONLY).

Two independent restatements of the reference's W4A16 arithmetic live here:

* the C library ``oracle/w4a16_oracle.c`` loaded through ctypes (fast, multi-threaded), and
* plain numpy versions (``np_*``) written separately, used to cross-check the C code.

Only ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline legs of ``bench.py`` may import
this module. 16-bit floats travel as ``uint16`` bit patterns so fp16 and bf16 share one interface.
"""

from __future__ import annotations

import ctypes
import subprocess
from functools import lru_cache
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
LIB_PATH = HERE / "libw4a16_oracle.so"
REF_LIB_PATH = HERE / "_ref" / "libfk_reference.so"

F16 = 0
BF16 = 1
TILE = 128


def build(force: bool = False) -> Path:
    """Compile the C oracle if it is missing or older than its source."""
    src = HERE / "w4a16_oracle.c"
    if force or not LIB_PATH.exists() or LIB_PATH.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(HERE), "oracle"] + (["-B"] if force else []), check=True,
                       capture_output=True)
    return LIB_PATH


@lru_cache(maxsize=1)
def lib() -> ctypes.CDLL:
    build()
    handle = ctypes.CDLL(str(LIB_PATH))
    vp, ci = ctypes.c_void_p, ctypes.c_int
    handle.oracle_packet_stride.restype = ci
    handle.oracle_packet_stride.argtypes = [ci]
    handle.oracle_num_threads.restype = ci
    handle.oracle_set_threads.argtypes = [ci]
    handle.oracle_half_to_float.restype = ctypes.c_float
    handle.oracle_half_to_float.argtypes = [ctypes.c_uint16, ci]
    handle.oracle_float_to_half.restype = ctypes.c_uint16
    handle.oracle_float_to_half.argtypes = [ctypes.c_float, ci]
    handle.oracle_dequant_rowmajor.argtypes = [vp, vp, vp, vp, ci, ci, ci, ci]
    handle.oracle_pack_packets.argtypes = [vp, vp, vp, vp, ci, ci, ci]
    handle.oracle_dequant_packets.argtypes = [vp, vp, ci, ci, ci, ci]
    handle.oracle_group_sums.argtypes = [vp, vp, ci, ci, ci, ci]
    handle.oracle_gemv_f64.argtypes = [vp, vp, vp, vp, vp, ci, ci, ci, ci, ci]
    handle.oracle_gemv_ref_order.argtypes = [vp, vp, vp, vp, vp, ci, ci, ci, ci, ci]
    handle.oracle_gemv_explicit.argtypes = [vp, vp, vp, vp, vp, vp, ci, ci, ci, ci, ci]
    return handle


def _ptr(array: np.ndarray) -> ctypes.c_void_p:
    return ctypes.c_void_p(array.ctypes.data)


def _c(array: np.ndarray, dtype: type) -> np.ndarray:
    return np.ascontiguousarray(array, dtype=dtype)


def bits_of(tensor) -> np.ndarray:  # noqa: ANN001 - torch is optional here
    """uint16 bit patterns of a torch fp16 / bf16 tensor (on any device)."""
    import torch

    return tensor.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def tensor_of(bits: np.ndarray, dtype_code: int):  # noqa: ANN201
    import torch

    target = torch.bfloat16 if dtype_code == BF16 else torch.float16
    return torch.from_numpy(bits.view(np.int16).copy()).view(target)


def dtype_code(name_or_dtype) -> int:  # noqa: ANN001
    text = str(name_or_dtype)
    return BF16 if "bf" in text or "bfloat" in text else F16


def packet_stride(group: int) -> int:
    return int(lib().oracle_packet_stride(group))


def num_threads() -> int:
    return int(lib().oracle_num_threads())


def set_threads(threads: int) -> None:
    lib().oracle_set_threads(int(threads))


# ---- C-backed functions ------------------------------------------------------------------
def dequant_rowmajor(q_u8, alpha_bits, beta_bits, group: int, dtype: int) -> np.ndarray:
    q_u8, alpha_bits, beta_bits = _c(q_u8, np.uint8), _c(alpha_bits, np.uint16), _c(beta_bits, np.uint16)
    n, k = q_u8.shape[0], q_u8.shape[1] * 2
    out = np.empty((n, k), dtype=np.uint16)
    lib().oracle_dequant_rowmajor(_ptr(q_u8), _ptr(alpha_bits), _ptr(beta_bits), _ptr(out), n, k, group, dtype)
    return out


def pack_packets(q_u8, alpha_bits, beta_bits, group: int) -> np.ndarray:
    q_u8, alpha_bits, beta_bits = _c(q_u8, np.uint8), _c(alpha_bits, np.uint16), _c(beta_bits, np.uint16)
    n, k = q_u8.shape[0], q_u8.shape[1] * 2
    out = np.empty(((n // TILE) * (k // group), packet_stride(group)), dtype=np.uint8)
    lib().oracle_pack_packets(_ptr(q_u8), _ptr(alpha_bits), _ptr(beta_bits), _ptr(out), n, k, group)
    return out


def dequant_packets(packets, n: int, k: int, group: int, dtype: int) -> np.ndarray:
    packets = _c(packets, np.uint8)
    out = np.empty((n, k), dtype=np.uint16)
    lib().oracle_dequant_packets(_ptr(packets), _ptr(out), n, k, group, dtype)
    return out


def group_sums(act_bits, group: int, dtype: int) -> np.ndarray:
    act_bits = _c(act_bits, np.uint16)
    batch, k = act_bits.shape
    out = np.empty((batch, k // group), dtype=np.float32)
    lib().oracle_group_sums(_ptr(act_bits), _ptr(out), batch, k, group, dtype)
    return out


def gemv_f64(act_bits, q_u8, alpha_bits, beta_bits, group: int, dtype: int) -> np.ndarray:
    act_bits, q_u8 = _c(act_bits, np.uint16), _c(q_u8, np.uint8)
    alpha_bits, beta_bits = _c(alpha_bits, np.uint16), _c(beta_bits, np.uint16)
    batch, k = act_bits.shape
    n = q_u8.shape[0]
    out = np.empty((batch, n), dtype=np.float64)
    lib().oracle_gemv_f64(_ptr(act_bits), _ptr(q_u8), _ptr(alpha_bits), _ptr(beta_bits), _ptr(out),
                          batch, n, k, group, dtype)
    return out


def gemv_ref_order(act_bits, q_u8, alpha_bits, beta_bits, group: int, dtype: int) -> np.ndarray:
    act_bits, q_u8 = _c(act_bits, np.uint16), _c(q_u8, np.uint8)
    alpha_bits, beta_bits = _c(alpha_bits, np.uint16), _c(beta_bits, np.uint16)
    batch, k = act_bits.shape
    n = q_u8.shape[0]
    out = np.empty((batch, n), dtype=np.uint16)
    lib().oracle_gemv_ref_order(_ptr(act_bits), _ptr(q_u8), _ptr(alpha_bits), _ptr(beta_bits),
                                _ptr(out), batch, n, k, group, dtype)
    return out


def gemv_explicit(act_bits, q_u8, alpha_bits, beta_bits, group: int, dtype: int,
                  scratch: np.ndarray | None = None) -> np.ndarray:
    """The reference's CPU-runnable expression: fp32 W = alpha*q + beta, y = round16(a @ W^T)."""
    act_bits, q_u8 = _c(act_bits, np.uint16), _c(q_u8, np.uint8)
    alpha_bits, beta_bits = _c(alpha_bits, np.uint16), _c(beta_bits, np.uint16)
    batch, k = act_bits.shape
    n = q_u8.shape[0]
    if scratch is None or scratch.size < (n + 1) * k:
        scratch = np.empty((n + 1) * k, dtype=np.float32)
    out = np.empty((batch, n), dtype=np.uint16)
    lib().oracle_gemv_explicit(_ptr(act_bits), _ptr(q_u8), _ptr(alpha_bits), _ptr(beta_bits),
                               _ptr(scratch), _ptr(out), batch, n, k, group, dtype)
    return out


# ---- numpy restatements (independent of the C file) -------------------------------------
def np_to_f32(bits: np.ndarray, dtype: int) -> np.ndarray:
    bits = np.asarray(bits, dtype=np.uint16)
    if dtype == BF16:
        return (bits.astype(np.uint32) << 16).view(np.float32)
    return bits.view(np.float16).astype(np.float32)


def np_from_f32(values: np.ndarray, dtype: int) -> np.ndarray:
    values = np.asarray(values, dtype=np.float32)
    if dtype == BF16:
        raw = values.view(np.uint32).astype(np.uint64)
        rounded = (raw + 0x7FFF + ((raw >> 16) & 1)) >> 16
        return rounded.astype(np.uint16)
    return values.astype(np.float16).view(np.uint16)


def np_nibbles(q_u8: np.ndarray) -> np.ndarray:
    """[n, k] integer weights; the low nibble of a byte is the even k."""
    q_u8 = np.asarray(q_u8, dtype=np.uint8)
    out = np.empty((q_u8.shape[0], q_u8.shape[1] * 2), dtype=np.uint8)
    out[:, 0::2] = q_u8 & 0x0F
    out[:, 1::2] = q_u8 >> 4
    return out


def np_dequant(q_u8, alpha_bits, beta_bits, group: int, dtype: int) -> np.ndarray:
    q = np_nibbles(q_u8).astype(np.float32)
    a = np.repeat(np_to_f32(alpha_bits, dtype), group, axis=1)
    b = np.repeat(np_to_f32(beta_bits, dtype), group, axis=1)
    return np_from_f32(a * q + b, dtype)


def np_pack(q_u8, alpha_bits, beta_bits, group: int) -> np.ndarray:
    q_u8 = np.asarray(q_u8, dtype=np.uint8)
    n, kb = q_u8.shape
    k = kb * 2
    ng = k // group
    tiles = n // TILE
    words = q_u8.reshape(tiles, TILE, ng, group // 8, 4)       # [t, c, g, r, byte]
    words = words.transpose(0, 2, 3, 1, 4).reshape(tiles, ng, -1)  # [t, g, (r, c, byte)]
    a = np.asarray(alpha_bits, dtype=np.uint16).reshape(tiles, TILE, ng).transpose(0, 2, 1)
    b = np.asarray(beta_bits, dtype=np.uint16).reshape(tiles, TILE, ng).transpose(0, 2, 1)
    packets = np.concatenate(
        [words, np.ascontiguousarray(a).view(np.uint8).reshape(tiles, ng, -1),
         np.ascontiguousarray(b).view(np.uint8).reshape(tiles, ng, -1)], axis=2)
    return np.ascontiguousarray(packets.reshape(tiles * ng, -1))


def np_gemv_f64(act_bits, q_u8, alpha_bits, beta_bits, group: int, dtype: int) -> np.ndarray:
    q = np_nibbles(q_u8).astype(np.float64)
    a = np.repeat(np_to_f32(alpha_bits, dtype).astype(np.float64), group, axis=1)
    b = np.repeat(np_to_f32(beta_bits, dtype).astype(np.float64), group, axis=1)
    x = np_to_f32(act_bits, dtype).astype(np.float64)
    return x @ (a * q + b).T


def max_rel_err(actual: np.ndarray, expected_f64: np.ndarray) -> float:
    """max_n |y - y64| / max(|y64|, eps) with eps = 1e-3 * max|y64| per output row.

    The stated tolerance is a "max relative error" without a rule for outputs that happen to land
    near zero; the floor ties the denominator to the row's scale so that such entries are judged
    by their absolute error against the size of the vector.
    """
    actual = np.asarray(actual, dtype=np.float64)
    expected = np.asarray(expected_f64, dtype=np.float64)
    floor = 1e-3 * np.max(np.abs(expected), axis=-1, keepdims=True)
    denom = np.maximum(np.abs(expected), np.maximum(floor, 1e-30))
    return float(np.max(np.abs(actual - expected) / denom))
