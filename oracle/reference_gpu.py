"""ctypes face of the reference's OWN CUDA kernels (TEST INFRASTRUCTURE ONLY).

``oracle/_ref/libfk_reference.so`` is the reference's ``csrc/kernels/decode_quant_linear/arc_w4a16.cu``
compiled for sm_100a from where it lies in a reference checkout (``make -C oracle ref REF=...``),
behind the C shim ``oracle/ref_shim.cu``. Nothing is copied into this repository and the shipped
library never links or loads it. It exists so that tests (and the bench's baseline legs) can run
the unmodified reference kernels on exactly the inputs the new library sees:

* ``pack``            -> pack_arc_w4a16_packets            (arc_w4a16.cu:649-669)
* ``group_sums``      -> compute_arc_w4a16_group_sums      (:671-685)
* ``forward``         -> arc_w4a16_forward                 (:687-707)
* ``forward_split_k`` -> arc_w4a16_forward_split_k         (:709-737)
* ``reduce``          -> reduce_arc_w4a16_split_k_partials (:739-751)
* ``dequant``         -> dequant_w4a16_to_fp16             (:753-770)
* ``dequant_packets`` -> dequant_arc_w4a16_packets_to_fp16 (:772-789)
* ``cublaslt_after_packet_dequant`` -> the vendor subject  (:805-816)

The reference is fp16 only with group sizes 64 and 128. All pointers are device addresses.
"""

from __future__ import annotations

import ctypes
from functools import lru_cache
from pathlib import Path

REF_LIB_PATH = Path(__file__).resolve().parent / "_ref" / "libfk_reference.so"


def available() -> bool:
    return REF_LIB_PATH.exists()


@lru_cache(maxsize=1)
def lib() -> ctypes.CDLL:
    if not available():
        raise FileNotFoundError(f"{REF_LIB_PATH} is not built (make -C oracle ref REF=<reference checkout>)")
    handle = ctypes.CDLL(str(REF_LIB_PATH))
    u, i, z = ctypes.c_uint64, ctypes.c_int, ctypes.c_size_t
    handle.fkref_last_error.restype = ctypes.c_char_p
    handle.fkref_pack.argtypes = [u, u, u, u, i, i, i, i, u]
    handle.fkref_group_sums.argtypes = [u, u, i, i, i, u]
    handle.fkref_forward.argtypes = [u, u, u, u, i, i, i, i, i, u]
    handle.fkref_forward_split_k.argtypes = [u, u, u, u, i, i, i, i, i, i, u]
    handle.fkref_reduce.argtypes = [u, u, i, i, i, u]
    handle.fkref_dequant.argtypes = [u, u, u, u, i, i, i, u]
    handle.fkref_dequant_packets.argtypes = [u, u, i, i, i, i, u]
    handle.fkref_cublaslt_after_dequant.argtypes = [u, u, u, u, u, u, u, z, i, i, i, i, u]
    if hasattr(handle, "fkref_cublaslt_after_packet_dequant"):
        handle.fkref_cublaslt_after_packet_dequant.argtypes = [u, u, u, u, u, z, i, i, i, i, i, u]
    return handle


def check(rc: int) -> None:
    if rc != 0:
        raise RuntimeError("reference kernel call failed: " + lib().fkref_last_error().decode(errors="replace"))


def stride(group: int) -> int:
    return 64 * group + 512


def pack(q, alpha, beta, packets, n: int, k: int, group: int, stream: int = 0) -> None:
    check(lib().fkref_pack(q, alpha, beta, packets, n, k, group, stride(group), stream))


def group_sums(act, sums, batch: int, k: int, group: int, stream: int = 0) -> None:
    check(lib().fkref_group_sums(act, sums, batch, k, group, stream))


def forward(act, packets, sums, out, batch: int, n: int, k: int, group: int, stream: int = 0) -> None:
    check(lib().fkref_forward(act, packets, sums, out, batch, n, k, group, stride(group), stream))


def forward_split_k(act, packets, sums, partials, batch: int, n: int, k: int, group: int, slices: int,
                    stream: int = 0) -> None:
    check(lib().fkref_forward_split_k(act, packets, sums, partials, batch, n, k, group, stride(group),
                                      slices, stream))


def reduce(partials, out, batch: int, n: int, slices: int, stream: int = 0) -> None:
    check(lib().fkref_reduce(partials, out, batch, n, slices, stream))


def dequant(q, alpha, beta, weight, n: int, k: int, group: int, stream: int = 0) -> None:
    check(lib().fkref_dequant(q, alpha, beta, weight, n, k, group, stream))


def dequant_packets(packets, weight, n: int, k: int, group: int, stream: int = 0) -> None:
    check(lib().fkref_dequant_packets(packets, weight, n, k, group, stride(group), stream))


def cublaslt_after_packet_dequant(act, packets, out, weight, workspace, workspace_bytes: int, batch: int,
                                  n: int, k: int, group: int, stream: int = 0) -> None:
    check(lib().fkref_cublaslt_after_packet_dequant(act, packets, out, weight, workspace, workspace_bytes,
                                                    batch, n, k, group, stride(group), stream))
