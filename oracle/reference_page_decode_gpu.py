"""ctypes face of the reference's OWN paged-KV decode kernels (TEST INFRASTRUCTURE ONLY).

``oracle/_ref/libfk_reference_page_decode.so`` is the reference's
``csrc/kernels/clustered_page_decode/clustered_page_decode.cu`` compiled for sm_100a from where it
lies in a reference checkout (``make -C oracle ref_page_decode REF=...``), behind the C shim
``oracle/ref_page_decode_shim.cu``. Nothing is copied into this repository and the shipped library
never links or loads it. ``forward`` is ``clustered_page_decode_forward``
(clustered_page_decode.cu:1085-1160): ``use_clustered_kernel`` = 0 selects its one-warp-per-head
kernel (:111-328), 1 its cluster kernel (:330-669) with ``cluster_size`` blocks per task.
"""

from __future__ import annotations

import ctypes
from functools import lru_cache
from pathlib import Path

REF_LIB_PATH = Path(__file__).resolve().parent / "_ref" / "libfk_reference_page_decode.so"


def available() -> bool:
    return REF_LIB_PATH.exists()


@lru_cache(maxsize=1)
def lib() -> ctypes.CDLL:
    if not available():
        raise FileNotFoundError(f"{REF_LIB_PATH} is not built (make -C oracle ref_page_decode REF=<reference checkout>)")
    handle = ctypes.CDLL(str(REF_LIB_PATH))
    u, i, f = ctypes.c_uint64, ctypes.c_int, ctypes.c_float
    handle.fkref_page_decode_last_error.restype = ctypes.c_char_p
    handle.fkref_page_decode_forward.argtypes = [u] * 12 + [i] * 11 + [f, f, u]
    return handle


def forward(*, query, key_pages, value_pages, key_scales, value_scales, runs, seq_lens, output, batch, num_q_heads,
            num_kv_heads, head_dim, page_size, group_tile, use_clustered_kernel, cluster_size, kv_format,
            keys_are_rotated, softmax_scale, rope_theta, stream) -> None:
    """All tensor arguments are torch CUDA tensors (or None for absent scales)."""

    def address(t) -> int:
        return 0 if t is None else int(t.data_ptr())

    rc = lib().fkref_page_decode_forward(
        address(query), address(key_pages), address(value_pages), address(key_scales), address(value_scales),
        address(runs["run_base_pages"]), address(runs["run_page_counts"]), address(runs["run_logical_starts"]),
        address(runs["run_last_page_lens"]), address(runs["request_run_offsets"]), address(seq_lens), address(output),
        batch, int(runs["run_base_pages"].numel()), num_q_heads, num_kv_heads, head_dim, page_size, group_tile,
        use_clustered_kernel, cluster_size, kv_format, int(keys_are_rotated), softmax_scale, rope_theta, stream)
    if rc != 0:
        raise RuntimeError("reference kernel call failed: " + lib().fkref_page_decode_last_error().decode(errors="replace"))
