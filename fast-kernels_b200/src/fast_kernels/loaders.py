"""Weight-preparation path: common on-disk int4 tensor layouts -> the packer's inputs.

The reference only ever synthesises weights (benchmarking/decode_linear_w4a16.py:152-174); a model
that was quantised elsewhere arrives as three tensors per linear layer. This module turns the two
widespread layouts into what ``pack_arc_w4a16_packets`` takes -- ``q_u8[N, K/2]`` (low nibble = even
k), ``alpha[N, K/G]`` and ``beta[N, K/G] = -(alpha * zero_point)`` evaluated in the 16-bit type, the
same expression the reference's input recipe uses -- with plain tensor arithmetic, so it runs on
CPU or CUDA tensors alike and is bit-exact by construction.

Layouts (K input features, N output features, G group size, all nibbles unsigned 0..15):

* ``gptq``: ``qweight`` int32 ``[K/8, N]``, eight consecutive k of one column per word, k = 8r + i
  in bits 4i..4i+3; ``qzeros`` int32 ``[K/G, N/8]``, eight consecutive columns per word, stored as
  ``zero_point - 1`` (the format's v1 convention; pass ``zero_offset=0`` for files that store the
  zero point itself); ``scales`` 16-bit ``[K/G, N]``. Weight = scale * (q - zero_point).
* ``awq``: ``qweight`` int32 ``[K, N/8]`` and ``qzeros`` int32 ``[K/G, N/8]``, eight columns per
  word in the interleaved order (0, 2, 4, 6, 1, 3, 5, 7): column 8c + order[i] in bits 4i..4i+3;
  zero points stored as they are; ``scales`` 16-bit ``[K/G, N]``.

Activation reordering (``g_idx`` that is not the identity grouping) is refused: the packet format
has one scale per (column, contiguous group).
"""

from __future__ import annotations

from typing import Any

AWQ_ORDER = (0, 2, 4, 6, 1, 3, 5, 7)


def _torch() -> Any:
    import torch

    return torch


def _nibbles_of_words(words: Any) -> Any:
    """int32 ``[..., W]`` -> uint8 ``[..., W, 8]``: nibble i of every word."""
    torch = _torch()
    shifts = torch.arange(0, 32, 4, dtype=torch.int32, device=words.device)
    return ((words.to(torch.int32).unsqueeze(-1) >> shifts) & 0xF).to(torch.uint8)


def _pack_rows(q: Any) -> Any:
    """uint8 nibbles ``[N, K]`` -> ``q_u8[N, K/2]`` with the even k in the low nibble."""
    return (q[:, 0::2] | (q[:, 1::2] << 4)).contiguous()


def _affine(scales: Any, zero_points: Any, dtype: Any) -> tuple[Any, Any]:
    """``scales``, ``zero_points`` as ``[K/G, N]`` -> ``alpha``, ``beta`` as ``[N, K/G]`` in `dtype`."""
    alpha = scales.to(dtype).t().contiguous()
    beta = -(alpha * zero_points.t().to(dtype))
    return alpha, beta.contiguous()


def _check_common(k: int, n: int, group_size: int, scales: Any) -> None:
    if group_size not in (32, 64, 128):
        raise ValueError("group_size must be one of {32, 64, 128}")
    if n % 128 != 0:
        raise ValueError("n must be a multiple of 128")
    if k % group_size != 0:
        raise ValueError("k must be divisible by group_size")
    if tuple(scales.shape) != (k // group_size, n):
        raise ValueError(f"scales must have shape {(k // group_size, n)}")


def from_gptq(qweight: Any, qzeros: Any, scales: Any, *, group_size: int, dtype: Any | None = None,
              g_idx: Any | None = None, zero_offset: int = 1) -> tuple[Any, Any, Any]:
    """GPTQ-style tensors -> ``(q_u8, alpha, beta)``."""
    torch = _torch()
    if qweight.ndim != 2 or qzeros.ndim != 2:
        raise ValueError("qweight and qzeros must be rank-2 tensors")
    k, n = qweight.shape[0] * 8, qweight.shape[1]
    _check_common(k, n, group_size, scales)
    groups = k // group_size
    if tuple(qzeros.shape) != (groups, n // 8):
        raise ValueError(f"qzeros must have shape {(groups, n // 8)}")
    if g_idx is not None:
        expected = torch.arange(k, device=g_idx.device) // group_size
        if g_idx.numel() != k or not torch.equal(g_idx.to(expected.dtype).flatten(), expected):
            raise ValueError("activation reordering (a non-trivial g_idx) is not supported")
    dtype = dtype or scales.dtype
    # [K/8, N, 8] -> k = 8 r + i -> [N, K]
    q = _nibbles_of_words(qweight).permute(1, 0, 2).reshape(n, k)
    # a stored 15 with zero_offset = 1 means zero point 16; W = s (q - 16) still holds
    zeros = _nibbles_of_words(qzeros).reshape(groups, n).to(torch.int32) + zero_offset
    alpha, beta = _affine(scales, zeros, dtype)
    return _pack_rows(q), alpha, beta


def from_awq(qweight: Any, qzeros: Any, scales: Any, *, group_size: int,
             dtype: Any | None = None) -> tuple[Any, Any, Any]:
    """AWQ-style (GEMM layout) tensors -> ``(q_u8, alpha, beta)``."""
    torch = _torch()
    if qweight.ndim != 2 or qzeros.ndim != 2:
        raise ValueError("qweight and qzeros must be rank-2 tensors")
    k, n = qweight.shape[0], qweight.shape[1] * 8
    _check_common(k, n, group_size, scales)
    groups = k // group_size
    if tuple(qzeros.shape) != (groups, n // 8):
        raise ValueError(f"qzeros must have shape {(groups, n // 8)}")
    dtype = dtype or scales.dtype
    # nibble i of a word is column 8 c + AWQ_ORDER[i]: undo the interleave with a gather
    inverse = torch.empty(8, dtype=torch.long, device=qweight.device)
    inverse[torch.tensor(AWQ_ORDER, device=qweight.device)] = torch.arange(8, device=qweight.device)
    q = _nibbles_of_words(qweight).index_select(-1, inverse).reshape(k, n).t().contiguous()
    zeros = _nibbles_of_words(qzeros).index_select(-1, inverse).reshape(groups, n).to(torch.int32)
    alpha, beta = _affine(scales, zeros, dtype)
    return _pack_rows(q), alpha, beta


def load_linear(tensors: dict[str, Any], *, layout: str, group_size: int, dtype: Any | None = None,
                prefix: str = "") -> tuple[Any, Any, Any]:
    """Picks ``<prefix>qweight / qzeros / scales`` (and ``g_idx``) out of a checkpoint's tensor
    dictionary and converts them; `layout` is ``"gptq"`` or ``"awq"``."""
    try:
        qweight, qzeros, scales = (tensors[prefix + name] for name in ("qweight", "qzeros", "scales"))
    except KeyError as exc:
        raise KeyError(f"checkpoint has no tensor {exc.args[0]!r}") from None
    if layout == "gptq":
        return from_gptq(qweight, qzeros, scales, group_size=group_size, dtype=dtype,
                         g_idx=tensors.get(prefix + "g_idx"))
    if layout == "awq":
        return from_awq(qweight, qzeros, scales, group_size=group_size, dtype=dtype)
    raise ValueError("layout must be 'gptq' or 'awq'")
