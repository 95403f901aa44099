"""Tensor-level API of the W4A16 decode ops.

Mirrors ``src/fast_kernels/ops/decode_quant_linear.py`` of SamMausberg/fast-kernels: the same
function names, keyword arguments, argument checks and error types (``TypeError`` for a wrong
tensor type or dtype, ``ValueError`` for shapes, devices and option strings, ``RuntimeError`` when
the native module is missing). What differs:

* there is one implementation, the sm_100a kernel. The ``impl`` argument and the
  ``FK_ARC_W4A16_IMPL`` variable still accept ``auto | scalar | tc | wgmma`` (the reference's
  tests pass them) but all of them run the same kernel; the cuBLASLt route stays available only
  as the baseline subject ``cublaslt_fp16_after_dequant``;
* no autotuning and no separate group-sum launch: ``arc_w4a16_forward`` is a single kernel launch
  that also finishes split-K; ``split_k_slices > 1`` selects the caller-visible partials path;
* ``torch.bfloat16`` tensors and ``group_size=32`` are accepted everywhere (the 16-bit dtype of
  activations, scales, offsets and outputs must agree).

Every call is enqueued on ``torch.cuda.current_stream()`` and never synchronises.
"""

from __future__ import annotations

import os
from typing import TYPE_CHECKING, Any

from fast_kernels.native import native_build_info, native_module

if TYPE_CHECKING:  # pragma: no cover
    import torch

_ARC_IMPL_ENV = "FK_ARC_W4A16_IMPL"
_ARC_IMPLS = ("auto", "scalar", "tc", "wgmma")
_VENDOR_WORKSPACE_BYTES = 8 * 1024 * 1024

LAYOUT_TO_GROUP_SIZE: dict[str, int] = {
    "groupwise_32": 32,
    "groupwise_64": 64,
    "groupwise_128": 128,
}

# Scratch owned by this module, keyed like the reference's caches (device, and stream for the
# buffers a kernel writes): tensors are reused across calls and never freed while the process
# lives, so a kernel still in flight can never see its scratch recycled.
_WORKSPACES: dict[tuple[int, int], Any] = {}
_WEIGHT_BUFFERS: dict[tuple[int, int, int, Any], Any] = {}
_VENDOR_WORKSPACES: dict[tuple[int, int], Any] = {}
_PARTIALS: dict[tuple[int, int, int, int, int], Any] = {}


def _require_torch() -> Any:
    try:
        import torch
    except ImportError as exc:  # pragma: no cover
        raise RuntimeError("PyTorch is required for decode_quant_linear ops") from exc
    return torch


def cuda_decode_available() -> bool:
    info = native_build_info()
    return bool(info.get("available", False)) and bool(info.get("compiled_with_cuda", False))


def group_size_for_layout(layout: str) -> int:
    try:
        return LAYOUT_TO_GROUP_SIZE[layout]
    except KeyError as exc:
        raise ValueError(f"unsupported layout: {layout}") from exc


def arc_packet_stride_bytes(group_size: int) -> int:
    if group_size not in {32, 64, 128}:
        raise ValueError("group_size must be 32, 64 or 128")
    return (128 * (group_size // 2)) + (2 * 128 * 2)


def _require_cuda_backend() -> Any:
    if not cuda_decode_available():
        raise RuntimeError("fast-kernels native module was built without CUDA support")
    return native_module()


def _float_dtypes() -> tuple[Any, Any]:
    torch = _require_torch()
    return (torch.float16, torch.bfloat16)


def _check_cuda_tensor(tensor: Any, *, name: str, dtype: Any, ndim: int) -> None:
    """dtype may be one torch dtype or a tuple of accepted ones."""
    torch = _require_torch()
    if not isinstance(tensor, torch.Tensor):
        raise TypeError(f"{name} must be a torch.Tensor")
    accepted = dtype if isinstance(dtype, tuple) else (dtype,)
    if tensor.dtype not in accepted:
        wanted = " or ".join(str(d) for d in accepted)
        raise TypeError(f"{name} must have dtype {wanted}")
    if tensor.ndim != ndim:
        raise ValueError(f"{name} must be {ndim}D")
    if not tensor.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor")
    if not tensor.is_contiguous():
        raise ValueError(f"{name} must be contiguous")


def _check_same_cuda_device(*named_tensors: tuple[str, Any]) -> None:
    devices = {tensor.device for _, tensor in named_tensors}
    if len(devices) <= 1:
        return
    summary = ", ".join(f"{name}={tensor.device}" for name, tensor in named_tensors)
    raise ValueError(f"all CUDA tensors must be on the same device: {summary}")


def _check_same_dtype(*named_tensors: tuple[str, Any]) -> None:
    dtypes = {tensor.dtype for _, tensor in named_tensors}
    if len(dtypes) > 1:
        summary = ", ".join(f"{name}={tensor.dtype}" for name, tensor in named_tensors)
        raise TypeError(f"16-bit tensors must share one dtype: {summary}")


def _element_type(native: Any, dtype: Any) -> int:
    torch = _require_torch()
    return int(native.ELEMENT_BFLOAT16 if dtype == torch.bfloat16 else native.ELEMENT_FLOAT16)


def _current_stream_ptr(device: Any) -> int:
    torch = _require_torch()
    return int(torch.cuda.current_stream(device=device).cuda_stream)


def _device_index(device: Any) -> int:
    torch = _require_torch()
    return int(device.index if device.index is not None else torch.cuda.current_device())


def arc_w4a16_supported_impls(device: Any | None = None) -> tuple[str, ...]:
    """Option strings ``arc_w4a16_forward`` accepts. All of them run the sm_100a kernel."""
    del device
    if not cuda_decode_available():
        return ("auto", "scalar")
    return _ARC_IMPLS


def _resolve_arc_impl(device: Any, impl: str | None) -> str:
    if impl is None:
        impl = os.environ.get(_ARC_IMPL_ENV, "auto")
    normalized = impl.strip().lower()
    if normalized not in _ARC_IMPLS:
        raise ValueError(f"impl must be one of {sorted(_ARC_IMPLS)} or omitted; received {impl!r}")
    supported = set(arc_w4a16_supported_impls(device))
    if normalized != "auto" and normalized not in supported:
        raise ValueError(
            f"impl={normalized!r} is unsupported on device {device}; "
            f"supported implementations are {sorted(supported)}"
        )
    return normalized


def _gemv_workspace(native: Any, device: Any, stream_ptr: int, need: int) -> Any:
    """Zero-initialised GEMV scratch for (device, stream); grows, never shrinks."""
    torch = _require_torch()
    key = (_device_index(device), stream_ptr)
    buffer = _WORKSPACES.get(key)
    if buffer is None or buffer.numel() < need:
        # Sized generously so that shape changes do not reallocate; the old tensor is dropped only
        # after the allocator has ordered its reuse behind work already queued on this stream.
        buffer = torch.zeros(max(need * 2, 4 << 20), device=device, dtype=torch.uint8)
        _WORKSPACES[key] = buffer
    return buffer


def pack_arc_w4a16_packets(
    q_u8: torch.Tensor,
    alpha: torch.Tensor,
    beta: torch.Tensor,
    *,
    group_size: int,
    packets: torch.Tensor | None = None,
) -> torch.Tensor:
    torch = _require_torch()
    native = _require_cuda_backend()
    _check_cuda_tensor(q_u8, name="q_u8", dtype=torch.uint8, ndim=2)
    _check_cuda_tensor(alpha, name="alpha", dtype=_float_dtypes(), ndim=2)
    _check_cuda_tensor(beta, name="beta", dtype=_float_dtypes(), ndim=2)
    _check_same_dtype(("alpha", alpha), ("beta", beta))

    n, packed_k = q_u8.shape
    k = packed_k * 2
    num_groups = k // group_size
    if alpha.shape != (n, num_groups):
        raise ValueError("alpha must have shape [n, k // group_size]")
    if beta.shape != (n, num_groups):
        raise ValueError("beta must have shape [n, k // group_size]")

    packet_stride = arc_packet_stride_bytes(group_size)
    num_tiles = n // 128
    if n % 128 != 0:
        raise ValueError("n must be divisible by 128")
    expected_shape = (num_tiles * num_groups, packet_stride)

    if packets is None:
        packets = torch.empty(expected_shape, device=q_u8.device, dtype=torch.uint8)
    else:
        _check_cuda_tensor(packets, name="packets", dtype=torch.uint8, ndim=2)
        if packets.shape != expected_shape:
            raise ValueError(f"packets must have shape {expected_shape}")

    _check_same_cuda_device(("q_u8", q_u8), ("alpha", alpha), ("beta", beta), ("packets", packets))
    native.pack_arc_w4a16_packets(
        q_u8.data_ptr(),
        alpha.data_ptr(),
        beta.data_ptr(),
        packets.data_ptr(),
        n,
        k,
        group_size,
        packet_stride,
        _current_stream_ptr(q_u8.device),
    )
    return packets


def arc_w4a16_forward(
    activations: torch.Tensor,
    packets: torch.Tensor,
    *,
    n: int,
    k: int,
    group_size: int,
    output: torch.Tensor | None = None,
    split_k_slices: int | None = None,
    partials: torch.Tensor | None = None,
    impl: str | None = None,
) -> torch.Tensor:
    torch = _require_torch()
    native = _require_cuda_backend()
    _check_cuda_tensor(activations, name="activations", dtype=_float_dtypes(), ndim=2)
    _check_cuda_tensor(packets, name="packets", dtype=torch.uint8, ndim=2)

    batch = activations.shape[0]
    if activations.shape[1] != k:
        raise ValueError("activations.shape[1] must match k")

    packet_stride = arc_packet_stride_bytes(group_size)
    num_groups = k // group_size
    expected_packets = ((n // 128) * num_groups, packet_stride)
    if packets.shape != expected_packets:
        raise ValueError(f"packets must have shape {expected_packets}")

    if output is None:
        output = torch.empty((batch, n), device=activations.device, dtype=activations.dtype)
    else:
        _check_cuda_tensor(output, name="output", dtype=activations.dtype, ndim=2)
        if output.shape != (batch, n):
            raise ValueError(f"output must have shape {(batch, n)}")

    _check_same_cuda_device(("activations", activations), ("packets", packets), ("output", output))

    resolved_impl = _resolve_arc_impl(activations.device, impl)
    if split_k_slices is not None and split_k_slices < 1:
        raise ValueError("split_k_slices must be positive")
    if resolved_impl in {"tc", "wgmma"} and split_k_slices not in {None, 1}:
        raise ValueError("split_k_slices is only supported by impl='scalar'")

    element_type = _element_type(native, activations.dtype)
    stream_ptr = _current_stream_ptr(activations.device)

    if split_k_slices is None or split_k_slices <= 1:
        need = int(native.arc_w4a16_workspace_bytes(batch, n, k, group_size))
        workspace = _gemv_workspace(native, activations.device, stream_ptr, need)
        native.arc_w4a16_forward_fused(
            activations.data_ptr(),
            packets.data_ptr(),
            output.data_ptr(),
            workspace.data_ptr(),
            workspace.numel(),
            batch,
            n,
            k,
            group_size,
            packet_stride,
            element_type,
            stream_ptr,
        )
        return output

    if partials is None:
        key = (_device_index(activations.device), stream_ptr, batch, n, split_k_slices)
        partials = _PARTIALS.get(key)
        if partials is None:
            partials = torch.empty(
                (split_k_slices, batch, n), device=activations.device, dtype=torch.float32
            )
            _PARTIALS[key] = partials
    else:
        _check_cuda_tensor(partials, name="partials", dtype=torch.float32, ndim=3)
        if tuple(partials.shape) != (split_k_slices, batch, n):
            raise ValueError(f"partials must have shape {(split_k_slices, batch, n)}")
        _check_same_cuda_device(
            ("activations", activations),
            ("packets", packets),
            ("output", output),
            ("partials", partials),
        )
    native.arc_w4a16_forward_split_k_typed(
        activations.data_ptr(),
        packets.data_ptr(),
        partials.data_ptr(),
        batch,
        n,
        k,
        group_size,
        packet_stride,
        split_k_slices,
        element_type,
        stream_ptr,
    )
    native.reduce_arc_w4a16_split_k_partials_typed(
        partials.data_ptr(), output.data_ptr(), batch, n, split_k_slices, element_type, stream_ptr
    )
    return output


def dequant_w4a16_to_fp16(
    q_u8: torch.Tensor,
    alpha: torch.Tensor,
    beta: torch.Tensor,
    *,
    group_size: int,
    output: torch.Tensor | None = None,
) -> torch.Tensor:
    """W[n, k] = alpha * q + beta in the dtype of ``alpha`` (fp16 as in the reference, or bf16)."""
    torch = _require_torch()
    native = _require_cuda_backend()
    _check_cuda_tensor(q_u8, name="q_u8", dtype=torch.uint8, ndim=2)
    _check_cuda_tensor(alpha, name="alpha", dtype=_float_dtypes(), ndim=2)
    _check_cuda_tensor(beta, name="beta", dtype=alpha.dtype, ndim=2)

    n, packed_k = q_u8.shape
    k = packed_k * 2
    num_groups = k // group_size
    if alpha.shape != (n, num_groups):
        raise ValueError("alpha must have shape [n, k // group_size]")
    if beta.shape != (n, num_groups):
        raise ValueError("beta must have shape [n, k // group_size]")

    if output is None:
        output = torch.empty((n, k), device=q_u8.device, dtype=alpha.dtype)
    else:
        _check_cuda_tensor(output, name="output", dtype=alpha.dtype, ndim=2)
        if output.shape != (n, k):
            raise ValueError(f"output must have shape {(n, k)}")

    _check_same_cuda_device(("q_u8", q_u8), ("alpha", alpha), ("beta", beta), ("output", output))
    native.dequant_w4a16_typed(
        q_u8.data_ptr(),
        alpha.data_ptr(),
        beta.data_ptr(),
        output.data_ptr(),
        n,
        k,
        group_size,
        _element_type(native, alpha.dtype),
        _current_stream_ptr(q_u8.device),
    )
    return output


def dequant_arc_w4a16_packets(
    packets: torch.Tensor,
    *,
    n: int,
    k: int,
    group_size: int,
    dtype: Any | None = None,
    output: torch.Tensor | None = None,
) -> torch.Tensor:
    """The same weight matrix, recovered from ARC packets."""
    torch = _require_torch()
    native = _require_cuda_backend()
    _check_cuda_tensor(packets, name="packets", dtype=torch.uint8, ndim=2)
    packet_stride = arc_packet_stride_bytes(group_size)
    expected_packets = ((n // 128) * (k // group_size), packet_stride)
    if packets.shape != expected_packets:
        raise ValueError(f"packets must have shape {expected_packets}")
    if output is None:
        output = torch.empty((n, k), device=packets.device, dtype=dtype or torch.float16)
    else:
        _check_cuda_tensor(output, name="output", dtype=_float_dtypes(), ndim=2)
        if output.shape != (n, k):
            raise ValueError(f"output must have shape {(n, k)}")
    _check_same_cuda_device(("packets", packets), ("output", output))
    native.dequant_arc_w4a16_packets_typed(
        packets.data_ptr(),
        output.data_ptr(),
        n,
        k,
        group_size,
        packet_stride,
        _element_type(native, output.dtype),
        _current_stream_ptr(packets.device),
    )
    return output


def cublaslt_fp16_after_dequant(
    activations: torch.Tensor,
    q_u8: torch.Tensor,
    alpha: torch.Tensor,
    beta: torch.Tensor,
    *,
    group_size: int,
    output: torch.Tensor | None = None,
    weight_buffer: torch.Tensor | None = None,
    workspace: torch.Tensor | None = None,
) -> torch.Tensor:
    """Vendor baseline subject: dequantise to a 16-bit weight, then a cuBLASLt GEMM (fp32 compute)."""
    torch = _require_torch()
    native = _require_cuda_backend()
    _check_cuda_tensor(activations, name="activations", dtype=_float_dtypes(), ndim=2)
    _check_cuda_tensor(q_u8, name="q_u8", dtype=torch.uint8, ndim=2)
    _check_cuda_tensor(alpha, name="alpha", dtype=activations.dtype, ndim=2)
    _check_cuda_tensor(beta, name="beta", dtype=activations.dtype, ndim=2)

    batch, k = activations.shape
    n, packed_k = q_u8.shape
    if packed_k * 2 != k:
        raise ValueError("q_u8.shape[1] must match activations.shape[1] / 2")
    num_groups = k // group_size
    if alpha.shape != (n, num_groups):
        raise ValueError("alpha must have shape [n, k // group_size]")
    if beta.shape != (n, num_groups):
        raise ValueError("beta must have shape [n, k // group_size]")

    if output is None:
        output = torch.empty((batch, n), device=activations.device, dtype=activations.dtype)
    else:
        _check_cuda_tensor(output, name="output", dtype=activations.dtype, ndim=2)
        if output.shape != (batch, n):
            raise ValueError(f"output must have shape {(batch, n)}")

    stream_ptr = _current_stream_ptr(activations.device)
    if weight_buffer is None:
        key = (_device_index(activations.device), n, k, activations.dtype)
        weight_buffer = _WEIGHT_BUFFERS.get(key)
        if weight_buffer is None:
            weight_buffer = torch.empty((n, k), device=activations.device, dtype=activations.dtype)
            _WEIGHT_BUFFERS[key] = weight_buffer
    else:
        _check_cuda_tensor(weight_buffer, name="weight_buffer", dtype=activations.dtype, ndim=2)
        if weight_buffer.shape != (n, k):
            raise ValueError(f"weight_buffer must have shape {(n, k)}")

    if workspace is None:
        key2 = (_device_index(activations.device), stream_ptr)
        workspace = _VENDOR_WORKSPACES.get(key2)
        if workspace is None:
            workspace = torch.empty(_VENDOR_WORKSPACE_BYTES, device=activations.device, dtype=torch.uint8)
            _VENDOR_WORKSPACES[key2] = workspace
    else:
        _check_cuda_tensor(workspace, name="workspace", dtype=torch.uint8, ndim=1)

    _check_same_cuda_device(
        ("activations", activations),
        ("q_u8", q_u8),
        ("alpha", alpha),
        ("beta", beta),
        ("output", output),
        ("weight_buffer", weight_buffer),
        ("workspace", workspace),
    )
    element_type = _element_type(native, activations.dtype)
    native.dequant_w4a16_typed(
        q_u8.data_ptr(), alpha.data_ptr(), beta.data_ptr(), weight_buffer.data_ptr(), n, k,
        group_size, element_type, stream_ptr,
    )
    native.cublaslt_with_weight_typed(
        activations.data_ptr(), weight_buffer.data_ptr(), output.data_ptr(), workspace.data_ptr(),
        workspace.numel(), batch, n, k, element_type, stream_ptr,
    )
    return output
