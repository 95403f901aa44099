"""The Python op layer (fast_kernels.ops) keeps the reference's public surface and error
behaviour. CPU-only checks here; numerics are in the gpu-marked tests."""

from __future__ import annotations

import inspect

import pytest
import torch
from fast_kernels import ops
from fast_kernels.native import native_available, native_build_info, native_module


def test_native_module_reports_build_info() -> None:
    # mirrors tests/cpu_smoke/test_import.py:4-7 of the reference
    info = native_build_info()
    assert "available" in info
    assert native_available()
    for key in ("project_version", "compiled_with_cuda", "cxx_compiler_id", "cxx_compiler_version",
                "cuda_compiler_version", "cuda_architectures"):
        assert key in info  # the reference's build_info keys (python_module.cpp:17-26)
    assert info["compiled_with_cuda"] is True
    assert info["cuda_architectures"] == "100a"


def test_native_module_exports_the_reference_binding_names() -> None:
    native = native_module()
    for name in (
        "build_info", "compute_arc_w4a16_group_sums", "pack_arc_w4a16_packets", "arc_w4a16_forward",
        "arc_w4a16_forward_split_k", "reduce_arc_w4a16_split_k_partials", "dequant_w4a16_to_fp16",
        "dequant_arc_w4a16_packets_to_fp16", "cublaslt_fp16_with_weight",
        "cublaslt_fp16_after_packet_dequant", "cublaslt_fp16_after_dequant",
    ):
        assert hasattr(native, name), name
    # keyword names equal the C++ parameter names, as in the reference bindings
    doc = native.arc_w4a16_forward.__doc__
    for kw in ("activations_ptr", "packets_ptr", "group_sums_ptr", "output_ptr", "batch", "n", "k",
               "group_size", "packet_stride_bytes", "stream_ptr"):
        assert kw in doc
    with pytest.raises(ValueError, match="batch and k must be positive"):
        native.arc_w4a16_forward(activations_ptr=256, packets_ptr=256, group_sums_ptr=0, output_ptr=256,
                                 batch=0, n=128, k=256, group_size=128, packet_stride_bytes=8704,
                                 stream_ptr=0)
    with pytest.raises(ValueError, match="packet_stride_bytes=1 does not match expected 4608"):
        native.pack_arc_w4a16_packets(256, 256, 256, 256, 128, 256, 64, 1, 0)


def test_public_names_and_signatures() -> None:
    for name in ("arc_packet_stride_bytes", "arc_w4a16_forward", "arc_w4a16_supported_impls",
                 "pack_arc_w4a16_packets", "dequant_w4a16_to_fp16", "cublaslt_fp16_after_dequant",
                 "cuda_decode_available", "group_size_for_layout"):
        assert hasattr(ops, name), name
    forward = inspect.signature(ops.arc_w4a16_forward)
    assert list(forward.parameters) == ["activations", "packets", "n", "k", "group_size", "output",
                                        "split_k_slices", "partials", "impl"]
    assert all(p.kind is inspect.Parameter.KEYWORD_ONLY for p in list(forward.parameters.values())[2:])
    pack = inspect.signature(ops.pack_arc_w4a16_packets)
    assert list(pack.parameters) == ["q_u8", "alpha", "beta", "group_size", "packets"]


def test_layouts_strides_and_impl_strings() -> None:
    assert ops.group_size_for_layout("groupwise_64") == 64
    assert ops.group_size_for_layout("groupwise_128") == 128
    assert ops.group_size_for_layout("groupwise_32") == 32
    with pytest.raises(ValueError, match="unsupported layout"):
        ops.group_size_for_layout("rowwise")
    assert ops.arc_packet_stride_bytes(128) == 8704
    assert ops.arc_packet_stride_bytes(64) == 4608
    with pytest.raises(ValueError):
        ops.arc_packet_stride_bytes(48)
    assert ops.cuda_decode_available()
    assert set(ops.arc_w4a16_supported_impls()) == {"auto", "scalar", "tc", "wgmma"}


def test_tensor_validation_errors_without_a_gpu() -> None:
    act = torch.zeros((1, 256), dtype=torch.float16)
    packets = torch.zeros((2, 8704), dtype=torch.uint8)
    with pytest.raises(ValueError, match="activations must be a CUDA tensor"):
        ops.arc_w4a16_forward(act, packets, n=128, k=256, group_size=128)
    with pytest.raises(TypeError, match="activations must have dtype"):
        ops.arc_w4a16_forward(act.float(), packets, n=128, k=256, group_size=128)
    with pytest.raises(TypeError, match="must be a torch.Tensor"):
        ops.arc_w4a16_forward([1, 2], packets, n=128, k=256, group_size=128)
    with pytest.raises(ValueError, match="must be 2D"):
        ops.arc_w4a16_forward(act[0], packets, n=128, k=256, group_size=128)
    q = torch.zeros((128, 128), dtype=torch.uint8)
    scales = torch.zeros((128, 2), dtype=torch.float16)
    with pytest.raises(ValueError, match="q_u8 must be a CUDA tensor"):
        ops.pack_arc_w4a16_packets(q, scales, scales, group_size=128)
    with pytest.raises(ValueError, match="q_u8 must be a CUDA tensor"):
        ops.dequant_w4a16_to_fp16(q, scales, scales, group_size=128)
