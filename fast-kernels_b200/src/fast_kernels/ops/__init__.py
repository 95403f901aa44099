"""Python ops of the W4A16 decode path (same public names as the reference's ``fast_kernels.ops``
for this kernel family, plus the bf16 / explicit-dtype additions)."""

from fast_kernels.ops.decode_quant_linear import (
    LAYOUT_TO_GROUP_SIZE,
    arc_packet_stride_bytes,
    arc_w4a16_forward,
    arc_w4a16_supported_impls,
    cublaslt_fp16_after_dequant,
    cuda_decode_available,
    dequant_arc_w4a16_packets,
    dequant_w4a16_to_fp16,
    group_size_for_layout,
    pack_arc_w4a16_packets,
)

__all__ = [
    "LAYOUT_TO_GROUP_SIZE",
    "arc_packet_stride_bytes",
    "arc_w4a16_forward",
    "arc_w4a16_supported_impls",
    "cublaslt_fp16_after_dequant",
    "cuda_decode_available",
    "dequant_arc_w4a16_packets",
    "dequant_w4a16_to_fp16",
    "group_size_for_layout",
    "pack_arc_w4a16_packets",
]
