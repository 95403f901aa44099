"""Python ops of the decode path: the W4A16 linear layer and the paged-KV attention (same public names as the reference's ``fast_kernels.ops``
for this kernel family, plus the bf16 / explicit-dtype additions)."""

from fast_kernels.ops.clustered_page_decode import (
    ClusteredPageDecodePlan,
    PagedKVCache,
    clustered_page_decode,
    cuda_clustered_decode_available,
    estimate_page_decode_metrics,
    materialize_reference_dense_kv,
    pack_paged_kv_bf16,
    plan_clustered_page_decode,
    quantize_paged_kv_fp8,
    quantize_paged_kv_int8,
    reference_clustered_page_decode,
)
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
    "ClusteredPageDecodePlan",
    "PagedKVCache",
    "clustered_page_decode",
    "cuda_clustered_decode_available",
    "estimate_page_decode_metrics",
    "materialize_reference_dense_kv",
    "pack_paged_kv_bf16",
    "plan_clustered_page_decode",
    "quantize_paged_kv_fp8",
    "quantize_paged_kv_int8",
    "reference_clustered_page_decode",
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
