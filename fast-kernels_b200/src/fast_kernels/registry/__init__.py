"""Kernel and baseline ids a suite may name (``fk verify`` checks suites against these).

The W4A16 and paged-decode ids are the reference's (src/fast_kernels/registry/kernels.py:17-49 and
baselines.py:16-27); here all four kernel ids run the one sm_100a kernel. ``template/noop_gemm``
and its two baselines stay registered because the reference's CLI smoke test benches the
scaffold suite that names them.
"""

from __future__ import annotations

from dataclasses import dataclass

__all__ = ["BaselineSpec", "KernelSpec", "baseline_registry", "kernel_registry"]


@dataclass(frozen=True, slots=True)
class KernelSpec:
    kernel_id: str
    family: str
    description: str
    maturity: str
    impl: str | None = None  # the ``impl=`` string the op is called with


@dataclass(frozen=True, slots=True)
class BaselineSpec:
    baseline_id: str
    source: str
    family: str
    description: str


_ONE_KERNEL = "sm_100a streaming W4A16 GEMV (bulk-copy ring, LOP3 unpack, mixed-precision FMA, in-launch split-K)"


def kernel_registry() -> dict[str, KernelSpec]:
    specs = [
        KernelSpec("decode/w4a16_linear", "decode_quant_linear", _ONE_KERNEL + "; impl=auto", "beta", None),
        KernelSpec("decode/w4a16_linear_scalar", "decode_quant_linear", _ONE_KERNEL + "; impl=scalar", "beta", "scalar"),
        KernelSpec("decode/w4a16_linear_tc", "decode_quant_linear", _ONE_KERNEL + "; impl=tc (same kernel)", "beta", "tc"),
        KernelSpec("decode/w4a16_linear_wgmma", "decode_quant_linear", _ONE_KERNEL + "; impl=wgmma (same kernel)", "beta", "wgmma"),
        KernelSpec("decode/clustered_page_decode_auto", "clustered_page_decode",
                   "sm_100a paged-KV decode attention (bulk-copy unit ring per warp, split over blocks); force_impl=auto", "beta", "auto"),
        KernelSpec("decode/clustered_page_decode_direct", "clustered_page_decode",
                   "the same kernel, one block per (request, kv head, head tile); force_impl=direct", "beta", "direct"),
        KernelSpec("decode/clustered_page_decode_clustered", "clustered_page_decode",
                   "the same kernel, pages cut over as many blocks as fill the device; force_impl=clustered", "beta", "clustered"),
        KernelSpec("decode/prefix_union_decode_auto", "prefix_union_decode",
                   "shared-prefix paged decode; below compute capability 12 the plan's fallback (the paged-KV decode kernel)", "beta", "auto"),
        KernelSpec("decode/prefix_union_decode_union", "prefix_union_decode",
                   "registered as in the reference; its union kernel needs compute capability 12, reported as skipped", "scaffold", "union"),
        KernelSpec("decode/prefix_union_decode_fallback", "prefix_union_decode",
                   "shared-prefix paged decode through the paged-KV decode kernel", "beta", "fallback"),
        KernelSpec("template/noop_gemm", "gemm", "scaffold entry used by the template suite", "scaffold", None),
    ]
    return {spec.kernel_id: spec for spec in specs}


def baseline_registry() -> dict[str, BaselineSpec]:
    specs = [
        BaselineSpec("torch/reference_w4a16_linear", "torch", "decode_quant_linear",
                     "dequantise to a 16-bit weight with the native kernel, then torch.mm"),
        BaselineSpec("vendor/cublaslt_fp16_after_dequant", "vendor", "decode_quant_linear",
                     "dequantise, then a cuBLASLt GEMM with fp32 compute"),
        BaselineSpec("torch/reference_clustered_page_decode", "torch", "clustered_page_decode",
                     "dense gather through the page table, rotary embedding, softmax attention in PyTorch"),
        BaselineSpec("vendor/flashinfer_clustered_page_decode", "vendor", "clustered_page_decode",
                     "registered as in the reference; reported as skipped (no cache-layout converter here)"),
        BaselineSpec("torch/reference_prefix_union_decode", "torch", "prefix_union_decode",
                     "the PyTorch statement of the paged decode (sharing pages does not change the mathematics)"),
        BaselineSpec("torch/reference_gemm", "torch", "gemm", "scaffold baseline of the template suite"),
        BaselineSpec("vendor/cublaslt_gemm", "vendor", "gemm", "scaffold baseline of the template suite"),
    ]
    return {spec.baseline_id: spec for spec in specs}
