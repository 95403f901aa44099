"""The reference's own GPU tests for this path (tests/gpu/test_decode_quant_linear.py in
SamMausberg/fast-kernels), re-stated against this build's ``fast_kernels.ops``: same shapes, seed
formulas, value recipes, option strings and tolerances (atol = rtol = 1e-2; dequant 1e-3 there,
bit-exact here). Inputs are drawn on the CPU so the oracle sees the same bits. bf16 and group 32
are added as extra parameters."""

from __future__ import annotations

import numpy as np
import pytest
import torch
from fast_kernels.native import native_module
from fast_kernels.ops import (
    arc_w4a16_forward,
    arc_w4a16_supported_impls,
    cublaslt_fp16_after_dequant,
    dequant_arc_w4a16_packets,
    dequant_w4a16_to_fp16,
    pack_arc_w4a16_packets,
)
from oracle import w4a16_oracle as oracle

pytestmark = pytest.mark.gpu


def _inputs(seed: int, batch: int, n: int, k: int, group: int, lo: float, span: float, dtype=torch.float16):
    torch.manual_seed(seed)
    groups = k // group
    activations = torch.randn((batch, k), dtype=torch.float32).to(dtype).contiguous()
    q_u8 = torch.randint(0, 256, (n, k // 2), dtype=torch.uint8).contiguous()
    alpha = (lo + (span * torch.rand((n, groups), dtype=torch.float32))).to(dtype)
    zero_points = torch.randint(0, 16, (n, groups), dtype=torch.int16)
    beta = -(alpha * zero_points.to(dtype=dtype))
    return activations, q_u8, alpha, beta


def _explicit_reference_output(activations, q_u8, alpha, beta, *, group_size: int):
    """The reference's expectation (its test file, :46-60), evaluated on CPU tensors."""
    low = torch.bitwise_and(q_u8, 0x0F).to(torch.float32)
    high = torch.bitwise_right_shift(q_u8, 4).to(torch.float32)
    q_values = torch.stack((low, high), dim=-1).reshape(q_u8.shape[0], q_u8.shape[1] * 2)
    alpha_expanded = alpha.to(torch.float32).repeat_interleave(group_size, dim=1)
    beta_expanded = beta.to(torch.float32).repeat_interleave(group_size, dim=1)
    weights = (alpha_expanded * q_values) + beta_expanded
    return torch.matmul(activations.to(torch.float32), weights.transpose(0, 1)).to(activations.dtype)


def _assert_matches(out, cpu_inputs, group: int, atol: float = 1e-2, rtol: float = 1e-2) -> None:
    activations, q_u8, alpha, beta = cpu_inputs
    expected = _explicit_reference_output(activations, q_u8, alpha, beta, group_size=group)
    if activations.dtype == torch.bfloat16:
        atol, rtol = 4 * atol, 2 * rtol  # bf16 has 8 mantissa bits: one output ulp is 2^-8 relative
    torch.testing.assert_close(out.cpu(), expected, atol=atol, rtol=rtol)
    code = oracle.dtype_code(activations.dtype)
    y64 = oracle.gemv_f64(oracle.bits_of(activations), q_u8.numpy(), oracle.bits_of(alpha),
                          oracle.bits_of(beta), group, code)
    assert oracle.max_rel_err(out.float().cpu().numpy(), y64) <= 1e-2


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("group_size", [32, 64, 128])
@pytest.mark.parametrize("batch", [1, 4])
@pytest.mark.parametrize("impl", [None, "scalar", "tc", "wgmma"])
def test_arc_kernel_matches_explicit_reference(group_size, batch, impl, dtype) -> None:
    cpu = _inputs(7 + batch + group_size, batch, 128, group_size * 2, group_size, 0.05, 0.1, dtype)
    activations, q_u8, alpha, beta = (t.cuda() for t in cpu)
    packets = pack_arc_w4a16_packets(q_u8, alpha, beta, group_size=group_size)
    out = arc_w4a16_forward(activations, packets, n=128, k=group_size * 2, group_size=group_size, impl=impl)
    assert out.dtype == dtype and out.shape == (batch, 128)
    _assert_matches(out, cpu, group_size)


@pytest.mark.parametrize("group_size", [64, 128])
@pytest.mark.parametrize("batch", [8, 16])
def test_arc_scalar_direct_matches_reference(group_size: int, batch: int) -> None:
    cpu = _inputs(90 + batch + group_size, batch, 4096, group_size * 4, group_size, 0.03, 0.12)
    activations, q_u8, alpha, beta = (t.cuda() for t in cpu)
    packets = pack_arc_w4a16_packets(q_u8, alpha, beta, group_size=group_size)
    out = arc_w4a16_forward(activations, packets, n=4096, k=group_size * 4, group_size=group_size,
                            split_k_slices=1, impl="scalar")
    _assert_matches(out, cpu, group_size)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("group_size", [32, 64, 128])
def test_native_dequant_matches_explicit_reference(group_size: int, dtype) -> None:
    _, q_cpu, alpha_cpu, beta_cpu = _inputs(123 + group_size, 1, 128, group_size * 2, group_size, 0.03, 0.2, dtype)
    q_u8, alpha, beta = q_cpu.cuda(), alpha_cpu.cuda(), beta_cpu.cuda()
    native_weight = dequant_w4a16_to_fp16(q_u8, alpha, beta, group_size=group_size)
    low = torch.bitwise_and(q_cpu, 0x0F).to(torch.float32)
    high = torch.bitwise_right_shift(q_cpu, 4).to(torch.float32)
    q_values = torch.stack((low, high), dim=-1).reshape(128, group_size * 2)
    expected = (alpha_cpu.float().repeat_interleave(group_size, dim=1) * q_values
                + beta_cpu.float().repeat_interleave(group_size, dim=1)).to(dtype)
    assert torch.equal(native_weight.cpu(), expected)  # the reference asks for 1e-3; this is exact
    packets = pack_arc_w4a16_packets(q_u8, alpha, beta, group_size=group_size)
    from_packets = dequant_arc_w4a16_packets(packets, n=128, k=group_size * 2, group_size=group_size, dtype=dtype)
    assert torch.equal(from_packets.cpu(), expected)


def test_arc_split_k_override_matches_explicit_reference() -> None:
    cpu = _inputs(4242, 8, 128, 512, 128, 0.04, 0.12)
    activations, q_u8, alpha, beta = (t.cuda() for t in cpu)
    packets = pack_arc_w4a16_packets(q_u8, alpha, beta, group_size=128)
    partials = torch.empty((4, 8, 128), device="cuda", dtype=torch.float32)
    out = arc_w4a16_forward(activations, packets, n=128, k=512, group_size=128, split_k_slices=4,
                            partials=partials)
    _assert_matches(out, cpu, 128)
    assert torch.equal(out, (partials[0] + partials[1] + partials[2] + partials[3]).half())


def test_arc_impl_env_override_matches_explicit_reference(monkeypatch: pytest.MonkeyPatch) -> None:
    cpu = _inputs(5150, 4, 128, 512, 128, 0.04, 0.12)
    activations, q_u8, alpha, beta = (t.cuda() for t in cpu)
    packets = pack_arc_w4a16_packets(q_u8, alpha, beta, group_size=128)
    assert "wgmma" in arc_w4a16_supported_impls(torch.device("cuda"))
    monkeypatch.setenv("FK_ARC_W4A16_IMPL", "wgmma")
    out = arc_w4a16_forward(activations, packets, n=128, k=512, group_size=128)
    _assert_matches(out, cpu, 128)
    monkeypatch.setenv("FK_ARC_W4A16_IMPL", "nonsense")
    with pytest.raises(ValueError, match="impl must be one of"):
        arc_w4a16_forward(activations, packets, n=128, k=512, group_size=128)


def test_arc_kernel_respects_current_stream() -> None:
    cpu = _inputs(2112, 1, 128, 256, 128, 0.05, 0.1)
    expected_activations, q_u8, alpha, beta = (t.cuda() for t in cpu)
    activations = torch.zeros_like(expected_activations)
    packets = pack_arc_w4a16_packets(q_u8, alpha, beta, group_size=128)
    torch.cuda.synchronize()
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        torch.cuda._sleep(50_000_000)
        activations.copy_(expected_activations)
        out = arc_w4a16_forward(activations, packets, n=128, k=256, group_size=128)
    stream.synchronize()
    torch.cuda.synchronize()
    _assert_matches(out, cpu, 128)


def test_shape_and_option_errors_on_device() -> None:
    cpu = _inputs(1, 2, 128, 256, 128, 0.05, 0.1)
    activations, q_u8, alpha, beta = (t.cuda() for t in cpu)
    packets = pack_arc_w4a16_packets(q_u8, alpha, beta, group_size=128)
    with pytest.raises(ValueError, match=r"activations.shape\[1\] must match k"):
        arc_w4a16_forward(activations, packets, n=128, k=512, group_size=128)
    with pytest.raises(ValueError, match="packets must have shape"):
        arc_w4a16_forward(activations, packets, n=256, k=256, group_size=128)
    with pytest.raises(ValueError, match="split_k_slices must be positive"):
        arc_w4a16_forward(activations, packets, n=128, k=256, group_size=128, split_k_slices=0)
    with pytest.raises(ValueError, match="only supported by impl='scalar'"):
        arc_w4a16_forward(activations, packets, n=128, k=256, group_size=128, split_k_slices=2, impl="tc")
    with pytest.raises(ValueError, match="must not exceed the number of groups"):
        arc_w4a16_forward(activations, packets, n=128, k=256, group_size=128, split_k_slices=3)
    with pytest.raises(ValueError, match="output must have shape"):
        arc_w4a16_forward(activations, packets, n=128, k=256, group_size=128,
                          output=torch.empty((1, 128), device="cuda", dtype=torch.float16))
    with pytest.raises(ValueError, match="alpha must have shape"):
        pack_arc_w4a16_packets(q_u8, alpha[:, :1].contiguous(), beta, group_size=128)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_vendor_subject_and_cpp_launcher_without_workspace(dtype) -> None:
    """cublaslt_fp16_after_dequant (baseline subject) and the reference-signature C++ launcher,
    which owns its scratch because that signature has no parameter for it."""
    cpu = _inputs(77, 3, 256, 1024, 128, 0.005, 0.015, dtype)
    activations, q_u8, alpha, beta = (t.cuda() for t in cpu)
    vendor = cublaslt_fp16_after_dequant(activations, q_u8, alpha, beta, group_size=128)
    expected = _explicit_reference_output(*cpu, group_size=128)
    torch.testing.assert_close(vendor.cpu(), expected, atol=4e-2, rtol=2e-2)
    if dtype == torch.float16:
        native = native_module()
        packets = pack_arc_w4a16_packets(q_u8, alpha, beta, group_size=128)
        out = torch.full((3, 256), float("nan"), device="cuda", dtype=dtype)
        stream = int(torch.cuda.current_stream().cuda_stream)
        for _ in range(2):
            native.arc_w4a16_forward(activations.data_ptr(), packets.data_ptr(), 0, out.data_ptr(), 3, 256,
                                     1024, 128, 8704, stream)
        _assert_matches(out, cpu, 128)
        assert native.arc_w4a16_device_status() == 0


def test_native_forward_can_be_captured_after_one_warm_up_call() -> None:
    """The reference's arc_w4a16_forward takes no scratch, so the launcher layer owns one workspace
    per (device, stream). Its rule: the first call on a stream allocates (outside capture); every
    later call allocates nothing -- so it can be recorded into a CUDA graph -- and a first call
    made DURING capture fails with a RuntimeError instead of allocating."""
    native = native_module()
    group, n, k = 128, 1024, 2048
    cpu = _inputs(77, 1, n, k, group, 0.05, 0.1)
    activations, q_u8, alpha, beta = (t.cuda() for t in cpu)
    packets = pack_arc_w4a16_packets(q_u8, alpha, beta, group_size=group)
    stride = packets.shape[1]
    out = torch.zeros((1, n), dtype=torch.float16, device="cuda")
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())

    def call(stream: torch.cuda.Stream) -> None:
        native.arc_w4a16_forward(activations_ptr=activations.data_ptr(), packets_ptr=packets.data_ptr(),
                                 group_sums_ptr=0, output_ptr=out.data_ptr(), batch=1, n=n, k=k,
                                 group_size=group, packet_stride_bytes=stride, stream_ptr=stream.cuda_stream)

    with torch.cuda.stream(side):
        call(side)  # warm-up: allocates this stream's workspace
        side.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        out.zero_()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            call(side)
        graph.replay()
        side.synchronize()
        # nothing was allocated for the capture (torch may hand cached blocks back meanwhile)
        assert torch.cuda.mem_get_info()[0] >= free_before
    _assert_matches(out, cpu, group)

    fresh = torch.cuda.Stream()
    fresh.wait_stream(torch.cuda.current_stream())
    graph2 = torch.cuda.CUDAGraph()
    with pytest.raises(RuntimeError, match="outside capture"):
        with torch.cuda.stream(fresh):
            with torch.cuda.graph(graph2, stream=fresh):
                call(fresh)
    torch.cuda.synchronize()
