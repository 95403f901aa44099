"""GPU parity against the reference's OWN CUDA kernels, run here on the same inputs.

``oracle/_ref/libfk_reference.so`` is the reference's arc_w4a16.cu compiled unmodified for sm_100a
(see oracle/reference_gpu.py). On the recipes of the reference's six GPU tests
(tests/gpu/test_decode_quant_linear.py:63-281), three of its bench cases and the single
CPU-runnable configuration (4096 x 4096, group 128, fp16, seed 0), these tests pin:

* packets from fk_w4a16_pack_packets are byte-equal to pack_arc_packets_kernel's (arc_w4a16.cu:87-122),
  and packets produced by the reference's packer feed fk_w4a16_gemv unchanged;
* both dequantisers are bit-equal to dequant_w4a16_kernel / dequant_arc_packets_kernel (:160-220);
* group sums are bit-equal to compute_arc_group_sums_kernel (:124-158);
* fk_w4a16_gemv is within the reference tests' atol = rtol = 1e-2 of arc_w4a16_forward (:687-707),
  and the reference kernel itself is within 1e-2 of the fp64 oracle -- which pins the oracle from
  the other side;
* the caller-visible split-K pair against arc_w4a16_forward_split_k + reduce (:709-751).

The reference is fp16 only, group sizes 64 and 128. Skipped when the library was not built.
"""

from __future__ import annotations

import numpy as np
import pytest
import torch
from fast_kernels import capi
from fast_kernels.workloads import REFERENCE_CASE, make_problem
from oracle import reference_gpu as ref
from oracle import w4a16_oracle as oracle
from w4a16_testlib import (
    Workspace,
    capi_gemv,
    capi_pack,
    dev_bits,
    golden_case_names,
    host_bits,
    load_golden,
    stream_ptr,
)

pytestmark = [
    pytest.mark.gpu,
    pytest.mark.skipif(not ref.available(), reason="oracle/_ref/libfk_reference.so is not built"),
]

WS = Workspace()
F16 = 0


def _case(name: str) -> dict:
    if name == "config0_4096x4096_g128_seed0":
        problem = make_problem(REFERENCE_CASE, seed=0)
        return {
            "q_u8": problem["q_u8"].numpy(),
            "alpha": oracle.bits_of(problem["alpha"]),
            "beta": oracle.bits_of(problem["beta"]),
            "activations": oracle.bits_of(problem["activations"]),
            "meta": {"group_size": 128, "n": 4096, "k": 4096, "batch": 1},
        }
    case = load_golden(name)
    if case is None:
        pytest.skip("this torch build does not reproduce the fixture's seeded inputs")
    return case


CASES = [*golden_case_names(), "config0_4096x4096_g128_seed0"]


def _device_inputs(case: dict):
    q = torch.from_numpy(case["q_u8"]).cuda()
    alpha, beta, act = (dev_bits(case[key], F16) for key in ("alpha", "beta", "activations"))
    return q, alpha, beta, act


def _ref_packets(q, alpha, beta, n: int, k: int, group: int) -> torch.Tensor:
    packets = torch.full(((n // 128) * (k // group), ref.stride(group)), 0xA5, dtype=torch.uint8, device="cuda")
    ref.pack(q.data_ptr(), alpha.data_ptr(), beta.data_ptr(), packets.data_ptr(), n, k, group, stream_ptr())
    return packets


def _ref_forward(act, packets, n: int, k: int, group: int) -> torch.Tensor:
    batch = act.shape[0]
    sums = torch.empty((batch, k // group), dtype=torch.float32, device="cuda")
    out = torch.full((batch, n), float("nan"), dtype=torch.float16, device="cuda")
    ref.group_sums(act.data_ptr(), sums.data_ptr(), batch, k, group, stream_ptr())
    ref.forward(act.data_ptr(), packets.data_ptr(), sums.data_ptr(), out.data_ptr(), batch, n, k, group,
                stream_ptr())
    return out


@pytest.mark.parametrize("name", CASES)
def test_pack_is_byte_equal_to_the_reference_packer(name: str) -> None:
    case = _case(name)
    meta = case["meta"]
    group, n, k = meta["group_size"], meta["n"], meta["k"]
    q, alpha, beta, act = _device_inputs(case)
    ours = capi_pack(capi, q, alpha, beta, group)
    theirs = _ref_packets(q, alpha, beta, n, k, group)
    torch.cuda.synchronize()
    assert torch.equal(ours, theirs)
    # and the reference's packets drive the new GEMV as they are
    from_theirs = capi_gemv(capi, WS, act, theirs, n, k, group, F16)
    from_ours = capi_gemv(capi, WS, act, ours, n, k, group, F16)
    torch.cuda.synchronize()
    assert torch.equal(from_theirs.view(torch.int16), from_ours.view(torch.int16))


@pytest.mark.parametrize("name", CASES)
def test_dequantisers_are_bit_equal_to_the_reference_kernels(name: str) -> None:
    case = _case(name)
    meta = case["meta"]
    group, n, k = meta["group_size"], meta["n"], meta["k"]
    q, alpha, beta, _ = _device_inputs(case)
    lib = capi.load_library()
    theirs = torch.empty((n, k), dtype=torch.float16, device="cuda")
    ours = torch.empty_like(theirs)
    ref.dequant(q.data_ptr(), alpha.data_ptr(), beta.data_ptr(), theirs.data_ptr(), n, k, group, stream_ptr())
    capi.check(lib.fk_w4a16_dequant_rowmajor(q.data_ptr(), alpha.data_ptr(), beta.data_ptr(), ours.data_ptr(),
                                             n, k, group, F16, stream_ptr()))
    torch.cuda.synchronize()
    assert torch.equal(ours.view(torch.int16), theirs.view(torch.int16))
    # the CPU oracle agrees with the reference kernel bit for bit as well
    want = oracle.dequant_rowmajor(case["q_u8"], case["alpha"], case["beta"], group, F16)
    assert np.array_equal(host_bits(theirs), want)

    packets = _ref_packets(q, alpha, beta, n, k, group)
    theirs.zero_()
    ours.zero_()
    ref.dequant_packets(packets.data_ptr(), theirs.data_ptr(), n, k, group, stream_ptr())
    capi.check(lib.fk_w4a16_dequant_packets(packets.data_ptr(), ours.data_ptr(), n, k, group,
                                            ref.stride(group), F16, stream_ptr()))
    torch.cuda.synchronize()
    assert torch.equal(ours.view(torch.int16), theirs.view(torch.int16))
    assert np.array_equal(host_bits(theirs), want)


@pytest.mark.parametrize("name", CASES)
def test_group_sums_are_bit_equal_to_the_reference_kernel(name: str) -> None:
    case = _case(name)
    meta = case["meta"]
    group, k, batch = meta["group_size"], meta["k"], meta["batch"]
    act = dev_bits(case["activations"], F16)
    theirs = torch.empty((batch, k // group), dtype=torch.float32, device="cuda")
    ours = torch.empty_like(theirs)
    ref.group_sums(act.data_ptr(), theirs.data_ptr(), batch, k, group, stream_ptr())
    capi.check(capi.load_library().fk_w4a16_group_sums(act.data_ptr(), ours.data_ptr(), batch, k, group, F16,
                                                       stream_ptr()))
    torch.cuda.synchronize()
    assert torch.equal(ours.view(torch.int32), theirs.view(torch.int32))
    assert np.array_equal(theirs.cpu().numpy().view(np.uint32),
                          oracle.group_sums(case["activations"], group, F16).view(np.uint32))


@pytest.mark.parametrize("name", CASES)
def test_gemv_matches_the_reference_forward_kernel(name: str) -> None:
    case = _case(name)
    meta = case["meta"]
    group, n, k = meta["group_size"], meta["n"], meta["k"]
    q, alpha, beta, act = _device_inputs(case)
    packets = _ref_packets(q, alpha, beta, n, k, group)
    theirs = _ref_forward(act, packets, n, k, group)
    ours = capi_gemv(capi, WS, act, packets, n, k, group, F16)
    torch.cuda.synchronize()
    assert torch.isfinite(theirs.float()).all() and torch.isfinite(ours.float()).all()
    # the reference tests' own bar (tests/gpu/test_decode_quant_linear.py:102)
    torch.testing.assert_close(ours, theirs, atol=1e-2, rtol=1e-2)
    # both against the fp64 oracle: pins the oracle to the reference kernel, and us to both
    y64 = oracle.gemv_f64(case["activations"], case["q_u8"], case["alpha"], case["beta"], group, F16)
    assert oracle.max_rel_err(theirs.float().cpu().numpy(), y64) <= 1e-2
    assert oracle.max_rel_err(ours.float().cpu().numpy(), y64) <= 1e-2
    # the oracle's restatement of the reference kernel's own fp32 summation order gives its bits
    # up to the last place of the 16-bit result (the kernel's FMA contraction is the compiler's)
    restated = oracle.gemv_ref_order(case["activations"], case["q_u8"], case["alpha"], case["beta"], group, F16)
    restated_f = oracle.np_to_f32(restated, F16).astype(np.float64)
    assert oracle.max_rel_err(theirs.float().cpu().numpy(), restated_f) <= 2e-3


@pytest.mark.parametrize("slices", [2, 4])
def test_split_k_pair_matches_the_reference_pair(slices: int) -> None:
    case = _case("ref_test_split_k")
    meta = case["meta"]
    group, n, k, batch = meta["group_size"], meta["n"], meta["k"], meta["batch"]
    if slices > k // group:
        pytest.skip("more slices than groups")
    q, alpha, beta, act = _device_inputs(case)
    packets = _ref_packets(q, alpha, beta, n, k, group)
    lib = capi.load_library()
    sums = torch.empty((batch, k // group), dtype=torch.float32, device="cuda")
    ref.group_sums(act.data_ptr(), sums.data_ptr(), batch, k, group, stream_ptr())
    theirs_partials = torch.full((slices, batch, n), float("nan"), dtype=torch.float32, device="cuda")
    ref.forward_split_k(act.data_ptr(), packets.data_ptr(), sums.data_ptr(), theirs_partials.data_ptr(), batch,
                        n, k, group, slices, stream_ptr())
    theirs = torch.empty((batch, n), dtype=torch.float16, device="cuda")
    ref.reduce(theirs_partials.data_ptr(), theirs.data_ptr(), batch, n, slices, stream_ptr())

    ours_partials = torch.full_like(theirs_partials, float("nan"))
    capi.check(lib.fk_w4a16_gemv_split_k(act.data_ptr(), packets.data_ptr(), ours_partials.data_ptr(), batch, n,
                                         k, group, ref.stride(group), slices, F16, stream_ptr()))
    ours = torch.empty_like(theirs)
    capi.check(lib.fk_w4a16_reduce_partials(ours_partials.data_ptr(), ours.data_ptr(), batch, n, slices, F16,
                                            stream_ptr()))
    # our reduce kernel on THEIR partials gives their bits: same slice order, one rounding
    cross = torch.empty_like(theirs)
    capi.check(lib.fk_w4a16_reduce_partials(theirs_partials.data_ptr(), cross.data_ptr(), batch, n, slices, F16,
                                            stream_ptr()))
    torch.cuda.synchronize()
    assert torch.equal(cross.view(torch.int16), theirs.view(torch.int16))
    scale = theirs_partials.abs().max().item()
    assert (ours_partials - theirs_partials).abs().max().item() <= 1e-4 * scale  # same slices, fp32
    torch.testing.assert_close(ours, theirs, atol=1e-2, rtol=1e-2)
