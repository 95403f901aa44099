"""Pins the CPU oracle (oracle/w4a16_oracle.c) to the reference's own arithmetic.

The fixtures under tests/golden/ are outputs of the reference's `_explicit_reference_output`
(tests/gpu/test_decode_quant_linear.py:46-60 in SamMausberg/fast-kernels) and of its dequant
expectation (:158-166), produced by tests/golden/make_golden.py. Every oracle function is checked
against them, and the C code is cross-checked against separate numpy restatements.
"""

from __future__ import annotations

import numpy as np
import pytest
import torch
from oracle import w4a16_oracle as oracle
from w4a16_testlib import golden_case_names, load_golden

ALL_CASES = golden_case_names()
STORED_CASES = golden_case_names(stored_only=True)


def _case(name: str):
    data = load_golden(name)
    if data is None:
        pytest.skip("this torch build does not reproduce the fixture's seeded inputs")
    return data


def test_half_conversions_match_numpy_exhaustively() -> None:
    lib = oracle.lib()
    all_bits = np.arange(0, 1 << 16, dtype=np.uint16)
    floats = all_bits.view(np.float16).astype(np.float32)
    for bits in (0x0000, 0x0001, 0x03FF, 0x0400, 0x3C00, 0x7BFF, 0x7C00, 0x8001, 0xFBFF):
        assert lib.oracle_half_to_float(bits, oracle.F16) == floats[bits]
    # fp32 -> fp16 on every fp16 value, its neighbours' midpoints and random floats
    rng = np.random.default_rng(0)
    probes = np.concatenate([
        floats[np.isfinite(floats)],
        (floats[:-1] + floats[1:])[np.isfinite(floats[:-1] + floats[1:])] / 2,
        rng.standard_normal(20000).astype(np.float32) * 100,
        rng.standard_normal(20000).astype(np.float32) * 1e-5,
        np.array([65504.0, 65519.9, 65520.0, 70000.0, 2.0**-25, 2.0**-24, 1.5 * 2.0**-25], dtype=np.float32),
    ]).astype(np.float32)
    with np.errstate(over="ignore"):
        expected = probes.astype(np.float16).view(np.uint16)
    got = np.array([lib.oracle_float_to_half(float(x), oracle.F16) for x in probes], dtype=np.uint16)
    assert np.array_equal(got, expected)


def test_bf16_conversions_match_torch() -> None:
    lib = oracle.lib()
    rng = np.random.default_rng(1)
    probes = np.concatenate([rng.standard_normal(5000), rng.standard_normal(5000) * 1e-3,
                             np.array([1.0, 1.00390625, 1.01171875, 3.3895e38])]).astype(np.float32)
    expected = torch.from_numpy(probes).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    got = np.array([lib.oracle_float_to_half(float(x), oracle.BF16) for x in probes], dtype=np.uint16)
    assert np.array_equal(got, expected)
    back = np.array([lib.oracle_half_to_float(int(b), oracle.BF16) for b in expected], dtype=np.float32)
    assert np.array_equal(back, torch.from_numpy(probes).to(torch.bfloat16).float().numpy())


@pytest.mark.parametrize("name", STORED_CASES)
def test_dequant_is_bit_exact_with_reference_expression(name: str) -> None:
    case = _case(name)
    group = case["meta"]["group_size"]
    got = oracle.dequant_rowmajor(case["q_u8"], case["alpha"], case["beta"], group, oracle.F16)
    assert np.array_equal(got, case["weight"])
    assert np.array_equal(oracle.np_dequant(case["q_u8"], case["alpha"], case["beta"], group, oracle.F16),
                          case["weight"])


@pytest.mark.parametrize("name", STORED_CASES)
def test_pack_then_dequant_round_trips(name: str) -> None:
    case = _case(name)
    meta = case["meta"]
    group = meta["group_size"]
    packets = oracle.pack_packets(case["q_u8"], case["alpha"], case["beta"], group)
    assert packets.shape == ((meta["n"] // 128) * (meta["k"] // group), 64 * group + 512)
    assert np.array_equal(packets, oracle.np_pack(case["q_u8"], case["alpha"], case["beta"], group))
    from_packets = oracle.dequant_packets(packets, meta["n"], meta["k"], group, oracle.F16)
    assert np.array_equal(from_packets, case["weight"])


@pytest.mark.parametrize("name", ALL_CASES)
def test_gemv_oracles_match_reference_output(name: str) -> None:
    case = _case(name)
    group = case["meta"]["group_size"]
    args = (case["activations"], case["q_u8"], case["alpha"], case["beta"], group, oracle.F16)
    expected = oracle.np_to_f32(case["output"], oracle.F16).astype(np.float64)

    y64 = oracle.gemv_f64(*args)
    # The reference output is fp16-rounded fp32 math; fp64 differs from it by that rounding only.
    assert np.allclose(y64, expected, rtol=2e-3, atol=2e-3)
    if case["meta"]["n"] * case["meta"]["k"] <= 1 << 20:
        assert np.allclose(y64, oracle.np_gemv_f64(*args), rtol=1e-12, atol=1e-12)

    # The two fp32 restatements land on the reference's fp16 output up to one rounding step.
    for fn in (oracle.gemv_explicit, oracle.gemv_ref_order):
        got = oracle.np_to_f32(fn(*args), oracle.F16).astype(np.float64)
        # the reference's tests use atol = rtol = 1e-2; the restatements sit far inside that
        assert np.allclose(got, expected, rtol=2e-3, atol=2e-3)
    assert oracle.max_rel_err(expected, y64) < 1e-2


def test_group_sums_follow_the_reference_tree() -> None:
    rng = np.random.default_rng(3)
    for group in (32, 64, 128):
        act = torch.from_numpy(rng.standard_normal((3, group * 5)).astype(np.float32)).to(torch.float16)
        bits = oracle.bits_of(act)
        sums = oracle.group_sums(bits, group, oracle.F16)
        assert sums.shape == (3, 5)
        exact = act.double().reshape(3, 5, group).sum(-1).numpy()
        assert np.allclose(sums, exact, rtol=1e-5, atol=1e-4)
        # pairing order: (a0+a1) first, then slots i and i+stride
        first = act[0, :group].float().numpy()
        slots = np.zeros(128, dtype=np.float32)
        slots[: group // 2] = first[0::2] + first[1::2]
        stride = 64
        while stride:
            slots[:stride] = slots[:stride] + slots[stride: 2 * stride]
            stride //= 2
        assert sums[0, 0] == slots[0]


def test_bf16_dequant_and_gemv_agree_with_torch() -> None:
    gen = torch.Generator().manual_seed(11)
    n, k, group = 256, 512, 64
    act = torch.randn((2, k), generator=gen).to(torch.bfloat16)
    q = torch.randint(0, 256, (n, k // 2), generator=gen, dtype=torch.uint8)
    alpha = (0.005 + 0.015 * torch.rand((n, k // group), generator=gen)).to(torch.bfloat16)
    zero = torch.randint(0, 16, (n, k // group), generator=gen).to(torch.bfloat16)
    beta = -(alpha * zero)
    low = (q & 0x0F).float()
    high = (q >> 4).float()
    qv = torch.stack((low, high), dim=-1).reshape(n, k)
    weight = alpha.float().repeat_interleave(group, 1) * qv + beta.float().repeat_interleave(group, 1)
    got = oracle.dequant_rowmajor(q.numpy(), oracle.bits_of(alpha), oracle.bits_of(beta), group, oracle.BF16)
    assert np.array_equal(got, oracle.bits_of(weight.to(torch.bfloat16)))
    y64 = oracle.gemv_f64(oracle.bits_of(act), q.numpy(), oracle.bits_of(alpha), oracle.bits_of(beta),
                          group, oracle.BF16)
    assert np.allclose(y64, (act.double() @ weight.double().T).numpy(), rtol=1e-10, atol=1e-10)
