"""Checkpoint-layout loaders (fast_kernels.loaders) against independent numpy packers of the two
layouts: the packer inputs they produce must be bit-identical to the ones built directly from the
integer weights, zero points and scales, and must dequantise (oracle) to scale * (q - zero)."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from fast_kernels import loaders
from oracle import w4a16_oracle as oracle


def _synth(n: int, k: int, group: int, dtype: torch.dtype, seed: int, max_zero: int = 15):
    gen = torch.Generator().manual_seed(seed)
    q = torch.randint(0, 16, (n, k), generator=gen, dtype=torch.int32)
    zeros = torch.randint(0, max_zero + 1, (k // group, n), generator=gen, dtype=torch.int32)
    scales = (0.005 + 0.015 * torch.rand((k // group, n), generator=gen)).to(dtype)
    return q, zeros, scales


def _words(nibbles: np.ndarray) -> np.ndarray:
    """[..., 8] nibbles -> int32 words, nibble i in bits 4i..4i+3."""
    acc = np.zeros(nibbles.shape[:-1], dtype=np.uint32)
    for i in range(8):
        acc |= nibbles[..., i].astype(np.uint32) << np.uint32(4 * i)
    return acc.view(np.int32)


def _gptq_tensors(q, zeros, scales, zero_offset=1):
    n, k = q.shape
    qn = q.numpy().T.reshape(k // 8, 8, n).transpose(0, 2, 1)             # [K/8, N, 8]: k = 8 r + i
    zn = ((zeros.numpy() - zero_offset) & 0xF).reshape(zeros.shape[0], n // 8, 8)
    return torch.from_numpy(_words(qn)), torch.from_numpy(_words(zn)), scales


def _awq_tensors(q, zeros, scales):
    n, k = q.shape
    order = np.array(loaders.AWQ_ORDER)
    qn = q.numpy().T.reshape(k, n // 8, 8)[..., order]                    # nibble i <- column order[i]
    zn = zeros.numpy().reshape(zeros.shape[0], n // 8, 8)[..., order]
    return torch.from_numpy(_words(qn)), torch.from_numpy(_words(zn)), scales


def _expected(q, zeros, scales, dtype):
    q8 = q.to(torch.uint8)
    q_u8 = q8[:, 0::2] | (q8[:, 1::2] << 4)
    alpha = scales.to(dtype).t().contiguous()
    beta = -(alpha * zeros.t().to(dtype))
    return q_u8, alpha, beta


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("group", [32, 64, 128])
@pytest.mark.parametrize("layout", ["gptq", "awq"])
def test_loader_is_bit_exact(layout: str, group: int, dtype: torch.dtype) -> None:
    n, k = 256, 3 * group
    q, zeros, scales = _synth(n, k, group, dtype, seed=group + (1 if layout == "awq" else 0),
                              max_zero=15 if layout == "awq" else 16)
    if layout == "gptq":
        zeros = zeros.clamp(min=1)  # stored as zero - 1 in a nibble
        tensors = dict(zip(("qweight", "qzeros", "scales"), _gptq_tensors(q, zeros, scales)))
    else:
        tensors = dict(zip(("qweight", "qzeros", "scales"), _awq_tensors(q, zeros, scales)))
    q_u8, alpha, beta = loaders.load_linear(tensors, layout=layout, group_size=group)
    want_q, want_alpha, want_beta = _expected(q, zeros, scales, dtype)
    assert torch.equal(q_u8, want_q)
    assert torch.equal(alpha.view(torch.int16), want_alpha.view(torch.int16))
    assert torch.equal(beta.view(torch.int16), want_beta.view(torch.int16))
    # and the packer's inputs mean what the checkpoint means: W = scale * (q - zero), to 16-bit rounding
    code = oracle.dtype_code("fp16" if dtype == torch.float16 else "bf16")
    w_bits = oracle.dequant_rowmajor(q_u8.numpy(), oracle.bits_of(alpha), oracle.bits_of(beta), group, code)
    w = torch.from_numpy(w_bits.view(np.int16)).view(dtype).double()
    ideal = scales.double().t().repeat_interleave(group, dim=1) * (q.double() - zeros.t().double().repeat_interleave(group, dim=1))
    tol = 2.0 ** (-9 if dtype == torch.float16 else -6)
    assert float((w - ideal).abs().max()) <= tol * float(ideal.abs().max())


def test_loader_refusals() -> None:
    q, zeros, scales = _synth(128, 128, 128, torch.float16, seed=3)
    qweight, qzeros, _ = _gptq_tensors(q, zeros.clamp(min=1), scales)
    with pytest.raises(ValueError, match="g_idx"):
        loaders.from_gptq(qweight, qzeros, scales, group_size=128, g_idx=torch.arange(128).flip(0) // 128 + 1)
    loaders.from_gptq(qweight, qzeros, scales, group_size=128, g_idx=torch.arange(128) // 128)
    with pytest.raises(ValueError, match="scales must have shape"):
        loaders.from_gptq(qweight, qzeros, scales[:, :64], group_size=128)
    with pytest.raises(ValueError, match="group_size"):
        loaders.from_awq(qweight, qzeros, scales, group_size=16)
    with pytest.raises(KeyError, match="qzeros"):
        loaders.load_linear({"qweight": qweight, "scales": scales}, layout="gptq", group_size=128)
    with pytest.raises(ValueError, match="layout"):
        loaders.load_linear({"qweight": qweight, "qzeros": qzeros, "scales": scales}, layout="x", group_size=128)
