"""Seeded synthetic W4A16 problems.

The shapes are those of Llama-3-8B / 70B-style / 13B decoder layers; no checkpoint or dataset is
involved, only the distributions the benchmark configurations state. Values are drawn on the CPU
with a ``torch.Generator`` (CPU and CUDA generators produce different streams for one seed), then
moved to the device, so every implementation sees identical bits.

The zero-point convention is the reference's (benchmarking/decode_linear_w4a16.py:152-174 in
SamMausberg/fast-kernels): ``beta = -(alpha * zero_point)`` evaluated in the 16-bit type.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch

TORCH_DTYPES = {"fp16": torch.float16, "bf16": torch.bfloat16}


@dataclass(frozen=True)
class LayerShape:
    name: str
    n: int
    k: int
    group_size: int = 128
    batch: int = 1
    dtype: str = "bf16"
    scale_range: tuple[float, float] = (0.005, 0.02)
    zero_point: int | None = 8  # None -> uniform uint4 zero points per group

    def algorithmic_bytes(self) -> int:
        """Bytes one call must move: nibbles + 16-bit scale and offset per group + activations
        + outputs. Split-K scratch is not counted."""
        groups = self.k // self.group_size
        return (
            self.n * self.k // 2
            + 2 * self.n * groups * 2
            + self.batch * self.k * 2
            + self.batch * self.n * 2
        )


# The Llama-3-8B decode layer set at M=1 (the headline workload).
LLAMA3_8B_LAYERS = (
    LayerShape("qkv", 6144, 4096),
    LayerShape("o_proj", 4096, 4096),
    LayerShape("gate_up", 28672, 4096),
    LayerShape("down_proj", 4096, 14336),
)
# The single CPU-runnable case of the reference: 4096 x 4096, fp16, seed 0.
REFERENCE_CASE = LayerShape("ref_4096", 4096, 4096, dtype="fp16")
# Batched decode sweep on a 70B-style MLP up projection, per-group uint4 zero points.
BATCH_SWEEP = tuple(
    LayerShape(f"mlp_up_m{m}", 28672, 8192, batch=m, zero_point=None) for m in (1, 2, 4, 8, 16)
)
# Layers large enough to shard over the GPUs of a node (N-split, K-split).
SHARDED_COLUMN = LayerShape("gate_up_70b", 57344, 8192)
SHARDED_ROW = LayerShape("down_70b", 8192, 28672)
# Edge and large shapes: a 13B MLP at three group sizes (fp16, asymmetric zeros), an LM head.
EDGE_SHAPES = tuple(
    LayerShape(f"mlp13b_g{g}", 13824, 5120, group_size=g, dtype="fp16", scale_range=(0.001, 0.05),
               zero_point=None)
    for g in (32, 64, 128)
) + (LayerShape("lm_head", 128256, 4096),)


def seed_for(shape: LayerShape) -> int:
    """The reference's per-case seed (benchmarking/decode_linear_w4a16.py:148-149)."""
    return (shape.batch * 1_000_003 + shape.n * 1009 + shape.k * 101 + shape.group_size) % (2**31 - 1)


def make_problem(shape: LayerShape, *, seed: int | None = None, device: Any = "cpu") -> dict[str, Any]:
    """Returns activations [batch,k], q_u8 [n,k/2], alpha/beta [n,k/G] on `device`."""
    gen = torch.Generator().manual_seed(seed_for(shape) if seed is None else seed)
    dtype = TORCH_DTYPES[shape.dtype]
    groups = shape.k // shape.group_size
    activations = torch.randn((shape.batch, shape.k), generator=gen, dtype=torch.float32).to(dtype)
    q_u8 = torch.randint(0, 256, (shape.n, shape.k // 2), generator=gen, dtype=torch.uint8)
    lo, hi = shape.scale_range
    alpha = (lo + (hi - lo) * torch.rand((shape.n, groups), generator=gen, dtype=torch.float32)).to(dtype)
    if shape.zero_point is None:
        zero = torch.randint(0, 16, (shape.n, groups), generator=gen, dtype=torch.int16).to(dtype)
    else:
        zero = torch.full((shape.n, groups), float(shape.zero_point), dtype=dtype)
    beta = -(alpha * zero)
    out = {
        "activations": activations.contiguous(),
        "q_u8": q_u8.contiguous(),
        "alpha": alpha.contiguous(),
        "beta": beta.contiguous(),
    }
    return {key: value.to(device) for key, value in out.items()}
