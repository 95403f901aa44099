"""Helpers shared by the W4A16 tests: golden-fixture loading and thin C-ABI call wrappers."""

from __future__ import annotations

import hashlib
import json
from pathlib import Path
from typing import Any

import numpy as np
import torch

GOLDEN = Path(__file__).resolve().parent / "golden"


def manifest() -> dict[str, Any]:
    return json.loads((GOLDEN / "manifest.json").read_text())


def golden_case_names(stored_only: bool = False) -> list[str]:
    return [c["name"] for c in manifest()["cases"] if c["inputs_stored"] or not stored_only]


def _bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().view(np.uint16).copy()


def _regenerate(meta: dict[str, Any]) -> dict[str, np.ndarray]:
    """Re-draw a fixture's inputs from its recorded recipe (CPU generator)."""
    recipe = meta["recipe"]
    batch, n, k, group = meta["batch"], meta["n"], meta["k"], meta["group_size"]
    groups = k // group
    torch.manual_seed(recipe["seed"])
    if recipe["kind"] == "test":
        activations = torch.randn((batch, k), dtype=torch.float16)
        q_u8 = torch.randint(0, 256, (n, k // 2), dtype=torch.uint8)
        alpha = (recipe["lo"] + recipe["span"] * torch.rand((n, groups), dtype=torch.float32)).to(torch.float16)
    else:
        activations = (0.25 * torch.randn((batch, k), dtype=torch.float32)).to(torch.float16)
        q_u8 = torch.randint(0, 256, (n, k // 2), dtype=torch.uint8)
        alpha = (0.02 + 0.18 * torch.rand((n, groups), dtype=torch.float32)).to(torch.float16)
    zero_points = torch.randint(0, 16, (n, groups), dtype=torch.int16)
    beta = -(alpha * zero_points.to(dtype=torch.float16))
    return {
        "activations": _bits(activations),
        "q_u8": q_u8.numpy().copy(),
        "alpha": _bits(alpha),
        "beta": _bits(beta),
    }


def load_golden(name: str) -> dict[str, Any] | None:
    """Inputs and reference outputs of one fixture as numpy arrays (16-bit floats as uint16).

    Returns None when the inputs were stored as a seed only and this torch build no longer
    reproduces them (the recorded SHA-256 does not match).
    """
    meta = next(c for c in manifest()["cases"] if c["name"] == name)
    data = dict(np.load(GOLDEN / f"{name}.npz"))
    if not meta["inputs_stored"]:
        inputs = _regenerate(meta)
        digest = hashlib.sha256()
        for key in ("activations", "q_u8", "alpha", "beta"):
            digest.update(np.ascontiguousarray(inputs[key]).tobytes())
        if digest.hexdigest() != meta["inputs_sha256"]:
            return None
        data.update(inputs)
    data["meta"] = meta
    return data


# ---- C-ABI call helpers (torch tensors supply device memory; nothing else) --------------------
def torch_dtype(code: int) -> torch.dtype:
    return torch.bfloat16 if code == 1 else torch.float16


def dev_bits(bits: np.ndarray, code: int, device: str = "cuda") -> torch.Tensor:
    return torch.from_numpy(bits.view(np.int16).copy()).view(torch_dtype(code)).to(device)


def host_bits(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def stream_ptr() -> int:
    return int(torch.cuda.current_stream().cuda_stream)


class Workspace:
    """A zero-initialised GEMV workspace that grows on demand (one per test process)."""

    def __init__(self) -> None:
        self.buffer: torch.Tensor | None = None

    def get(self, capi: Any, batch: int, n: int, k: int, group: int) -> torch.Tensor:
        need = int(capi.load_library().fk_w4a16_workspace_bytes(batch, n, k, group))
        assert need > 0
        if self.buffer is None or self.buffer.numel() < need:
            self.buffer = torch.zeros(need, dtype=torch.uint8, device="cuda")
        return self.buffer


def capi_pack(capi: Any, q: torch.Tensor, alpha: torch.Tensor, beta: torch.Tensor, group: int) -> torch.Tensor:
    lib = capi.load_library()
    n, k = q.shape[0], q.shape[1] * 2
    stride = capi.packet_stride_bytes(group)
    packets = torch.empty(((n // 128) * (k // group), stride), dtype=torch.uint8, device=q.device)
    capi.check(lib.fk_w4a16_pack_packets(q.data_ptr(), alpha.data_ptr(), beta.data_ptr(),
                                         packets.data_ptr(), n, k, group, stride, stream_ptr()))
    return packets


def capi_gemv(capi: Any, ws: Workspace, act: torch.Tensor, packets: torch.Tensor, n: int, k: int,
              group: int, code: int) -> torch.Tensor:
    lib = capi.load_library()
    batch = act.shape[0]
    out = torch.full((batch, n), float("nan"), dtype=act.dtype, device=act.device)
    workspace = ws.get(capi, batch, n, k, group)
    capi.check(lib.fk_w4a16_gemv(act.data_ptr(), packets.data_ptr(), out.data_ptr(),
                                 workspace.data_ptr(), workspace.numel(), batch, n, k, group,
                                 capi.packet_stride_bytes(group), code, stream_ptr()))
    return out
