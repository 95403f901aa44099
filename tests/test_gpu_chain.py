"""fk_w4a16_gemv_chain: several dependent GEMVs in one persistent launch.

The chain must give the results of the same steps issued one after another as fk_w4a16_gemv_ex
calls: bit for bit against the packet-stream kernel (same work split and summation order; the
cluster kernel is switched off for the comparison), and within the usual 1e-2 of the fp64 oracle.
"""

from __future__ import annotations

import ctypes

import numpy as np
import pytest
import torch
from fast_kernels import capi
from fast_kernels.workloads import LayerShape, make_problem
from oracle import w4a16_oracle as oracle
from w4a16_testlib import Workspace, capi_pack, stream_ptr

pytestmark = pytest.mark.gpu

WS = Workspace()


@pytest.fixture(autouse=True)
def _stream_kernel_only_and_clean_status():
    lib = capi.load_library()
    capi.check(lib.fk_w4a16_set_tuning(b"cluster", 0))
    capi.check(lib.fk_w4a16_set_tuning(b"mma_min_batch", 5))
    yield
    capi.check(lib.fk_w4a16_set_tuning(b"cluster", 1))
    capi.check(lib.fk_w4a16_set_tuning(b"mma_min_batch", 0))
    torch.cuda.synchronize()
    assert capi.device_status() == 0, "a bounded device-side wait timed out"


def _layer(n: int, k: int, group: int, dtype: str, seed: int):
    shape = LayerShape("t", n, k, group_size=group, dtype=dtype, zero_point=None)
    problem = make_problem(shape, seed=seed)
    q, alpha, beta = (problem[key].cuda() for key in ("q_u8", "alpha", "beta"))
    return problem, capi_pack(capi, q, alpha, beta, group)


def _chain_workspace(batch: int, group: int) -> torch.Tensor:
    need = int(capi.load_library().fk_w4a16_chain_workspace_bytes(batch, group))
    assert need > 0
    return torch.zeros(need, dtype=torch.uint8, device="cuda")


def _run_chain(steps: list[dict], batch: int, group: int, code: int, workspace: torch.Tensor) -> None:
    array = (capi.ChainStep * len(steps))()
    for slot, step in zip(array, steps):
        slot.activations, slot.packets, slot.output = (step[key].data_ptr() for key in ("act", "packets", "out"))
        slot.n, slot.k = step["n"], step["k"]
        slot.residual = step["residual"].data_ptr() if step.get("residual") is not None else None
        slot.epilogue = step.get("epilogue", 0)
        slot.norm_weight = step["norm_weight"].data_ptr() if step.get("norm_weight") is not None else None
        slot.norm_eps = step.get("norm_eps", 0.0)
    capi.check(capi.load_library().fk_w4a16_gemv_chain(array, len(steps), workspace.data_ptr(), workspace.numel(),
                                                       batch, group, 64 * group + 512, code, stream_ptr()))


def _run_separately(steps: list[dict], batch: int, group: int, code: int) -> None:
    lib = capi.load_library()
    for step in steps:
        args = capi.GemvArgs()
        ws = WS.get(capi, batch, step["n"], step["k"], group)
        args.activations, args.packets, args.output = (step[key].data_ptr() for key in ("act", "packets", "out"))
        args.workspace, args.workspace_bytes = ws.data_ptr(), ws.numel()
        args.batch, args.n, args.k, args.group_size = batch, step["n"], step["k"], group
        args.packet_stride_bytes, args.dtype = 64 * group + 512, code
        args.residual = step["residual"].data_ptr() if step.get("residual") is not None else None
        args.epilogue = step.get("epilogue", 0)
        args.norm_weight = step["norm_weight"].data_ptr() if step.get("norm_weight") is not None else None
        args.norm_eps = step.get("norm_eps", 0.0)
        args.stream = stream_ptr()
        capi.check(lib.fk_w4a16_gemv_ex(args))


@pytest.mark.parametrize(("batch", "group", "dtype"), [(1, 128, "bf16"), (2, 64, "fp16"), (4, 128, "bf16"),
                                                        (3, 32, "bf16")])
def test_chain_of_a_decoder_block_matches_separate_calls(batch: int, group: int, dtype: str) -> None:
    """o_proj (+ residual) -> RMSNorm + [gate; up] with SiLU-and-multiply -> down_proj (+ residual,
    in place) -> RMSNorm + qkv of the next layer: every step reads what the step before wrote."""
    code = oracle.dtype_code(dtype)
    tdtype = torch.bfloat16 if code else torch.float16
    hidden, inter, qkv = 1024, 2816, 1536
    layers = {
        "o": _layer(hidden, hidden, group, dtype, 1),
        "gate_up": _layer(2 * inter, hidden, group, dtype, 2),
        "down": _layer(hidden, inter, group, dtype, 3),
        "qkv": _layer(qkv, hidden, group, dtype, 4),
    }
    gen = torch.Generator().manual_seed(11 + batch)
    attn = torch.randn((batch, hidden), generator=gen).to(tdtype).cuda()
    h0 = torch.randn((batch, hidden), generator=gen).to(tdtype).cuda()
    norm1 = (1.0 + 0.1 * torch.randn((hidden,), generator=gen)).to(tdtype).cuda()
    norm2 = (1.0 + 0.1 * torch.randn((hidden,), generator=gen)).to(tdtype).cuda()

    def build():
        h = h0.clone()
        mlp = torch.full((batch, inter), float("nan"), dtype=tdtype, device="cuda")
        out = torch.full((batch, qkv), float("nan"), dtype=tdtype, device="cuda")
        steps = [
            {"act": attn, "packets": layers["o"][1], "out": h, "n": hidden, "k": hidden, "residual": h},
            {"act": h, "packets": layers["gate_up"][1], "out": mlp, "n": 2 * inter, "k": hidden,
             "epilogue": capi.EPILOGUE_SILU_MUL, "norm_weight": norm1, "norm_eps": 1e-5},
            {"act": mlp, "packets": layers["down"][1], "out": h, "n": hidden, "k": inter, "residual": h},
            {"act": h, "packets": layers["qkv"][1], "out": out, "n": qkv, "k": hidden,
             "norm_weight": norm2, "norm_eps": 1e-5},
        ]
        return steps, h, mlp, out

    want_steps, want_h, want_mlp, want_out = build()
    _run_separately(want_steps, batch, group, code)
    torch.cuda.synchronize()
    workspace = _chain_workspace(batch, group)
    for _ in range(2):  # twice on one workspace: the barrier counter resets itself
        got_steps, got_h, got_mlp, got_out = build()
        _run_chain(got_steps, batch, group, code, workspace)
        torch.cuda.synchronize()
        assert torch.isfinite(got_out.float()).all() and torch.isfinite(got_mlp.float()).all()
        assert torch.equal(got_mlp.view(torch.int16), want_mlp.view(torch.int16))
        assert torch.equal(got_h.view(torch.int16), want_h.view(torch.int16))
        assert torch.equal(got_out.view(torch.int16), want_out.view(torch.int16))
    # the last step against the fp64 oracle, fed with what the chain itself produced for it
    x = got_h.float().cpu().numpy().astype(np.float64)
    inv = 1.0 / np.sqrt((x ** 2).mean(axis=1, keepdims=True) + 1e-5)
    x_norm = torch.from_numpy((got_h.float().cpu().numpy() * inv.astype(np.float32))).to(tdtype)
    normed = (norm2.cpu().float() * x_norm.float()).to(tdtype)
    problem = layers["qkv"][0]
    y64 = oracle.gemv_f64(oracle.bits_of(normed), problem["q_u8"].numpy(), oracle.bits_of(problem["alpha"]),
                          oracle.bits_of(problem["beta"]), group, code)
    assert oracle.max_rel_err(got_out.float().cpu().numpy(), y64) <= 1e-2


def test_chain_of_the_8b_layer_set_matches_separate_calls() -> None:
    """The four layer shapes of the headline workload as one chain (independent inputs here: the
    barrier between the steps is there all the same)."""
    shapes = [("qkv", 6144, 4096), ("o_proj", 4096, 4096), ("gate_up", 28672, 4096), ("down_proj", 4096, 14336)]
    steps_want, steps_got, problems = [], [], []
    for index, (_, n, k) in enumerate(shapes):
        problem, packets = _layer(n, k, 128, "bf16", 20 + index)
        act = problem["activations"].cuda()
        problems.append(problem)
        for steps in (steps_want, steps_got):
            steps.append({"act": act, "packets": packets, "n": n, "k": k,
                          "out": torch.full((1, n), float("nan"), dtype=torch.bfloat16, device="cuda")})
    _run_separately(steps_want, 1, 128, 1)
    workspace = _chain_workspace(1, 128)
    _run_chain(steps_got, 1, 128, 1, workspace)
    torch.cuda.synchronize()
    for want, got, problem, (name, n, _) in zip(steps_want, steps_got, problems, shapes):
        assert torch.equal(got["out"].view(torch.int16), want["out"].view(torch.int16)), name
        rows = slice(0, 512)
        y64 = oracle.gemv_f64(oracle.bits_of(problem["activations"]), problem["q_u8"][rows].numpy(),
                              oracle.bits_of(problem["alpha"][rows]), oracle.bits_of(problem["beta"][rows]), 128, 1)
        assert oracle.max_rel_err(got["out"][:, rows].float().cpu().numpy(), y64) <= 1e-2, name


def test_chain_refusals() -> None:
    lib = capi.load_library()
    _, packets = _layer(256, 256, 128, "bf16", 5)
    act = torch.zeros((1, 256), dtype=torch.bfloat16, device="cuda")
    out = torch.zeros((1, 256), dtype=torch.bfloat16, device="cuda")
    workspace = _chain_workspace(1, 128)
    step = {"act": act, "packets": packets, "out": out, "n": 256, "k": 256}
    with pytest.raises(ValueError, match="between 1 and 8"):
        _run_chain([step] * 9, 1, 128, 1, workspace)
    with pytest.raises(ValueError, match="at most 4"):
        _run_chain([step], 5, 128, 1, workspace)
    with pytest.raises(ValueError, match="workspace_bytes"):
        _run_chain([step], 1, 128, 1, workspace[: 1 << 20])
    assert int(lib.fk_w4a16_chain_workspace_bytes(5, 128)) == 0
    _run_chain([step], 1, 128, 1, workspace)  # and a chain of one step is just a GEMV
    torch.cuda.synchronize()
