"""fk_w4a16_gemv_static: the GEMV entry point that brings its own scratch.

Some hosts of this library cannot allocate device memory when they call it -- a server whose own
pools already own all free HBM, or a decode loop that must never hit an allocation's device-wide
stall -- so this variant keeps its scratch in a fixed array inside the library. The tests call it
through the C ABI twice in a row per shape, alternating shapes on the one shared array (which keeps
what the previous call left), and check each result against the workspace-taking entry point and
against the fp64 oracle; they also check that the calls leave the device's free memory untouched.
Collected last on purpose, so a failure here cannot hide results of the other tests under -x.
"""

from __future__ import annotations

import pytest
import torch
from fast_kernels import capi
from fast_kernels.workloads import LayerShape, make_problem
from oracle import w4a16_oracle as oracle
from w4a16_testlib import Workspace, capi_pack, stream_ptr

pytestmark = pytest.mark.gpu


def _gemv_cuda_cores(ws: Workspace, act, packets, n, k, group, code):
    """The workspace-taking entry point on the kernels the static one uses: the launch plan is the
    same, so the bits must agree. (For batch 3-4 on large layers fk_w4a16_gemv itself would pick
    the tensor-core kernel; the tuning knob "mma_min_batch" = 5 keeps it off.)"""
    lib = capi.load_library()
    batch = act.shape[0]
    out = torch.full((batch, n), float("nan"), dtype=act.dtype, device=act.device)
    workspace = ws.get(capi, batch, n, k, group)
    capi.check(lib.fk_w4a16_gemv(act.data_ptr(), packets.data_ptr(), out.data_ptr(), workspace.data_ptr(),
                                 workspace.numel(), batch, n, k, group, capi.packet_stride_bytes(group), code,
                                 stream_ptr()))
    return out


def _prepare(shape: LayerShape, seed: int):
    problem = make_problem(shape, seed=seed)
    q, alpha, beta, act = (problem[key].cuda() for key in ("q_u8", "alpha", "beta", "activations"))
    packets = capi_pack(capi, q, alpha, beta, shape.group_size)
    return problem, act, packets


@pytest.mark.parametrize(("dtype", "batch"), [("bf16", 1), ("fp16", 2), ("bf16", 3), ("bf16", 4)])
def test_static_scratch_entry_point_matches_the_workspace_one_twice(dtype: str, batch: int) -> None:
    lib = capi.load_library()
    capi.check(lib.fk_w4a16_set_tuning(b"mma_min_batch", 5))
    capi.check(lib.fk_w4a16_set_tuning(b"umma_min_batch", 0))
    try:
        _static_against_workspace(dtype, batch)
    finally:
        capi.check(lib.fk_w4a16_set_tuning(b"mma_min_batch", 0))
        capi.check(lib.fk_w4a16_set_tuning(b"umma_min_batch", -1))


def _static_against_workspace(dtype: str, batch: int) -> None:
    code = oracle.dtype_code(dtype)
    # 100 tiles of 9 packets over 148 CTAs: the packet-stream kernel with most tiles split over two
    # or three CTAs, i.e. the ticket finish on the shared array; then the 8B gate_up layer (224
    # tiles, every CTA boundary inside a tile); then a small layer that takes the cluster kernel
    shapes = [LayerShape("a", 128 * 100, 128 * 9, batch=batch, dtype=dtype, zero_point=None),
              LayerShape("b", 28672, 4096, batch=batch, dtype=dtype, zero_point=None),
              LayerShape("c", 4096, 4096, batch=batch, dtype=dtype, zero_point=None)]
    ws = Workspace()
    prepared = []
    for shape in shapes:
        problem, act, packets = _prepare(shape, seed=31 + batch)
        expected = _gemv_cuda_cores(ws, act, packets, shape.n, shape.k, 128, code)
        rows = slice(0, 640)
        y64 = oracle.gemv_f64(oracle.bits_of(problem["activations"]), problem["q_u8"][rows].numpy(),
                              oracle.bits_of(problem["alpha"][rows]), oracle.bits_of(problem["beta"][rows]),
                              128, code)
        prepared.append((shape, act, packets, expected, rows, y64))
    torch.cuda.synchronize()
    lib = capi.load_library()
    outs = [torch.empty((batch, s.n), dtype=prepared[0][1].dtype, device="cuda") for s in shapes]
    for _ in range(2):  # a, a, b, b, c, c, a, a, ... on the one shared array
        for (shape, act, packets, expected, rows, y64), out in zip(prepared, outs):
            for _ in range(2):
                out.fill_(float("nan"))
                capi.check(lib.fk_w4a16_gemv_static(act.data_ptr(), packets.data_ptr(), out.data_ptr(), batch,
                                                    shape.n, shape.k, 128, 8704, code, stream_ptr()))
                torch.cuda.synchronize()
                # same kernels, same launch plan, fixed summation order: the bits agree, and so does
                # the 1e-2 bound against the fp64 oracle that every GEMV test here uses
                assert torch.equal(out.view(torch.int16), expected.view(torch.int16)), shape.name
                assert oracle.max_rel_err(out[:, rows].float().cpu().numpy(), y64) <= 1e-2
    assert capi.device_status() == 0


def test_static_scratch_entry_point_leaves_free_memory_alone() -> None:
    """No allocation of any kind inside the call: free device memory reads the same before and
    after a burst of calls made with nothing else running."""
    shape = LayerShape("d", 128 * 100, 128 * 9, batch=2, dtype="bf16", zero_point=None)
    _, act, packets = _prepare(shape, seed=3)
    lib = capi.load_library()
    out = torch.empty((2, shape.n), dtype=torch.bfloat16, device="cuda")
    capi.check(lib.fk_w4a16_gemv_static(act.data_ptr(), packets.data_ptr(), out.data_ptr(), 2, shape.n,
                                        shape.k, 128, 8704, 1, stream_ptr()))
    torch.cuda.synchronize()
    before = torch.cuda.mem_get_info()[0]
    for _ in range(8):
        capi.check(lib.fk_w4a16_gemv_static(act.data_ptr(), packets.data_ptr(), out.data_ptr(), 2, shape.n,
                                            shape.k, 128, 8704, 1, stream_ptr()))
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] >= before  # never less: the calls allocated nothing


def test_static_scratch_entry_point_refuses_what_does_not_fit() -> None:
    lib = capi.load_library()
    shape = LayerShape("big_batch", 4096, 4096, batch=16, dtype="bf16")
    act = torch.zeros((16, shape.k), dtype=torch.bfloat16, device="cuda")
    packets = torch.zeros(((shape.n // 128) * (shape.k // 128), 8704), dtype=torch.uint8, device="cuda")
    out = torch.zeros((16, shape.n), dtype=torch.bfloat16, device="cuda")
    code = lib.fk_w4a16_gemv_static(act.data_ptr(), packets.data_ptr(), out.data_ptr(), 16, shape.n, shape.k,
                                    128, 8704, 1, stream_ptr())
    assert code == capi.ERR_INVALID_ARGUMENT
    message = lib.fk_w4a16_last_error().decode()
    assert "static array holds 1048576" in message and "bytes of scratch" in message
