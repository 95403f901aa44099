"""fk_w4a16_gemv_static: the GEMV entry point that brings its own scratch.

Some hosts of this library cannot allocate device memory when they call it -- a server whose own
pools already own all free HBM, or a decode loop that must never hit an allocation's device-wide
stall -- so this variant keeps its scratch in a fixed array inside the library. The test calls it
through the C ABI twice in a row (the array is shared and keeps what the previous call left) and
checks each result against the workspace-taking entry point and against the fp64 oracle.
Collected last on purpose, so a failure here cannot hide results of the other tests under -x.
"""

from __future__ import annotations

import numpy as np
import pytest
import torch
from fast_kernels import capi
from fast_kernels.workloads import LayerShape, make_problem
from oracle import w4a16_oracle as oracle
from w4a16_testlib import Workspace, capi_gemv, capi_pack, stream_ptr

pytestmark = pytest.mark.gpu


def _gemv_static(act, packets, n, k, group, code):
    lib = capi.load_library()
    out = torch.full((act.shape[0], n), float("nan"), dtype=act.dtype, device=act.device)
    capi.check(lib.fk_w4a16_gemv_static(act.data_ptr(), packets.data_ptr(), out.data_ptr(), act.shape[0],
                                        n, k, group, capi.packet_stride_bytes(group), code, stream_ptr()))
    return out


@pytest.mark.parametrize(("dtype", "batch"), [("bf16", 1), ("fp16", 3)])
def test_static_scratch_entry_point_matches_the_workspace_one_twice(dtype: str, batch: int) -> None:
    code = oracle.dtype_code(dtype)
    # first a shape whose tiles are shared between CTAs, then a different one on the same array
    shapes = [LayerShape("a", 128 * 37, 128 * 9, batch=batch, dtype=dtype, zero_point=None),
              LayerShape("b", 4096, 4096, batch=batch, dtype=dtype, zero_point=None)]
    ws = Workspace()
    for shape in shapes:
        problem = make_problem(shape, seed=31 + batch)
        q, alpha, beta, act = (problem[key].cuda() for key in ("q_u8", "alpha", "beta", "activations"))
        packets = capi_pack(capi, q, alpha, beta, 128)
        expected = capi_gemv(capi, ws, act, packets, shape.n, shape.k, 128, code)
        y64 = oracle.gemv_f64(oracle.bits_of(problem["activations"]), problem["q_u8"].numpy(),
                              oracle.bits_of(problem["alpha"]), oracle.bits_of(problem["beta"]), 128, code)
        for _ in range(2):
            got = _gemv_static(act, packets, shape.n, shape.k, 128, code)
            torch.cuda.synchronize()
            # same kernel, same launch plan, fixed summation order: the bits agree, and so does
            # the 1e-2 bound against the fp64 oracle that every GEMV test here uses
            assert torch.equal(got.view(torch.int16), expected.view(torch.int16))
            assert oracle.max_rel_err(got.float().cpu().numpy(), y64) <= 1e-2
    assert capi.device_status() == 0


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
