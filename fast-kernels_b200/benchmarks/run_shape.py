#!/usr/bin/env python3
"""Runs one W4A16 problem a few times through the C ABI -- the small, fixed workload to put under
a profiler (``ncu -k regex:gemv_stream ... python run_shape.py 28672 4096 128 1 bf16 3``).

    run_shape.py N K GROUP BATCH fp16|bf16 LAUNCHES [WARPS STAGES CTAS]

Launches alternate between two copies of the weights; the optional last three numbers override
the launch plan (see fk_w4a16_set_launch_config).
"""

from __future__ import annotations

import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT / "src"))

import torch  # noqa: E402
from fast_kernels import capi  # noqa: E402
from fast_kernels.workloads import LayerShape, make_problem  # noqa: E402


def main() -> int:
    if len(sys.argv) < 7:
        print(__doc__)
        return 2
    n, k, group, batch = (int(x) for x in sys.argv[1:5])
    dtype, launches = sys.argv[5], int(sys.argv[6])
    lib = capi.load_library()
    if len(sys.argv) >= 10:
        capi.check(lib.fk_w4a16_set_launch_config(*(int(x) for x in sys.argv[7:10])))
    shape = LayerShape("profiled", n, k, group_size=group, batch=batch, dtype=dtype)
    problem = make_problem(shape)
    q, alpha, beta, act = (problem[key].cuda() for key in ("q_u8", "alpha", "beta", "activations"))
    stride = capi.packet_stride_bytes(group)
    packets = torch.empty(((n // 128) * (k // group), stride), dtype=torch.uint8, device="cuda")
    capi.check(lib.fk_w4a16_pack_packets(q.data_ptr(), alpha.data_ptr(), beta.data_ptr(), packets.data_ptr(),
                                         n, k, group, stride, 0))
    copies = [packets, packets.clone()]
    out = torch.empty((batch, n), dtype=act.dtype, device="cuda")
    need = int(lib.fk_w4a16_workspace_bytes(batch, n, k, group))
    workspace = torch.zeros(need, dtype=torch.uint8, device="cuda")
    code = capi.DTYPE_BF16 if dtype == "bf16" else capi.DTYPE_F16
    torch.cuda.synchronize()
    for i in range(launches):
        capi.check(lib.fk_w4a16_gemv(act.data_ptr(), copies[i % 2].data_ptr(), out.data_ptr(), workspace.data_ptr(),
                                     workspace.numel(), batch, n, k, group, stride, code, 0))
    torch.cuda.synchronize()
    print("device status", capi.device_status(), "max |y|", float(out.float().abs().max()))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
