"""Sharded layers on real GPUs (needs at least two; skipped otherwise): both splits, both
exchanges, against the fp64 oracle, one process per GPU over NCCL."""

from __future__ import annotations

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port() -> int:
    with socket.socket() as sock:
        sock.bind(("127.0.0.1", 0))
        return int(sock.getsockname()[1])


def _rank_main(rank: int, world: int, port: int) -> None:
    from fast_kernels import capi
    from fast_kernels.dist import ShardedW4A16Linear
    from fast_kernels.workloads import LayerShape, make_problem
    from oracle import w4a16_oracle as oracle
    from w4a16_testlib import capi_pack

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        for dtype_name, group, batch, n, k in (("bf16", 128, 1, 128 * 16 * world, 128 * 24 * world),
                                                ("fp16", 64, 3, 128 * 4 * world, 64 * 10 * world)):
            code = oracle.dtype_code(dtype_name)
            dtype = torch.bfloat16 if code else torch.float16
            shape = LayerShape("t", n, k, group_size=group, batch=batch, dtype=dtype_name, zero_point=None)
            problem = make_problem(shape, seed=21)
            q, alpha, beta, act = (problem[key].cuda() for key in ("q_u8", "alpha", "beta", "activations"))
            packets = capi_pack(capi, q, alpha, beta, group)
            y64 = oracle.gemv_f64(oracle.bits_of(problem["activations"]), problem["q_u8"].numpy(),
                                  oracle.bits_of(problem["alpha"]), oracle.bits_of(problem["beta"]), group, code)
            for mode in ("column", "row"):
                results = {}
                for exchange in ("nccl", "peer"):
                    layer = ShardedW4A16Linear(packets, n=n, k=k, group_size=group, mode=mode, dtype=dtype,
                                               exchange=exchange)
                    for _ in range(3):  # repeated calls: tickets, counters and double buffering
                        out = layer(act)
                    torch.cuda.synchronize()
                    assert out.shape == (batch, n) and out.dtype == dtype
                    err = oracle.max_rel_err(out.float().cpu().numpy(), y64)
                    assert err <= 1e-2, (mode, exchange, dtype_name, err)
                    results[exchange] = out.clone()
                    bits = out.view(torch.int16).to(torch.int32).contiguous()
                    gathered = [torch.empty_like(bits) for _ in range(world)]
                    dist.all_gather(gathered, bits)
                    assert all(torch.equal(g, bits) for g in gathered), "ranks disagree"
                # the two exchanges may run different local kernels (cluster vs stream finish), so
                # their fp32 sums can differ in the last bit before the 16-bit rounding
                pair_err = oracle.max_rel_err(results["peer"].float().cpu().numpy(),
                                              results["nccl"].double().cpu().numpy())
                assert pair_err <= 1e-2, (mode, dtype_name, pair_err)
        assert capi.device_status() == 0
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least two GPUs")
def test_sharded_layers_on_all_visible_gpus() -> None:
    world = min(torch.cuda.device_count(), 8)
    world = 1 << (world.bit_length() - 1)
    mp.spawn(_rank_main, args=(world, _free_port()), nprocs=world, join=True)
