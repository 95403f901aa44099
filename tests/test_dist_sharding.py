"""Sharded layers: the shard arithmetic and the N > 1 host path, on CPU.

The two-rank cases run as real ``torch.distributed`` processes over gloo (127.0.0.1); the local
GEMV is supplied by the CPU oracle so that no GPU is needed -- what is under test is the slicing of
packets and activations, the gather / reduce step and the error handling, not the kernel.
"""

from __future__ import annotations

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
from fast_kernels.dist import (
    ShardedW4A16Linear,
    activation_shard,
    check_shardable,
    column_shard_packets,
    row_shard_packets,
)
from fast_kernels.workloads import LayerShape, make_problem
from oracle import w4a16_oracle as oracle


def _packed_problem(shape: LayerShape, seed: int):
    problem = make_problem(shape, seed=seed)
    packets = oracle.pack_packets(problem["q_u8"].numpy(), oracle.bits_of(problem["alpha"]),
                                  oracle.bits_of(problem["beta"]), shape.group_size)
    return problem, torch.from_numpy(packets)


def _oracle_local_forward(group: int, code: int, dtype: torch.dtype):
    """A CPU stand-in for the CUDA GEMV, built on the oracle: fp64 matvec of the shard."""

    def forward(act, packets, n_local, k_local, want_f32):
        weight_bits = oracle.dequant_packets(packets.numpy(), n_local, k_local, group, code)
        # use exact alpha*q+beta rather than the rounded weights: recompute from the packet fields
        tiles, groups = n_local // 128, k_local // group
        view = packets.numpy().reshape(tiles, groups, -1)
        words = view[:, :, : 64 * group].reshape(tiles, groups, group // 8, 128, 4)
        q = np.empty((tiles, groups, group // 8, 128, 8), dtype=np.float64)
        for byte in range(4):
            q[..., 2 * byte] = words[..., byte] & 0x0F
            q[..., 2 * byte + 1] = words[..., byte] >> 4
        q = q.transpose(0, 3, 1, 2, 4).reshape(n_local, k_local)
        scales = np.ascontiguousarray(view[:, :, 64 * group:]).view(np.uint16).reshape(tiles, groups, 2, 128)
        alpha = oracle.np_to_f32(scales[:, :, 0], code).astype(np.float64).transpose(0, 2, 1).reshape(n_local, groups)
        beta = oracle.np_to_f32(scales[:, :, 1], code).astype(np.float64).transpose(0, 2, 1).reshape(n_local, groups)
        weight = np.repeat(alpha, group, axis=1) * q + np.repeat(beta, group, axis=1)
        assert weight_bits.shape == weight.shape
        y = act.double().numpy() @ weight.T
        out = torch.from_numpy(y)
        return out.float() if want_f32 else out.to(dtype)

    return forward


def test_shard_arithmetic_against_the_oracle() -> None:
    shape = LayerShape("t", 512, 1024, group_size=64, dtype="fp16", zero_point=None)
    problem, packets = _packed_problem(shape, 3)
    full = oracle.dequant_packets(packets.numpy(), shape.n, shape.k, 64, oracle.F16)
    world = 4
    column_parts = [column_shard_packets(packets, n=512, k=1024, group_size=64, rank=r, world=world)
                    for r in range(world)]
    assert torch.equal(torch.cat(column_parts), packets)
    for r, part in enumerate(column_parts):
        local = oracle.dequant_packets(part.numpy(), 128, 1024, 64, oracle.F16)
        assert np.array_equal(local, full[r * 128:(r + 1) * 128])
    for r in range(world):
        part = row_shard_packets(packets, n=512, k=1024, group_size=64, rank=r, world=world)
        assert part.shape == (4 * 4, 4608) and part.is_contiguous()
        local = oracle.dequant_packets(part.numpy(), 512, 256, 64, oracle.F16)
        assert np.array_equal(local, full[:, r * 256:(r + 1) * 256])
    act = problem["activations"]
    assert activation_shard(act, rank=1, world=4, mode="column") is act
    assert torch.equal(activation_shard(act, rank=1, world=4, mode="row"), act[:, 256:512])


def test_unshardable_layers_are_refused_on_the_host() -> None:
    with pytest.raises(ValueError, match="tiles to divide"):
        check_shardable(384, 1024, 128, 2, "column")       # 3 tiles over 2 ranks
    with pytest.raises(ValueError, match="groups to divide"):
        check_shardable(512, 128 * 3, 128, 2, "row")        # 3 groups over 2 ranks
    with pytest.raises(ValueError, match="mode must be"):
        check_shardable(512, 1024, 128, 2, "diagonal")
    with pytest.raises(ValueError, match="multiple of 128"):
        check_shardable(500, 1024, 128, 2, "column")
    with pytest.raises(ValueError, match="packets must have shape"):
        column_shard_packets(torch.zeros((3, 8704), dtype=torch.uint8), n=256, k=256, group_size=128,
                             rank=0, world=2)
    with pytest.raises(ValueError, match="rank out of range"):
        row_shard_packets(torch.zeros((4, 8704), dtype=torch.uint8), n=256, k=256, group_size=128,
                          rank=2, world=2)
    with pytest.raises(RuntimeError, match="must be initialised"):
        ShardedW4A16Linear(torch.zeros((4, 8704), dtype=torch.uint8), n=256, k=256, group_size=128,
                           mode="column", dtype=torch.float16)


def _free_port() -> int:
    with socket.socket() as sock:
        sock.bind(("127.0.0.1", 0))
        return int(sock.getsockname()[1])


def _rank_main(rank: int, world: int, port: int) -> None:
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        for dtype_name, group, batch in (("bf16", 128, 1), ("fp16", 64, 3)):
            code = oracle.dtype_code(dtype_name)
            dtype = torch.bfloat16 if code else torch.float16
            shape = LayerShape("t", 512, 1024, group_size=group, batch=batch, dtype=dtype_name, zero_point=None)
            problem, packets = _packed_problem(shape, 11)
            y64 = oracle.gemv_f64(oracle.bits_of(problem["activations"]), problem["q_u8"].numpy(),
                                  oracle.bits_of(problem["alpha"]), oracle.bits_of(problem["beta"]), group, code)
            for mode in ("column", "row"):
                layer = ShardedW4A16Linear(packets, n=512, k=1024, group_size=group, mode=mode, dtype=dtype,
                                           local_forward=_oracle_local_forward(group, code, dtype))
                assert layer.n_local == (256 if mode == "column" else 512)
                out = layer(problem["activations"])
                assert out.shape == (batch, 512) and out.dtype == dtype
                assert oracle.max_rel_err(out.float().numpy(), y64) <= 1e-2, (mode, dtype_name)
                # every rank holds the same bits
                mine = out.view(torch.int16).to(torch.int32)
                theirs = [torch.empty_like(mine) for _ in range(world)]
                dist.all_gather(theirs, mine)
                assert all(torch.equal(t, mine) for t in theirs)
            # argument errors surface on the host, on every rank, before any exchange
            layer = ShardedW4A16Linear(packets, n=512, k=1024, group_size=group, mode="row", dtype=dtype,
                                       local_forward=_oracle_local_forward(group, code, dtype))
            with pytest.raises(ValueError, match="activations must have shape"):
                layer(problem["activations"][:, :512])
            with pytest.raises(TypeError, match="must have dtype"):
                layer(problem["activations"].float())
        with pytest.raises(ValueError, match="groups to divide"):
            ShardedW4A16Linear(torch.zeros((4 * 3, 8704), dtype=torch.uint8), n=512, k=384, group_size=128,
                               mode="row", dtype=torch.float16)
        with pytest.raises(ValueError, match="needs CUDA tensors"):
            ShardedW4A16Linear(torch.zeros((4 * 2, 8704), dtype=torch.uint8), n=512, k=256, group_size=128,
                               mode="row", dtype=torch.float16, exchange="peer")
    finally:
        dist.destroy_process_group()


def test_two_ranks_over_gloo() -> None:
    mp.spawn(_rank_main, args=(2, _free_port()), nprocs=2, join=True)
