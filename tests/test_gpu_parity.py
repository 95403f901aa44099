"""GPU parity: the CUDA library, called through its C ABI, against the CPU oracle.

Bars: bit-exact for pack / dequant / group sums (integer and byte work, plus the fixed-order fp32
sums); for the GEMV, max relative error <= 1e-2 against the fp64 dequant-matvec oracle (floor on
the denominator: 1e-3 of the row's largest |y|), and the reference tests' own
assert_close(atol=1e-2, rtol=1e-2) against the golden outputs.
"""

from __future__ import annotations

import numpy as np
import pytest
import torch
from fast_kernels import capi
from fast_kernels.workloads import LayerShape, make_problem
from oracle import w4a16_oracle as oracle
from w4a16_testlib import (
    Workspace,
    capi_gemv,
    capi_pack,
    dev_bits,
    golden_case_names,
    host_bits,
    load_golden,
    stream_ptr,
)

pytestmark = pytest.mark.gpu

GEMV_REL_TOL = 1e-2
WS = Workspace()


@pytest.fixture(autouse=True)
def _device_status_is_clean():
    yield
    torch.cuda.synchronize()
    assert capi.device_status() == 0, "a bounded device-side wait timed out"


def _check_gemv(problem: dict, shape: LayerShape, code: int) -> None:
    q, alpha, beta, act = (problem[k].cuda() for k in ("q_u8", "alpha", "beta", "activations"))
    packets = capi_pack(capi, q, alpha, beta, shape.group_size)
    out = capi_gemv(capi, WS, act, packets, shape.n, shape.k, shape.group_size, code)
    torch.cuda.synchronize()
    got = out.float().cpu().numpy().astype(np.float64)
    assert np.isfinite(got).all(), "some outputs were never written"
    y64 = oracle.gemv_f64(oracle.bits_of(problem["activations"]), problem["q_u8"].numpy(),
                          oracle.bits_of(problem["alpha"]), oracle.bits_of(problem["beta"]),
                          shape.group_size, code)
    err = oracle.max_rel_err(got, y64)
    assert err <= GEMV_REL_TOL, f"max relative error {err:.3e} for {shape}"
    # a second call on the same workspace must give the same bits (tickets reset themselves)
    again = capi_gemv(capi, WS, act, packets, shape.n, shape.k, shape.group_size, code)
    torch.cuda.synchronize()
    assert torch.equal(again.view(torch.int16), out.view(torch.int16))


@pytest.mark.parametrize("name", golden_case_names())
def test_gemv_matches_reference_golden_outputs(name: str) -> None:
    case = load_golden(name)
    if case is None:
        pytest.skip("this torch build does not reproduce the fixture's seeded inputs")
    meta = case["meta"]
    group, n, k = meta["group_size"], meta["n"], meta["k"]
    q = torch.from_numpy(case["q_u8"]).cuda()
    alpha, beta, act = (dev_bits(case[key], 0) for key in ("alpha", "beta", "activations"))
    packets = capi_pack(capi, q, alpha, beta, group)
    out = capi_gemv(capi, WS, act, packets, n, k, group, 0)
    expected = dev_bits(case["output"], 0)
    # the reference's own bar (tests/gpu/test_decode_quant_linear.py:102)
    torch.testing.assert_close(out, expected, atol=1e-2, rtol=1e-2)
    y64 = oracle.gemv_f64(case["activations"], case["q_u8"], case["alpha"], case["beta"], group, 0)
    assert oracle.max_rel_err(out.float().cpu().numpy(), y64) <= GEMV_REL_TOL


@pytest.mark.parametrize("group", [32, 64, 128])
@pytest.mark.parametrize("dtype", ["fp16", "bf16"])
def test_pack_and_dequant_are_bit_exact(group: int, dtype: str) -> None:
    code = oracle.dtype_code(dtype)
    shape = LayerShape("t", 384, group * 6, group_size=group, dtype=dtype, zero_point=None,
                       scale_range=(0.001, 0.05))
    problem = make_problem(shape, seed=100 + group)
    q, alpha, beta = (problem[k].cuda() for k in ("q_u8", "alpha", "beta"))
    lib = capi.load_library()
    packets = capi_pack(capi, q, alpha, beta, group)
    want_packets = oracle.pack_packets(problem["q_u8"].numpy(), oracle.bits_of(problem["alpha"]),
                                       oracle.bits_of(problem["beta"]), group)
    assert np.array_equal(packets.cpu().numpy(), want_packets)

    want_weight = oracle.dequant_rowmajor(problem["q_u8"].numpy(), oracle.bits_of(problem["alpha"]),
                                          oracle.bits_of(problem["beta"]), group, code)
    weight = torch.empty((shape.n, shape.k), dtype=alpha.dtype, device="cuda")
    capi.check(lib.fk_w4a16_dequant_rowmajor(q.data_ptr(), alpha.data_ptr(), beta.data_ptr(),
                                             weight.data_ptr(), shape.n, shape.k, group, code, stream_ptr()))
    assert np.array_equal(host_bits(weight), want_weight)
    weight.zero_()
    capi.check(lib.fk_w4a16_dequant_packets(packets.data_ptr(), weight.data_ptr(), shape.n, shape.k,
                                            group, capi.packet_stride_bytes(group), code, stream_ptr()))
    assert np.array_equal(host_bits(weight), want_weight)


@pytest.mark.parametrize("group", [32, 64, 128])
@pytest.mark.parametrize("dtype", ["fp16", "bf16"])
def test_group_sums_are_bit_exact(group: int, dtype: str) -> None:
    code = oracle.dtype_code(dtype)
    gen = torch.Generator().manual_seed(5 + group)
    act = torch.randn((5, group * 9), generator=gen).to(torch.float16 if code == 0 else torch.bfloat16)
    dev = act.cuda()
    sums = torch.empty((5, 9), dtype=torch.float32, device="cuda")
    capi.check(capi.load_library().fk_w4a16_group_sums(dev.data_ptr(), sums.data_ptr(), 5, group * 9,
                                                       group, code, stream_ptr()))
    want = oracle.group_sums(oracle.bits_of(act), group, code)
    assert np.array_equal(sums.cpu().numpy().view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("dtype", ["fp16", "bf16"])
@pytest.mark.parametrize("group", [32, 64, 128])
@pytest.mark.parametrize("batch", [1, 2, 3, 4, 7])
def test_gemv_small_shapes(group: int, batch: int, dtype: str) -> None:
    # odd tile/group counts so that warp runs start and end inside tiles
    shape = LayerShape("t", 128 * 5, group * 7, group_size=group, batch=batch, dtype=dtype,
                       zero_point=None, scale_range=(0.001, 0.05))
    _check_gemv(make_problem(shape, seed=7 * group + batch), shape, oracle.dtype_code(dtype))


@pytest.mark.parametrize(
    ("n", "k", "group", "dtype"),
    [
        (128, 128, 128, "fp16"),      # a single packet
        (128, 64, 32, "bf16"),        # two tiny packets
        (4096, 4096, 128, "fp16"),    # the reference case: fewer packets than resident warps
        (6144, 4096, 128, "bf16"),    # Llama-3-8B qkv
        (4096, 14336, 128, "bf16"),   # down_proj: long K, runs shorter than a tile
        (13824, 5120, 32, "fp16"),    # 13B MLP, smallest group
        (13824, 5120, 64, "fp16"),
    ],
)
def test_gemv_layer_shapes(n: int, k: int, group: int, dtype: str) -> None:
    shape = LayerShape("t", n, k, group_size=group, dtype=dtype, zero_point=None)
    _check_gemv(make_problem(shape), shape, oracle.dtype_code(dtype))


@pytest.mark.parametrize(("warps", "stages", "ctas"), [(1, 2, 3), (3, 2, 0), (8, 3, 0), (16, 2, 0), (5, 4, 11)])
def test_gemv_is_independent_of_launch_shape(warps: int, stages: int, ctas: int) -> None:
    lib = capi.load_library()
    shape = LayerShape("t", 128 * 9, 128 * 11, batch=2, dtype="fp16", zero_point=None)
    problem = make_problem(shape, seed=99)
    try:
        capi.check(lib.fk_w4a16_set_launch_config(warps, stages, ctas))
        _check_gemv(problem, shape, 0)
    finally:
        capi.check(lib.fk_w4a16_set_launch_config(0, 0, 0))


def test_gemv_full_size_properties() -> None:
    """At a size the CPU oracle would take too long on: linearity in the activations and
    agreement between the fused path and the caller-visible split-K path."""
    lib = capi.load_library()
    shape = LayerShape("mlp_up", 28672, 8192, dtype="bf16")
    problem = make_problem(shape)
    q, alpha, beta, act = (problem[k].cuda() for k in ("q_u8", "alpha", "beta", "activations"))
    packets = capi_pack(capi, q, alpha, beta, 128)
    del q
    y1 = capi_gemv(capi, WS, act, packets, shape.n, shape.k, 128, 1).float()
    y2 = capi_gemv(capi, WS, (act * 2).contiguous(), packets, shape.n, shape.k, 128, 1).float()
    scale = y1.abs().max().item()
    assert (y2 - 2 * y1).abs().max().item() <= 2e-2 * scale  # doubling is exact up to bf16 rounding of y
    partials = torch.empty((4, 1, shape.n), dtype=torch.float32, device="cuda")
    capi.check(lib.fk_w4a16_gemv_split_k(act.data_ptr(), packets.data_ptr(), partials.data_ptr(), 1,
                                         shape.n, shape.k, 128, 8704, 4, 1, stream_ptr()))
    via_split = partials.sum(0)
    assert (via_split - y1).abs().max().item() <= 1e-2 * scale
    # and a sample of rows against the fp64 oracle
    rows = slice(0, 512)
    y64 = oracle.gemv_f64(oracle.bits_of(problem["activations"]), problem["q_u8"][rows].numpy(),
                          oracle.bits_of(problem["alpha"][rows]), oracle.bits_of(problem["beta"][rows]), 128, 1)
    assert oracle.max_rel_err(y1[:, rows].cpu().numpy(), y64) <= GEMV_REL_TOL


def _oracle_rows(problem: dict, rows: slice, group: int, code: int) -> np.ndarray:
    return oracle.gemv_f64(oracle.bits_of(problem["activations"]), problem["q_u8"][rows].numpy(),
                           oracle.bits_of(problem["alpha"][rows]), oracle.bits_of(problem["beta"][rows]),
                           group, code)


def test_gemv_lm_head_against_the_oracle() -> None:
    """The largest configured shape, 128256 x 4096 (1002 tiles, 32064 packets): row slices at the
    start, across the middle and at the very end of the output against the fp64 oracle; every
    output written; a second call gives the same bits."""
    shape = LayerShape("lm_head", 128256, 4096, dtype="bf16")
    problem = make_problem(shape)
    q, alpha, beta, act = (problem[k].cuda() for k in ("q_u8", "alpha", "beta", "activations"))
    packets = capi_pack(capi, q, alpha, beta, 128)
    del q
    out = capi_gemv(capi, WS, act, packets, shape.n, shape.k, 128, 1)
    again = capi_gemv(capi, WS, act, packets, shape.n, shape.k, 128, 1)
    torch.cuda.synchronize()
    assert torch.isfinite(out.float()).all(), "some outputs were never written"
    assert torch.equal(out.view(torch.int16), again.view(torch.int16))
    got = out.float().cpu().numpy()
    for rows in (slice(0, 384), slice(64000, 64512), slice(128256 - 384, 128256)):
        assert oracle.max_rel_err(got[:, rows], _oracle_rows(problem, rows, 128, 1)) <= GEMV_REL_TOL, rows


@pytest.mark.parametrize("batch", [2, 4, 8])
def test_gemv_batched_sweep_shape_against_the_oracle(batch: int) -> None:
    """28672 x 8192 with per-group uint4 zero points at batches 2, 4 and 8 (4 is where the launch
    plan switches to the tensor-core kernel on a layer this large)."""
    shape = LayerShape("mlp_up", 28672, 8192, batch=batch, dtype="bf16", zero_point=None)
    problem = make_problem(shape)
    q, alpha, beta, act = (problem[k].cuda() for k in ("q_u8", "alpha", "beta", "activations"))
    packets = capi_pack(capi, q, alpha, beta, 128)
    del q
    out = capi_gemv(capi, WS, act, packets, shape.n, shape.k, 128, 1)
    again = capi_gemv(capi, WS, act, packets, shape.n, shape.k, 128, 1)
    torch.cuda.synchronize()
    assert torch.isfinite(out.float()).all(), "some outputs were never written"
    assert torch.equal(out.view(torch.int16), again.view(torch.int16))
    got = out.float().cpu().numpy()
    for rows in (slice(0, 256), slice(14200, 14456), slice(28672 - 256, 28672)):
        assert oracle.max_rel_err(got[:, rows], _oracle_rows(problem, rows, 128, 1)) <= GEMV_REL_TOL, rows


def test_gemv_13b_mlp_group_128() -> None:
    shape = LayerShape("mlp13b_g128", 13824, 5120, group_size=128, dtype="fp16", scale_range=(0.001, 0.05),
                       zero_point=None)
    _check_gemv(make_problem(shape), shape, 0)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_column_shards_of_the_fused_gate_up_layer(world: int) -> None:
    """57344 x 8192 split by output columns over 2, 4 and 8 ranks, every rank's shard run on this
    GPU: each shard's outputs land in its slice of the full row (output_ld / output_col0), and the
    assembled row meets the fp64 oracle on slices that straddle shard boundaries."""
    from fast_kernels.dist import column_shard_packets

    lib = capi.load_library()
    shape = LayerShape("gate_up_70b", 57344, 8192, dtype="bf16")
    problem = make_problem(shape)
    q, alpha, beta, act = (problem[k].cuda() for k in ("q_u8", "alpha", "beta", "activations"))
    packets = capi_pack(capi, q, alpha, beta, 128)
    del q
    n_local = shape.n // world
    full = torch.full((1, shape.n), float("nan"), dtype=torch.bfloat16, device="cuda")
    for rank in range(world):
        shard = column_shard_packets(packets, n=shape.n, k=shape.k, group_size=128, rank=rank, world=world)
        args = capi.GemvArgs()
        ws = WS.get(capi, 1, n_local, shape.k, 128)
        args.activations, args.packets, args.output = act.data_ptr(), shard.data_ptr(), full.data_ptr()
        args.workspace, args.workspace_bytes = ws.data_ptr(), ws.numel()
        args.batch, args.n, args.k, args.group_size = 1, n_local, shape.k, 128
        args.packet_stride_bytes, args.dtype = 8704, 1
        args.output_ld, args.output_col0 = shape.n, rank * n_local
        args.stream = stream_ptr()
        capi.check(lib.fk_w4a16_gemv_ex(args))
    torch.cuda.synchronize()
    assert torch.isfinite(full.float()).all(), "some outputs were never written"
    got = full.float().cpu().numpy()
    edge = n_local  # the boundary between rank 0 and rank 1
    for rows in (slice(0, 256), slice(edge - 128, edge + 128), slice(shape.n - 256, shape.n)):
        assert oracle.max_rel_err(got[:, rows], _oracle_rows(problem, rows, 128, 1)) <= GEMV_REL_TOL, rows


@pytest.mark.parametrize("world", [2, 4, 8])
def test_row_shards_of_the_down_projection(world: int) -> None:
    """8192 x 28672 split by input features over 2, 4 and 8 ranks, every rank's shard run on this
    GPU with unrounded fp32 outputs; the partials, added in rank order and rounded once, meet the
    fp64 oracle."""
    from fast_kernels.dist import activation_shard, row_shard_packets

    lib = capi.load_library()
    shape = LayerShape("down_70b", 8192, 28672, dtype="bf16")
    problem = make_problem(shape)
    q, alpha, beta, act = (problem[k].cuda() for k in ("q_u8", "alpha", "beta", "activations"))
    packets = capi_pack(capi, q, alpha, beta, 128)
    del q
    k_local = shape.k // world
    partials = torch.full((world, 1, shape.n), float("nan"), dtype=torch.float32, device="cuda")
    for rank in range(world):
        shard = row_shard_packets(packets, n=shape.n, k=shape.k, group_size=128, rank=rank, world=world)
        local_act = activation_shard(act, rank=rank, world=world, mode="row")
        args = capi.GemvArgs()
        ws = WS.get(capi, 1, shape.n, k_local, 128)
        args.activations, args.packets = local_act.data_ptr(), shard.data_ptr()
        args.output = partials[rank].data_ptr()
        args.workspace, args.workspace_bytes = ws.data_ptr(), ws.numel()
        args.batch, args.n, args.k, args.group_size = 1, shape.n, k_local, 128
        args.packet_stride_bytes, args.dtype = 8704, 1
        args.output_f32 = 1
        args.stream = stream_ptr()
        capi.check(lib.fk_w4a16_gemv_ex(args))
        torch.cuda.synchronize()
    assert torch.isfinite(partials).all(), "some partial sums were never written"
    total = partials[0].clone()
    for rank in range(1, world):
        total = total + partials[rank]
    got = total.to(torch.bfloat16).float().cpu().numpy()
    for rows in (slice(0, 512), slice(4000, 4256), slice(shape.n - 256, shape.n)):
        assert oracle.max_rel_err(got[:, rows], _oracle_rows(problem, rows, 128, 1)) <= GEMV_REL_TOL, rows


@pytest.mark.parametrize("dtype", ["fp16", "bf16"])
@pytest.mark.parametrize(("batch", "slices"), [(1, 2), (8, 4), (3, 7)])
def test_split_k_and_reduce(batch: int, slices: int, dtype: str) -> None:
    """The caller-visible split-K pair (reference: arc_w4a16.cu:709-751; its test :171-207)."""
    code = oracle.dtype_code(dtype)
    lib = capi.load_library()
    shape = LayerShape("t", 256, 128 * 7, batch=batch, dtype=dtype, zero_point=None)
    problem = make_problem(shape, seed=4242)
    q, alpha, beta, act = (problem[k].cuda() for k in ("q_u8", "alpha", "beta", "activations"))
    packets = capi_pack(capi, q, alpha, beta, 128)
    partials = torch.full((slices, batch, shape.n), float("nan"), dtype=torch.float32, device="cuda")
    capi.check(lib.fk_w4a16_gemv_split_k(act.data_ptr(), packets.data_ptr(), partials.data_ptr(), batch,
                                         shape.n, shape.k, 128, 8704, slices, code, stream_ptr()))
    out = torch.empty((batch, shape.n), dtype=act.dtype, device="cuda")
    capi.check(lib.fk_w4a16_reduce_partials(partials.data_ptr(), out.data_ptr(), batch, shape.n, slices,
                                            code, stream_ptr()))
    torch.cuda.synchronize()
    # reduce: slices added in index order, one rounding
    want = partials[0].clone()
    for s in range(1, slices):
        want = want + partials[s]
    assert torch.equal(out, want.to(act.dtype))
    y64 = oracle.gemv_f64(oracle.bits_of(problem["activations"]), problem["q_u8"].numpy(),
                          oracle.bits_of(problem["alpha"]), oracle.bits_of(problem["beta"]), 128, code)
    assert oracle.max_rel_err(out.float().cpu().numpy(), y64) <= GEMV_REL_TOL


@pytest.mark.parametrize("dtype", ["fp16", "bf16"])
def test_cublaslt_subject_matches_oracle(dtype: str) -> None:
    code = oracle.dtype_code(dtype)
    lib = capi.load_library()
    shape = LayerShape("t", 512, 1024, batch=4, dtype=dtype, zero_point=None)
    problem = make_problem(shape, seed=17)
    q, alpha, beta, act = (problem[k].cuda() for k in ("q_u8", "alpha", "beta", "activations"))
    weight = torch.empty((shape.n, shape.k), dtype=act.dtype, device="cuda")
    capi.check(lib.fk_w4a16_dequant_rowmajor(q.data_ptr(), alpha.data_ptr(), beta.data_ptr(),
                                             weight.data_ptr(), shape.n, shape.k, 128, code, stream_ptr()))
    out = torch.empty((4, shape.n), dtype=act.dtype, device="cuda")
    lt_ws = torch.empty(8 << 20, dtype=torch.uint8, device="cuda")
    capi.check(lib.fk_w4a16_cublaslt_matmul(act.data_ptr(), weight.data_ptr(), out.data_ptr(),
                                            lt_ws.data_ptr(), lt_ws.numel(), 4, shape.n, shape.k, code,
                                            stream_ptr()))
    torch.cuda.synchronize()
    y64 = oracle.gemv_f64(oracle.bits_of(problem["activations"]), problem["q_u8"].numpy(),
                          oracle.bits_of(problem["alpha"]), oracle.bits_of(problem["beta"]), 128, code)
    # the weight is rounded to 16 bits before the GEMM here, hence the looser bar (reference: 1e-2 abs/rel)
    assert np.allclose(out.float().cpu().numpy(), y64, rtol=2e-2, atol=2e-2)


def test_gemv_respects_the_stream() -> None:
    """Work is enqueued on the stream it is given (reference test :248-281)."""
    shape = LayerShape("t", 128, 256, dtype="fp16", zero_point=None)
    problem = make_problem(shape, seed=2112)
    q, alpha, beta = (problem[k].cuda() for k in ("q_u8", "alpha", "beta"))
    packets = capi_pack(capi, q, alpha, beta, 128)
    expected_act = problem["activations"].cuda()
    act = torch.zeros_like(expected_act)
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        torch.cuda._sleep(50_000_000)
        act.copy_(expected_act)
        out = capi_gemv(capi, WS, act, packets, shape.n, shape.k, 128, 0)
    side.synchronize()
    torch.cuda.synchronize()
    y64 = oracle.gemv_f64(oracle.bits_of(problem["activations"]), problem["q_u8"].numpy(),
                          oracle.bits_of(problem["alpha"]), oracle.bits_of(problem["beta"]), 128, 0)
    assert oracle.max_rel_err(out.float().cpu().numpy(), y64) <= GEMV_REL_TOL


def test_gemv_host_buffers_match_device_call() -> None:
    """fk_w4a16_gemv_host: pinned host activations in, pinned host result out, same bits as the
    device-pointer call; nothing synchronises inside the call."""
    lib = capi.load_library()
    shape = LayerShape("t", 128 * 9, 128 * 7, batch=3, dtype="bf16", zero_point=None)
    problem = make_problem(shape, seed=515)
    q, alpha, beta, act = (problem[k].cuda() for k in ("q_u8", "alpha", "beta", "activations"))
    packets = capi_pack(capi, q, alpha, beta, 128)
    plain = capi_gemv(capi, WS, act, packets, shape.n, shape.k, 128, 1)
    host_in = problem["activations"].pin_memory()
    host_out = torch.zeros((3, shape.n), dtype=torch.bfloat16).pin_memory()
    dev_in = torch.zeros_like(act)
    dev_out = torch.zeros_like(plain)
    ws = WS.get(capi, 3, shape.n, shape.k, 128)
    capi.check(lib.fk_w4a16_gemv_host(host_in.data_ptr(), packets.data_ptr(), host_out.data_ptr(),
                                      dev_in.data_ptr(), dev_out.data_ptr(), ws.data_ptr(), ws.numel(),
                                      3, shape.n, shape.k, 128, 8704, 1, stream_ptr()))
    torch.cuda.synchronize()
    assert torch.equal(host_out, plain.cpu())
    assert torch.equal(dev_in, act)
    assert torch.equal(dev_out, plain)
    # pageable host memory takes the copy path; same bits
    paged_in = problem["activations"].clone()
    paged_out = torch.zeros((3, shape.n), dtype=torch.bfloat16)
    dev_in.zero_()
    dev_out.zero_()
    capi.check(lib.fk_w4a16_gemv_host(paged_in.data_ptr(), packets.data_ptr(), paged_out.data_ptr(),
                                      dev_in.data_ptr(), dev_out.data_ptr(), ws.data_ptr(), ws.numel(),
                                      3, shape.n, shape.k, 128, 8704, 1, stream_ptr()))
    torch.cuda.synchronize()
    assert torch.equal(paged_out, plain.cpu()) and torch.equal(dev_out, plain)
    # back-to-back calls that reuse one staging buffer see their own activations
    host_in2 = (problem["activations"] * 0.5).pin_memory()
    host_out2 = torch.zeros_like(host_out).pin_memory()
    for h_in, h_out in ((host_in, host_out), (host_in2, host_out2), (host_in, host_out)):
        capi.check(lib.fk_w4a16_gemv_host(h_in.data_ptr(), packets.data_ptr(), h_out.data_ptr(),
                                          dev_in.data_ptr(), dev_out.data_ptr(), ws.data_ptr(), ws.numel(),
                                          3, shape.n, shape.k, 128, 8704, 1, stream_ptr()))
    torch.cuda.synchronize()
    half = capi_gemv(capi, WS, act * 0.5, packets, shape.n, shape.k, 128, 1)
    assert torch.equal(host_out, plain.cpu()) and torch.equal(host_out2, half.cpu())
    with pytest.raises(ValueError, match="host_output"):
        capi.check(lib.fk_w4a16_gemv_host(host_in.data_ptr(), packets.data_ptr(), None,
                                          dev_in.data_ptr(), dev_out.data_ptr(), ws.data_ptr(), ws.numel(),
                                          3, shape.n, shape.k, 128, 8704, 1, stream_ptr()))


def _grid_ctas(batch: int, n: int, k: int, group: int, code: int) -> int:
    """CTAs of the launch fk_w4a16_gemv makes for a problem ("... grid=AxB ...")."""
    text = capi.describe_plan(batch, n, k, group, code)
    a, b = text.split(" grid=")[1].split(" ")[0].split("x")
    return int(a) * int(b)


@pytest.mark.parametrize(("n", "k"), [(128 * 6, 128 * 5), (128 * 100, 128 * 9)])  # cluster / stream kernel
def test_gemv_ex_output_placement_fp32_and_peer_stores(n: int, k: int) -> None:
    """fk_w4a16_gemv_ex: fp32 partial outputs, a slice of a wider matrix, a second destination
    and the completion counters -- here with both destinations on this GPU. Every CTA adds one to
    every counter; the kernel completes once its own counter shows wait_value x CTAs."""
    lib = capi.load_library()
    shape = LayerShape("t", n, k, batch=2, dtype="bf16", zero_point=None)
    problem = make_problem(shape, seed=808)
    q, alpha, beta, act = (problem[k_].cuda() for k_ in ("q_u8", "alpha", "beta", "activations"))
    packets = capi_pack(capi, q, alpha, beta, 128)
    plain = capi_gemv(capi, WS, act, packets, shape.n, shape.k, 128, 1)
    ctas = _grid_ctas(2, shape.n, shape.k, 128, 1)
    ld, col0 = shape.n * 3, shape.n
    signals = torch.zeros(64, dtype=torch.int32, device="cuda")
    for want_f32 in (0, 1):
        dtype = torch.float32 if want_f32 else torch.bfloat16
        wide = torch.full((2, ld), -7.0, dtype=dtype, device="cuda")
        mirror = torch.full((2, ld), -7.0, dtype=dtype, device="cuda")
        args = capi.GemvArgs()
        ws = WS.get(capi, 2, shape.n, shape.k, 128)
        args.activations, args.packets, args.output = act.data_ptr(), packets.data_ptr(), wide.data_ptr()
        args.workspace, args.workspace_bytes = ws.data_ptr(), ws.numel()
        args.batch, args.n, args.k, args.group_size = 2, shape.n, shape.k, 128
        args.packet_stride_bytes, args.dtype = 8704, 1
        args.output_f32, args.output_ld, args.output_col0 = want_f32, ld, col0
        args.num_peers = 1
        args.peer_outputs[0] = mirror.data_ptr()
        args.peer_signals[0] = signals.data_ptr() + 4
        args.local_signal = signals.data_ptr()
        args.wait_value = want_f32 + 1  # calls so far x (GPUs in the group = 1)
        args.stream = stream_ptr()
        capi.check(lib.fk_w4a16_gemv_ex(args))
        torch.cuda.synchronize()
        assert signals[0].item() == (want_f32 + 1) * ctas and signals[1].item() == (want_f32 + 1) * ctas
        for buf in (wide, mirror):
            assert (buf[:, :col0] == -7.0).all() and (buf[:, col0 + shape.n:] == -7.0).all()
        assert torch.equal(wide, mirror)
        got = wide[:, col0:col0 + shape.n]
        if want_f32:
            assert torch.equal(got.to(torch.bfloat16), plain)  # same sums, rounded once
        else:
            assert torch.equal(got, plain)
    with pytest.raises(ValueError, match="output_ld"):
        args.output_col0 = ld
        capi.check(lib.fk_w4a16_gemv_ex(args))


@pytest.mark.parametrize(("n", "k"), [(128 * 6, 128 * 5), (128 * 100, 128 * 9)])
def test_gemv_ex_fused_reduction_behind_the_exchange(n: int, k: int) -> None:
    """reduce_slots: a K-split layer's sum over GPUs inside the GEMV launch. One GPU plays one of
    two ranks: its partial goes to slot 0 of a [2][batch][n] fp32 buffer, slot 1 holds what the
    other rank would have delivered; the kernel waits for its own CTAs' signals, then writes
    round16(slot 0 + slot 1)."""
    lib = capi.load_library()
    shape = LayerShape("t", n, k, batch=2, dtype="bf16", zero_point=None)
    problem = make_problem(shape, seed=909)
    q, alpha, beta, act = (problem[k_].cuda() for k_ in ("q_u8", "alpha", "beta", "activations"))
    packets = capi_pack(capi, q, alpha, beta, 128)
    y32 = torch.empty((2, n), dtype=torch.float32, device="cuda")
    _gemv_ex(lib, act, packets, y32, shape, 1, f32=1)
    gen = torch.Generator().manual_seed(4)
    other = torch.randn((2, n), generator=gen).cuda()
    slots = torch.full((2, 2, n), float("nan"), dtype=torch.float32, device="cuda")
    slots[1] = other
    signals = torch.zeros(8, dtype=torch.int32, device="cuda")
    for call in (1, 2):  # twice: the counter keeps counting
        slots[0].fill_(float("nan"))
        out = torch.full((2, n), float("nan"), dtype=torch.bfloat16, device="cuda")
        args = capi.GemvArgs()
        ws = WS.get(capi, 2, n, k, 128)
        args.activations, args.packets, args.output = act.data_ptr(), packets.data_ptr(), slots.data_ptr()
        args.workspace, args.workspace_bytes = ws.data_ptr(), ws.numel()
        args.batch, args.n, args.k, args.group_size = 2, n, k, 128
        args.packet_stride_bytes, args.dtype = 8704, 1
        args.output_f32 = 1
        args.local_signal = signals.data_ptr()
        args.wait_value = call
        args.reduce_input, args.reduce_output, args.reduce_slots = slots.data_ptr(), out.data_ptr(), 2
        args.stream = stream_ptr()
        capi.check(lib.fk_w4a16_gemv_ex(args))
        torch.cuda.synchronize()
        assert torch.equal(slots[0], y32)
        assert torch.equal(out, (y32 + other).to(torch.bfloat16))
    args.local_signal = 0
    with pytest.raises(ValueError, match="reduce_slots"):
        capi.check(lib.fk_w4a16_gemv_ex(args))


def _ll_words(values: torch.Tensor, epoch: int) -> torch.Tensor:
    """fp32 values -> 8-byte words {value, epoch} as an int64 tensor."""
    bits = values.contiguous().view(torch.int32).to(torch.int64) & 0xFFFFFFFF
    return bits | (epoch << 32)


@pytest.mark.parametrize(("n", "k"), [(128 * 6, 128 * 5), (128 * 100, 128 * 9)])  # cluster / stream kernel
@pytest.mark.parametrize("reduce", [0, 1])
def test_gemv_ex_flag_in_data_exchange(n: int, k: int, reduce: int) -> None:
    """The ll_* exchange with one GPU playing rank 0 of two: its results go out as 8-byte words
    {fp32 value, epoch} into slot 0 of its own receive area, slot 1 holds the words the other rank
    would have stored, and the kernel's first CTAs assemble the final output -- the two slots'
    columns side by side (an N-split) or their sum (a K-split). With the epoch kept on the device:
    three calls in a row alternate between the two receive areas, and the calls are recorded into
    a CUDA graph and replayed."""
    lib = capi.load_library()
    batch = 2
    shape = LayerShape("t", n, k, batch=batch, dtype="bf16", zero_point=None)
    problem = make_problem(shape, seed=1212)
    q, alpha, beta, act = (problem[k_].cuda() for k_ in ("q_u8", "alpha", "beta", "activations"))
    packets = capi_pack(capi, q, alpha, beta, 128)
    y32 = torch.empty((batch, n), dtype=torch.float32, device="cuda")
    _gemv_ex(lib, act, packets, y32, shape, 1, f32=1)
    gen = torch.Generator().manual_seed(8)
    other = torch.randn((batch, n), generator=gen).cuda()
    want = (y32 + other).to(torch.bfloat16) if reduce else torch.cat([y32, other], dim=1).to(torch.bfloat16)

    slot_words = batch * n
    area_words = 2 * slot_words
    control = torch.zeros(4, dtype=torch.int32, device="cuda")          # epoch counter, ticket
    areas = torch.zeros((2, 2, batch, n), dtype=torch.int64, device="cuda")  # [parity][slot][m][n]
    out = torch.full(want.shape, float("nan"), dtype=torch.bfloat16, device="cuda")
    ws = WS.get(capi, batch, n, k, 128)

    def call() -> None:
        args = capi.GemvArgs()
        args.activations, args.packets, args.output = act.data_ptr(), packets.data_ptr(), areas.data_ptr()
        args.workspace, args.workspace_bytes = ws.data_ptr(), ws.numel()
        args.batch, args.n, args.k, args.group_size = batch, n, k, 128
        args.packet_stride_bytes, args.dtype = 8704, 1
        args.ll_epoch_counter = control.data_ptr()
        args.ll_parity_words = area_words
        args.ll_input, args.ll_output = areas.data_ptr(), out.data_ptr()
        args.ll_slots, args.ll_slot_cols, args.ll_reduce = 2, n, reduce
        args.stream = stream_ptr()
        capi.check(lib.fk_w4a16_gemv_ex(args))

    for epoch in (1, 2, 3):
        areas[epoch & 1, 1] = _ll_words(other, epoch)  # what the other rank stores for this call
        out.fill_(float("nan"))
        call()
        torch.cuda.synchronize()
        assert control[0].item() == epoch and control[1].item() == 0
        assert torch.equal(out, want), epoch
        mine = areas[epoch & 1, 0]
        assert torch.equal((mine >> 32).to(torch.int32), torch.full_like(mine, epoch, dtype=torch.int32))
        assert torch.equal((mine & 0xFFFFFFFF).to(torch.int32).view(torch.float32), y32)
    # recorded once, replayed twice: epochs 4/5 while recording is not run, then 4 and 5
    areas[0, 1] = _ll_words(other, 4)
    areas[1, 1] = _ll_words(other, 5)
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            call()
    torch.cuda.current_stream().wait_stream(side)
    for epoch in (4, 5):
        out.fill_(float("nan"))
        graph.replay()
        torch.cuda.synchronize()
        assert control[0].item() == epoch
        assert torch.equal(out, want), epoch
    # a word that never arrives: bounded wait, status 2, the context stays usable
    capi.check(lib.fk_w4a16_set_tuning(b"peer_wait_ms", 20))
    try:
        areas[0, 1] = 0
        call()  # epoch 6 expects slot 1 of area 0
        torch.cuda.synchronize()
        assert capi.device_status() == 2
    finally:
        capi.check(lib.fk_w4a16_set_tuning(b"peer_wait_ms", 2000))


def test_peer_wait_gives_up_and_reports_through_the_status_word() -> None:
    """Failure detection without a fault: a call whose counter can never reach its target (it is
    told to wait for one more group-wide delivery than will ever come) returns after the bounded
    wait -- shortened to 20 ms here -- with device status 2; reading the status clears it, and after
    re-initialising the workspace the same buffers serve a normal call."""
    lib = capi.load_library()
    shape = LayerShape("t", 128 * 6, 128 * 5, batch=1, dtype="bf16", zero_point=None)
    problem = make_problem(shape, seed=606)
    q, alpha, beta, act = (problem[k_].cuda() for k_ in ("q_u8", "alpha", "beta", "activations"))
    packets = capi_pack(capi, q, alpha, beta, 128)
    plain = capi_gemv(capi, WS, act, packets, shape.n, shape.k, 128, 1)
    signals = torch.zeros(8, dtype=torch.int32, device="cuda")
    out = torch.zeros((1, shape.n), dtype=torch.bfloat16, device="cuda")
    ws = WS.get(capi, 1, shape.n, shape.k, 128)

    def call(wait_value: int) -> None:
        args = capi.GemvArgs()
        args.activations, args.packets, args.output = act.data_ptr(), packets.data_ptr(), out.data_ptr()
        args.workspace, args.workspace_bytes = ws.data_ptr(), ws.numel()
        args.batch, args.n, args.k, args.group_size = 1, shape.n, shape.k, 128
        args.packet_stride_bytes, args.dtype = 8704, 1
        args.local_signal = signals.data_ptr()
        args.wait_value = wait_value
        args.stream = stream_ptr()
        capi.check(lib.fk_w4a16_gemv_ex(args))

    capi.check(lib.fk_w4a16_set_tuning(b"peer_wait_ms", 20))
    try:
        call(2)  # only one delivery (this call's own) will ever arrive
        torch.cuda.synchronize()
        assert capi.device_status() == 2  # kStatusPeerWaitTimeout
        assert capi.device_status() == 0  # reading it cleared it
        assert torch.equal(out, plain)    # this GPU's own outputs were complete all the same
        capi.check(lib.fk_w4a16_workspace_init(ws.data_ptr(), ws.numel(), stream_ptr()))
        out.zero_()
        call(2)  # the counter now holds two rounds of signals: a normal call
        torch.cuda.synchronize()
        assert capi.device_status() == 0
        assert torch.equal(out, plain)
    finally:
        capi.check(lib.fk_w4a16_set_tuning(b"peer_wait_ms", 2000))
    with pytest.raises(ValueError, match="peer_wait_ms"):
        capi.check(lib.fk_w4a16_set_tuning(b"peer_wait_ms", 0))
    with pytest.raises(ValueError, match="unknown tuning knob"):
        capi.check(lib.fk_w4a16_set_tuning(b"no_such_knob", 1))


def _gemv_ex(lib, act, packets, out, shape, code, *, f32=0, residual=None):
    args = capi.GemvArgs()
    ws = WS.get(capi, shape.batch, shape.n, shape.k, shape.group_size)
    args.activations, args.packets, args.output = act.data_ptr(), packets.data_ptr(), out.data_ptr()
    args.workspace, args.workspace_bytes = ws.data_ptr(), ws.numel()
    args.batch, args.n, args.k, args.group_size = shape.batch, shape.n, shape.k, shape.group_size
    args.packet_stride_bytes, args.dtype = 64 * shape.group_size + 512, code
    args.output_f32 = f32
    args.residual = 0 if residual is None else residual.data_ptr()
    args.stream = stream_ptr()
    capi.check(lib.fk_w4a16_gemv_ex(args))


@pytest.mark.parametrize(
    ("n", "k", "batch", "dtype", "variant"),
    [
        (128 * 6, 128 * 5, 1, "bf16", 0),      # stream kernel, tiles shared between CTAs
        (128 * 6, 128 * 5, 3, "fp16", 0),
        (4096, 4096, 1, "bf16", 0),            # cluster kernel
        (28672, 4096, 2, "bf16", 0),           # pair-exchange finish
        (128 * 6, 128 * 5, 8, "bf16", 0),      # mma.sync kernel
        (128 * 6, 128 * 5, 2, "bf16", 1),      # tcgen05 kernel
    ],
)
def test_gemv_ex_fused_residual_add(n: int, k: int, batch: int, dtype: str, variant: int) -> None:
    """residual: out = round16(y + residual) with ONE rounding, also in place."""
    lib = capi.load_library()
    shape = LayerShape("t", n, k, batch=batch, dtype=dtype, zero_point=None)
    problem = make_problem(shape, seed=31 + batch)
    code = oracle.dtype_code(dtype)
    q, alpha, beta, act = (problem[key].cuda() for key in ("q_u8", "alpha", "beta", "activations"))
    packets = capi_pack(capi, q, alpha, beta, 128)
    gen = torch.Generator().manual_seed(5)
    residual = torch.randn((batch, n), generator=gen).to(act.dtype).cuda()
    capi.check(lib.fk_w4a16_set_variant(variant))
    try:
        y32 = torch.empty((batch, n), dtype=torch.float32, device="cuda")
        _gemv_ex(lib, act, packets, y32, shape, code, f32=1)
        fused = torch.empty((batch, n), dtype=act.dtype, device="cuda")
        _gemv_ex(lib, act, packets, fused, shape, code, residual=residual)
        in_place = residual.clone()
        _gemv_ex(lib, act, packets, in_place, shape, code, residual=in_place)
        sum32 = torch.empty_like(y32)
        _gemv_ex(lib, act, packets, sum32, shape, code, f32=1, residual=residual)
        torch.cuda.synchronize()
    finally:
        capi.check(lib.fk_w4a16_set_variant(capi.VARIANT_AUTO))
    expected32 = y32 + residual.float()
    assert torch.equal(sum32, expected32)
    assert torch.equal(fused, expected32.to(act.dtype))
    assert torch.equal(in_place, fused)


@pytest.mark.parametrize(
    ("n", "k", "batch", "dtype", "variant"),
    [
        (128 * 6, 128 * 5, 1, "bf16", 0),      # stream kernel, tiles shared between CTAs
        (128 * 6, 128 * 5, 3, "fp16", 0),
        (4096, 4096, 2, "bf16", 0),            # cluster kernel
        (28672, 4096, 1, "bf16", 0),           # the 8B gate_up layer
        (128 * 6, 128 * 5, 8, "bf16", 0),      # mma.sync kernel
        (128 * 6, 128 * 5, 2, "fp16", 1),      # tcgen05 kernel
    ],
)
def test_gemv_ex_fused_silu_mul(n: int, k: int, batch: int, dtype: str, variant: int) -> None:
    """epilogue = SILU_MUL: out[:, j] = silu(y[:, j]) * y[:, j + n/2], from the unrounded sums."""
    lib = capi.load_library()
    shape = LayerShape("t", n, k, batch=batch, dtype=dtype, zero_point=None)
    problem = make_problem(shape, seed=77 + batch)
    code = oracle.dtype_code(dtype)
    q, alpha, beta, act = (problem[key].cuda() for key in ("q_u8", "alpha", "beta", "activations"))
    packets = capi_pack(capi, q, alpha, beta, 128)
    half = n // 2
    capi.check(lib.fk_w4a16_set_variant(variant))
    try:
        outs = []
        for _ in range(2):  # twice on one workspace: the meeting words clear themselves
            out = torch.full((batch, half), float("nan"), dtype=act.dtype, device="cuda")
            args = capi.GemvArgs()
            ws = WS.get(capi, batch, n, k, 128)
            args.activations, args.packets, args.output = act.data_ptr(), packets.data_ptr(), out.data_ptr()
            args.workspace, args.workspace_bytes = ws.data_ptr(), ws.numel()
            args.batch, args.n, args.k, args.group_size = batch, n, k, 128
            args.packet_stride_bytes, args.dtype = 8704, code
            args.epilogue = capi.EPILOGUE_SILU_MUL
            args.stream = stream_ptr()
            capi.check(lib.fk_w4a16_gemv_ex(args))
            torch.cuda.synchronize()
            outs.append(out)
        plain = capi_gemv(capi, WS, act, packets, n, k, 128, code)  # the workspace still works
        torch.cuda.synchronize()
    finally:
        capi.check(lib.fk_w4a16_set_variant(capi.VARIANT_AUTO))
    y64 = oracle.gemv_f64(oracle.bits_of(problem["activations"]), problem["q_u8"].numpy(),
                          oracle.bits_of(problem["alpha"]), oracle.bits_of(problem["beta"]), 128, code)
    gate, up = y64[:, :half], y64[:, half:]
    want = gate / (1.0 + np.exp(-gate)) * up
    got = outs[0].float().cpu().numpy().astype(np.float64)
    assert np.isfinite(got).all(), "some outputs were never written"
    assert oracle.max_rel_err(got, want) <= GEMV_REL_TOL
    assert torch.equal(outs[0].view(torch.int16), outs[1].view(torch.int16))
    assert oracle.max_rel_err(plain.float().cpu().numpy(), y64) <= GEMV_REL_TOL


@pytest.mark.parametrize(
    ("n", "k", "batch", "dtype"),
    [
        (128 * 6, 128 * 5, 1, "bf16"),   # stream kernel
        (128 * 6, 128 * 5, 3, "fp16"),
        (4096, 4096, 2, "bf16"),         # cluster kernel
        (28672, 4096, 1, "bf16"),        # the 8B gate_up layer behind its post-attention norm
        (28672, 4096, 4, "bf16"),        # a batch the plain call would send to the mma.sync kernel
    ],
)
def test_gemv_ex_fused_rmsnorm(n: int, k: int, batch: int, dtype: str) -> None:
    """norm_weight: the GEMV multiplies round16(w * round16(x * rsqrt(mean(x^2) + eps)))."""
    lib = capi.load_library()
    shape = LayerShape("t", n, k, batch=batch, dtype=dtype, zero_point=None)
    problem = make_problem(shape, seed=55 + batch)
    code = oracle.dtype_code(dtype)
    q, alpha, beta = (problem[key].cuda() for key in ("q_u8", "alpha", "beta"))
    packets = capi_pack(capi, q, alpha, beta, 128)
    gen = torch.Generator().manual_seed(9)
    torch_dtype_ = torch.bfloat16 if code else torch.float16
    x = (3.0 * torch.randn((batch, k), generator=gen)).to(torch_dtype_)
    weight = (1.0 + 0.1 * torch.randn((k,), generator=gen)).to(torch_dtype_)
    eps = 1e-5
    # the module's arithmetic, with the sum of squares in fp64
    inv = 1.0 / np.sqrt((x.double().numpy() ** 2).mean(axis=1, keepdims=True) + eps)
    x_norm = torch.from_numpy(x.float().numpy() * inv.astype(np.float32)).to(torch_dtype_)
    normed = (weight.float() * x_norm.float()).to(torch_dtype_)
    y64 = oracle.gemv_f64(oracle.bits_of(normed), problem["q_u8"].numpy(), oracle.bits_of(problem["alpha"]),
                          oracle.bits_of(problem["beta"]), 128, code)

    out = torch.full((batch, n), float("nan"), dtype=torch_dtype_, device="cuda")
    x_dev, w_dev = x.cuda(), weight.cuda()
    args = capi.GemvArgs()
    ws = WS.get(capi, batch, n, k, 128)
    args.activations, args.packets, args.output = x_dev.data_ptr(), packets.data_ptr(), out.data_ptr()
    args.workspace, args.workspace_bytes = ws.data_ptr(), ws.numel()
    args.batch, args.n, args.k, args.group_size = batch, n, k, 128
    args.packet_stride_bytes, args.dtype = 8704, code
    args.norm_weight, args.norm_eps = w_dev.data_ptr(), eps
    args.stream = stream_ptr()
    capi.check(lib.fk_w4a16_gemv_ex(args))
    torch.cuda.synchronize()
    got = out.float().cpu().numpy().astype(np.float64)
    assert np.isfinite(got).all()
    assert oracle.max_rel_err(got, y64) <= GEMV_REL_TOL
    # and it equals the unfused pipeline on the same normalised activations up to the rare element
    # whose first rounding falls the other way (the sum of squares is added in another order)
    unfused = capi_gemv(capi, WS, normed.cuda(), packets, n, k, 128, code)
    torch.cuda.synchronize()
    assert oracle.max_rel_err(got, unfused.double().cpu().numpy()) <= GEMV_REL_TOL
    args.batch = 5
    with pytest.raises(ValueError, match="RMSNorm"):
        capi.check(lib.fk_w4a16_gemv_ex(args))


def test_gemv_ex_silu_mul_refusals() -> None:
    lib = capi.load_library()
    shape = LayerShape("t", 128 * 3, 128, batch=1, dtype="bf16", zero_point=None)
    problem = make_problem(shape, seed=1)
    q, alpha, beta, act = (problem[key].cuda() for key in ("q_u8", "alpha", "beta", "activations"))
    packets = capi_pack(capi, q, alpha, beta, 128)
    out = torch.empty((1, shape.n), dtype=act.dtype, device="cuda")
    args = capi.GemvArgs()
    ws = WS.get(capi, 1, shape.n, shape.k, 128)
    args.activations, args.packets, args.output = act.data_ptr(), packets.data_ptr(), out.data_ptr()
    args.workspace, args.workspace_bytes = ws.data_ptr(), ws.numel()
    args.batch, args.n, args.k, args.group_size = 1, shape.n, shape.k, 128
    args.packet_stride_bytes, args.dtype = 8704, 1
    args.epilogue = capi.EPILOGUE_SILU_MUL
    with pytest.raises(ValueError, match="multiple of 256"):
        capi.check(lib.fk_w4a16_gemv_ex(args))
    args.epilogue = 9
    with pytest.raises(ValueError, match="epilogue"):
        capi.check(lib.fk_w4a16_gemv_ex(args))


@pytest.mark.parametrize("dtype", ["fp16", "bf16"])
@pytest.mark.parametrize("group", [32, 64, 128])
@pytest.mark.parametrize("batch", [5, 8, 9, 16, 19])
def test_gemm_tensor_core_batches(group: int, batch: int, dtype: str) -> None:
    """Batches above 4 take the MMA kernel (rows in tiles of 8 or 16, the last one padded)."""
    shape = LayerShape("t", 128 * 5, group * 9, group_size=group, batch=batch, dtype=dtype,
                       zero_point=None, scale_range=(0.001, 0.05))
    _check_gemv(make_problem(shape, seed=13 * group + batch), shape, oracle.dtype_code(dtype))


@pytest.mark.parametrize(("n", "k", "batch"), [(4096, 4096, 8), (28672, 8192, 16), (4096, 14336, 8)])
def test_gemm_tensor_core_layer_shapes(n: int, k: int, batch: int) -> None:
    shape = LayerShape("t", n, k, batch=batch, dtype="bf16", zero_point=None)
    problem = make_problem(shape)
    if n * k > 64 * 1024 * 1024:  # keep the CPU oracle to a slice of the rows at the largest size
        q, alpha, beta, act = (problem[key].cuda() for key in ("q_u8", "alpha", "beta", "activations"))
        packets = capi_pack(capi, q, alpha, beta, 128)
        out = capi_gemv(capi, WS, act, packets, n, k, 128, 1)
        torch.cuda.synchronize()
        assert torch.isfinite(out.float()).all()
        rows = slice(1024, 1536)
        y64 = oracle.gemv_f64(oracle.bits_of(problem["activations"]), problem["q_u8"][rows].numpy(),
                              oracle.bits_of(problem["alpha"][rows]), oracle.bits_of(problem["beta"][rows]), 128, 1)
        assert oracle.max_rel_err(out[:, rows].float().cpu().numpy(), y64) <= GEMV_REL_TOL
        return
    _check_gemv(problem, shape, 1)


@pytest.mark.parametrize("dtype", ["fp16", "bf16"])
@pytest.mark.parametrize("group", [32, 64, 128])
@pytest.mark.parametrize("batch", [1, 2])
def test_warp_mma_variant_matches_the_oracle(group: int, batch: int, dtype: str) -> None:
    """Tuning knob "wmma" (FK_W4A16_WMMA=1): the stream kernel with its inner product on mma.sync
    (batches 1 and 2)."""
    lib = capi.load_library()
    capi.check(lib.fk_w4a16_set_tuning(b"wmma", 1))
    try:
        shape = LayerShape("t", 128 * 5, group * 9, group_size=group, batch=batch, dtype=dtype,
                           zero_point=None)
        _check_gemv(make_problem(shape, seed=777 + batch), shape, oracle.dtype_code(dtype))
        big = LayerShape("gate_up", 28672, 4096, batch=batch, dtype=dtype, zero_point=None)
        if group == 128:
            _check_gemv(make_problem(big, seed=778), big, oracle.dtype_code(dtype))
    finally:
        capi.check(lib.fk_w4a16_set_tuning(b"wmma", 0))


@pytest.mark.parametrize("dtype", ["fp16", "bf16"])
@pytest.mark.parametrize("group", [32, 64, 128])
@pytest.mark.parametrize("batch", [1, 2, 3, 4, 8, 16, 19])
def test_tcgen05_variant_matches_the_oracle(group: int, batch: int, dtype: str) -> None:
    """The warp-specialised tcgen05 / tensor-memory kernel meets the same bar as the other kernels
    for every group size, type and batch (more than 16 rows: 16 at a time)."""
    lib = capi.load_library()
    capi.check(lib.fk_w4a16_set_variant(capi.VARIANT_TCGEN05))
    try:
        shape = LayerShape("t", 128 * 5, group * 9, group_size=group, batch=batch, dtype=dtype,
                           zero_point=None)
        _check_gemv(make_problem(shape, seed=5150 + batch), shape, oracle.dtype_code(dtype))
        assert capi.device_status() == 0
    finally:
        capi.check(lib.fk_w4a16_set_variant(capi.VARIANT_AUTO))


@pytest.mark.parametrize(("n", "k", "batch"), [(4096, 4096, 1), (6144, 4096, 2), (4096, 14336, 4),
                                                 (28672, 4096, 8), (13824, 5120, 16)])
def test_tcgen05_variant_on_layer_shapes(n: int, k: int, batch: int) -> None:
    lib = capi.load_library()
    capi.check(lib.fk_w4a16_set_variant(capi.VARIANT_TCGEN05))
    try:
        shape = LayerShape("t", n, k, batch=batch, dtype="bf16", zero_point=None)
        _check_gemv(make_problem(shape, seed=99), shape, oracle.dtype_code("bf16"))
    finally:
        capi.check(lib.fk_w4a16_set_variant(capi.VARIANT_AUTO))
    with pytest.raises(ValueError, match="variant"):
        capi.check(lib.fk_w4a16_set_variant(7))
