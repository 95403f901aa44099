"""Paged-KV decode attention on the GPU: the kernel through the C ABI and through the
reference-compatible Python op, against the fp64 oracle, the fixtures the reference's own Python
produced, and -- where it is built -- the reference's own CUDA kernels.

Tolerances. Against the fp64 oracle ON THE SAME (quantised) DATA: |y - y64| <= 2e-3 + 8e-3 |y64|
(one bf16 rounding of the output is 2^-9 relative; the arithmetic is fp32). Against the reference's
PyTorch expectation, which for 8-bit pages is computed from the unquantised pages: the reference's
own atol = 0.125, rtol = 0.03 (tests/gpu/test_clustered_page_decode.py:156 there)."""

from __future__ import annotations

import ctypes
import importlib

import numpy as np
import pytest
import torch
from fast_kernels import page_decode_capi as pdc
from oracle import page_decode_oracle as oracle
from oracle import reference_page_decode_gpu as refgpu
from page_decode_testlib import KV_IDS, DeviceCase, case_on_device, load_case, manifest

pytestmark = pytest.mark.gpu
ops = importlib.import_module("fast_kernels.ops.clustered_page_decode")
CASES = manifest()
IDS = [m["name"] for m in CASES]
ATOL, RTOL = 2e-3, 8e-3


def _assert_close_to_oracle(out: torch.Tensor, want: np.ndarray, what: str = "") -> None:
    got = out.float().cpu().numpy().astype(np.float64)
    assert np.isfinite(got).all(), what
    worst, scaled = oracle.max_abs_and_scaled_error(got, want, ATOL, RTOL)
    assert scaled <= 1.0, f"{what}: max abs error {worst:.3e}, {scaled:.2f} x tolerance"


def _status_ok() -> None:
    torch.cuda.synchronize()
    assert pdc.device_status() == 0


# ---- fixtures: the kernel on the reference's inputs --------------------------------------------------
@pytest.mark.parametrize("splits", [1, 0, 3, 8])
@pytest.mark.parametrize("meta", CASES, ids=IDS)
def test_kernel_on_the_reference_fixtures(meta, splits) -> None:
    case = load_case(meta["name"])
    dev = case_on_device(meta, case)
    out = dev.forward(pdc, splits=splits)
    _assert_close_to_oracle(out, dev.oracle(oracle), meta["name"])
    expected = torch.from_numpy(case["expected"].view(np.int16).copy()).view(torch.bfloat16).float()
    torch.testing.assert_close(out.float().cpu(), expected, atol=1.25e-1, rtol=3e-2)
    _status_ok()


# ---- seeded problems of every shape the kernel is instantiated for -----------------------------------
def _random_problem(*, batch, q_heads, kv_heads, head_dim, page_size, lens, layout, rotated, seed, fragment=True):
    generator = torch.Generator().manual_seed(seed)
    max_len = max(max(lens), 1)
    query = torch.randn((batch, q_heads, head_dim), generator=generator).to(torch.bfloat16)
    keys = torch.randn((batch, kv_heads, max_len, head_dim), generator=generator).to(torch.bfloat16)
    values = torch.randn((batch, kv_heads, max_len, head_dim), generator=generator).to(torch.bfloat16)
    build = {"bf16_kv": ops.pack_paged_kv_bf16, "int8_kv": ops.quantize_paged_kv_int8,
             "fp8_kv": ops.quantize_paged_kv_fp8}[layout]
    cache = build(keys, values, torch.tensor(lens, dtype=torch.int32), page_size=page_size, fragment_pages=fragment,
                  seed=seed, key_rope_theta=10000.0 if rotated else None)
    plan = ops.plan_clustered_page_decode(page_table=cache.page_table, seq_lens=cache.seq_lens, num_q_heads=q_heads,
                                          num_kv_heads=kv_heads, head_dim=head_dim, page_size=page_size,
                                          kv_layout=layout, use_cache=False)
    return query, cache, plan


def _device_case(query, cache, plan) -> DeviceCase:
    def raw(t):
        if t.dtype == torch.bfloat16:
            return t.contiguous().view(torch.int16).numpy().view(np.uint16)
        return t.contiguous().view(torch.uint8).numpy()

    runs = {name: getattr(plan, f"{name}_cpu").numpy() for name in
            ("run_base_pages", "run_page_counts", "run_logical_starts", "run_last_page_lens", "request_run_offsets")}
    return DeviceCase(query=raw(query), key_pages=raw(cache.key_pages), value_pages=raw(cache.value_pages),
                      key_scales=None if cache.key_scales is None else cache.key_scales.numpy(),
                      value_scales=None if cache.value_scales is None else cache.value_scales.numpy(),
                      runs=runs, seq_lens=cache.seq_lens.numpy(), kv_format=KV_IDS[cache.kv_layout],
                      keys_are_rotated=cache.keys_are_rotated, page_size=cache.page_size)


@pytest.mark.parametrize("rotated", [False, True])
@pytest.mark.parametrize("layout", ["bf16_kv", "fp8_kv", "int8_kv"])
@pytest.mark.parametrize(("head_dim", "page_size"), [(64, 16), (64, 32), (128, 16), (128, 32)])
@pytest.mark.parametrize("group", [1, 2, 3, 4, 8, 12])
def test_every_instantiation_against_the_oracle(group, head_dim, page_size, layout, rotated) -> None:
    """Group sizes 3 and 12 leave a head tile partly empty; 12 also needs two tiles."""
    kv_heads = 2
    lens = [5 * page_size + 3, 1, 2 * page_size]  # ragged, a single token, an exact multiple
    query, cache, plan = _random_problem(batch=3, q_heads=group * kv_heads, kv_heads=kv_heads, head_dim=head_dim,
                                         page_size=page_size, lens=lens, layout=layout, rotated=rotated,
                                         seed=group * 1000 + head_dim + page_size)
    dev = _device_case(query, cache, plan)
    want = dev.oracle(oracle)
    for splits in (1, 2, 3):  # one block; a cluster of two; three blocks through the workspace
        _assert_close_to_oracle(dev.forward(pdc, splits=splits), want, f"splits={splits}")
    _status_ok()


@pytest.mark.parametrize(("name", "shape"), [
    # the shapes of the reference's benchmark suite (benchmarks/suites/clustered_page_decode.toml there)
    ("gqa4_short_page16", dict(batch=4, page_size=16, max_len=256, q_heads=32, kv_heads=8, head_dim=128)),
    ("gqa4_long_page16", dict(batch=4, page_size=16, max_len=2048, q_heads=32, kv_heads=8, head_dim=128)),
    ("mqa8_long_page32", dict(batch=2, page_size=32, max_len=4096, q_heads=32, kv_heads=4, head_dim=128)),
    ("mqa32_long_page32", dict(batch=2, page_size=32, max_len=4096, q_heads=32, kv_heads=1, head_dim=128)),
    ("gqa2_short_page32_h64", dict(batch=8, page_size=32, max_len=512, q_heads=16, kv_heads=8, head_dim=64)),
])
@pytest.mark.parametrize("layout", ["bf16_kv", "int8_kv", "fp8_kv"])
def test_benchmark_suite_shapes_through_the_python_op(name, shape, layout) -> None:
    generator = torch.Generator().manual_seed(len(name))
    lens = torch.randint(max(shape["page_size"], shape["max_len"] - shape["page_size"] + 1), shape["max_len"] + 1,
                         (shape["batch"],), generator=generator).tolist()
    query, cache, plan = _random_problem(batch=shape["batch"], q_heads=shape["q_heads"], kv_heads=shape["kv_heads"],
                                         head_dim=shape["head_dim"], page_size=shape["page_size"], lens=lens,
                                         layout=layout, rotated=False, seed=7)
    want = _device_case(query, cache, plan).oracle(oracle)
    gpu_cache = _cache_to(cache, "cuda")
    out = ops.clustered_page_decode(query.cuda(), gpu_cache, plan=plan)
    _assert_close_to_oracle(out, want, name)
    reference = ops.reference_clustered_page_decode(query.cuda(), gpu_cache)
    torch.testing.assert_close(out, reference, atol=1.25e-1, rtol=3e-2)
    _status_ok()


def _cache_to(cache, device):
    def move(t):
        return None if t is None else t.to(device)

    return ops.PagedKVCache(
        key_pages=move(cache.key_pages), value_pages=move(cache.value_pages), page_table=cache.page_table,
        seq_lens=cache.seq_lens, key_scales=move(cache.key_scales), value_scales=move(cache.value_scales),
        reference_key_pages=move(cache.reference_key_pages), reference_value_pages=move(cache.reference_value_pages),
        kv_layout=cache.kv_layout, page_size=cache.page_size, num_kv_heads=cache.num_kv_heads, head_dim=cache.head_dim,
        keys_are_rotated=cache.keys_are_rotated, key_rope_theta=cache.key_rope_theta)


# ---- the reference's own GPU tests, restated against this op -----------------------------------------
def _reference_test_case(layout, force_impl, *, batch, num_q_heads, num_kv_heads, head_dim, max_seq_len, page_size,
                         cluster_size, key_rope_theta=None):
    """_assert_case of the reference (tests/gpu/test_clustered_page_decode.py:113-156 there)."""
    torch.manual_seed(batch + num_q_heads + num_kv_heads + head_dim + max_seq_len + page_size)
    query = torch.randn((batch, num_q_heads, head_dim), device="cuda").to(torch.bfloat16)
    keys = torch.randn((batch, num_kv_heads, max_seq_len, head_dim), device="cuda").to(torch.bfloat16)
    values = torch.randn((batch, num_kv_heads, max_seq_len, head_dim), device="cuda").to(torch.bfloat16)
    seq_lens = torch.randint(max(page_size, max_seq_len - page_size + 1), max_seq_len + 1, (batch,), dtype=torch.int32)
    build = {"bf16_kv": ops.pack_paged_kv_bf16, "int8_kv": ops.quantize_paged_kv_int8,
             "fp8_kv": ops.quantize_paged_kv_fp8}[layout]
    cache = build(keys, values, seq_lens, page_size=page_size, fragment_pages=True, seed=1, key_rope_theta=key_rope_theta)
    plan = ops.plan_clustered_page_decode(page_table=cache.page_table, seq_lens=cache.seq_lens, num_q_heads=num_q_heads,
                                          num_kv_heads=cache.num_kv_heads, head_dim=cache.head_dim,
                                          page_size=cache.page_size, kv_layout=cache.kv_layout, cluster_size=cluster_size)
    actual = ops.clustered_page_decode(query, cache, plan=plan, force_impl=force_impl)
    expected = ops.reference_clustered_page_decode(query, cache)
    torch.testing.assert_close(actual, expected, atol=1.25e-1, rtol=3e-2)
    return query, cache


SMALL_DIRECT = dict(batch=2, num_q_heads=16, num_kv_heads=4, head_dim=64, max_seq_len=128, page_size=16, cluster_size=1)
SMALL_CLUSTERED = dict(batch=2, num_q_heads=32, num_kv_heads=1, head_dim=128, max_seq_len=256, page_size=32, cluster_size=2)


@pytest.mark.parametrize(("layout", "force_impl", "shape"), [
    ("bf16_kv", "direct", dict(batch=2, num_q_heads=4, num_kv_heads=4, head_dim=64, max_seq_len=64, page_size=16, cluster_size=1)),
    ("bf16_kv", "direct", SMALL_DIRECT),
    ("int8_kv", "clustered", dict(batch=2, num_q_heads=32, num_kv_heads=4, head_dim=128, max_seq_len=256, page_size=32, cluster_size=2)),
    ("bf16_kv", "clustered", SMALL_CLUSTERED),
    ("fp8_kv", "clustered", dict(batch=2, num_q_heads=32, num_kv_heads=4, head_dim=128, max_seq_len=256, page_size=32, cluster_size=2)),
])
def test_op_matches_the_pytorch_reference(layout, force_impl, shape) -> None:
    _reference_test_case(layout, force_impl, **shape)
    _status_ok()


@pytest.mark.parametrize("layout", ["bf16_kv", "fp8_kv", "int8_kv"])
@pytest.mark.parametrize("force_impl", ["direct", "clustered"])
def test_op_with_keys_rotated_ahead_of_time(layout, force_impl) -> None:
    shape = SMALL_DIRECT if force_impl == "direct" else SMALL_CLUSTERED
    _reference_test_case(layout, force_impl, key_rope_theta=10000.0, **shape)
    _status_ok()


def test_op_argument_errors() -> None:
    query, cache = _reference_test_case("bf16_kv", "direct", key_rope_theta=10000.0, **SMALL_DIRECT)
    with pytest.raises(ValueError, match="rope_theta must match"):
        ops.clustered_page_decode(query, cache, rope_theta=5000.0, force_impl="direct")
    with pytest.raises(ValueError, match="force_impl must be one of"):
        ops.clustered_page_decode(query, cache, force_impl="fast")
    with pytest.raises(TypeError, match="query must have dtype"):
        ops.clustered_page_decode(query.float(), cache)
    with pytest.raises(ValueError, match="query must be a CUDA tensor"):
        ops.clustered_page_decode(query.cpu(), cache)
    with pytest.raises(ValueError, match="head_dim must match"):
        ops.clustered_page_decode(torch.zeros((2, 16, 128), dtype=torch.bfloat16, device="cuda"), cache)
    torch.manual_seed(5)
    wide = torch.randn((1, 32, 128), device="cuda").to(torch.bfloat16)
    kv = torch.randn((1, 1, 128, 128), device="cuda").to(torch.bfloat16)
    mqa = ops.pack_paged_kv_bf16(kv, kv, torch.tensor([100], dtype=torch.int32), page_size=32)
    with pytest.raises(ValueError, match='force_impl="direct" only supports group_size <= 8'):
        ops.clustered_page_decode(wide, mqa, force_impl="direct")


# ---- descriptors the planner never produces, long requests, determinism -------------------------------
def test_hand_written_runs_empty_requests_and_short_pages() -> None:
    """Runs in arbitrary order with gaps in the logical numbering, a run whose last page is short in
    the MIDDLE of a request, a request without runs, one with seq_len 0, and one of zero-length
    pages: the kernel follows the descriptors exactly as the reference's kernels do."""
    rng = np.random.default_rng(11)
    pages, kv_heads, page_size, head_dim = 12, 2, 16, 64
    keys = oracle.f32_to_bf16_bits(rng.standard_normal((pages, kv_heads, page_size, head_dim)).astype(np.float32))
    values = oracle.f32_to_bf16_bits(rng.standard_normal((pages, kv_heads, page_size, head_dim)).astype(np.float32))
    query = oracle.f32_to_bf16_bits(rng.standard_normal((5, 6, head_dim)).astype(np.float32))
    runs = {
        "run_base_pages": [7, 2, 10, 0, 5, 4],
        "run_page_counts": [2, 3, 1, 1, 2, 1],
        "run_logical_starts": [0, 5, 9, 0, 0, 0],
        "run_last_page_lens": [9, 16, 1, 16, 7, 0],
        "request_run_offsets": [0, 3, 3, 4, 5, 6],
    }
    dev = DeviceCase(query=query, key_pages=keys, value_pages=values, key_scales=None, value_scales=None,
                     runs={k: np.asarray(v, dtype=np.int32) for k, v in runs.items()},
                     seq_lens=np.asarray([150, 40, 0, 23, 1], dtype=np.int32), kv_format=0, keys_are_rotated=False,
                     page_size=page_size)
    want = dev.oracle(oracle)
    assert not want[1].any() and not want[2].any() and not want[4].any()
    for splits in (1, 0, 5):
        out = dev.forward(pdc, splits=splits)
        _assert_close_to_oracle(out, want, f"splits={splits}")
        assert not out[1].float().abs().sum().item() and not out[2].float().abs().sum().item()
    _status_ok()


def test_request_longer_than_one_block_lists_at_a_time() -> None:
    """1300 pages in ONE block (splits = 1) exceed the 1024 page entries a block keeps in shared
    memory, so the list is rebuilt for a second round; with splits the same request takes one."""
    query, cache, plan = _random_problem(batch=1, q_heads=4, kv_heads=1, head_dim=64, page_size=16, lens=[1300 * 16 - 5],
                                         layout="bf16_kv", rotated=False, seed=3)
    dev = _device_case(query, cache, plan)
    want = dev.oracle(oracle)
    for splits in (1, 0):
        _assert_close_to_oracle(dev.forward(pdc, splits=splits), want, f"splits={splits}")
    _status_ok()


def test_results_do_not_depend_on_timing_and_the_workspace_stays_clean() -> None:
    query, cache, plan = _random_problem(batch=4, q_heads=32, kv_heads=8, head_dim=128, page_size=16,
                                         lens=[2048, 1999, 1777, 2040], layout="int8_kv", rotated=False, seed=9)
    dev = _device_case(query, cache, plan)
    first = dev.forward(pdc)
    header = dev.workspace[: 64 * 1024].clone()
    for _ in range(5):
        assert torch.equal(dev.forward(pdc).view(torch.int16), first.view(torch.int16))
    torch.cuda.synchronize()
    assert not header.any().item() and not dev.workspace[: 64 * 1024].any().item()  # tickets are zero again
    info = pdc.describe_plan(dev.args(pdc, first))
    assert int(info["splits"]) > 1 and int(info["blocks"]) == int(info["tasks"]) * int(info["splits"])
    assert info["merge"] == "cluster"  # 32 tasks x 4 blocks
    through_workspace = dev.forward(pdc, splits=5)
    for _ in range(3):
        assert torch.equal(dev.forward(pdc, splits=5).view(torch.int16), through_workspace.view(torch.int16))
    torch.cuda.synchronize()
    assert not dev.workspace[: 64 * 1024].any().item()
    one = dev.forward(pdc, splits=1)
    for other in (first, through_workspace):
        assert (one.float() - other.float()).abs().max().item() <= 2e-2  # another order of the same sums
    _status_ok()


def test_call_recorded_into_a_cuda_graph_replays() -> None:
    query, cache, plan = _random_problem(batch=2, q_heads=16, kv_heads=2, head_dim=128, page_size=32,
                                         lens=[700, 650], layout="fp8_kv", rotated=True, seed=21)
    dev = _device_case(query, cache, plan)
    eager = dev.forward(pdc)
    out = torch.zeros_like(eager)
    args = dev.args(pdc, out)
    stream = torch.cuda.Stream()
    args.stream = int(stream.cuda_stream)
    graph = torch.cuda.CUDAGraph()
    torch.cuda.synchronize()
    with torch.cuda.graph(graph, stream=stream):
        pdc.check(pdc.load_library().fk_page_decode_forward(ctypes.byref(args)))
    for _ in range(3):
        out.zero_()
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(out.view(torch.int16), eager.view(torch.int16))
    _status_ok()


def test_early_descriptor_reads_give_the_same_bits_in_a_busy_stream() -> None:
    """With FK_PAGE_DECODE_FLAG_EARLY_DESCRIPTORS the kernel sorts the request's runs before it waits
    for the kernel ahead of it in the stream; queries, pages and outputs are still read after the
    wait. Here the kernel ahead WRITES the query (a copy from a staging buffer) and the call before
    that used the same workspace, several times in a row: every result must equal the plain one."""
    query, cache, plan = _random_problem(batch=4, q_heads=16, kv_heads=4, head_dim=128, page_size=16,
                                         lens=[900, 640, 17, 1024], layout="bf16_kv", rotated=False, seed=5)
    dev = _device_case(query, cache, plan)
    plain = dev.forward(pdc)
    staged = dev.query.clone()
    for _ in range(6):
        dev.query.zero_()
        dev.query.copy_(staged)  # a kernel that writes the query, right ahead of the decode
        out = dev.forward(pdc, flags=pdc.FLAG_EARLY_DESCRIPTORS)
        assert torch.equal(out.view(torch.int16), plain.view(torch.int16))
    _status_ok()


@pytest.mark.parametrize(("layout", "rotated"),
                         [("bf16_kv", True), ("bf16_kv", False), ("fp8_kv", True), ("fp8_kv", False)])
def test_whatever_lies_past_a_page_s_last_token_does_not_matter(layout, rotated) -> None:
    """Page tails past the last token are nobody's data: fill them with NaN bit patterns (bf16
    0x7fc0, e4m3 0x7f) in keys and values. Logits of those tokens are masked, and neither path may
    let a zero weight meet a NaN value (the tensor-core path zeroes such value rows in shared
    memory first -- for 8-bit pages while it converts them; the fp32 path never reads them)."""
    query, cache, plan = _random_problem(batch=3, q_heads=8, kv_heads=2, head_dim=128, page_size=32,
                                         lens=[45, 7, 100], layout=layout, rotated=rotated, seed=13)
    dev = _device_case(query, cache, plan)
    want = dev.oracle(oracle)
    info = pdc.describe_plan(dev.args(pdc, torch.empty_like(dev.query)))
    assert info["kernel"] == ("page_decode_mma" if rotated else "page_decode")
    poison = torch.tensor(0x7FC0, dtype=torch.int16) if layout == "bf16_kv" else torch.tensor(0x7F, dtype=torch.uint8)
    table, lens = cache.page_table.numpy(), cache.seq_lens.numpy()
    for request in range(3):
        last_slot = (int(lens[request]) - 1) // 32
        live = int(lens[request]) - last_slot * 32
        page = int(table[request, last_slot])
        for pages in (dev.key_pages, dev.value_pages):
            raw = pages.view(torch.int16) if layout == "bf16_kv" else pages
            raw[page, :, live:, :] = poison.to(raw.device)
    for splits in (1, 3):
        _assert_close_to_oracle(dev.forward(pdc, splits=splits), want, f"{layout} splits={splits}")
    _status_ok()


@pytest.mark.parametrize("layout", ["bf16_kv", "fp8_kv", "int8_kv"])
def test_tensor_core_variant_on_the_suite_shapes_with_rotated_keys(layout) -> None:
    """Pages whose keys carry their rotation take the mma.sync form of the kernel: same bound
    against the fp64 oracle as the fp32 form (query and probabilities enter as bf16 head +
    remainder, nothing else is rounded; e4m3 and int8 elements are bf16 values exactly, their
    scales stay in fp32)."""
    for batch, page, max_len, q_heads, kv_heads, dim in ((4, 16, 2048, 32, 8, 128), (2, 32, 4096, 32, 1, 128),
                                                          (8, 32, 512, 16, 8, 64), (3, 16, 300, 24, 2, 128)):
        generator = torch.Generator().manual_seed(batch + max_len)
        lens = torch.randint(max_len // 2, max_len + 1, (batch,), generator=generator).tolist()
        query, cache, plan = _random_problem(batch=batch, q_heads=q_heads, kv_heads=kv_heads, head_dim=dim,
                                             page_size=page, lens=lens, layout=layout, rotated=True, seed=23)
        dev = _device_case(query, cache, plan)
        out = dev.forward(pdc, max_pages_hint=plan.max_pages)
        info = pdc.describe_plan(dev.args(pdc, out, max_pages_hint=plan.max_pages))
        assert info["kernel"] == "page_decode_mma" and info["group_tile"] == "8"
        _assert_close_to_oracle(out, dev.oracle(oracle), f"{batch}x{kv_heads}x{max_len}")
        assert torch.equal(dev.forward(pdc, max_pages_hint=plan.max_pages).view(torch.int16), out.view(torch.int16))
    _status_ok()


@pytest.mark.parametrize("layout", ["fp8_kv", "int8_kv"])
def test_tensor_core_variant_with_scales_and_elements_at_the_ends_of_their_ranges(layout) -> None:
    """8-bit pages enter the tensor cores as f16, with powers of two taken out of the query and out
    of the value scales (a running exponent). Here the value scales of neighbouring tokens differ by
    up to 2^30 and grow along the sequence, the query is large, and the e4m3 pages hold subnormals
    (bytes 0x01-0x07), which the f16 operands must carry exactly: an operand flushed to zero, or a
    weight that left the f16 range, shows as an error relative to the output's own magnitude."""
    for seed, query_gain in ((3, 64.0), (4, 2.0**-12)):
        query, cache, plan = _random_problem(batch=3, q_heads=16, kv_heads=2, head_dim=128, page_size=16,
                                             lens=[700, 33, 512], layout=layout, rotated=True, seed=seed)
        generator = torch.Generator().manual_seed(100 + seed)
        query = (query.float() * query_gain).to(torch.bfloat16)
        # per-token value scales: 2^(-20 .. +10), drifting upwards with the slot inside the page
        shape = cache.value_scales.shape  # [pages, kv_heads, page_size, blocks]
        exponent = torch.randint(-20, 0, shape, generator=generator).float()
        exponent += torch.arange(shape[2]).float().view(1, 1, -1, 1) * (10.0 / shape[2])
        cache.value_scales.copy_(torch.exp2(exponent))
        # logits are degree-0 in (query gain x key scale): keep them in a softmax's working range
        cache.key_scales.mul_(1.0 / query_gain)
        if layout == "fp8_kv":
            tiny = torch.randint(1, 8, cache.value_pages.shape, generator=generator, dtype=torch.uint8)
            sign = torch.randint(0, 2, cache.value_pages.shape, generator=generator, dtype=torch.uint8) << 7
            every_other_page = (torch.arange(cache.value_pages.shape[0]) % 2 == 0).view(-1, 1, 1, 1)
            raw = cache.value_pages.view(torch.uint8)
            raw.copy_(torch.where(every_other_page, tiny | sign, raw))
            # and keys: subnormals in half of the dimensions of every third page (their logits
            # then come from the other half, which keeps them apart from one another)
            third = (torch.arange(cache.key_pages.shape[0]) % 3 == 0).view(-1, 1, 1, 1)
            odd_dims = (torch.arange(cache.key_pages.shape[3]) % 2 == 1).view(1, 1, 1, -1)
            raw = cache.key_pages.view(torch.uint8)
            raw.copy_(torch.where(third & odd_dims, tiny | sign, raw))
        dev = _device_case(query, cache, plan)
        want = dev.oracle(oracle)
        info = pdc.describe_plan(dev.args(pdc, torch.empty_like(dev.query)))
        assert info["kernel"] == "page_decode_mma"
        for splits in (1, 0):
            got = dev.forward(pdc, splits=splits).float().cpu().numpy().astype(np.float64)
            assert np.isfinite(got).all()
            for request in range(3):
                size = np.abs(want[request]).max()
                assert size > 0.0
                assert np.abs(got[request] - want[request]).max() <= 1.0e-2 * size, (layout, seed, splits, request)
    _status_ok()


def test_e4m3_subnormal_values_alone_survive_the_tensor_core_path() -> None:
    """Every value element an e4m3 subnormal (|x| <= 7 * 2^-9), value scales 1: the output is of that
    size and must match the oracle to bf16 rounding -- not zero, as it would be if the f16 operands
    of the MMA lost their subnormals."""
    query, cache, plan = _random_problem(batch=2, q_heads=8, kv_heads=2, head_dim=64, page_size=32,
                                         lens=[200, 96], layout="fp8_kv", rotated=True, seed=9)
    generator = torch.Generator().manual_seed(9)
    tiny = torch.randint(1, 8, cache.value_pages.shape, generator=generator, dtype=torch.uint8)
    sign = torch.randint(0, 2, cache.value_pages.shape, generator=generator, dtype=torch.uint8) << 7
    cache.value_pages.view(torch.uint8).copy_(tiny | sign)
    cache.value_scales.fill_(1.0)
    dev = _device_case(query, cache, plan)
    want = dev.oracle(oracle)
    got = dev.forward(pdc).float().cpu().numpy().astype(np.float64)
    size = np.abs(want).max()
    assert 2.0**-12 < size < 2.0**-6
    assert np.abs(got - want).max() <= 1.0e-2 * size
    _status_ok()


@pytest.mark.parametrize("layout", ["bf16_kv", "int8_kv"])
def test_tensor_core_variant_block_size_follows_the_wave_count(layout) -> None:
    """With more tasks than SMs the tensor-core form uses blocks of 6 warps (two to an SM) unless
    that adds more than a fifth to the number of waves; otherwise 12 warps, or 8 when fewer than
    half of the SMs have a task. Every such plan must give the oracle's result."""
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    kv_heads = 8
    for batch in (sms // (4 * kv_heads), sms // kv_heads, sms // kv_heads + 6, 2 * sms // kv_heads + 3,
                  3 * sms // kv_heads + 1):
        batch = max(batch, 1)
        tasks = batch * kv_heads
        generator = torch.Generator().manual_seed(tasks)
        lens = torch.randint(20, 70, (batch,), generator=generator).tolist()
        query, cache, plan = _random_problem(batch=batch, q_heads=32, kv_heads=kv_heads, head_dim=128,
                                             page_size=16, lens=lens, layout=layout, rotated=True, seed=tasks)
        dev = _device_case(query, cache, plan)
        out = dev.forward(pdc)
        info = pdc.describe_plan(dev.args(pdc, out))
        whole, halved = -(-tasks // sms), -(-tasks // (2 * sms))
        if tasks * 2 <= sms:
            expected = 8
        elif tasks > sms and 10 * halved <= 6 * whole:
            expected = 6
        else:
            expected = 12
        assert info["kernel"] == "page_decode_mma" and int(info["warps"]) == expected, (tasks, info)
        _assert_close_to_oracle(out, dev.oracle(oracle), f"{layout} tasks={tasks}")
    # few tasks: 8 warps while a block's share is short, 12 once a warp of 12 would see 8 units or more
    # (the plan only; `dev` is the last problem above, the hint stands for the length of the requests)
    query, cache, plan = _random_problem(batch=1, q_heads=16, kv_heads=2, head_dim=128, page_size=16,
                                         lens=[40], layout=layout, rotated=True, seed=1)
    dev = _device_case(query, cache, plan)
    out = torch.empty_like(dev.query)
    for hint, expected in ((64, 8), (1024, 8), (16384, 12)):
        info = pdc.describe_plan(dev.args(pdc, out, max_pages_hint=hint))
        assert int(info["warps"]) == expected, (hint, info)
    _status_ok()


@pytest.mark.parametrize("layout", ["fp8_kv", "int8_kv", "bf16_kv"])
def test_tensor_core_variant_fills_the_device_with_resident_thirds(layout) -> None:
    """8-bit pages, more than half and at most two thirds of the SMs with a task, long requests (by
    the caller's hint): three 6-warp blocks per task, merged through the workspace. bf16 pages keep
    one 12-warp block per task. The hint is an upper bound -- the requests here are short, so some
    blocks get no unit at all -- and the result must not depend on it."""
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    kv_heads = 2
    batch = (sms * 5 // 9) // kv_heads + 1  # tasks just above half of the SMs
    tasks = batch * kv_heads
    assert sms < 2 * tasks and 3 * tasks <= 2 * sms
    generator = torch.Generator().manual_seed(tasks)
    lens = torch.randint(1, 120, (batch,), generator=generator).tolist()
    query, cache, plan = _random_problem(batch=batch, q_heads=8, kv_heads=kv_heads, head_dim=128, page_size=16,
                                         lens=lens, layout=layout, rotated=True, seed=77)
    dev = _device_case(query, cache, plan)
    out = dev.forward(pdc, max_pages_hint=512)
    info = pdc.describe_plan(dev.args(pdc, out, max_pages_hint=512))
    if layout == "bf16_kv":
        assert (info["splits"], info["warps"]) == ("1", "12"), info
    else:
        assert (info["splits"], info["warps"], info["merge"]) == ("3", "6", "global"), info
    want = dev.oracle(oracle)
    _assert_close_to_oracle(out, want, layout)
    _assert_close_to_oracle(dev.forward(pdc, max_pages_hint=plan.max_pages), want, f"{layout}, true hint")
    _status_ok()


def test_group_tile_and_launch_overrides_keep_the_result() -> None:
    query, cache, plan = _random_problem(batch=2, q_heads=16, kv_heads=2, head_dim=128, page_size=16,
                                         lens=[333, 200], layout="bf16_kv", rotated=False, seed=2)
    dev = _device_case(query, cache, plan)
    want = dev.oracle(oracle)
    lib = pdc.load_library()
    for tile in (1, 2, 4, 8):
        _assert_close_to_oracle(dev.forward(pdc, group_tile=tile), want, f"group_tile={tile}")
    try:
        for warps, stages in ((1, 1), (3, 2), (8, 3), (4, 4)):
            pdc.check(lib.fk_page_decode_set_launch_config(warps, stages))
            _assert_close_to_oracle(dev.forward(pdc), want, f"warps={warps} stages={stages}")
    finally:
        pdc.check(lib.fk_page_decode_set_launch_config(0, 0))
    _status_ok()


def test_workspace_that_is_too_small_is_refused() -> None:
    query, cache, plan = _random_problem(batch=2, q_heads=16, kv_heads=2, head_dim=128, page_size=16,
                                         lens=[333, 200], layout="bf16_kv", rotated=False, seed=2)
    dev = _device_case(query, cache, plan)
    out = dev.forward(pdc)
    args = dev.args(pdc, out, splits=3)  # 3 blocks per task merge through the workspace (2 or 4: a cluster)
    args.workspace_bytes = 64 * 1024
    assert pdc.load_library().fk_page_decode_forward(ctypes.byref(args)) == pdc.ERR_INVALID_ARGUMENT
    assert "workspace too small" in pdc.load_library().fk_page_decode_last_error().decode()
    for splits in (1, 4):  # one block per task needs no scratch, nor does a cluster of 4
        args.splits, args.workspace, args.workspace_bytes = splits, 0, 0
        out.fill_(float("nan"))
        pdc.check(pdc.load_library().fk_page_decode_forward(ctypes.byref(args)))
        _assert_close_to_oracle(out, dev.oracle(oracle), f"splits={splits}")
    _status_ok()


# ---- shared prefixes: the reference's prefix_union_decode op ------------------------------------------
@pytest.mark.parametrize("layout", ["bf16_kv", "fp8_kv", "int8_kv"])
def test_prefix_union_op_on_requests_that_share_pages(layout) -> None:
    """The recipe of the reference's tests (tests/gpu/test_prefix_union_decode.py:48-98 there): groups
    of four requests repeat their leader's first pages, identical pages are stored once, keys are
    rotated ahead of time. On a device below compute capability 12 the reference computes the op
    through its fallback plan and refuses force_impl="union"; so does this build."""
    union = importlib.import_module("fast_kernels.ops.prefix_union_decode")
    batch, q_heads, kv_heads, dim, max_len, page, shared_pages, group = 8, 32, 8, 128, 512, 16, 4, 4
    torch.manual_seed(batch + q_heads + kv_heads + dim + max_len + page + shared_pages + group)
    query = torch.randn((batch, q_heads, dim), device="cuda").to(torch.bfloat16)
    keys = torch.randn((batch, kv_heads, max_len, dim), device="cuda").to(torch.bfloat16)
    values = torch.randn((batch, kv_heads, max_len, dim), device="cuda").to(torch.bfloat16)
    lens = torch.randint(shared_pages * page + 1, max_len + 1, (batch,), dtype=torch.int32)
    for start in range(0, batch, group):
        keys[start + 1 : start + group, :, : shared_pages * page] = keys[start, :, : shared_pages * page]
        values[start + 1 : start + group, :, : shared_pages * page] = values[start, :, : shared_pages * page]
    build = {"bf16_kv": ops.pack_paged_kv_bf16, "int8_kv": ops.quantize_paged_kv_int8,
             "fp8_kv": ops.quantize_paged_kv_fp8}[layout]
    cache = build(keys, values, lens, page_size=page, fragment_pages=True, seed=3, key_rope_theta=10000.0,
                  deduplicate_identical_pages=True)
    assert cache.total_pages < int(((lens + page - 1) // page).sum())  # shared pages are stored once
    plan = union.plan_prefix_union_decode(page_table=cache.page_table, seq_lens=cache.seq_lens, num_q_heads=q_heads,
                                          num_kv_heads=kv_heads, head_dim=dim, page_size=page, kv_layout=layout,
                                          keys_are_rotated=True)
    assert plan.launch_mode == "fallback" and plan.estimated_saved_hbm_bytes > 0
    assert int(plan.tasks_cpu[:, 1].max()) == shared_pages
    actual = union.prefix_union_decode(query, cache, plan=plan)
    expected = union.reference_prefix_union_decode(query, cache)
    torch.testing.assert_close(actual, expected, atol=1.25e-1, rtol=3e-2)
    cpu_cache = _cache_to(cache, "cpu")
    want = _device_case(query.cpu(), cpu_cache, plan.fallback_plan).oracle(oracle)
    _assert_close_to_oracle(actual, want, layout)
    assert torch.equal(union.prefix_union_decode(query, cache, force_impl="fallback").view(torch.int16),
                       actual.view(torch.int16))
    with pytest.raises(RuntimeError, match="Blackwell-class GPU for union mode"):
        union.prefix_union_decode(query, cache, plan=plan, force_impl="union")
    with pytest.raises(ValueError, match="force_impl must be one of"):
        union.prefix_union_decode(query, cache, plan=plan, force_impl="clustered")
    _status_ok()


# ---- beside the reference's own CUDA kernels ----------------------------------------------------------
@pytest.mark.skipif(not refgpu.available(), reason="oracle/_ref/libfk_reference_page_decode.so is not built")
@pytest.mark.parametrize(("layout", "clustered", "cluster_size", "rotated", "shape"), [
    ("bf16_kv", 0, 1, False, dict(batch=2, q_heads=16, kv_heads=4, head_dim=64, page_size=16, lens=[128, 117])),
    ("bf16_kv", 1, 2, False, dict(batch=2, q_heads=32, kv_heads=1, head_dim=128, page_size=32, lens=[256, 230])),
    ("int8_kv", 1, 2, False, dict(batch=2, q_heads=32, kv_heads=4, head_dim=128, page_size=32, lens=[256, 250])),
    ("fp8_kv", 1, 4, True, dict(batch=2, q_heads=32, kv_heads=4, head_dim=128, page_size=32, lens=[1024, 1000])),
    ("int8_kv", 0, 1, True, dict(batch=3, q_heads=8, kv_heads=4, head_dim=64, page_size=32, lens=[70, 33, 96])),
    ("bf16_kv", 1, 4, False, dict(batch=4, q_heads=32, kv_heads=8, head_dim=128, page_size=16, lens=[2048, 2000, 1500, 2047])),
])
def test_beside_the_reference_cuda_kernels(layout, clustered, cluster_size, rotated, shape) -> None:
    """Both kernels see the same bytes; both are compared with the fp64 oracle. The reference's
    cluster kernel rounds rotated / dequantised keys and values to bf16 before multiplying
    (clustered_page_decode.cu:522-525 there), so it is given the looser of the two bounds."""
    query, cache, plan = _random_problem(**shape, layout=layout, rotated=rotated, seed=17)
    dev = _device_case(query, cache, plan)
    want = dev.oracle(oracle)
    ours = dev.forward(pdc)
    theirs = torch.full_like(ours, float("nan"))
    refgpu.forward(query=dev.query, key_pages=dev.key_pages, value_pages=dev.value_pages, key_scales=dev.key_scales,
                   value_scales=dev.value_scales, runs=dev.runs, seq_lens=dev.seq_lens, output=theirs, batch=dev.batch,
                   num_q_heads=dev.num_q_heads, num_kv_heads=dev.num_kv_heads, head_dim=dev.head_dim,
                   page_size=dev.page_size, group_tile=plan.group_tile, use_clustered_kernel=clustered,
                   cluster_size=cluster_size, kv_format=dev.kv_format, keys_are_rotated=rotated,
                   softmax_scale=dev.softmax_scale, rope_theta=dev.rope_theta,
                   stream=int(torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    _assert_close_to_oracle(ours, want, "this library")
    _, scaled = oracle.max_abs_and_scaled_error(theirs.float().cpu().numpy().astype(np.float64), want, 2e-2, 2e-2)
    assert scaled <= 1.0, "the reference kernel is off the oracle: the oracle or the call is wrong"
    torch.testing.assert_close(ours, theirs, atol=2e-2, rtol=2e-2)
    _status_ok()
