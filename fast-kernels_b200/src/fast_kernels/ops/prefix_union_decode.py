"""Shared-prefix paged decode: the reference's Python surface for this op.

Same public names, arguments, defaults and errors as the reference's
``src/fast_kernels/ops/prefix_union_decode.py`` (``PrefixUnionDecodePlan`` :31-69,
``plan_prefix_union_decode`` :155-343, ``prefix_union_decode`` :346-451,
``estimate_prefix_union_decode_metrics`` :454-466, ``reference_prefix_union_decode`` :469-483).

The planner groups requests whose page tables begin with the same physical pages (a prompt prefix
stored once) and emits the reference's four descriptor tables -- tasks, shared pages, tail pages,
consumers -- with the same rows in the same order.

Which kernel runs: the reference's union kernel refuses devices below compute capability 12
(``csrc/kernels/prefix_union_decode/prefix_union_decode.cu:843-846`` there) and its planner picks
``launch_mode = "fallback"`` on them (:322-324), so on a B200 (10.0) the reference ALWAYS computes
this op with ``clustered_page_decode`` on the plan's ``fallback_plan``, and ``force_impl="union"``
raises. This module does exactly that, over this build's paged-KV decode kernel; no separate union
kernel is built.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Literal

from fast_kernels.ops.clustered_page_decode import (
    ClusteredPageDecodePlan,
    PagedKVCache,
    _check_cuda_tensor,
    _check_same_cuda_device,
    _require_layout,
    _torch,
    clustered_page_decode,
    cuda_clustered_decode_available,
    estimate_page_decode_metrics,
    plan_clustered_page_decode,
    reference_clustered_page_decode,
)

FORCE_IMPLS = {"auto", "union", "fallback"}
DEFAULT_MIN_SHARED_PAGES = 2
DEFAULT_MIN_CONSUMERS = 2
_PLAN_CACHE: dict[tuple[Any, ...], "PrefixUnionDecodePlan"] = {}

# Row formats of the descriptor tables (int32), as the reference's kernel reads them:
#   tasks        [shared_page_offset, shared_page_count, consumer_offset, consumer_count, kv_head, 0, 0, 0]
#   shared_pages [physical page, valid tokens]
#   tail_pages   [physical page, valid tokens | logical page << 16]
#   consumers    [query row, output row, tail_page_offset, query position, tail page count, 0, 0, 0]
_TASK_WIDTH, _PAGE_WIDTH, _CONSUMER_WIDTH = 8, 2, 8


@dataclass(slots=True)
class PrefixUnionDecodePlan:
    batch: int
    page_size: int
    num_q_heads: int
    num_kv_heads: int
    head_dim: int
    kv_layout: Literal["bf16_kv", "fp8_kv", "int8_kv"]
    cluster_size: int
    min_shared_pages: int
    min_consumers: int
    launch_mode: Literal["union", "fallback"]
    estimated_saved_hbm_bytes: int
    tasks_cpu: Any
    shared_pages_cpu: Any
    tail_pages_cpu: Any
    consumers_cpu: Any
    fallback_plan: ClusteredPageDecodePlan
    _device_cache: dict[str, dict[str, Any]] = field(default_factory=dict, repr=False)

    @property
    def num_tasks(self) -> int:
        return int(self.tasks_cpu.shape[0])

    def device_tensors(self, device: Any) -> dict[str, Any]:
        torch = _torch()
        key = str(device)
        if key not in self._device_cache:
            tables = {"tasks": self.tasks_cpu, "shared_pages": self.shared_pages_cpu,
                      "tail_pages": self.tail_pages_cpu, "consumers": self.consumers_cpu}
            tensors = {name: table.to(device=device, dtype=torch.int32) for name, table in tables.items()}
            tensors["scheduler_counter"] = torch.zeros((1,), device=device, dtype=torch.int32)
            self._device_cache[key] = tensors
        return self._device_cache[key]


def cuda_prefix_union_decode_available() -> bool:
    return cuda_clustered_decode_available()


def _union_kernel_supported() -> bool:
    """The reference's rule: compute capability 12 and up (`_is_blackwell_device`, :147-152 there)."""
    torch = _torch()
    return bool(torch.cuda.is_available()) and int(torch.cuda.get_device_capability(torch.device("cuda"))[0]) >= 12


def _table(rows: list[list[int]], width: int) -> Any:
    torch = _torch()
    if not rows:
        return torch.empty((0, width), dtype=torch.int32)
    return torch.tensor(rows, dtype=torch.int32).reshape(len(rows), width).contiguous()


def _shared_page_bytes(page_size: int, head_dim: int, kv_layout: str) -> int:
    """Bytes of one page of one kv head, keys + values + their scales."""
    if kv_layout == "bf16_kv":
        return 2 * page_size * head_dim * 2
    blocks = head_dim // 64
    return 2 * page_size * head_dim + 4 * blocks * (1 + page_size)


def _longest_shared_prefixes(pages_of: list[tuple[int, ...]], min_pages: int, min_requests: int) -> list[tuple[int, ...]]:
    """For every request the longest prefix of its page list (at least `min_pages` pages) that at
    least `min_requests` requests begin with; () if there is none."""
    population: dict[tuple[int, ...], int] = {}
    for pages in pages_of:
        for length in range(min_pages, len(pages) + 1):
            population[pages[:length]] = population.get(pages[:length], 0) + 1
    chosen = []
    for pages in pages_of:
        length = len(pages)
        while length >= min_pages and population.get(pages[:length], 0) < min_requests:
            length -= 1
        chosen.append(pages[:length] if length >= min_pages else ())
    return chosen


def plan_prefix_union_decode(
    *,
    page_table: Any,
    seq_lens: Any,
    num_q_heads: int,
    num_kv_heads: int,
    head_dim: int,
    page_size: int,
    kv_layout: str,
    keys_are_rotated: bool,
    cluster_size: int | None = None,
    min_shared_pages: int = DEFAULT_MIN_SHARED_PAGES,
    min_consumers: int = DEFAULT_MIN_CONSUMERS,
    use_cache: bool = True,
) -> PrefixUnionDecodePlan:
    torch = _torch()
    layout = _require_layout(kv_layout)
    table_cpu = page_table.to(device="cpu", dtype=torch.int32).contiguous()
    lens_cpu = seq_lens.to(device="cpu", dtype=torch.int32).contiguous()
    if table_cpu.ndim != 2:
        raise ValueError("page_table must be a 2D int tensor")
    if lens_cpu.ndim != 1 or int(lens_cpu.shape[0]) != int(table_cpu.shape[0]):
        raise ValueError("seq_lens must be a 1D tensor with one entry per request")
    if num_q_heads % num_kv_heads != 0:
        raise ValueError("num_q_heads must be divisible by num_kv_heads")
    if head_dim not in {64, 128}:
        raise ValueError("head_dim must be 64 or 128")
    if page_size not in {16, 32}:
        raise ValueError("page_size must be 16 or 32")
    if min_shared_pages < 1:
        raise ValueError("min_shared_pages must be >= 1")
    if min_consumers < 2:
        raise ValueError("min_consumers must be >= 2")

    lens = [int(v) for v in lens_cpu.tolist()]
    rows = table_cpu.tolist()
    cache_key = (tuple(lens), tuple(tuple(row) for row in rows), num_q_heads, num_kv_heads, head_dim, page_size,
                 layout, int(keys_are_rotated), min_shared_pages, min_consumers, cluster_size)
    if use_cache and cache_key in _PLAN_CACHE:
        return _PLAN_CACHE[cache_key]

    batch = len(lens)
    group_size = num_q_heads // num_kv_heads
    page_counts = [(length + page_size - 1) // page_size for length in lens]
    pages_of = [tuple(int(v) for v in rows[r][: page_counts[r]]) for r in range(batch)]
    # tokens that count in page `slot` of request r: a full page, except the last one
    tokens_of = [[page_size if slot < page_counts[r] - 1 else max(0, lens[r] - slot * page_size)
                  for slot in range(page_counts[r])] for r in range(batch)]
    prefixes = _longest_shared_prefixes(pages_of, min_shared_pages, min_consumers)

    # one task per (kv head, prefix); the requests of a task in request order; tasks with the most
    # shared pages x requests first (ties: more requests, then the higher kv head -- a stable
    # descending sort, so equal keys keep the order in which the groups were first seen)
    members: dict[tuple[int, tuple[int, ...]], list[int]] = {}
    for request, prefix in enumerate(prefixes):
        for kv_head in range(num_kv_heads):
            members.setdefault((kv_head, prefix), []).append(request)
    ordered = sorted(members.items(), key=lambda item: (len(item[0][1]) * len(item[1]), len(item[1]), item[0][0]),
                     reverse=True)

    tasks: list[list[int]] = []
    shared: list[list[int]] = []
    tails: list[list[int]] = []
    consumers: list[list[int]] = []
    saved_bytes = 0
    page_bytes = _shared_page_bytes(page_size, head_dim, layout)
    for (kv_head, prefix), requests in ordered:
        first_shared, first_consumer = len(shared), len(consumers)
        shared += [[page, tokens_of[requests[0]][slot]] for slot, page in enumerate(prefix)]
        for request in requests:
            tail_slots = range(len(prefix), page_counts[request])
            for q_head in range(kv_head * group_size, (kv_head + 1) * group_size):
                row = request * num_q_heads + q_head
                consumers.append([row, row, len(tails), max(0, lens[request] - 1), len(tail_slots), 0, 0, 0])
                tails += [[pages_of[request][slot], tokens_of[request][slot] | (slot << 16)] for slot in tail_slots]
        count = len(consumers) - first_consumer
        tasks.append([first_shared, len(prefix), first_consumer, count, kv_head, 0, 0, 0])
        if prefix and count > 1:
            saved_bytes += (count - 1) * len(prefix) * page_bytes

    chosen_cluster = 1 if cluster_size is None else int(cluster_size)
    if chosen_cluster not in {1, 2, 4, 8}:
        raise ValueError("cluster_size must be one of {1, 2, 4, 8}")
    fallback_plan = plan_clustered_page_decode(
        page_table=table_cpu, seq_lens=lens_cpu, num_q_heads=num_q_heads, num_kv_heads=num_kv_heads,
        head_dim=head_dim, page_size=page_size, kv_layout=layout, cluster_size=cluster_size, use_cache=use_cache)
    union = bool(keys_are_rotated) and _union_kernel_supported() and saved_bytes > 0
    plan = PrefixUnionDecodePlan(
        batch=batch, page_size=page_size, num_q_heads=num_q_heads, num_kv_heads=num_kv_heads, head_dim=head_dim,
        kv_layout=layout, cluster_size=chosen_cluster, min_shared_pages=min_shared_pages, min_consumers=min_consumers,
        launch_mode="union" if union else "fallback", estimated_saved_hbm_bytes=saved_bytes,
        tasks_cpu=_table(tasks, _TASK_WIDTH), shared_pages_cpu=_table(shared, _PAGE_WIDTH),
        tail_pages_cpu=_table(tails, _PAGE_WIDTH), consumers_cpu=_table(consumers, _CONSUMER_WIDTH),
        fallback_plan=fallback_plan)
    if use_cache:
        _PLAN_CACHE[cache_key] = plan
    return plan


def prefix_union_decode(
    query: Any,
    cache: PagedKVCache,
    *,
    plan: PrefixUnionDecodePlan | None = None,
    output: Any | None = None,
    softmax_scale: float | None = None,
    rope_theta: float = 10000.0,
    force_impl: str = "auto",
) -> Any:
    torch = _torch()
    if force_impl not in FORCE_IMPLS:
        raise ValueError(f"force_impl must be one of {sorted(FORCE_IMPLS)}")
    _check_cuda_tensor(query, name="query", dtype=torch.bfloat16, ndim=3)
    _check_same_cuda_device(("query", query), ("key_pages", cache.key_pages), ("value_pages", cache.value_pages),
                            ("key_scales", cache.key_scales), ("value_scales", cache.value_scales))
    num_q_heads, head_dim = int(query.shape[1]), int(query.shape[2])
    if num_q_heads % cache.num_kv_heads != 0:
        raise ValueError("query head count must be divisible by cache.num_kv_heads")
    if head_dim != cache.head_dim:
        raise ValueError("query head_dim must match cache head_dim")
    if plan is None:
        plan = plan_prefix_union_decode(
            page_table=cache.page_table, seq_lens=cache.seq_lens, num_q_heads=num_q_heads,
            num_kv_heads=cache.num_kv_heads, head_dim=head_dim, page_size=cache.page_size,
            kv_layout=cache.kv_layout, keys_are_rotated=cache.keys_are_rotated)
    if output is None:
        output = torch.empty_like(query)
    _check_cuda_tensor(output, name="output", dtype=torch.bfloat16, ndim=3)

    if force_impl == "union" or (force_impl == "auto" and plan.launch_mode == "union"):
        # the reference's checks, in its order (:394-412 there); the last one always fires here
        if not cache.keys_are_rotated:
            raise ValueError("prefix_union_decode requires pre-rotated key pages for the union path")
        if cache.key_rope_theta is None:
            raise ValueError("rotated key caches must record key_rope_theta")
        if float(cache.key_rope_theta) != float(rope_theta):
            raise ValueError("rope_theta must match the key_rope_theta used to build the cache")
        raise RuntimeError("prefix_union_decode requires a Blackwell-class GPU for union mode")
    return clustered_page_decode(query, cache, plan=plan.fallback_plan, output=output, softmax_scale=softmax_scale,
                                 rope_theta=rope_theta, force_impl="auto")


def estimate_prefix_union_decode_metrics(cache: PagedKVCache, plan: PrefixUnionDecodePlan) -> dict[str, float]:
    metrics = dict(estimate_page_decode_metrics(cache, plan.fallback_plan))
    saved_per_token = float(plan.estimated_saved_hbm_bytes) / max(1.0, float(plan.batch))
    metrics["hbm_bytes_per_token"] = max(0.0, metrics["hbm_bytes_per_token"] - saved_per_token)
    metrics["workspace_bytes_per_token"] = 0.0
    metrics["dsm_bytes_per_token"] = float(plan.cluster_size * plan.page_size * plan.head_dim * 4 * 2)
    metrics["estimated_saved_hbm_bytes"] = float(plan.estimated_saved_hbm_bytes)
    return metrics


def reference_prefix_union_decode(
    query: Any,
    cache: PagedKVCache,
    *,
    softmax_scale: float | None = None,
    rope_theta: float = 10000.0,
    output: Any | None = None,
) -> Any:
    """Sharing a prefix does not change the mathematics: the PyTorch reference of the paged decode."""
    return reference_clustered_page_decode(query, cache, softmax_scale=softmax_scale, rope_theta=rope_theta,
                                           output=output)

