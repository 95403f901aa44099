"""Paged-KV decode attention: the reference's Python surface for this op, over the sm_100a kernel.

Same public names, arguments, defaults and errors as the reference's
``src/fast_kernels/ops/clustered_page_decode.py`` (``PagedKVCache`` :21-40,
``ClusteredPageDecodePlan`` :43-87, ``pack_paged_kv_bf16`` :344-421, ``quantize_paged_kv_int8`` /
``_fp8`` :478-559, ``plan_clustered_page_decode`` :593-708, ``clustered_page_decode`` :715-811,
``reference_clustered_page_decode`` :857-903, ``estimate_page_decode_metrics`` :906-927), so a
caller of that module can import this one instead. The host-side preparation here is written with
whole-tensor operations instead of per-page Python loops and produces the same bytes: pages in
request order, zero past a request's last token, optionally spread over physical slots by a seeded
permutation, optionally with identical pages stored once.

Layouts: keys / values ``[pages, kv_heads, page_size, head_dim]`` as bf16, e4m3 (``uint8``
storage) or int8; quantised keys carry one fp32 scale per (page, kv head, 64-dim block), values one
per (page, kv head, token, 64-dim block).

The compute path is the CUDA library only (``fast_kernels._native``); without it the op raises.
``reference_clustered_page_decode`` is the plain PyTorch statement of the same attention, for tests
and for the benchmark's baseline column.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any, Literal

from fast_kernels.native import native_build_info, native_module

KV_LAYOUTS = {"bf16_kv", "fp8_kv", "int8_kv"}
KV_FORMAT_IDS = {"bf16_kv": 0, "fp8_kv": 1, "int8_kv": 2}
FORCE_IMPLS = {"auto", "direct", "clustered"}
DEFAULT_DIRECT_PAGE_THRESHOLD = 4
DEFAULT_PDL_PAGE_THRESHOLD = 256
_SCALE_BLOCK = 64
_PLAN_CACHE: dict[tuple[Any, ...], "ClusteredPageDecodePlan"] = {}

KvLayout = Literal["bf16_kv", "fp8_kv", "int8_kv"]


def _torch() -> Any:
    try:
        import torch
    except ImportError as exc:  # pragma: no cover
        raise RuntimeError("PyTorch is required for clustered_page_decode ops") from exc
    return torch


@dataclass(slots=True, frozen=True)
class PagedKVCache:
    key_pages: Any
    value_pages: Any
    page_table: Any
    seq_lens: Any
    key_scales: Any | None
    value_scales: Any | None
    reference_key_pages: Any
    reference_value_pages: Any
    kv_layout: KvLayout
    page_size: int
    num_kv_heads: int
    head_dim: int
    keys_are_rotated: bool = False
    key_rope_theta: float | None = None

    @property
    def total_pages(self) -> int:
        return int(self.key_pages.shape[0])


@dataclass(slots=True)
class ClusteredPageDecodePlan:
    batch: int
    page_size: int
    num_q_heads: int
    num_kv_heads: int
    head_dim: int
    kv_layout: KvLayout
    max_pages: int
    group_tile: int
    q_head_tiles: int
    cluster_size: int
    direct_page_threshold: int
    pdl_page_threshold: int
    launch_mode: Literal["direct", "clustered"]
    run_base_pages_cpu: Any
    run_page_counts_cpu: Any
    run_logical_starts_cpu: Any
    run_last_page_lens_cpu: Any
    request_run_offsets_cpu: Any
    seq_lens_cpu: Any
    _device_cache: dict[str, dict[str, Any]] = field(default_factory=dict, repr=False)

    @property
    def num_runs(self) -> int:
        return int(self.run_base_pages_cpu.shape[0])

    def device_tensors(self, device: Any) -> dict[str, Any]:
        """The six descriptor arrays as int32 tensors on `device`, uploaded once per device."""
        torch = _torch()
        key = str(device)
        if key not in self._device_cache:
            host = {
                "run_base_pages": self.run_base_pages_cpu,
                "run_page_counts": self.run_page_counts_cpu,
                "run_logical_starts": self.run_logical_starts_cpu,
                "run_last_page_lens": self.run_last_page_lens_cpu,
                "request_run_offsets": self.request_run_offsets_cpu,
                "seq_lens": self.seq_lens_cpu,
            }
            self._device_cache[key] = {
                name: tensor.to(device=device, dtype=torch.int32) for name, tensor in host.items()
            }
        return self._device_cache[key]


def cuda_clustered_decode_available() -> bool:
    info = native_build_info()
    return bool(info.get("available", False)) and bool(info.get("compiled_with_cuda", False))


def _require_cuda_backend() -> Any:
    if not cuda_clustered_decode_available():
        raise RuntimeError("fast-kernels native module was built without CUDA support")
    return native_module()


def _require_layout(layout: str) -> KvLayout:
    if layout not in KV_LAYOUTS:
        raise ValueError(f"layout must be one of {sorted(KV_LAYOUTS)}")
    return layout  # type: ignore[return-value]


def _layout_id(layout: str) -> int:
    if layout not in KV_FORMAT_IDS:
        raise ValueError(f"unsupported kv layout: {layout}")
    return KV_FORMAT_IDS[layout]


def _check_cuda_tensor(tensor: Any, *, name: str, dtype: Any, ndim: int) -> None:
    torch = _torch()
    if not isinstance(tensor, torch.Tensor):
        raise TypeError(f"{name} must be a torch.Tensor")
    if tensor.ndim != ndim:
        raise ValueError(f"{name} must be {ndim}D")
    if tensor.dtype != dtype:
        raise TypeError(f"{name} must have dtype {dtype}")
    if not tensor.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor")
    if not tensor.is_contiguous():
        raise ValueError(f"{name} must be contiguous")


def _check_same_cuda_device(*named: tuple[str, Any]) -> None:
    present = [(name, tensor) for name, tensor in named if tensor is not None]
    if len({tensor.device for _, tensor in present}) > 1:
        summary = ", ".join(f"{name}={tensor.device}" for name, tensor in present)
        raise ValueError(f"all CUDA tensors must be on the same device: {summary}")


def _pages_per_request(seq_lens: Any, page_size: int) -> Any:
    return (seq_lens + (page_size - 1)) // page_size


# ---------------------------------------------------------------------------------------------
# rotary embedding (Llama pairing: dimensions 2i and 2i+1 turn by position * theta^(-2i/d))
# ---------------------------------------------------------------------------------------------
def _apply_llama_rope_torch(x: Any, positions: Any, rope_theta: float) -> Any:
    torch = _torch()
    head_dim = int(x.shape[-1])
    half = head_dim // 2
    exponent = -2.0 * torch.arange(half, device=x.device, dtype=torch.float32) / head_dim
    inv_freq = rope_theta**exponent
    angle = positions.to(device=x.device, dtype=torch.float32)[..., None] * inv_freq
    cos, sin = torch.cos(angle), torch.sin(angle)
    pairs = x.to(torch.float32).reshape(*x.shape[:-1], half, 2)
    even, odd = pairs[..., 0], pairs[..., 1]
    return torch.stack((even * cos - odd * sin, even * sin + odd * cos), dim=-1).reshape_as(x)


def _rotate_dense_keys(keys: Any, rope_theta: float) -> Any:
    """Every token of every request rotated by its own position (tokens past a request's length
    never reach a page, so rotating them too changes nothing)."""
    torch = _torch()
    positions = torch.arange(int(keys.shape[2]), device=keys.device, dtype=torch.float32)
    return _apply_llama_rope_torch(keys, positions, rope_theta).to(keys.dtype)


# ---------------------------------------------------------------------------------------------
# dense [batch, kv_heads, seq, dim] -> pages
# ---------------------------------------------------------------------------------------------
def _logical_pages(dense: Any, seq_lens_cpu: Any, page_size: int) -> Any:
    """Pages in request order, ceil(len / page_size) per request, zero past the last token."""
    torch = _torch()
    batch, heads, seq, dim = (int(v) for v in dense.shape)
    counts = _pages_per_request(seq_lens_cpu, page_size).to(torch.int64)
    max_pages = max(int(counts.max().item()) if batch else 0, (seq + page_size - 1) // page_size)
    padded = torch.zeros((batch, heads, max_pages * page_size, dim), device=dense.device, dtype=dense.dtype)
    padded[:, :, :seq] = dense
    lens = seq_lens_cpu.to(device=dense.device, dtype=torch.int64)
    token = torch.arange(max_pages * page_size, device=dense.device)
    padded.masked_fill_((token[None, :] >= lens[:, None])[:, None, :, None], 0)  # +0.0, whatever was there
    paged = padded.reshape(batch, heads, max_pages, page_size, dim).permute(0, 2, 1, 3, 4)
    keep = torch.arange(max_pages)[None, :] < counts[:, None]
    return paged[keep.to(dense.device)].contiguous()


def _first_occurrence_ids(key_pages: Any, value_pages: Any) -> tuple[Any, Any]:
    """(indices of the pages that are the first of their content, page -> index into those)."""
    import numpy as np

    torch = _torch()
    total = int(key_pages.shape[0])
    if total == 0:
        empty = torch.empty((0,), dtype=torch.int64)
        return empty, empty
    rows = torch.cat(
        (key_pages.contiguous().view(torch.uint8).reshape(total, -1),
         value_pages.contiguous().view(torch.uint8).reshape(total, -1)), dim=1,
    ).cpu().numpy()
    _, first, inverse = np.unique(rows, axis=0, return_index=True, return_inverse=True)
    order = np.argsort(first, kind="stable")  # number the distinct pages by first appearance
    rank = np.empty_like(order)
    rank[order] = np.arange(order.size)
    return torch.from_numpy(first[order].astype(np.int64)), torch.from_numpy(rank[inverse.reshape(-1)].astype(np.int64))


def _page_table(seq_lens_cpu: Any, page_size: int, logical_to_stored: Any, stored_pages: int,
                fragment_pages: bool, seed: int | None, device: Any) -> tuple[Any, Any]:
    """(page_table [batch, max_pages] int32 with -1 padding, physical slot -> stored page)."""
    torch = _torch()
    batch = int(seq_lens_cpu.shape[0])
    counts = _pages_per_request(seq_lens_cpu, page_size).to(torch.int64)
    max_pages = int(counts.max().item()) if batch else 0
    table = torch.full((batch, max_pages), -1, dtype=torch.int32)
    if stored_pages == 0:
        return table, torch.empty((0,), device=device, dtype=torch.int64)
    if fragment_pages:
        generator = torch.Generator(device=device)
        if seed is not None:
            generator.manual_seed(seed)
        slot_to_stored = torch.randperm(stored_pages, generator=generator, device=device)
        stored_to_slot = torch.empty_like(slot_to_stored)
        stored_to_slot[slot_to_stored] = torch.arange(stored_pages, device=device)
    else:
        slot_to_stored = torch.arange(stored_pages, device=device)
        stored_to_slot = slot_to_stored
    physical = stored_to_slot[logical_to_stored.to(device)].to(device="cpu", dtype=torch.int32)
    keep = torch.arange(max_pages)[None, :] < counts[:, None]
    table[keep] = physical
    return table, slot_to_stored.to(torch.int64)


def pack_paged_kv_bf16(
    keys: Any,
    values: Any,
    seq_lens: Any,
    *,
    page_size: int,
    fragment_pages: bool = True,
    seed: int | None = None,
    key_rope_theta: float | None = None,
    deduplicate_identical_pages: bool = False,
) -> PagedKVCache:
    torch = _torch()
    if keys.ndim != 4 or values.ndim != 4:
        raise ValueError("keys and values must be 4D tensors shaped [batch, kv_heads, seq, head_dim]")
    if keys.shape != values.shape:
        raise ValueError("keys and values must share the same shape")
    if page_size not in {16, 32}:
        raise ValueError("page_size must be 16 or 32")
    if seq_lens.ndim != 1 or int(seq_lens.shape[0]) != int(keys.shape[0]):
        raise ValueError("seq_lens must be 1D with one length per request")

    seq_lens_cpu = seq_lens.to(device="cpu", dtype=torch.int32).contiguous()
    keys_bf16 = keys.to(torch.bfloat16).contiguous()
    values_bf16 = values.to(torch.bfloat16).contiguous()
    if key_rope_theta is not None:
        keys_bf16 = _rotate_dense_keys(keys_bf16, float(key_rope_theta))
    key_pages = _logical_pages(keys_bf16, seq_lens_cpu, page_size)
    value_pages = _logical_pages(values_bf16, seq_lens_cpu, page_size)
    total = int(key_pages.shape[0])
    if deduplicate_identical_pages:
        firsts, logical_to_stored = _first_occurrence_ids(key_pages, value_pages)
        firsts = firsts.to(key_pages.device)
        key_pages, value_pages = key_pages[firsts].contiguous(), value_pages[firsts].contiguous()
    else:
        logical_to_stored = torch.arange(total, dtype=torch.int64)
    table, slot_to_stored = _page_table(seq_lens_cpu, page_size, logical_to_stored, int(key_pages.shape[0]),
                                        fragment_pages, seed, keys_bf16.device)
    if int(slot_to_stored.numel()):
        key_pages = key_pages.index_select(0, slot_to_stored).contiguous()
        value_pages = value_pages.index_select(0, slot_to_stored).contiguous()
    return PagedKVCache(
        key_pages=key_pages,
        value_pages=value_pages,
        page_table=table.contiguous(),
        seq_lens=seq_lens_cpu,
        key_scales=None,
        value_scales=None,
        reference_key_pages=key_pages,
        reference_value_pages=value_pages,
        kv_layout="bf16_kv",
        page_size=page_size,
        num_kv_heads=int(keys.shape[1]),
        head_dim=int(keys.shape[3]),
        keys_are_rotated=key_rope_theta is not None,
        key_rope_theta=None if key_rope_theta is None else float(key_rope_theta),
    )


# ---------------------------------------------------------------------------------------------
# 8-bit pages: symmetric scales per 64-dim block (keys: over the page's tokens too)
# ---------------------------------------------------------------------------------------------
def _block_scales(pages: Any, limit: float) -> tuple[Any, Any, Any]:
    torch = _torch()
    blocks = pages.float().reshape(*pages.shape[:-1], int(pages.shape[-1]) // _SCALE_BLOCK, _SCALE_BLOCK)
    magnitude = blocks.abs()
    key_scales = torch.clamp(magnitude.amax(dim=(-3, -1)) / limit, min=1e-6)  # [pages, heads, blocks]
    value_scales = torch.clamp(magnitude.amax(dim=-1) / limit, min=1e-6)      # [pages, heads, tokens, blocks]
    return blocks, key_scales, value_scales


def _quantize_kv_int8(key_pages: Any, value_pages: Any) -> tuple[Any, Any, Any, Any]:
    torch = _torch()

    def to_int8(blocks: Any, scale: Any, like: Any) -> Any:
        return torch.clamp(torch.round(blocks / scale), min=-127, max=127).to(torch.int8).reshape_as(like).contiguous()

    key_blocks, key_scales, _ = _block_scales(key_pages, 127.0)
    value_blocks, _, value_scales = _block_scales(value_pages, 127.0)
    return (to_int8(key_blocks, key_scales[:, :, None, :, None], key_pages),
            to_int8(value_blocks, value_scales[..., None], value_pages),
            key_scales.contiguous(), value_scales.contiguous())


def _require_fp8_dtype() -> Any:
    torch = _torch()
    if not hasattr(torch, "float8_e4m3fn"):
        raise RuntimeError("This PyTorch build does not expose torch.float8_e4m3fn")
    return torch.float8_e4m3fn


def _quantize_kv_fp8(key_pages: Any, value_pages: Any) -> tuple[Any, Any, Any, Any]:
    torch = _torch()
    fp8 = _require_fp8_dtype()

    def to_fp8(blocks: Any, scale: Any, like: Any) -> Any:
        return (blocks / scale).to(fp8).view(torch.uint8).reshape_as(like).contiguous()

    key_blocks, key_scales, _ = _block_scales(key_pages, 448.0)
    value_blocks, _, value_scales = _block_scales(value_pages, 448.0)
    return (to_fp8(key_blocks, key_scales[:, :, None, :, None], key_pages),
            to_fp8(value_blocks, value_scales[..., None], value_pages),
            key_scales.contiguous(), value_scales.contiguous())


def _quantized_cache(packed: PagedKVCache, layout: KvLayout, quantize: Any) -> PagedKVCache:
    key_bytes, value_bytes, key_scales, value_scales = quantize(packed.reference_key_pages,
                                                                packed.reference_value_pages)
    return PagedKVCache(
        key_pages=key_bytes,
        value_pages=value_bytes,
        page_table=packed.page_table,
        seq_lens=packed.seq_lens,
        key_scales=key_scales,
        value_scales=value_scales,
        reference_key_pages=packed.reference_key_pages,
        reference_value_pages=packed.reference_value_pages,
        kv_layout=layout,
        page_size=packed.page_size,
        num_kv_heads=packed.num_kv_heads,
        head_dim=packed.head_dim,
        keys_are_rotated=packed.keys_are_rotated,
        key_rope_theta=packed.key_rope_theta,
    )


def quantize_paged_kv_int8(keys: Any, values: Any, seq_lens: Any, *, page_size: int, fragment_pages: bool = True,
                           seed: int | None = None, key_rope_theta: float | None = None,
                           deduplicate_identical_pages: bool = False) -> PagedKVCache:
    packed = pack_paged_kv_bf16(keys, values, seq_lens, page_size=page_size, fragment_pages=fragment_pages,
                                seed=seed, key_rope_theta=key_rope_theta,
                                deduplicate_identical_pages=deduplicate_identical_pages)
    return _quantized_cache(packed, "int8_kv", _quantize_kv_int8)


def quantize_paged_kv_fp8(keys: Any, values: Any, seq_lens: Any, *, page_size: int, fragment_pages: bool = True,
                          seed: int | None = None, key_rope_theta: float | None = None,
                          deduplicate_identical_pages: bool = False) -> PagedKVCache:
    packed = pack_paged_kv_bf16(keys, values, seq_lens, page_size=page_size, fragment_pages=fragment_pages,
                                seed=seed, key_rope_theta=key_rope_theta,
                                deduplicate_identical_pages=deduplicate_identical_pages)
    return _quantized_cache(packed, "fp8_kv", _quantize_kv_fp8)


# ---------------------------------------------------------------------------------------------
# plan: page table -> runs of physically consecutive pages
# ---------------------------------------------------------------------------------------------
def _default_group_tile(group_size: int) -> int:
    for tile in (1, 2, 4):
        if group_size <= tile:
            return tile
    return 8


def _default_cluster_size(max_pages: int, direct_page_threshold: int, group_size: int) -> int:
    """The reference's table (ops/clustered_page_decode.py:572-590 there), kept so that plans
    carry the same numbers. On this build the value is a hint: 1 = one block per (request, kv
    head, head tile), more = the launcher cuts the pages over as many blocks as fill the device."""
    torch = _torch()
    if max_pages <= direct_page_threshold or not torch.cuda.is_available():
        return 1
    major, _minor = torch.cuda.get_device_capability(torch.device("cuda"))
    if major >= 12:
        if max_pages >= 192:
            return 4
        if max_pages >= 128:
            return 2 if group_size > 8 else 4
        return 2 if max_pages >= 64 else 1
    if major >= 9:
        if max_pages >= 128:
            return 4 if group_size >= 8 else 2
        return 2 if group_size >= 8 and max_pages >= 64 else 1
    return 1


def plan_clustered_page_decode(
    *,
    page_table: Any,
    seq_lens: Any,
    num_q_heads: int,
    num_kv_heads: int,
    head_dim: int,
    page_size: int,
    kv_layout: str,
    cluster_size: int | None = None,
    direct_page_threshold: int = DEFAULT_DIRECT_PAGE_THRESHOLD,
    pdl_page_threshold: int = DEFAULT_PDL_PAGE_THRESHOLD,
    use_cache: bool = True,
) -> ClusteredPageDecodePlan:
    import numpy as np

    torch = _torch()
    layout = _require_layout(kv_layout)
    seq_lens_cpu = seq_lens.to(device="cpu", dtype=torch.int32).contiguous()
    table_cpu = page_table.to(device="cpu", dtype=torch.int32).contiguous()
    if table_cpu.ndim != 2:
        raise ValueError("page_table must be a 2D int tensor")
    if seq_lens_cpu.ndim != 1 or int(seq_lens_cpu.shape[0]) != int(table_cpu.shape[0]):
        raise ValueError("seq_lens must be a 1D tensor with one entry per request")
    if num_q_heads % num_kv_heads != 0:
        raise ValueError("num_q_heads must be divisible by num_kv_heads")
    if head_dim not in {64, 128}:
        raise ValueError("head_dim must be 64 or 128")
    if page_size not in {16, 32}:
        raise ValueError("page_size must be 16 or 32")

    batch = int(table_cpu.shape[0])
    lens = seq_lens_cpu.numpy().astype(np.int64)
    pages = (lens + page_size - 1) // page_size
    max_pages = int(pages.max())
    group_size = num_q_heads // num_kv_heads
    group_tile = _default_group_tile(group_size)
    chosen_cluster = (_default_cluster_size(max_pages, direct_page_threshold, group_size)
                      if cluster_size is None else int(cluster_size))
    launch_mode: Literal["direct", "clustered"] = (
        "clustered" if group_size > 8 or max_pages > direct_page_threshold else "direct")

    table = table_cpu.numpy()
    cache_key = (lens.tobytes(), table.tobytes(), table.shape, num_q_heads, num_kv_heads, head_dim, page_size,
                 layout, group_tile, chosen_cluster, direct_page_threshold, pdl_page_threshold)
    if use_cache and cache_key in _PLAN_CACHE:
        return _PLAN_CACHE[cache_key]

    bases: list[np.ndarray] = []
    counts: list[np.ndarray] = []
    starts: list[np.ndarray] = []
    lasts: list[np.ndarray] = []
    offsets = [0]
    for request in range(batch):
        n = int(pages[request])
        if n > 0:
            row = table[request, :n].astype(np.int64)
            # a new run begins wherever a page does not follow its predecessor physically
            begin = np.concatenate(([0], np.flatnonzero(np.diff(row) != 1) + 1))
            length = np.diff(np.concatenate((begin, [n])))
            last = np.full(begin.shape, page_size, dtype=np.int64)
            last[-1] = (int(lens[request]) - 1) % page_size + 1
            bases.append(row[begin])
            counts.append(length)
            starts.append(begin)
            lasts.append(last)
            offsets.append(offsets[-1] + int(begin.size))
        else:
            offsets.append(offsets[-1])

    def as_tensor(parts: list[np.ndarray]) -> Any:
        joined = np.concatenate(parts) if parts else np.empty((0,), dtype=np.int64)
        return torch.from_numpy(joined.astype(np.int32))

    plan = ClusteredPageDecodePlan(
        batch=batch,
        page_size=page_size,
        num_q_heads=num_q_heads,
        num_kv_heads=num_kv_heads,
        head_dim=head_dim,
        kv_layout=layout,
        max_pages=max_pages,
        group_tile=group_tile,
        q_head_tiles=int(math.ceil(group_size / group_tile)),
        cluster_size=chosen_cluster,
        direct_page_threshold=direct_page_threshold,
        pdl_page_threshold=pdl_page_threshold,
        launch_mode=launch_mode,
        run_base_pages_cpu=as_tensor(bases),
        run_page_counts_cpu=as_tensor(counts),
        run_logical_starts_cpu=as_tensor(starts),
        run_last_page_lens_cpu=as_tensor(lasts),
        request_run_offsets_cpu=torch.tensor(offsets, dtype=torch.int32),
        seq_lens_cpu=seq_lens_cpu,
    )
    if use_cache:
        _PLAN_CACHE[cache_key] = plan
    return plan


# ---------------------------------------------------------------------------------------------
# the op
# ---------------------------------------------------------------------------------------------
def clustered_page_decode(
    query: Any,
    cache: PagedKVCache,
    *,
    plan: ClusteredPageDecodePlan | None = None,
    output: Any | None = None,
    softmax_scale: float | None = None,
    rope_theta: float = 10000.0,
    force_impl: str = "auto",
) -> Any:
    torch = _torch()
    native = _require_cuda_backend()
    if force_impl not in FORCE_IMPLS:
        raise ValueError(f"force_impl must be one of {sorted(FORCE_IMPLS)}")
    _check_cuda_tensor(query, name="query", dtype=torch.bfloat16, ndim=3)
    _check_same_cuda_device(("query", query), ("key_pages", cache.key_pages), ("value_pages", cache.value_pages))
    batch, num_q_heads, head_dim = (int(v) for v in query.shape)
    if num_q_heads % cache.num_kv_heads != 0:
        raise ValueError("query head count must be divisible by cache.num_kv_heads")
    if head_dim != cache.head_dim:
        raise ValueError("query head_dim must match cache head_dim")
    if plan is None:
        plan = plan_clustered_page_decode(
            page_table=cache.page_table, seq_lens=cache.seq_lens, num_q_heads=num_q_heads,
            num_kv_heads=cache.num_kv_heads, head_dim=head_dim, page_size=cache.page_size,
            kv_layout=cache.kv_layout)
    group_size = num_q_heads // cache.num_kv_heads
    direct = force_impl == "direct" or (force_impl == "auto" and plan.launch_mode == "direct")
    if direct and group_size > 8:
        raise ValueError('force_impl="direct" only supports group_size <= 8; use auto or force_impl="clustered"')
    if output is None:
        output = torch.empty_like(query)
    _check_cuda_tensor(output, name="output", dtype=torch.bfloat16, ndim=3)
    if cache.keys_are_rotated:
        if cache.key_rope_theta is None:
            raise ValueError("rotated key caches must record key_rope_theta")
        if float(cache.key_rope_theta) != float(rope_theta):
            raise ValueError("rope_theta must match the key_rope_theta used to build the cache")
    if cache.key_scales is not None or cache.value_scales is not None:
        _check_same_cuda_device(("query", query), ("key_scales", cache.key_scales),
                                ("value_scales", cache.value_scales))
    descriptors = plan.device_tensors(query.device)
    scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(head_dim)

    def address(tensor: Any | None) -> int:
        return 0 if tensor is None else int(tensor.data_ptr())

    native.clustered_page_decode_forward(
        address(query), address(cache.key_pages), address(cache.value_pages), address(cache.key_scales),
        address(cache.value_scales), address(descriptors["run_base_pages"]),
        address(descriptors["run_page_counts"]), address(descriptors["run_logical_starts"]),
        address(descriptors["run_last_page_lens"]), address(descriptors["request_run_offsets"]),
        address(descriptors["seq_lens"]), address(output), batch, plan.num_runs, num_q_heads, cache.num_kv_heads,
        head_dim, cache.page_size, plan.group_tile, int(not direct),
        # "clustered" always may split; the plan's cluster_size of 1 is the reference's way of
        # saying "short request", which max_pages_hint tells the launcher more precisely
        max(2, plan.cluster_size) if not direct else 1,
        _layout_id(cache.kv_layout), int(cache.keys_are_rotated), float(scale), float(rope_theta),
        int(torch.cuda.current_stream(device=query.device).cuda_stream), max_pages_hint=plan.max_pages,
        early_descriptors=1,  # the descriptors were uploaded from the host when the plan was made
    )
    return output


# ---------------------------------------------------------------------------------------------
# plain PyTorch statement of the op (tests, baseline column)
# ---------------------------------------------------------------------------------------------
def materialize_reference_dense_kv(cache: PagedKVCache) -> tuple[Any, Any]:
    """[batch, kv_heads, max_seq_len, head_dim] keys and values gathered back through the page table
    from the unquantised pages."""
    torch = _torch()
    batch = int(cache.page_table.shape[0])
    max_len = int(cache.seq_lens.max().item())
    pages = cache.reference_key_pages
    slots = (max_len + cache.page_size - 1) // cache.page_size
    table = cache.page_table[:, :slots].to(device=pages.device, dtype=torch.int64).clamp(min=0)

    def gather(source: Any) -> Any:
        picked = source[table]  # [batch, slots, heads, page, dim]
        dense = picked.permute(0, 2, 1, 3, 4).reshape(batch, cache.num_kv_heads, slots * cache.page_size, cache.head_dim)
        token = torch.arange(slots * cache.page_size, device=pages.device)
        dead = token[None, :] >= cache.seq_lens.to(pages.device)[:, None]
        return dense.masked_fill(dead[:, None, :, None], 0)[:, :, :max_len].contiguous()

    return gather(cache.reference_key_pages), gather(cache.reference_value_pages)


def reference_clustered_page_decode(
    query: Any,
    cache: PagedKVCache,
    *,
    softmax_scale: float | None = None,
    rope_theta: float = 10000.0,
    output: Any | None = None,
) -> Any:
    torch = _torch()
    if query.ndim != 3:
        raise ValueError("query must be 3D [batch, q_heads, head_dim]")
    batch, num_q_heads, head_dim = (int(v) for v in query.shape)
    if head_dim != cache.head_dim:
        raise ValueError("query head_dim must match cache head_dim")
    group_size = num_q_heads // cache.num_kv_heads
    scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(head_dim)
    dense_keys, dense_values = materialize_reference_dense_kv(cache)
    result = torch.empty_like(query) if output is None else output
    for request in range(batch):
        length = int(cache.seq_lens[request].item())
        positions = torch.arange(length, device=query.device, dtype=torch.float32)
        q = _apply_llama_rope_torch(query[request], torch.full((num_q_heads,), length - 1, device=query.device),
                                    rope_theta).to(torch.float32)
        keys = dense_keys[request, :, :length]
        if not cache.keys_are_rotated:
            keys = _apply_llama_rope_torch(keys, positions, rope_theta)
        keys = keys.to(torch.float32).repeat_interleave(group_size, dim=0)       # [q_heads, len, dim]
        values = dense_values[request, :, :length].to(torch.float32).repeat_interleave(group_size, dim=0)
        logits = torch.einsum("htd,hd->ht", keys, q) * scale
        result[request] = torch.einsum("ht,htd->hd", torch.softmax(logits, dim=1), values).to(torch.bfloat16)
    return result


def estimate_page_decode_metrics(cache: PagedKVCache, plan: ClusteredPageDecodePlan) -> dict[str, float]:
    """Bytes per decoded token as the harness reports them. On this build every page of a kv head is
    read from HBM once per head TILE (one block carries up to 8 query heads), never once per head."""
    torch = _torch()
    element_bytes = {"bf16_kv": 2.0, "fp8_kv": 1.0, "int8_kv": 1.0}[cache.kv_layout]
    mean_tokens = float(cache.seq_lens.to(torch.float32).mean().item())
    reuse = float(plan.q_head_tiles)
    kv_bytes = mean_tokens * cache.num_kv_heads * cache.head_dim * 2.0 * element_bytes * reuse
    scale_bytes = 0.0
    if cache.kv_layout != "bf16_kv":
        scale_bytes = mean_tokens * cache.num_kv_heads * (cache.head_dim / _SCALE_BLOCK) * 4.0 * reuse
    return {
        "hbm_bytes_per_token": kv_bytes + scale_bytes,
        "workspace_bytes_per_token": 0.0,
        "dsm_bytes_per_token": 0.0,
    }
