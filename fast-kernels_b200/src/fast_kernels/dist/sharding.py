"""Cutting an ARC-packet weight matrix into per-rank shards. Pure tensor indexing: works on CPU
and CUDA tensors alike, touches no kernel.

Packets are stored tile-major, group-minor -- packet (tile t, group g) is row ``t * NG + g`` of the
``[T * NG, stride]`` packet tensor (T = n / 128 tiles, NG = k / group_size groups) -- so

* a **column shard** (output features split, "N-split") is a contiguous slice of rows: rank r of P
  owns tiles ``[r*T/P, (r+1)*T/P)``;
* a **row shard** (input features split, "K-split") owns groups ``[r*NG/P, (r+1)*NG/P)`` of every
  tile, a strided subset that is gathered into a local ``[T * NG/P, stride]`` tensor once at load.
"""

from __future__ import annotations

from typing import Any

MODES = ("column", "row")


def check_shardable(n: int, k: int, group_size: int, world: int, mode: str) -> None:
    """Raises ValueError, before anything is launched, if the layer cannot be split this way."""
    if mode not in MODES:
        raise ValueError(f"mode must be one of {MODES}; received {mode!r}")
    if world < 1:
        raise ValueError("world size must be positive")
    if n <= 0 or n % 128 != 0:
        raise ValueError("n must be a positive multiple of 128")
    if group_size not in (32, 64, 128) or k <= 0 or k % group_size != 0:
        raise ValueError("k must be a positive multiple of group_size (32, 64 or 128)")
    if mode == "column" and (n // 128) % world != 0:
        raise ValueError(f"column split needs n/128 = {n // 128} tiles to divide by the {world} ranks")
    if mode == "row" and (k // group_size) % world != 0:
        raise ValueError(
            f"row split needs k/group_size = {k // group_size} groups to divide by the {world} ranks"
        )


def _check_packets(packets: Any, n: int, k: int, group_size: int) -> tuple[int, int, int]:
    tiles, groups = n // 128, k // group_size
    stride = 64 * group_size + 512
    if tuple(packets.shape) != (tiles * groups, stride):
        raise ValueError(f"packets must have shape {(tiles * groups, stride)}")
    return tiles, groups, stride


def column_shard_packets(packets: Any, *, n: int, k: int, group_size: int, rank: int, world: int) -> Any:
    """Rank's packets for an N-split: a view of ``n / world`` output columns, all of k."""
    check_shardable(n, k, group_size, world, "column")
    if not 0 <= rank < world:
        raise ValueError("rank out of range")
    tiles, groups, _ = _check_packets(packets, n, k, group_size)
    per_rank = tiles // world
    return packets[rank * per_rank * groups:(rank + 1) * per_rank * groups]


def row_shard_packets(packets: Any, *, n: int, k: int, group_size: int, rank: int, world: int) -> Any:
    """Rank's packets for a K-split: all n output columns, ``k / world`` input features (a copy)."""
    check_shardable(n, k, group_size, world, "row")
    if not 0 <= rank < world:
        raise ValueError("rank out of range")
    tiles, groups, stride = _check_packets(packets, n, k, group_size)
    per_rank = groups // world
    view = packets.reshape(tiles, groups, stride)[:, rank * per_rank:(rank + 1) * per_rank]
    return view.reshape(tiles * per_rank, stride).contiguous()


def activation_shard(activations: Any, *, rank: int, world: int, mode: str) -> Any:
    """The part of ``activations[m, k]`` a rank multiplies with: all of it (column split) or its
    contiguous k-range (row split, copied so that rows are dense)."""
    if mode == "column":
        return activations
    k = activations.shape[1]
    if k % world != 0:
        raise ValueError("activations' k must divide by the world size")
    per_rank = k // world
    return activations[:, rank * per_rank:(rank + 1) * per_rank].contiguous()
