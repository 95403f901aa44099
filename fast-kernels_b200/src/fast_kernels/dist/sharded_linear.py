"""A W4A16 linear layer split over the ranks of one ``torch.distributed`` group.

Two splits, as tensor-parallel decoders use them:

* ``mode="column"`` (N-split): each rank holds ``n / P`` output columns and the full activation
  vector; local GEMV, then the outputs are gathered so that every rank ends with ``[m, n]``.
* ``mode="row"`` (K-split): each rank holds ``k / P`` input features of every column; the local
  GEMV yields an unrounded fp32 partial ``[m, n]``, the partials are summed over ranks (in rank
  order for the ``peer`` exchange, hence reproducible) and rounded once to the 16-bit type.

Two exchanges:

* ``exchange="nccl"``: ``all_gather_into_tensor`` / ``all_reduce`` on the group, enqueued on the
  GEMV's stream. Works on any backend (the CPU tests run it over gloo).
* ``exchange="peer"`` (CUDA, one node): the GEMV kernel itself stores every finished tile into all
  ranks' receive areas through peer-mapped symmetric memory while it is still streaming weights,
  as 8-byte words that carry the call's epoch beside the value (an 8-byte store is atomic, so
  there is nothing to fence and nothing to signal); the kernel's first CTAs turn the words into
  the final 16-bit result as they arrive (bounded wait) -- side by side for a column split, added
  in rank order for a row split. One launch does compute, exchange and reduction, no collective
  call, and because the call count lives on the device a captured call can be replayed.

One process per GPU; all ranks must call ``forward`` the same number of times in the same order.
"""

from __future__ import annotations

from typing import Any, Callable

from fast_kernels.dist.sharding import (
    activation_shard,
    check_shardable,
    column_shard_packets,
    row_shard_packets,
)

LocalForward = Callable[[Any, Any, int, int, bool], Any]
"""(activations_local, packets_local, n_local, k_local, want_f32) -> [m, n_local] tensor."""


def _torch() -> Any:
    import torch

    return torch


class ShardedW4A16Linear:
    def __init__(
        self,
        packets: Any,
        *,
        n: int,
        k: int,
        group_size: int,
        mode: str,
        dtype: Any,
        group: Any | None = None,
        exchange: str = "nccl",
        packets_are_local: bool = False,
        local_forward: LocalForward | None = None,
        max_batch: int = 4,
    ) -> None:
        torch = _torch()
        import torch.distributed as dist

        if not dist.is_initialized():
            raise RuntimeError("torch.distributed must be initialised before building a sharded layer")
        if exchange not in ("nccl", "peer"):
            raise ValueError("exchange must be 'nccl' or 'peer'")
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        check_shardable(n, k, group_size, self.world, mode)
        if exchange == "peer" and self.world - 1 > 7:
            raise ValueError("the peer exchange supports at most 8 ranks")
        self.n, self.k, self.group_size, self.mode, self.dtype = n, k, group_size, mode, dtype
        self.exchange = exchange
        self.max_batch = max_batch
        self.n_local = n // self.world if mode == "column" else n
        self.k_local = k if mode == "column" else k // self.world
        if packets_are_local:
            expected = ((self.n_local // 128) * (self.k_local // group_size), 64 * group_size + 512)
            if tuple(packets.shape) != expected:
                raise ValueError(f"local packets must have shape {expected}")
            self.packets = packets
        elif mode == "column":
            self.packets = column_shard_packets(packets, n=n, k=k, group_size=group_size,
                                                rank=self.rank, world=self.world)
        else:
            self.packets = row_shard_packets(packets, n=n, k=k, group_size=group_size,
                                             rank=self.rank, world=self.world)
        self.device = self.packets.device
        self._local_forward = local_forward or self._cuda_local_forward
        self._workspace = None
        self._calls = 0
        self._peer = None
        if exchange == "peer":
            if self.device.type != "cuda":
                raise ValueError("the peer exchange needs CUDA tensors")
            self._setup_peer_buffers(torch)

    # ---- local compute through the C ABI ---------------------------------------------------
    def _gemv_args(self, activations: Any, output: Any, want_f32: bool) -> Any:
        torch = _torch()
        from fast_kernels import capi

        lib = capi.load_library()
        batch = activations.shape[0]
        if self._workspace is None:
            need = int(lib.fk_w4a16_workspace_bytes(self.max_batch, self.n_local, self.k_local,
                                                    self.group_size))
            self._workspace = torch.zeros(need, dtype=torch.uint8, device=self.device)
        args = capi.GemvArgs()
        args.activations = activations.data_ptr()
        args.packets = self.packets.data_ptr()
        args.output = output.data_ptr()
        args.workspace = self._workspace.data_ptr()
        args.workspace_bytes = self._workspace.numel()
        args.batch = batch
        args.n = self.n_local
        args.k = self.k_local
        args.group_size = self.group_size
        args.packet_stride_bytes = 64 * self.group_size + 512
        args.dtype = capi.DTYPE_BF16 if self.dtype == torch.bfloat16 else capi.DTYPE_F16
        args.output_f32 = 1 if want_f32 else 0
        args.stream = int(torch.cuda.current_stream(self.device).cuda_stream)
        return args

    def _cuda_local_forward(self, activations: Any, packets: Any, n_local: int, k_local: int,
                            want_f32: bool) -> Any:
        torch = _torch()
        from fast_kernels import capi

        del packets, n_local, k_local  # the layer's own shard is what the arguments describe
        out = torch.empty((activations.shape[0], self.n_local), device=self.device,
                          dtype=torch.float32 if want_f32 else self.dtype)
        args = self._gemv_args(activations, out, want_f32)
        capi.check(capi.load_library().fk_w4a16_gemv_ex(args))
        return out

    # ---- public -----------------------------------------------------------------------------
    def forward(self, activations: Any) -> Any:
        """activations ``[m, k]`` (identical on every rank) -> ``[m, n]`` on every rank."""
        if activations.ndim != 2 or activations.shape[1] != self.k:
            raise ValueError(f"activations must have shape [m, {self.k}]")
        if activations.shape[0] > self.max_batch:
            raise ValueError(f"batch {activations.shape[0]} exceeds max_batch={self.max_batch}")
        if activations.dtype != self.dtype:
            raise TypeError(f"activations must have dtype {self.dtype}")
        local_act = activation_shard(activations, rank=self.rank, world=self.world, mode=self.mode)
        self._calls += 1
        if self.exchange == "peer":
            return self._forward_peer(local_act)
        return self._forward_collective(local_act)

    __call__ = forward

    # ---- exchange by collectives --------------------------------------------------------------
    def _forward_collective(self, local_act: Any) -> Any:
        torch = _torch()
        import torch.distributed as dist

        if self.mode == "column":
            local = self._local_forward(local_act, self.packets, self.n_local, self.k_local, False)
            m = local.shape[0]
            gathered = torch.empty((self.world * m, self.n_local), dtype=local.dtype, device=local.device)
            dist.all_gather_into_tensor(gathered, local.contiguous(), group=self.group)
            if m == 1:
                return gathered.view(1, self.n)
            return gathered.view(self.world, m, self.n_local).permute(1, 0, 2).reshape(m, self.n)
        partial = self._local_forward(local_act, self.packets, self.n_local, self.k_local, True)
        if partial.dtype != torch.float32:
            raise TypeError("a row-split local forward must return fp32 partial sums")
        dist.all_reduce(partial, op=dist.ReduceOp.SUM, group=self.group)
        return partial.to(self.dtype)

    # ---- exchange by peer stores inside the GEMV kernel -----------------------------------------
    _SIGNAL_BYTES = 256

    def _setup_peer_buffers(self, torch: Any) -> None:
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm

        # receive area: one slot of 8-byte words {fp32 value, epoch} per rank, two areas (epoch parity)
        cols = self.n_local if self.mode == "column" else self.n
        slot = self.world * self.max_batch * cols * 8
        slot = (slot + 255) & ~255
        total = self._SIGNAL_BYTES + 2 * slot
        group = self.group if self.group is not None else dist.group.WORLD
        buffer = symm.empty(total, dtype=torch.uint8, device=self.device)
        handle = symm.rendezvous(buffer, group)
        buffer.zero_()
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        self._peer = {
            "buffer": buffer,
            "handle": handle,
            "slot": slot,
            "ptrs": [int(handle.buffer_ptrs[r]) for r in range(self.world)],
        }

    def _forward_peer(self, local_act: Any) -> Any:
        """Flag-in-data exchange: every result travels as an 8-byte word {fp32 value, call epoch}
        into slot `rank` of every rank's receive area; the kernel's first CTAs assemble the final
        16-bit output from the words as they arrive -- concatenated (column split) or added in
        rank order (row split). No fence, no counters, one launch. The call count lives on the
        device (first words of the symmetric buffer), so a captured call can be replayed."""
        torch = _torch()
        from fast_kernels import capi

        lib = capi.load_library()
        peer = self._peer
        m = local_act.shape[0]
        cols = self.n_local if self.mode == "column" else self.n
        area_offset = self._SIGNAL_BYTES  # the even-epoch area; the odd one lies `slot` bytes behind
        slot_offset = area_offset + self.rank * m * cols * 8
        ptrs = peer["ptrs"]
        others = [r for r in range(self.world) if r != self.rank]
        out = torch.empty((m, self.n), dtype=self.dtype, device=self.device)
        args = self._gemv_args(local_act, out, False)
        args.output = ptrs[self.rank] + slot_offset
        args.output_ld = cols
        args.num_peers = len(others)
        for i, r in enumerate(others):
            args.peer_outputs[i] = ptrs[r] + slot_offset
        args.ll_epoch_counter = ptrs[self.rank]
        args.ll_parity_words = peer["slot"] // 8
        args.ll_input = ptrs[self.rank] + area_offset
        args.ll_output = out.data_ptr()
        args.ll_slots = self.world
        args.ll_slot_cols = cols
        args.ll_reduce = 1 if self.mode == "row" else 0
        capi.check(lib.fk_w4a16_gemv_ex(args))
        return out
