#!/usr/bin/env python3
"""The four linear layers of one Llama-3-8B decoder layer at batch 1, fused against unfused.

    decode_layer_chain.py [LAYERS] [REPLAYS]

fused:    [RMSNorm + qkv]  [o_proj + residual]  [RMSNorm + gate/up + SiLU*mul]  [down + residual]
          = 4 launches through fk_w4a16_gemv_ex
unfused:  rmsnorm, qkv, o_proj, add, rmsnorm, gate/up, silu*mul, down, add
          = 4 launches through fk_w4a16_gemv + 5 elementwise torch kernels (their fastest form here:
          torch.nn.functional.rms_norm, a fused silu*mul expression, in-place add)

Attention itself is out of scope: its output is a fixed tensor of the right shape. LAYERS sets of
distinct weights are chained (the working set exceeds L2), captured in one CUDA graph per variant
and replayed; device time per decoder layer is printed for both, with the worst relative
difference between their final hidden states.
"""

from __future__ import annotations

import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT / "src"))

import torch  # noqa: E402
from fast_kernels import capi  # noqa: E402
from fast_kernels.workloads import LayerShape, make_problem  # noqa: E402

HIDDEN, QKV, INTER = 4096, 6144, 14336
EPS = 1e-5


def main() -> int:
    layers = int(sys.argv[1]) if len(sys.argv) > 1 else 16
    replays = int(sys.argv[2]) if len(sys.argv) > 2 else 20
    lib = capi.load_library()
    device = torch.device("cuda")
    dtype = torch.bfloat16
    stride = capi.packet_stride_bytes(128)
    stream = torch.cuda.Stream()

    def packed(n: int, k: int, seed: int) -> torch.Tensor:
        problem = make_problem(LayerShape("w", n, k, dtype="bf16"), seed=seed)
        q, alpha, beta = (problem[key].to(device) for key in ("q_u8", "alpha", "beta"))
        out = torch.empty(((n // 128) * (k // 128), stride), dtype=torch.uint8, device=device)
        capi.check(lib.fk_w4a16_pack_packets(q.data_ptr(), alpha.data_ptr(), beta.data_ptr(), out.data_ptr(),
                                             n, k, 128, stride, 0))
        return out

    base = {"qkv": packed(QKV, HIDDEN, 1), "o": packed(HIDDEN, HIDDEN, 2),
            "gate_up": packed(2 * INTER, HIDDEN, 3), "down": packed(HIDDEN, INTER, 4)}
    weights = [{name: (w if i == 0 else w.clone()) for name, w in base.items()} for i in range(layers)]
    gen = torch.Generator().manual_seed(0)
    norm1 = (1.0 + 0.05 * torch.randn(HIDDEN, generator=gen)).to(dtype).to(device)
    norm2 = (1.0 + 0.05 * torch.randn(HIDDEN, generator=gen)).to(dtype).to(device)
    hidden0 = torch.randn((1, HIDDEN), generator=gen).to(dtype).to(device)
    attn_out = (0.5 * torch.randn((1, HIDDEN), generator=gen)).to(dtype).to(device)
    need = max(int(lib.fk_w4a16_workspace_bytes(1, n, k, 128))
               for n, k in ((QKV, HIDDEN), (HIDDEN, HIDDEN), (2 * INTER, HIDDEN), (HIDDEN, INTER)))
    workspace = torch.zeros(need, dtype=torch.uint8, device=device)

    def gemv(act, packets, out, n, k, *, residual=None, norm=None, silu_mul=False) -> None:
        args = capi.GemvArgs()
        args.activations, args.packets, args.output = act.data_ptr(), packets.data_ptr(), out.data_ptr()
        args.workspace, args.workspace_bytes = workspace.data_ptr(), workspace.numel()
        args.batch, args.n, args.k, args.group_size = 1, n, k, 128
        args.packet_stride_bytes, args.dtype = stride, capi.DTYPE_BF16
        args.residual = 0 if residual is None else residual.data_ptr()
        if norm is not None:
            args.norm_weight, args.norm_eps = norm.data_ptr(), EPS
        args.epilogue = capi.EPILOGUE_SILU_MUL if silu_mul else capi.EPILOGUE_NONE
        args.stream = stream.cuda_stream
        capi.check(lib.fk_w4a16_gemv_ex(args))

    qkv = torch.empty((1, QKV), dtype=dtype, device=device)
    gate_up = torch.empty((1, 2 * INTER), dtype=dtype, device=device)
    mlp_in = torch.empty((1, INTER), dtype=dtype, device=device)
    normed = torch.empty((1, HIDDEN), dtype=dtype, device=device)

    def fused(hidden: torch.Tensor) -> None:
        for w in weights:
            gemv(hidden, w["qkv"], qkv, QKV, HIDDEN, norm=norm1)
            gemv(attn_out, w["o"], hidden, HIDDEN, HIDDEN, residual=hidden)
            gemv(hidden, w["gate_up"], mlp_in, 2 * INTER, HIDDEN, norm=norm2, silu_mul=True)
            gemv(mlp_in, w["down"], hidden, HIDDEN, INTER, residual=hidden)

    proj = torch.empty((1, HIDDEN), dtype=dtype, device=device)

    def unfused(hidden: torch.Tensor) -> None:
        for w in weights:
            normed.copy_(torch.nn.functional.rms_norm(hidden, (HIDDEN,), norm1, EPS))
            gemv(normed, w["qkv"], qkv, QKV, HIDDEN)
            gemv(attn_out, w["o"], proj, HIDDEN, HIDDEN)
            hidden.add_(proj)
            normed.copy_(torch.nn.functional.rms_norm(hidden, (HIDDEN,), norm2, EPS))
            gemv(normed, w["gate_up"], gate_up, 2 * INTER, HIDDEN)
            torch.mul(torch.nn.functional.silu(gate_up[:, :INTER]), gate_up[:, INTER:], out=mlp_in)
            gemv(mlp_in, w["down"], proj, HIDDEN, INTER)
            hidden.add_(proj)

    results = {}
    for name, chain in (("fused", fused), ("unfused", unfused)):
        hidden = hidden0.clone()
        with torch.cuda.stream(stream):
            chain(hidden)  # warm-up: function attributes, allocator
            stream.synchronize()
            hidden.copy_(hidden0)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                chain(hidden)
            hidden.copy_(hidden0)
            graph.replay()
            stream.synchronize()
            final = hidden.clone()
            start = torch.cuda.Event(enable_timing=True)
            stop = torch.cuda.Event(enable_timing=True)
            start.record()
            for _ in range(replays):
                graph.replay()
            stop.record()
            stream.synchronize()
        results[name] = (start.elapsed_time(stop) * 1e3 / (replays * layers), final)
    fused_us, fused_out = results["fused"]
    unfused_us, unfused_out = results["unfused"]
    scale = float(unfused_out.float().abs().max())
    diff = float((fused_out.float() - unfused_out.float()).abs().max()) / scale
    print(f"decoder layer, 4 linear layers + norms/activation/residuals, batch 1, {layers} layers chained:")
    print(f"  fused   (4 launches): {fused_us:7.2f} us per layer")
    print(f"  unfused (9 launches): {unfused_us:7.2f} us per layer")
    print(f"  final hidden state: max |fused - unfused| / max |unfused| = {diff:.3e}")
    print("device status", capi.device_status())
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
