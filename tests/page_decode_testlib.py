"""Helpers shared by the page decode tests: fixture loading and calls through the C ABI."""

from __future__ import annotations

import json
from pathlib import Path
from typing import Any

import numpy as np

GOLDEN = Path(__file__).resolve().parent / "golden"
KV_IDS = {"bf16_kv": 0, "fp8_kv": 1, "int8_kv": 2}


def manifest() -> list[dict[str, Any]]:
    return json.loads((GOLDEN / "page_decode_manifest.json").read_text())


def load_case(name: str) -> dict[str, np.ndarray]:
    with np.load(GOLDEN / f"page_decode_{name}.npz") as data:
        return {key: data[key] for key in data.files}


def oracle_on_case(oracle: Any, meta: dict[str, Any], case: dict[str, np.ndarray]) -> np.ndarray:
    return oracle.page_decode_f64(
        case["query"], case["key_pages"], case["value_pages"], case.get("key_scales"), case.get("value_scales"),
        case["run_base_pages"], case["run_page_counts"], case["run_logical_starts"], case["run_last_page_lens"],
        case["request_run_offsets"], case["seq_lens"], kv_format=KV_IDS[meta["layout"]],
        keys_are_rotated=meta["key_rope_theta"] is not None, softmax_scale=1.0 / np.sqrt(meta["head_dim"]),
        rope_theta=10000.0)


class DeviceCase:
    """A problem on the device plus the call through fk_page_decode_forward."""

    def __init__(self, *, query, key_pages, value_pages, key_scales, value_scales, runs, seq_lens, kv_format,
                 keys_are_rotated, page_size, softmax_scale=None, rope_theta=10000.0):
        import torch

        dev = "cuda"
        self.torch = torch
        self.query = torch.from_numpy(query.view(np.int16)).to(dev).view(torch.bfloat16)
        if kv_format == 0:
            self.key_pages = torch.from_numpy(key_pages.view(np.int16)).to(dev).view(torch.bfloat16)
            self.value_pages = torch.from_numpy(value_pages.view(np.int16)).to(dev).view(torch.bfloat16)
        else:
            self.key_pages = torch.from_numpy(key_pages.view(np.uint8)).to(dev)
            self.value_pages = torch.from_numpy(value_pages.view(np.uint8)).to(dev)
        self.key_scales = None if key_scales is None else torch.from_numpy(key_scales).to(dev)
        self.value_scales = None if value_scales is None else torch.from_numpy(value_scales).to(dev)
        self.runs = {name: torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).to(dev) for name, a in runs.items()}
        self.seq_lens = torch.from_numpy(np.ascontiguousarray(seq_lens, dtype=np.int32)).to(dev)
        self.kv_format = kv_format
        self.keys_are_rotated = keys_are_rotated
        self.page_size = page_size
        self.batch, self.num_q_heads, self.head_dim = (int(v) for v in self.query.shape)
        self.num_kv_heads = int(self.key_pages.shape[1])
        self.softmax_scale = float(softmax_scale if softmax_scale is not None else 1.0 / np.sqrt(self.head_dim))
        self.rope_theta = float(rope_theta)
        self.workspace = None

    def args(self, pdc: Any, output: Any, *, splits: int = 0, group_tile: int = 0, max_pages_hint: int = 0,
             flags: int = 0) -> Any:
        torch = self.torch
        lib = pdc.load_library()
        if self.workspace is None:
            need = int(lib.fk_page_decode_workspace_bytes(self.batch, self.num_q_heads, self.num_kv_heads, self.head_dim))
            self.workspace = torch.zeros(need, dtype=torch.uint8, device="cuda")
        a = pdc.PageDecodeArgs()
        a.query = self.query.data_ptr()
        a.key_pages = self.key_pages.data_ptr()
        a.value_pages = self.value_pages.data_ptr()
        a.key_scales = 0 if self.key_scales is None else self.key_scales.data_ptr()
        a.value_scales = 0 if self.value_scales is None else self.value_scales.data_ptr()
        a.run_base_pages = self.runs["run_base_pages"].data_ptr()
        a.run_page_counts = self.runs["run_page_counts"].data_ptr()
        a.run_logical_starts = self.runs["run_logical_starts"].data_ptr()
        a.run_last_page_lens = self.runs["run_last_page_lens"].data_ptr()
        a.request_run_offsets = self.runs["request_run_offsets"].data_ptr()
        a.seq_lens = self.seq_lens.data_ptr()
        a.output = output.data_ptr()
        a.workspace = self.workspace.data_ptr()
        a.workspace_bytes = self.workspace.numel()
        a.batch = self.batch
        a.num_runs = int(self.runs["run_base_pages"].numel())
        a.num_q_heads = self.num_q_heads
        a.num_kv_heads = self.num_kv_heads
        a.head_dim = self.head_dim
        a.page_size = self.page_size
        a.group_tile = group_tile
        a.kv_format = self.kv_format
        a.keys_are_rotated = int(self.keys_are_rotated)
        a.splits = splits
        a.max_pages_hint = max_pages_hint
        a.flags = flags
        a.softmax_scale = self.softmax_scale
        a.rope_theta = self.rope_theta
        a.stream = int(torch.cuda.current_stream().cuda_stream)
        return a

    def forward(self, pdc: Any, **kwargs: Any) -> Any:
        import ctypes

        torch = self.torch
        out = torch.full((self.batch, self.num_q_heads, self.head_dim), float("nan"), dtype=torch.bfloat16, device="cuda")
        a = self.args(pdc, out, **kwargs)
        pdc.check(pdc.load_library().fk_page_decode_forward(ctypes.byref(a)))
        return out

    def oracle(self, oracle: Any) -> np.ndarray:
        def raw(t: Any) -> np.ndarray:
            if t.dtype == self.torch.bfloat16:
                return t.view(self.torch.int16).cpu().numpy().view(np.uint16)
            return t.cpu().numpy()

        runs = {name: t.cpu().numpy() for name, t in self.runs.items()}
        return oracle.page_decode_f64(
            raw(self.query), raw(self.key_pages), raw(self.value_pages),
            None if self.key_scales is None else self.key_scales.cpu().numpy(),
            None if self.value_scales is None else self.value_scales.cpu().numpy(),
            runs["run_base_pages"], runs["run_page_counts"], runs["run_logical_starts"], runs["run_last_page_lens"],
            runs["request_run_offsets"], self.seq_lens.cpu().numpy(), kv_format=self.kv_format,
            keys_are_rotated=self.keys_are_rotated, softmax_scale=self.softmax_scale, rope_theta=self.rope_theta)


def case_on_device(meta: dict[str, Any], case: dict[str, np.ndarray]) -> DeviceCase:
    runs = {name: case[name] for name in ("run_base_pages", "run_page_counts", "run_logical_starts",
                                          "run_last_page_lens", "request_run_offsets")}
    return DeviceCase(query=case["query"], key_pages=case["key_pages"], value_pages=case["value_pages"],
                      key_scales=case.get("key_scales"), value_scales=case.get("value_scales"), runs=runs,
                      seq_lens=case["seq_lens"], kv_format=KV_IDS[meta["layout"]],
                      keys_are_rotated=meta["key_rope_theta"] is not None, page_size=meta["page_size"])
