"""Generates the golden fixtures in this directory by running the REFERENCE's own CPU-runnable
W4A16 arithmetic (SamMausberg/fast-kernels) on seeded inputs.

The reference stores no golden vectors: its tests recompute expectations with the torch
expression ``_explicit_reference_output`` (tests/gpu/test_decode_quant_linear.py:46-60), and its
bench does the same with ``_make_case_inputs`` / ``_explicit_reference_output``
(src/fast_kernels/benchmarking/decode_linear_w4a16.py:152-192). This script imports exactly those
functions from a reference checkout, calls them on CPU tensors, and stores inputs and outputs as
bit patterns. It needs the checkout; the tests that consume the fixtures do not.

    python tests/golden/make_golden.py [--reference <path of the reference checkout>]

Cases mirror the reference's six GPU tests (same shapes, same seed formulas, same value recipes;
drawn with the CPU generator because CUDA draws cannot be reproduced off-GPU) plus three cases
from its bench input generator. Large inputs are stored as a seed and a SHA-256 instead of bytes.
"""

from __future__ import annotations

import argparse
import hashlib
import importlib.util
import json
import os
import sys
import types
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
MAX_STORED_INPUT_BYTES = 300_000


def _load_reference(reference: Path):
    sys.path.insert(0, str(reference / "src"))
    # The reference's reporting package imports matplotlib at module import; it is not installed
    # here and is irrelevant to the arithmetic, so give the import chain an empty stand-in.
    if "matplotlib" not in sys.modules:
        fake = types.ModuleType("matplotlib")
        fake.use = lambda *a, **k: None  # type: ignore[attr-defined]
        pyplot = types.ModuleType("matplotlib.pyplot")
        fake.pyplot = pyplot  # type: ignore[attr-defined]
        sys.modules["matplotlib"] = fake
        sys.modules["matplotlib.pyplot"] = pyplot
    spec = importlib.util.spec_from_file_location(
        "ref_gpu_tests", reference / "tests" / "gpu" / "test_decode_quant_linear.py"
    )
    tests_mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(tests_mod)  # type: ignore[union-attr]
    import fast_kernels.benchmarking.decode_linear_w4a16 as bench_mod  # noqa: PLC0415

    return tests_mod, bench_mod


def _bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().view(np.uint16).copy()


def _test_recipe(seed: int, batch: int, n: int, k: int, group: int, lo: float, span: float):
    """The value recipe shared by the reference's GPU tests (e.g. :70-83), on the CPU generator."""
    torch.manual_seed(seed)
    groups = k // group
    activations = torch.randn((batch, k), dtype=torch.float16).contiguous()
    q_u8 = torch.randint(0, 256, (n, k // 2), dtype=torch.uint8).contiguous()
    alpha = (lo + (span * torch.rand((n, groups), dtype=torch.float32))).to(torch.float16)
    zero_points = torch.randint(0, 16, (n, groups), dtype=torch.int16)
    beta = -(alpha * zero_points.to(dtype=torch.float16))
    return activations, q_u8, alpha, beta


def _sha(*arrays: np.ndarray) -> str:
    digest = hashlib.sha256()
    for array in arrays:
        digest.update(np.ascontiguousarray(array).tobytes())
    return digest.hexdigest()


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--reference", default=os.environ.get("FK_REFERENCE_ROOT"), required="FK_REFERENCE_ROOT" not in os.environ,
                        help="checkout of the reference project (or set FK_REFERENCE_ROOT)")
    ns = parser.parse_args()
    tests_mod, bench_mod = _load_reference(Path(ns.reference))
    explicit = tests_mod._explicit_reference_output

    cases = []

    def add(name: str, origin: str, recipe: dict, activations, q_u8, alpha, beta, group: int) -> None:
        output = explicit(activations, q_u8, alpha, beta, group_size=group)
        # the dequant expectation of test_native_dequant_matches_explicit_reference (:158-166)
        low = torch.bitwise_and(q_u8, 0x0F).to(torch.float32)
        high = torch.bitwise_right_shift(q_u8, 4).to(torch.float32)
        q_values = torch.stack((low, high), dim=-1).reshape(q_u8.shape[0], q_u8.shape[1] * 2)
        weight = (
            alpha.to(torch.float32).repeat_interleave(group, dim=1) * q_values
            + beta.to(torch.float32).repeat_interleave(group, dim=1)
        ).to(torch.float16)
        arrays = {
            "activations": _bits(activations),
            "q_u8": q_u8.numpy().copy(),
            "alpha": _bits(alpha),
            "beta": _bits(beta),
        }
        stored = {"output": _bits(output)}
        input_bytes = sum(a.nbytes for a in arrays.values())
        meta = {
            "name": name,
            "origin": origin,
            "recipe": recipe,
            "batch": int(activations.shape[0]),
            "n": int(q_u8.shape[0]),
            "k": int(q_u8.shape[1] * 2),
            "group_size": group,
            "dtype": "fp16",
            "inputs_sha256": _sha(*arrays.values()),
            "weight_sha256": _sha(_bits(weight)),
            "inputs_stored": input_bytes <= MAX_STORED_INPUT_BYTES,
        }
        if meta["inputs_stored"]:
            stored.update(arrays)
            stored["weight"] = _bits(weight)
        np.savez_compressed(HERE / f"{name}.npz", **stored)
        cases.append(meta)

    for group in (64, 128):
        for batch in (1, 4):
            seed = 7 + batch + group
            args = _test_recipe(seed, batch, 128, group * 2, group, 0.05, 0.1)
            add(f"ref_test_arc_g{group}_b{batch}", "tests/gpu/test_decode_quant_linear.py:63-102",
                {"kind": "test", "seed": seed, "lo": 0.05, "span": 0.1}, *args, group)
    for group in (64, 128):
        for batch in (8, 16):
            seed = 90 + batch + group
            args = _test_recipe(seed, batch, 4096, group * 4, group, 0.03, 0.12)
            add(f"ref_test_direct_g{group}_b{batch}", "tests/gpu/test_decode_quant_linear.py:105-140",
                {"kind": "test", "seed": seed, "lo": 0.03, "span": 0.12}, *args, group)
    for group in (64, 128):
        seed = 123 + group
        args = _test_recipe(seed, 1, 128, group * 2, group, 0.03, 0.2)
        add(f"ref_test_dequant_g{group}", "tests/gpu/test_decode_quant_linear.py:143-168",
            {"kind": "test", "seed": seed, "lo": 0.03, "span": 0.2}, *args, group)
    args = _test_recipe(4242, 8, 128, 512, 128, 0.04, 0.12)
    add("ref_test_split_k", "tests/gpu/test_decode_quant_linear.py:171-207",
        {"kind": "test", "seed": 4242, "lo": 0.04, "span": 0.12}, *args, 128)
    args = _test_recipe(5150, 4, 128, 512, 128, 0.04, 0.12)
    add("ref_test_env_impl", "tests/gpu/test_decode_quant_linear.py:210-245",
        {"kind": "test", "seed": 5150, "lo": 0.04, "span": 0.12}, *args, 128)

    # The reference bench's own input generator and seed rule, on CPU.
    for batch, n, k, group in ((1, 256, 1024, 128), (2, 128, 512, 64), (1, 4096, 4096, 128)):
        activations, q_u8, alpha, beta = bench_mod._make_case_inputs(
            torch, batch=batch, n=n, k=k, group_size=group, device=torch.device("cpu")
        )
        add(f"ref_bench_b{batch}_n{n}_k{k}_g{group}",
            "src/fast_kernels/benchmarking/decode_linear_w4a16.py:152-192",
            {"kind": "bench", "seed": bench_mod._seed_for_case(batch, n, k, group)},
            activations, q_u8, alpha, beta, group)

    manifest = {
        "generator": "tests/golden/make_golden.py",
        "torch": torch.__version__,
        "note": "outputs of the reference's _explicit_reference_output on CPU tensors",
        "cases": cases,
    }
    (HERE / "manifest.json").write_text(json.dumps(manifest, indent=2) + "\n")
    print(f"wrote {len(cases)} cases to {HERE}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
