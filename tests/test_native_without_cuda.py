"""A `_native` module built WITHOUT CUDA keeps the whole binding surface and refuses to compute.

Contract of the reference's CPU-only build (csrc/bindings/python_module.cpp:241-287 there, used by
its CI with FK_ENABLE_CUDA=OFF): every op name is still exported, calling one raises
RuntimeError("fast-kernels was built without CUDA support"), and build_info() says
compiled_with_cuda = False. Built here with g++ alone into a temporary directory and imported in a
child process, so the CUDA build of the same module name stays untouched.
"""

from __future__ import annotations

import importlib.util
import json
import subprocess
import sys
from pathlib import Path

REPO = Path(__file__).resolve().parent.parent

REFERENCE_OPS = [
    "pack_arc_w4a16_packets", "compute_arc_w4a16_group_sums", "arc_w4a16_forward",
    "arc_w4a16_forward_split_k", "reduce_arc_w4a16_split_k_partials", "dequant_w4a16_to_fp16",
    "dequant_arc_w4a16_packets_to_fp16", "cublaslt_fp16_with_weight",
    "cublaslt_fp16_after_packet_dequant", "cublaslt_fp16_after_dequant", "clustered_page_decode_forward", "prefix_union_decode_forward",
]

CHILD = r"""
import json, sys
sys.path.insert(0, sys.argv[1])
import _native
info = dict(_native.build_info())
names = sorted(n for n in dir(_native) if not n.startswith("_"))
raised = {}
calls = {
    "arc_w4a16_forward": dict(activations_ptr=0, packets_ptr=0, group_sums_ptr=0, output_ptr=0, batch=1,
                              n=128, k=128, group_size=128, packet_stride_bytes=8704, stream_ptr=0),
    "pack_arc_w4a16_packets": dict(q_ptr=0, alpha_ptr=0, beta_ptr=0, packets_ptr=0, n=128, k=128,
                                   group_size=128, packet_stride_bytes=8704, stream_ptr=0),
    "compute_arc_w4a16_group_sums": dict(activations_ptr=0, sums_ptr=0, batch=1, k=128, group_size=128,
                                         stream_ptr=0),
    "dequant_w4a16_to_fp16": dict(q_ptr=0, alpha_ptr=0, beta_ptr=0, output_ptr=0, n=128, k=128,
                                  group_size=128, stream_ptr=0),
    "clustered_page_decode_forward": dict(
        query_ptr=0, key_ptr=0, value_ptr=0, key_scales_ptr=0, value_scales_ptr=0, run_base_pages_ptr=0,
        run_page_counts_ptr=0, run_logical_starts_ptr=0, run_last_page_lens_ptr=0, request_run_offsets_ptr=0,
        seq_lens_ptr=0, output_ptr=0, batch=1, num_runs=1, num_q_heads=8, num_kv_heads=2, head_dim=128,
        page_size=16, group_tile=4, use_clustered_kernel=1, cluster_size=2, kv_format=0, keys_are_rotated=0,
        softmax_scale=0.1, rope_theta=10000.0, stream_ptr=0),
}
for name, kwargs in calls.items():
    try:
        getattr(_native, name)(**kwargs)
        raised[name] = "no error"
    except RuntimeError as exc:
        raised[name] = str(exc)
print(json.dumps({"info": info, "names": names, "raised": raised}))
"""


def test_native_module_without_cuda_exports_every_name_and_raises(tmp_path: Path) -> None:
    spec = importlib.util.spec_from_file_location("fk_build", REPO / "fast-kernels_b200" / "build.py")
    build = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(build)  # type: ignore[union-attr]
    build.build_python_module_without_cuda(tmp_path)
    done = subprocess.run([sys.executable, "-c", CHILD, str(tmp_path)], capture_output=True, text=True, check=True)
    report = json.loads(done.stdout.strip().splitlines()[-1])
    assert report["info"]["compiled_with_cuda"] is False
    for key in ("project_version", "cxx_compiler_id", "cxx_compiler_version", "cuda_compiler_version",
                "cuda_architectures"):
        assert key in report["info"]
    for name in REFERENCE_OPS:
        assert name in report["names"], name
    for name, message in report["raised"].items():
        assert message == "fast-kernels was built without CUDA support", (name, message)
