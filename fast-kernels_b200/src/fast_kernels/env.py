"""Environment snapshot recorded with every benchmark run (``fk env``)."""

from __future__ import annotations

import json
import platform
import shutil
import subprocess
import sys
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Any

from fast_kernels.native import native_build_info


@dataclass
class EnvironmentSnapshot:
    python_version: str
    platform: str
    machine: str
    git_sha: str | None = None
    git_dirty: bool | None = None
    torch_version: str | None = None
    nvcc_version: str | None = None
    nvidia_smi: dict[str, str] | None = None
    native: dict[str, Any] = field(default_factory=dict)

    def to_json(self) -> str:
        return json.dumps(asdict(self), indent=2, sort_keys=True)


def _run(cmd: list[str], cwd: Path | None = None) -> str | None:
    try:
        out = subprocess.run(cmd, cwd=cwd, capture_output=True, text=True, timeout=20, check=False)
    except (OSError, subprocess.SubprocessError):
        return None
    return out.stdout.strip() if out.returncode == 0 else None


def collect_environment(repo: Path | None = None) -> EnvironmentSnapshot:
    snapshot = EnvironmentSnapshot(
        python_version=sys.version.split()[0],
        platform=platform.platform(),
        machine=platform.machine(),
        native=native_build_info(),
    )
    sha = _run(["git", "rev-parse", "--short", "HEAD"], cwd=repo)
    if sha:
        snapshot.git_sha = sha
        snapshot.git_dirty = bool(_run(["git", "status", "--porcelain"], cwd=repo))
    try:
        import torch

        snapshot.torch_version = str(torch.__version__)
    except ImportError:
        pass
    if shutil.which("nvcc"):
        text = _run(["nvcc", "--version"]) or ""
        if "release" in text:
            snapshot.nvcc_version = text.split("release")[-1].split(",")[0].strip()
    if shutil.which("nvidia-smi"):
        row = _run(["nvidia-smi", "--query-gpu=name,driver_version,memory.total", "--format=csv,noheader"])
        if row:
            name, driver, memory = (part.strip() for part in row.splitlines()[0].split(",")[:3])
            snapshot.nvidia_smi = {"name": name, "driver_version": driver, "memory_total": memory}
    return snapshot
