"""Suite and result schemas: the TOML contract of ``fk verify`` / ``fk bench``.

Field names follow the reference's schemas (src/fast_kernels/schemas/suite.py:8-74 and
results.py:8-51 in SamMausberg/fast-kernels) so its suite files load here and result bundles
written here load there; only the fields the W4A16 family uses are spelled out, anything else a
suite carries is kept as an extra.
"""

from __future__ import annotations

from typing import Any, Literal

from pydantic import BaseModel, ConfigDict, Field

__all__ = [
    "BenchmarkCase",
    "BenchmarkSuite",
    "RegistryConfig",
    "ResultBundle",
    "RunMetadata",
    "ShapeCase",
    "ToleranceConfig",
]


class ShapeCase(BaseModel):
    """One problem size. For W4A16 suites ``m`` must be 1 and ``batch`` carries the GEMV rows."""

    model_config = ConfigDict(extra="allow")

    name: str
    m: int | None = None
    n: int | None = None
    k: int | None = None
    batch: int = 1

    def dimensions(self) -> dict[str, int]:
        dims = {"batch": int(self.batch)}
        for key in ("m", "n", "k"):
            value = getattr(self, key)
            if value is not None:
                dims[key] = int(value)
        for key, value in (self.model_extra or {}).items():
            if isinstance(value, int):
                dims[key] = value
        return dims

    def require_dimension(self, name: str) -> int:
        value = getattr(self, name, None)
        if value is None:
            raise ValueError(f"shape {self.name!r} is missing required dimension {name!r}")
        return int(value)


class ToleranceConfig(BaseModel):
    atol: float = 1e-3
    rtol: float = 1e-3


class RegistryConfig(BaseModel):
    ids: list[str] = Field(default_factory=list)


class BenchmarkSuite(BaseModel):
    schema_version: int = 1
    id: str
    family: str
    description: str
    metric: str = "latency_us"
    tags: list[str] = Field(default_factory=list)
    dtypes: list[str] = Field(default_factory=list)
    layouts: list[str] = Field(default_factory=list)
    shapes: list[ShapeCase] = Field(default_factory=list)
    kernels: RegistryConfig = Field(default_factory=RegistryConfig)
    baselines: RegistryConfig = Field(default_factory=RegistryConfig)
    tolerances: ToleranceConfig = Field(default_factory=ToleranceConfig)
    metadata: dict[str, Any] = Field(default_factory=dict)


class RunMetadata(BaseModel):
    schema_version: int = 2
    run_id: str
    suite_id: str
    created_at: str
    git_sha: str | None = None
    python_version: str
    platform: str
    machine: str
    native: dict[str, Any] = Field(default_factory=dict)
    nvidia_smi: dict[str, str] | None = None
    nvcc_version: str | None = None
    torch_version: str | None = None
    notes: list[str] = Field(default_factory=list)


class BenchmarkCase(BaseModel):
    case_id: str
    subject_kind: Literal["kernel", "baseline"]
    subject_id: str
    dtype: str
    layout: str
    shape_name: str
    dimensions: dict[str, int]
    status: Literal["ok", "skipped", "not_implemented", "failed"]
    latency_us_median: float | None = None
    latency_us_p95: float | None = None
    wall_latency_us_median: float | None = None
    wall_latency_us_p95: float | None = None
    device_latency_us_median: float | None = None
    device_latency_us_p95: float | None = None
    throughput: float | None = None
    decode_tokens_per_second: float | None = None
    speedup_vs: dict[str, float] = Field(default_factory=dict)
    metrics: dict[str, float] = Field(default_factory=dict)
    reason: str | None = None


class ResultBundle(BaseModel):
    schema_version: int = 2
    metadata: RunMetadata
    cases: list[BenchmarkCase] = Field(default_factory=list)
