"""Per-request runtime snapshot the backend reads from ``transformer_options``
(reference: runtime/context.py:12,20-32,140-144)."""

from __future__ import annotations

from dataclasses import dataclass

RUNTIME_KEY = "h3_optimizations_runtime"


@dataclass(frozen=True)
class RuntimeSnapshot:
    request_id: int
    step_index: int
    total_steps: int
    layout: object | None
    compute_dtype: object | None
    device: object | None
    error: str | None = None

    @property
    def valid_layout(self):
        return self.layout is not None and self.error is None


def get_runtime_snapshot(transformer_options):
    if not transformer_options:
        return None
    value = transformer_options.get(RUNTIME_KEY)
    # the reference's own RuntimeSnapshot class is accepted as well (duck-typed)
    if value is not None and all(hasattr(value, n) for n in ("step_index", "total_steps", "layout")):
        return value
    return None


def runtime_options(layout, step_index=-1, total_steps=0, dtype=None, device=None):
    return {
        RUNTIME_KEY: RuntimeSnapshot(
            request_id=0, step_index=int(step_index), total_steps=int(total_steps),
            layout=layout, compute_dtype=dtype, device=device,
        )
    }
