"""Density parameters of the H3 Sparse Attention (and Advanced) nodes.

The field names, defaults, constants and error texts are the contract of the
reference's node parameters (attention/sparse/config.py:25-129); how a budget
is validated and resolved is organised here as a short list of rules, each a
function that either decides the budget of a (sampler step, layer) or passes.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

H3_LAYER_COUNT = 50
MODE_SAGE128 = "sage128"
MODE_SAGE128_FUSED_QKV = "sage128_fused_qkv"
IMPLEMENTED_MODES = (MODE_SAGE128, MODE_SAGE128_FUSED_QKV)
DENSITY_FIXED = "fixed"
DENSER_EARLY_LATE_STEP_COUNT = 2
DENSER_EARLY_LATE_BONUS = 0.30

_WINDOW_FIELDS = ("early_steps", "early_kv", "late_steps", "late_kv")


def _density(name, value):
    """A KV density as float; ``None`` passes through."""
    if value is None:
        return None
    number = float(value)
    if not (math.isfinite(number) and 0.01 <= number <= 1.0):
        raise ValueError("%s must be finite and in [0.01, 1]" % name)
    return number


def _step_count(name, value):
    if isinstance(value, bool) or int(value) != value or int(value) < 0:
        raise ValueError("%s must be a non-negative integer" % name)
    return int(value)


@dataclass(frozen=True)
class HybridSparseConfig:
    mode: str = MODE_SAGE128
    video_budget: float = 0.5
    strict: bool = True
    density_mode: str = DENSITY_FIXED
    denser_early_late_steps: bool = False
    early_steps: int | None = None
    early_kv: float | None = None
    late_steps: int | None = None
    late_kv: float | None = None
    layer_video_budgets: tuple | None = None

    def __post_init__(self):
        if self.mode not in IMPLEMENTED_MODES:
            raise ValueError("sparse mode %r is unavailable; implemented modes: %s"
                             % (self.mode, ", ".join(IMPLEMENTED_MODES)))
        if self.density_mode != DENSITY_FIXED:
            raise ValueError("only fixed Sparse Sage density is supported")
        for name in ("video_budget", "early_kv", "late_kv"):
            _density(name, getattr(self, name))

        table = self.layer_video_budgets
        if table is not None:
            table = tuple(float(entry) for entry in table)
            if len(table) != H3_LAYER_COUNT:
                raise ValueError("layer_video_budgets must contain exactly %d values" % H3_LAYER_COUNT)
            for layer, entry in enumerate(table):
                _density("layer_video_budgets[%d]" % layer, entry)
            object.__setattr__(self, "layer_video_budgets", table)

        given = [name for name in _WINDOW_FIELDS if getattr(self, name) is not None]
        if given:
            if len(given) != len(_WINDOW_FIELDS):
                raise ValueError("explicit early/late sparse schedule is incomplete")
            if self.denser_early_late_steps:
                raise ValueError("legacy and explicit early/late schedules cannot be combined")
            _step_count("early_steps", self.early_steps)
            _step_count("late_steps", self.late_steps)
        if table is not None and (given or self.denser_early_late_steps):
            raise ValueError("static per-layer budgets cannot be combined with early/late schedules")

    @property
    def has_windows(self):
        return self.early_steps is not None

    @property
    def signature(self):
        def cast(kind, value):
            return None if value is None else kind(value)

        return (
            self.mode, float(self.video_budget), bool(self.strict), self.density_mode,
            bool(self.denser_early_late_steps),
            cast(int, self.early_steps), cast(float, self.early_kv),
            cast(int, self.late_steps), cast(float, self.late_kv),
            self.layer_video_budgets,
        )


# -- budget rules, tried in this order; the first that answers wins -------------


def _from_layer_table(config, step, total, layer):
    table = config.layer_video_budgets
    if table is None:
        return None
    if layer is None:
        raise ValueError("layer_index is required for static per-layer budgets")
    if isinstance(layer, bool) or int(layer) != layer:
        raise ValueError("layer_index must be an integer")
    if not 0 <= int(layer) < len(table):
        raise ValueError("layer_index is outside the static per-layer budget table")
    return table[int(layer)]


def _outside_the_run(config, step, total, layer):
    """An unknown step (-1), an empty run or a step past its end: base budget."""
    if step < 0 or total <= 0 or step >= total:
        return float(config.video_budget)
    return None


def _from_windows(config, step, total, layer):
    if not config.has_windows:
        return None
    hits = []
    if step < int(config.early_steps):
        hits.append(float(config.early_kv))
    if step >= total - int(config.late_steps):
        hits.append(float(config.late_kv))
    # inside both windows the denser one applies; outside both the base budget
    return max(hits) if hits else float(config.video_budget)


def _from_legacy_bonus(config, step, total, layer):
    if not config.denser_early_late_steps:
        return None
    edge = DENSER_EARLY_LATE_STEP_COUNT
    if step < edge or step >= total - edge:
        return min(1.0, float(config.video_budget) + DENSER_EARLY_LATE_BONUS)
    return None


_RULES = (_from_layer_table, _outside_the_run, _from_windows, _from_legacy_bonus)


def resolve_video_budget(config, step_index, total_steps, layer_index=None):
    """Video-KV budget of one (sampler step, layer): static per-layer table,
    else the base budget outside ``[0, total_steps)``, else explicit early/late
    windows, else the legacy bonus on the first and last two steps, else the
    base budget (attention/sparse/config.py:94-129)."""
    step, total = int(step_index), int(total_steps)
    for rule in _RULES:
        budget = rule(config, step, total, layer_index)
        if budget is not None:
            return float(budget)
    return float(config.video_budget)
