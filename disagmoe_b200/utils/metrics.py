"""Per-step engine metrics as running means (the fields of the reference's ``Metric``, disagmoe/utils/metrics.py:3-21).

Every field keeps its own sum and sample count, so a field that is only fed on some steps (the queue snapshot exists
only with tracing on; timers that did not run in a step) is averaged over the steps that fed it, not over all steps.
``counter`` counts engine steps."""
from typing import Dict

FIELDS = ("effective_tokens", "queueing_tokens", "queueing_batches", "t_schedule", "t_step", "t_preprocess", "t_execute",
          "t_postprocess")


class Metric:
    def __init__(self) -> None:
        self.counter = 0
        self._sum: Dict[str, float] = dict.fromkeys(FIELDS, 0.0)
        self._n: Dict[str, int] = dict.fromkeys(FIELDS, 0)

    def step(self) -> None:
        self.counter += 1

    def update(self, field_name: str, value: float) -> None:
        if field_name not in self._sum:
            raise KeyError(f"unknown metric {field_name!r}; one of {FIELDS}")
        self._sum[field_name] += float(value)
        self._n[field_name] += 1

    def __getattr__(self, name: str) -> float:
        # only reached for names that are not real attributes: the metric fields read as their current mean
        if name.startswith("_") or name not in FIELDS:
            raise AttributeError(name)
        n = self._n[name]
        return self._sum[name] / n if n else 0.0

    def as_dict(self) -> Dict[str, float]:
        out = {f: getattr(self, f) for f in FIELDS}
        out["counter"] = self.counter
        return out

    def __repr__(self) -> str:
        return "Metric(" + ", ".join(f"{k}={v:.4g}" for k, v in self.as_dict().items()) + ")"
