"""Running means of per-step engine metrics (reference: disagmoe/utils/metrics.py:3-21)."""
from dataclasses import dataclass


@dataclass
class Metric:
    effective_tokens: float = 0
    queueing_tokens: float = 0
    queueing_batches: float = 0
    t_schedule: float = 0
    t_step: float = 0
    t_preprocess: float = 0
    t_execute: float = 0
    t_postprocess: float = 0
    counter: int = 0

    def step(self) -> None:
        self.counter += 1

    def update(self, field_name: str, value: float) -> None:
        """Folds ``value`` into the running mean of ``field_name`` (call :meth:`step` first)."""
        n = max(self.counter, 1)
        old = getattr(self, field_name)
        setattr(self, field_name, old + (value - old) / n)
