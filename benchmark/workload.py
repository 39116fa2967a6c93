"""Request arrival generators (reference: benchmark/workload.py:46-111): uniform, Poisson, offline (all at t = 0)
and incremental Poisson (the rate grows by ``increment`` every ``interval`` seconds)."""
from __future__ import annotations

from typing import List, Sequence, Tuple

import numpy as np


class Workload:
    def __init__(self, arrivals: Sequence[float], input_lens: Sequence[int], output_lens: Sequence[int] = ()):
        self.arrivals = list(map(float, arrivals))
        self.input_lens = list(map(int, input_lens))
        self.output_lens = list(map(int, output_lens))

    def __len__(self):
        return len(self.arrivals)

    def __getitem__(self, i) -> Tuple[float, int]:
        return self.arrivals[i], self.input_lens[i]

    def __iter__(self):
        for i in range(len(self)):
            yield self[i]


class Generator:
    def __init__(self, rate: float, cv: float, min_input_len: int, max_input_len: int, seed: int = 0,
                 min_output_len: int = 0, max_output_len: int = 0):
        self.rate, self.cv = rate, cv
        self.min_input_len, self.max_input_len = min_input_len, max_input_len
        self.min_output_len, self.max_output_len = min_output_len, max_output_len
        self.rng = np.random.default_rng(seed)

    def generate_arrivals(self, n_request: int) -> np.ndarray:
        raise NotImplementedError

    def generate_input_lens(self, n_request: int) -> np.ndarray:
        return self.rng.integers(self.min_input_len, max(self.max_input_len, self.min_input_len + 1), n_request)

    def generate_output_lens(self, n_request: int) -> np.ndarray:
        if self.max_output_len <= 0:
            return np.zeros(0, dtype=int)
        return self.rng.integers(self.min_output_len, max(self.max_output_len, self.min_output_len + 1), n_request)

    def get_num_requests(self, duration: float) -> int:
        return int(duration * self.rate)

    def generate_duration(self, duration: float) -> Workload:
        return self.generate_num(self.get_num_requests(duration))

    def generate_num(self, num: int) -> Workload:
        return Workload(self.generate_arrivals(num), self.generate_input_lens(num), self.generate_output_lens(num))


class UniformGenerator(Generator):
    def generate_arrivals(self, n_request):
        return np.arange(n_request) / self.rate


class PoissonGenerator(Generator):
    def generate_arrivals(self, n_request):
        return np.cumsum(self.rng.exponential(1.0 / self.rate, n_request))


class OfflineGenerator(Generator):
    def generate_arrivals(self, n_request):
        return np.zeros(n_request)


class IncrementalPoissonGenerator(Generator):
    increment: float = 2.0
    interval: float = 60.0

    def get_num_requests(self, duration):
        n, rate = 0, self.rate
        while duration > 0:
            span = min(self.interval, duration)
            n += int(span * rate)
            duration -= span
            rate += self.increment
        return n

    def generate_arrivals(self, n_request):
        out: List[float] = []
        t0, rate = 0.0, self.rate
        while len(out) < n_request:
            k = int(min(rate * self.interval, n_request - len(out)))
            if k <= 0:
                break
            out.extend((t0 + np.cumsum(self.rng.exponential(1.0 / rate, k))).tolist())
            rate += self.increment
            t0 += self.interval
        return np.asarray(out[:n_request])


def get_generator(name: str):
    return {"uniform": UniformGenerator, "poisson": PoissonGenerator, "offline": OfflineGenerator,
            "incremental_poisson": IncrementalPoissonGenerator}[name]
