"""Sampling options of a request, with celeg's names, meanings and defaults
(``GenerationConfig``: include/celeg/model/runtime_types.hpp:98-108; limits in
src/backend/cpu/sampler.cpp:26-101)."""
from __future__ import annotations

from dataclasses import dataclass

MAX_TOP_K = 128        # celeg's kMaxTopK


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.1          # <= 0: greedy
    top_k: int = 50                   # 1: greedy; at most 128
    top_p: float = 1.0                # (0, 1]
    repetition_penalty: float = 1.05  # >= 1; applies to tokens of the prompt and generated ones
    seed: int = 1                     # non-zero 64-bit state of the request's xorshift64* generator

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0 or self.top_k == 1

    def validate(self) -> None:
        if not self.temperature >= 0.0 and not self.temperature <= 0.0:
            raise ValueError("temperature must be a number")
        if not 1 <= self.top_k <= MAX_TOP_K:
            raise ValueError(f"top_k must lie in 1..{MAX_TOP_K}, got {self.top_k}")
        if not 0.0 < self.top_p <= 1.0:
            raise ValueError(f"top_p must lie in (0, 1], got {self.top_p}")
        if not self.repetition_penalty >= 1.0:
            raise ValueError(f"repetition_penalty must be at least 1, got {self.repetition_penalty}")
        if not 0 < self.seed < 2 ** 64:
            raise ValueError(f"seed must be a non-zero unsigned 64-bit integer, got {self.seed}")


GREEDY = SamplingParams(temperature=0.0, top_k=1, top_p=1.0, repetition_penalty=1.0, seed=1)
