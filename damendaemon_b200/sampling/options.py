"""Sampling options and per-request sampler state. Names, defaults and bounds are the
reference's (damendaemon/sampling.py:17-58); the random stream is per request and never
the global one (damendaemon/sampling.py:72-73)."""
from __future__ import annotations

import math
import random
from collections import Counter
from dataclasses import dataclass


def _finite(value):
    if type(value) not in (float, int):
        return False
    try:
        return math.isfinite(value)
    except OverflowError:
        return False


@dataclass(frozen=True)
class Sampling:
    temperature: float = 0
    top_p: float = 1
    top_k: int = 0
    seed: int | None = None
    presence_penalty: float = 0
    frequency_penalty: float = 0
    repetition_penalty: float = 1
    logit_bias: dict | None = None

    def __post_init__(self):
        for name in ("temperature", "top_p"):
            if not _finite(getattr(self, name)):
                raise ValueError(f"{name} must be a finite number")
        if self.temperature < 0 or not 0 < self.top_p <= 1:
            raise ValueError("temperature must be nonnegative and top_p must be in (0, 1]")
        if type(self.top_k) is not int or self.top_k < 0:
            raise ValueError("top_k must be a nonnegative integer")
        if self.seed is not None and (type(self.seed) is not int or not 0 <= self.seed < 2 ** 64):
            raise ValueError("seed must be an integer in [0, 2**64)")
        for name in ("presence_penalty", "frequency_penalty", "repetition_penalty"):
            value = getattr(self, name)
            if not _finite(value):
                raise ValueError(f"{name} must be finite")
            if (name == "repetition_penalty" and value <= 0) or (name != "repetition_penalty" and not -2 <= value <= 2):
                raise ValueError("invalid token penalty")
        bias = self.logit_bias
        if bias is not None:
            if not isinstance(bias, dict) or len(bias) > 1024:
                raise ValueError("logit_bias must contain at most 1024 token entries")
            normal = {}
            for key, value in bias.items():
                if isinstance(key, str) and key.isascii() and key.isdecimal() and str(int(key)) == key:
                    key = int(key)
                if type(key) is not int or key < 0 or key in normal or not _finite(value) or not -100 <= value <= 100:
                    raise ValueError("invalid logit bias token or value")
                normal[key] = value
            object.__setattr__(self, "logit_bias", normal)

    @property
    def greedy(self):
        return not self.temperature

    @property
    def has_penalties(self):
        return bool(self.presence_penalty or self.frequency_penalty or self.repetition_penalty != 1)

    @property
    def has_adjustments(self):
        return self.has_penalties or bool(self.logit_bias)


class Sampler:
    """One request's sampling state: its random stream and the tokens it has seen."""

    def __init__(self, options: Sampling):
        self.options = options
        self.random = random.Random(options.seed) if options.temperature else None
        self.prompt_tokens = set()
        self.counts = Counter()

    def prepare(self, prompt, vocab_size):
        if any(token >= vocab_size for token in (self.options.logit_bias or {})):
            raise ValueError("logit_bias token exceeds model vocabulary")
        if self.options.repetition_penalty != 1:
            self.prompt_tokens = set(prompt)
        self.counts.clear()

    def observe(self, token):
        if self.options.has_penalties:
            self.counts[token] += 1

    def draw(self) -> float:
        """The next uniform number of this request's stream, in [0, 1)."""
        return self.random.random() if self.random is not None else 0.0

    def adjustments(self):
        """[(token, generated count, bias, seen)] for every token whose logit changes."""
        o = self.options
        if not o.has_adjustments:
            return []
        tokens = set(self.counts)
        if o.repetition_penalty != 1:
            tokens |= self.prompt_tokens
        if o.logit_bias:
            tokens |= set(o.logit_bias)
        return [(t, float(self.counts.get(t, 0)), float((o.logit_bias or {}).get(t, 0.0)),
                 1 if (t in self.counts or t in self.prompt_tokens) else 0) for t in sorted(tokens)]
