"""Sampling options and per-request sampler state.

The option names, their defaults and their bounds are the reference's interface
(damendaemon/sampling.py:17-58): temperature 0 = greedy, top_p in (0, 1], top_k 0 = off, a seed
below 2**64, presence/frequency penalties in [-2, 2], a positive repetition penalty, at most 1,024
biased tokens with biases in [-100, 100]. How they are checked is this project's: one table of
(field, accepted type, range) walked once, and messages that quote the offending value.
The random stream is per request and never the global one (damendaemon/sampling.py:72-73).
"""
from __future__ import annotations

import random
from collections import Counter
from dataclasses import dataclass, fields

MAX_BIASED_TOKENS = 1024
INF = float("inf")


@dataclass(frozen=True)
class _Range:
    """An interval of real numbers with open or closed ends; ``whole`` asks for an int."""
    low: float
    high: float
    low_open: bool = False
    high_open: bool = False
    whole: bool = False
    optional: bool = False

    def holds(self, value) -> bool:
        if value is None:
            return self.optional
        # bool is an int to Python but not a number to a caller; huge ints compare exactly, no float() needed
        if type(value) is not int and (self.whole or type(value) is not float):
            return False
        if value != value:           # NaN
            return False
        if type(value) is int and not self.whole and value.bit_length() > 1000:
            return False             # an integer too large to become a float (JSON allows them)
        above = value > self.low if self.low_open else value >= self.low
        below = value < self.high if self.high_open else value <= self.high
        return above and below

    def __str__(self):
        kind = "an integer" if self.whole else "a number"
        left = "(" if self.low_open or self.low == -INF else "["
        right = ")" if self.high_open or self.high == INF else "]"
        text = f"{kind} in {left}{self.low:g}, {self.high:g}{right}"
        return text + " or None" if self.optional else text


RULES = {
    "temperature": _Range(0, INF, high_open=True),
    "top_p": _Range(0, 1, low_open=True),
    "top_k": _Range(0, INF, high_open=True, whole=True),
    "seed": _Range(0, 2 ** 64, high_open=True, whole=True, optional=True),
    "presence_penalty": _Range(-2, 2),
    "frequency_penalty": _Range(-2, 2),
    "repetition_penalty": _Range(0, INF, low_open=True, high_open=True),
}
BIAS_VALUE = _Range(-100, 100)


def _token_key(key):
    """A bias table may come from JSON, whose keys are strings: '17' means token 17. Anything that is not
    the canonical decimal spelling of a non-negative integer (' 17', '+17', '017', '١٧') is refused."""
    if type(key) is int:
        return key if key >= 0 else None
    if isinstance(key, str) and key.isascii() and key.isdigit() and (key == "0" or key[0] != "0"):
        return int(key)
    return None


def _checked_bias(table):
    if not isinstance(table, dict):
        raise ValueError(f"logit_bias: a dict of token id -> bias is expected, not {type(table).__name__}")
    if len(table) > MAX_BIASED_TOKENS:
        raise ValueError(f"logit_bias: {len(table)} tokens given, at most {MAX_BIASED_TOKENS} are taken")
    out = {}
    for key, value in table.items():
        token = _token_key(key)
        if token is None:
            raise ValueError(f"logit_bias: {key!r} is not a token id")
        if token in out:
            raise ValueError(f"logit_bias: token {token} is given twice")
        if not BIAS_VALUE.holds(value):
            raise ValueError(f"logit_bias: the bias of token {token} is {value!r}; {BIAS_VALUE} is expected")
        out[token] = value
    return out


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
        for f in fields(self):
            rule = RULES.get(f.name)
            value = getattr(self, f.name)
            if rule is not None and not rule.holds(value):
                raise ValueError(f"{f.name} is {value!r}; {rule} is expected")
        if self.logit_bias is not None:
            object.__setattr__(self, "logit_bias", _checked_bias(self.logit_bias))

    @property
    def greedy(self):
        return self.temperature == 0

    @property
    def has_penalties(self):
        return self.presence_penalty != 0 or self.frequency_penalty != 0 or self.repetition_penalty != 1

    @property
    def has_adjustments(self):
        return self.has_penalties or bool(self.logit_bias)


class Sampler:
    """One request's sampling state: its random stream and the tokens it has seen."""

    def __init__(self, options: Sampling):
        self.options = options
        self.random = None if options.greedy else random.Random(options.seed)
        self.prompt_tokens = frozenset()
        self.counts = Counter()

    def prepare(self, prompt, vocab_size):
        """Called once when the request is taken in: the bias table is held against the model's vocabulary and
        the prompt's tokens are remembered if the repetition penalty will want them."""
        beyond = [t for t in (self.options.logit_bias or ()) if t >= vocab_size]
        if beyond:
            raise ValueError(f"logit_bias: token {min(beyond)} is outside the vocabulary of {vocab_size}")
        self.prompt_tokens = frozenset(prompt) if self.options.repetition_penalty != 1 else frozenset()
        self.counts = Counter()

    def observe(self, token):
        """A token was generated for this request."""
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
