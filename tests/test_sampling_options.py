"""Sampling options: the bounds of damendaemon/sampling.py:17-58, checked by this project's own rules table."""
import pytest

from damendaemon_b200.sampling import Sampler, Sampling


def test_defaults_are_greedy_and_unadjusted():
    o = Sampling()
    assert o.greedy and not o.has_penalties and not o.has_adjustments
    assert (o.temperature, o.top_p, o.top_k, o.seed) == (0, 1, 0, None)
    assert (o.presence_penalty, o.frequency_penalty, o.repetition_penalty, o.logit_bias) == (0, 0, 1, None)


@pytest.mark.parametrize("kw", [
    {"temperature": -0.1}, {"temperature": float("nan")}, {"temperature": float("inf")}, {"temperature": True},
    {"temperature": "1"}, {"temperature": 10 ** 400},
    {"top_p": 0}, {"top_p": 1.01}, {"top_p": None}, {"top_k": -1}, {"top_k": 2.0}, {"top_k": False},
    {"seed": -1}, {"seed": 2 ** 64}, {"seed": 1.0},
    {"presence_penalty": 2.5}, {"frequency_penalty": -2.5}, {"frequency_penalty": float("nan")},
    {"repetition_penalty": 0}, {"repetition_penalty": -1}, {"repetition_penalty": float("inf")},
    {"logit_bias": [1, 2]}, {"logit_bias": {"x": 1}}, {"logit_bias": {-1: 1}}, {"logit_bias": {"07": 1}},
    {"logit_bias": {" 7": 1}}, {"logit_bias": {"+7": 1}}, {"logit_bias": {"١": 1}}, {"logit_bias": {7: 101}},
    {"logit_bias": {7: float("nan")}}, {"logit_bias": {7: None}}, {"logit_bias": {7: 1, "7": 2}},
    {"logit_bias": {i: 0.5 for i in range(1025)}},
])
def test_rejected(kw):
    with pytest.raises(ValueError) as info:
        Sampling(**kw)
    assert next(iter(kw)) in str(info.value)        # the message names the field


@pytest.mark.parametrize("kw", [
    {"temperature": 0}, {"temperature": 2.5}, {"top_p": 1e-9}, {"top_p": 1}, {"top_k": 10 ** 9}, {"seed": 0},
    {"seed": 2 ** 64 - 1}, {"presence_penalty": -2}, {"frequency_penalty": 2}, {"repetition_penalty": 1e-3},
    {"logit_bias": {}}, {"logit_bias": {"0": -100, 5: 100}}, {"logit_bias": {i: 0.5 for i in range(1024)}},
])
def test_accepted(kw):
    Sampling(**kw)


def test_bias_keys_become_integers():
    assert Sampling(logit_bias={"12": 1.5, 3: -2}).logit_bias == {12: 1.5, 3: -2}


def test_sampler_state():
    s = Sampler(Sampling(temperature=0.8, seed=7, repetition_penalty=1.3, frequency_penalty=0.5, logit_bias={9: 2.0}))
    with pytest.raises(ValueError, match="vocabulary"):
        s.prepare([1, 2], 9)
    s.prepare([1, 2, 2], 50)
    for t in (2, 4, 4):
        s.observe(t)
    assert s.adjustments() == [(1, 0.0, 0.0, 1), (2, 1.0, 0.0, 1), (4, 2.0, 0.0, 1), (9, 0.0, 2.0, 0)]
    import random
    stream = random.Random(7)
    assert [s.draw() for _ in range(3)] == [stream.random() for _ in range(3)]
    s.prepare([5], 50)                  # taken in again: counts start over
    assert s.adjustments() == [(5, 0.0, 0.0, 1), (9, 0.0, 2.0, 0)]
    greedy = Sampler(Sampling())
    greedy.observe(3)
    assert greedy.random is None and greedy.draw() == 0.0 and greedy.adjustments() == []
