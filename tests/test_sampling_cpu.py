"""Sampling options and the counter-based uniform numbers (CPU)."""
import pytest

from braidinfer_b200.sampling import SamplingParams, uniform


def test_defaults_and_greedy_are_the_references():
    p = SamplingParams()
    assert (p.temperature, p.top_k, p.top_p, p.repetition_penalty, p.seed, p.min_p, p.logit_bias) == \
           (1.0, 50, 1.0, 1.0, None, 0.0, None)
    g = SamplingParams.greedy()
    assert g.temperature == 0.0 and g.top_k == 0 and g.is_plain_greedy
    assert not SamplingParams(temperature=0.0, repetition_penalty=1.3).is_plain_greedy


@pytest.mark.parametrize("kw", [{"temperature": -1}, {"top_k": -2}, {"top_p": 0.0}, {"top_p": 1.5},
                                {"min_p": 2.0}, {"repetition_penalty": 0.0}])
def test_refuses_bad_options(kw):
    with pytest.raises(ValueError):
        SamplingParams(**kw)


def test_uniform_is_a_function_of_seed_sequence_and_step():
    a = uniform(1, 0, 0)
    assert a == uniform(1, 0, 0) and 0.0 < a < 1.0
    assert len({uniform(1, s, t) for s in range(20) for t in range(20)}) == 400
    assert uniform(2, 0, 0) != a
    xs = [uniform(9, 3, t) for t in range(4000)]
    assert abs(sum(xs) / len(xs) - 0.5) < 0.02
    import numpy as np
    assert all(float(np.float32(x)) == x for x in xs[:100])        # exact in float32
