"""The counter-based uniform numbers of temperature sampling (no GPU)."""
from beglin_b200.sampling import request_key, uniform


def test_uniform_is_a_pure_function_in_range():
    us = [uniform(1, "a", s) for s in range(2000)]
    assert all(0.0 <= u < 1.0 for u in us)
    assert us == [uniform(1, "a", s) for s in range(2000)]
    assert abs(sum(us) / len(us) - 0.5) < 0.03
    assert len(set(us)) > 1990
    assert uniform(1, "a", 5) != uniform(2, "a", 5) and uniform(1, "a", 5) != uniform(1, "b", 5)
    assert request_key(7) == 7 and request_key("x") == request_key("x")
