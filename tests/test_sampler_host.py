from imparo_b200.sampling import uniform_for


def test_uniform_is_a_pure_function_in_range():
    seen = set()
    for seed in range(20):
        for step in range(50):
            u = uniform_for(seed, step)
            assert 0.0 <= u < 1.0 and u == uniform_for(seed, step)
            seen.add(u)
    assert len(seen) > 990
    vals = [uniform_for(7, s) for s in range(4000)]
    assert 0.45 < sum(vals) / len(vals) < 0.55
