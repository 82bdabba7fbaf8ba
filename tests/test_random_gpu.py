"""Random replay traces and random generation runs against the plain implementation: tiny
configuration, dtype, request lengths, way of cutting, page size, pool size, slots and token
budget are all drawn from a seeded generator, so a failure names the draw that showed it."""
import random

import pytest

from tests import traces
from tests.gpu_helpers import check_trace, make_requests, model_dir, plain_model
from tests.plain import lfm2_plain as P
from tests.test_generate_gpu import agree
from tests.test_replay_gpu import PAGE

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("draw", range(48))
def test_random_trace(draw):
    from imparo_b200.engine import Engine
    rng = random.Random(1000 + draw)
    name = "ABCDEF"[draw % 6]
    dtype = ["float32", "bfloat16"][(draw // 6) % 2]
    lengths = [rng.randint(3, 260) for _ in range(rng.randint(2, 7))]
    weights_seed = rng.randint(1, 2)
    reqs = make_requests(name, lengths, seed=rng.randint(0, 10 ** 6))
    kind = rng.choice(["mixed", "mixed", "mixed", "portions", "tail"])
    if kind == "mixed":
        steps = traces.mixed(reqs, seed=rng.randint(0, 10 ** 6), max_live=rng.randint(1, 4), tail=rng.randint(0, 40),
                             max_portion=rng.choice([2, 3, 5, 17, 40, 64, 130]))
    elif kind == "portions":
        steps = traces.portions(reqs, tuple(rng.randint(1, rng.choice([4, 20, 70])) for _ in range(rng.randint(3, 12))))
    else:
        steps = traces.tail_one_by_one(reqs, tail=rng.randint(1, 50))
    page = rng.choice([PAGE[name], 4, 8, 16, 32, 64])
    max_tokens = traces.max_live_tokens(steps, 64)
    eng = Engine(model_dir(name, weights_seed), dtype=dtype, ctx=max_tokens, parallel=4, page_size=page,
                 num_pages=(max_tokens + page - 1) // page, max_step_tokens=max(256, max_tokens))
    check_trace(eng, steps, name, reqs, dtype, seed=weights_seed)


@pytest.mark.parametrize("draw", range(24))
def test_random_generation(draw):
    """Continuous batching with a pool between one request's need and everyone's: portions under
    a random token budget, slots and pages used again, preemptions; greedy and seeded
    temperature picks must be the ones each request gets alone."""
    from imparo_b200.engine import Engine
    rng = random.Random(2000 + draw)
    name = "ABCDEF"[draw % 6]
    dtype = "bfloat16" if draw % 4 == 3 else "float32"
    n = rng.randint(1, 12)
    lens = [rng.randint(1, 90) for _ in range(n)]
    news = [rng.randint(0, 24) for _ in range(n)]
    temps = [rng.choice([0.0, 0.0, 0.7, 1.3]) for _ in range(n)]
    seeds = [rng.randint(0, 1000) for _ in range(n)]
    page = rng.choice([4, 8, 16, 32, 64])
    parallel = rng.randint(1, 6)
    longest = max(a + b for a, b in zip(lens, news))
    one = (longest + page - 1) // page
    num_pages = one + rng.randint(0, one * parallel)
    prompts = list(make_requests(name, lens, seed=rng.randint(0, 10 ** 6)).values())
    eng = Engine(model_dir(name), dtype=dtype, ctx=max(64, longest + 8), parallel=parallel, page_size=page,
                 num_pages=num_pages, max_step_tokens=rng.choice([2, 5, 8, 24, 64, 256]))
    got = eng.generate(prompts, max_tokens=news, temperature=temps, seed=seeds)
    assert eng.stats()["failed"] == []
    for i, p in enumerate(prompts):
        want, margins = P.generate(plain_model(name), p, news[i], temps[i], seeds[i])
        if temps[i] == 0:
            agree(got[i], want, margins, 1e-5 if dtype == "float32" else 2e-2)
        else:
            agree(got[i], want, margins, 1e-4 if dtype == "float32" else 5e-3)
    assert eng.cache.free_pages(0) == num_pages and eng.cache.free_slots() == parallel and eng.cache.n_requests() == 0
    eng.cache.check()
