"""Shared pieces of the GPU tests: model folders, plain logits, running a trace through the
engine's step function, tolerances."""
import functools
import os
import tempfile

import numpy as np

from tests import traces
from tests.plain.lfm2_plain import PlainLfm2
from tests.tiny_configs import ALL

# Tolerances, as a fraction of the largest |logit| of the compared request.
# float32: every reduction is 32-bit; measured error is ~1e-6 of the scale.
# bfloat16: 8-bit mantissas on weights-times-activations through up to 6 layers; measured
# error is ~5e-3 of the scale.
TOL = {"float32": 2e-5, "bfloat16": 2.5e-2}

_tmp = tempfile.TemporaryDirectory(prefix="imparo_b200_tests_")


@functools.lru_cache(maxsize=None)
def model_dir(name, seed=1):
    from imparo_b200.weights import write_random_model
    d = os.path.join(_tmp.name, f"{name}_{seed}")
    write_random_model(d, ALL[name], seed=seed, dtype="bfloat16")
    return d


@functools.lru_cache(maxsize=None)
def plain_model(name, seed=1):
    return PlainLfm2(model_dir(name, seed), np.float64)


def make_requests(name, lengths, seed=0):
    rng = np.random.default_rng(seed)
    vocab = ALL[name]["vocab_size"]
    return {f"r{i}": rng.integers(0, vocab, n).tolist() for i, n in enumerate(lengths)}


_plain_cache = {}


def plain_logits(name, requests, seed=1):
    out = {}
    m = plain_model(name, seed)
    for rid, toks in requests.items():
        key = (name, seed, tuple(toks))
        if key not in _plain_cache:
            _plain_cache[key] = m.logits(toks)
        out[rid] = _plain_cache[key]
    return out


def run_trace(engine, steps):
    """Feeds a trace to Engine.step the way bin/trace_run does.  -> {step: logits array}"""
    from imparo_b200.engine import StepItem
    ids, out = {}, {}
    counter = [getattr(engine, "_test_next_id", 1)]
    for s in steps:
        items = []
        for e in s["entries"]:
            if e["id"] not in ids:
                ids[e["id"]] = counter[0]
                counter[0] += 1
                engine.add_request(ids[e["id"]])
            items.append(StepItem(ids[e["id"]], e["tokens"], e["want"]))
        logits = engine.step(items)
        if logits is not None:
            out[s["step"]] = logits.cpu().numpy()
        for name in s["end"]:
            engine.end_request(ids.pop(name))
    engine._test_next_id = counter[0]
    engine.check_device_status()
    engine.cache.check()
    return out


def check_trace(engine, steps, name, requests, dtype, seed=1):
    ref = plain_logits(name, requests, seed)
    want = traces.expected(steps, ref)
    got = run_trace(engine, steps)
    assert sorted(got) == sorted(want)
    scale = max(float(np.abs(v).max()) for v in ref.values())
    bad = traces.first_mismatch(steps, got, want, TOL[dtype] * scale)
    assert bad is None, (f"first wrong place: step {bad[0]}, request {bad[1]}, position {bad[2]}, "
                         f"error {bad[3]:.3e} > {TOL[dtype] * scale:.3e}")
    assert engine.cache.n_requests() == 0
    return got
