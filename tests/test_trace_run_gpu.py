"""bin/trace_run as a program: its input and output protocol, in 32-bit and bfloat16,
compared with the plain implementation."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

from tests import traces
from tests.gpu_helpers import TOL, make_requests, model_dir, plain_logits
from tests.tiny_configs import ALL

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def replay(model, dtype, steps, out_dir, max_tokens):
    p = subprocess.Popen([os.path.join(ROOT, "bin", "trace_run"), "--model", model, "--dtype", dtype, "--out", str(out_dir),
                          "--max-tokens", str(max_tokens)], stdin=subprocess.PIPE, stdout=subprocess.PIPE,
                         stderr=subprocess.PIPE, text=True)
    try:
        for s in steps:
            p.stdin.write(json.dumps(s) + "\n")
            p.stdin.flush()
            line = p.stdout.readline().strip()          # the next step may come only after this
            assert line == f"done {s['step']}", (line, p.stderr.read()[-3000:] if p.poll() is not None else "")
        p.stdin.close()
        assert p.wait(timeout=120) == 0, p.stderr.read()[-3000:]
    finally:
        if p.poll() is None:
            p.kill()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["B", "C"])
def test_trace_run_mixed_with_page_reuse(tmp_path, name, dtype):
    reqs = make_requests(name, [70, 33, 90, 41, 64, 52], seed=7)
    steps = traces.mixed(reqs, seed=1)
    max_tokens = traces.max_live_tokens(steps, 64)
    assert max_tokens < sum(traces.round_up(len(t), 64) for t in reqs.values())
    out = tmp_path / "out"
    replay(model_dir(name), dtype, steps, out, max_tokens)
    ref = plain_logits(name, reqs)
    want = traces.expected(steps, ref)
    vocab = ALL[name]["vocab_size"]
    got = {}
    for s in steps:
        f = out / f"{s['step']}.f32"
        assert f.exists() == (s["step"] in want)
        if f.exists():
            got[s["step"]] = np.fromfile(f, dtype="<f4").reshape(-1, vocab)
            assert got[s["step"]].shape == want[s["step"]].shape
    scale = max(float(np.abs(v).max()) for v in ref.values())
    bad = traces.first_mismatch(steps, got, want, TOL[dtype] * scale)
    assert bad is None, bad


def test_trace_run_whole_then_decode_and_nothing_wanted(tmp_path):
    name = "A"
    toks = make_requests(name, [50], seed=3)["r0"]
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": toks[:18], "want": []}], "end": []},
             {"step": 1, "entries": [{"id": "x", "tokens": toks[18:20], "want": [1]}], "end": []},
             {"step": 2, "entries": [], "end": []}]
    steps += [{"step": 3 + i, "entries": [{"id": "x", "tokens": [toks[20 + i]], "want": [0]}], "end": ["x"] if i == 29 else []}
              for i in range(30)]
    out = tmp_path / "out"
    replay(model_dir(name), "float32", steps, out, 64)
    ref = plain_logits(name, {"x": toks})["x"]
    assert not (out / "0.f32").exists() and not (out / "2.f32").exists()
    scale = float(np.abs(ref).max())
    assert np.abs(np.fromfile(out / "1.f32", dtype="<f4") - ref[19]).max() <= TOL["float32"] * scale
    for i in range(30):
        assert np.abs(np.fromfile(out / f"{3 + i}.f32", dtype="<f4") - ref[20 + i]).max() <= TOL["float32"] * scale
