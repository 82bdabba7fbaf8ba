"""Generation through the Python entry point and the command line against the plain
implementation: greedy and seeded temperature sampling, continuous batching with prompt
portions beside decode tokens, few pages."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

from tests.gpu_helpers import TOL, make_requests, model_dir, plain_model
from tests.plain import lfm2_plain as P

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def agree(got, want, margins, min_margin):
    """Same tokens, except that a pick the plain implementation made by less than
    min_margin may go the other way; after that the sequences legitimately differ."""
    for i, (g, w) in enumerate(zip(got, want)):
        if g != w:
            assert margins[i] < min_margin, f"token {i}: {g} != {w} with margin {margins[i]:.3e}"
            return
    if len(got) != len(want):       # one of them met a stop token where the other picked differently
        n = min(len(got), len(want))
        assert n < len(margins) and margins[n] < min_margin, f"{len(got)} tokens, expected {len(want)}"


@pytest.mark.parametrize("dtype,min_margin", [("float32", 1e-5), ("bfloat16", 2e-2)])
def test_tiny_a_greedy_16_plus_8(dtype, min_margin):
    from imparo_b200.engine import Engine
    prompt = make_requests("A", [16], seed=0)["r0"]
    eng = Engine(model_dir("A"), dtype=dtype, ctx=64, parallel=2, page_size=16, num_pages=4)
    got = eng.generate([prompt], max_tokens=8)[0]
    want, margins = P.generate(plain_model("A"), prompt, 8)
    agree(got, want, margins, min_margin)
    assert eng.cache.n_requests() == 0 and eng.cache.free_pages(0) == 4


@pytest.mark.parametrize("dtype,min_margin", [("float32", 1e-5), ("bfloat16", 2e-2)])
def test_tiny_b_mixed_batch_greedy_and_temperature(dtype, min_margin):
    """3 requests (5, 23, 40 tokens), portions of 8 beside running decodes, 12 new tokens
    each, greedy for one and temperature 0.8 (seeded) for two, pages of 4 tokens."""
    from imparo_b200.engine import Engine
    reqs = make_requests("B", [5, 23, 40], seed=1)
    prompts = list(reqs.values())
    temps, seeds = [0.0, 0.8, 0.8], [0, 11, 12]
    eng = Engine(model_dir("B"), dtype=dtype, ctx=64, parallel=3, page_size=4, num_pages=40, max_step_tokens=8)
    seen = []
    got = eng.generate(prompts, max_tokens=12, temperature=temps, seed=seeds, on_step=lambda plan: seen.append(plan))
    for i in range(3):
        want, margins = P.generate(plain_model("B"), prompts[i], 12, temps[i], seeds[i])
        agree(got[i], want, margins, min_margin if temps[i] == 0 else 1e-4 if dtype == "float32" else 5e-3)
    # portions ran beside decode tokens, under the budget
    assert all(sum(e.count for e in plan) <= 8 for plan in seen)
    assert any(any(e.count == 1 and e.want for e in plan) and any(e.count > 1 for e in plan) for plan in seen)
    assert eng.cache.n_requests() == 0 and eng.cache.free_pages(0) == 40
    eng.cache.check()


def test_pages_run_out_during_generation_requests_are_recomputed():
    """So few pages that running requests are preempted; every request still gets the
    tokens it would get alone."""
    from imparo_b200.engine import Engine
    reqs = make_requests("A", [30, 41, 22, 35], seed=4)
    prompts = list(reqs.values())
    eng = Engine(model_dir("A"), dtype="float32", ctx=128, parallel=4, page_size=4, num_pages=34, max_step_tokens=32)
    got = eng.generate(prompts, max_tokens=24)
    assert eng.stats()["preemptions"] >= 1
    for i, p in enumerate(prompts):
        want, margins = P.generate(plain_model("A"), p, 24)
        agree(got[i], want, margins, 1e-5)
    assert eng.cache.free_pages(0) == 34 and eng.cache.free_slots() == 4
    eng.cache.check()


def test_a_request_larger_than_the_pool_fails_alone():
    from imparo_b200.engine import Engine
    eng = Engine(model_dir("A"), dtype="float32", ctx=512, parallel=2, page_size=4, num_pages=8)
    reqs = make_requests("A", [60, 10], seed=6)
    got = eng.generate(list(reqs.values()), max_tokens=4)
    assert eng.stats()["failed"] == [0] and got[0] == [] and len(got[1]) == 4
    assert eng.cache.free_pages(0) == 8


def test_stop_token_and_zero_max_tokens():
    from imparo_b200.engine import Engine
    prompt = make_requests("A", [12], seed=2)["r0"]
    eng = Engine(model_dir("A"), dtype="float32", ctx=64, parallel=2)
    free = eng.generate([prompt], max_tokens=10)[0]
    stopped = eng.generate([prompt], max_tokens=10, stop_token_ids=[free[3]])[0]
    assert stopped == free[:free.index(free[3])]
    assert eng.generate([prompt, prompt], max_tokens=[0, 2]) == [[], free[:2]]


def test_command_line_generates_the_same_tokens(tmp_path):
    prompt = make_requests("A", [16], seed=0)["r0"]
    want, _ = P.generate(plain_model("A"), prompt, 8)
    tf = tmp_path / "tokens.txt"
    tf.write_text(" ".join(map(str, prompt)))
    r = subprocess.run([sys.executable, "-m", "imparo_b200", "-m", model_dir("A"), "--dtype", "float32", "--decode", "8",
                        "-c", "64", "-t", str(tf), "--json"], cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert json.loads(r.stdout.strip().splitlines()[-1])["tokens"] == [want]


def test_many_requests_few_pages_every_request_gets_its_own_tokens():
    """24 requests of random lengths through 5 slots and a pool far smaller than their sum:
    portions beside decode rows, slots and pages used again, preemptions.  Every request must
    get the tokens it gets alone (32-bit, greedy)."""
    from imparo_b200.engine import Engine
    rng = np.random.default_rng(9)
    lens = [int(x) for x in rng.integers(3, 60, 24)]
    reqs = make_requests("B", lens, seed=13)
    prompts = list(reqs.values())
    news = [int(x) for x in rng.integers(1, 20, 24)]
    eng = Engine(model_dir("B"), dtype="float32", ctx=96, parallel=5, page_size=4, num_pages=70, max_step_tokens=24)
    seen = []
    got = eng.generate(prompts, max_tokens=news, on_step=lambda plan: seen.append(plan))
    for i, p in enumerate(prompts):
        want, margins = P.generate(plain_model("B"), p, news[i])
        agree(got[i], want, margins, 1e-5)
    assert max(len(plan) for plan in seen) == 5                      # all slots were in use at once
    assert all(sum(e.count for e in plan) <= 24 for plan in seen)
    assert eng.stats()["failed"] == []
    assert eng.cache.free_pages(0) == 70 and eng.cache.free_slots() == 5 and eng.cache.n_requests() == 0
    eng.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("layer", [0, 1, 5])
def test_stage_probe_against_the_plain_implementation(dtype, layer):
    """Engine(probe_layer=i) shows the stages of one block; the plain implementation shows the same
    stages by the same names: a whole prompt, stage by stage."""
    from imparo_b200.engine import Engine, StepItem
    name = "B"
    toks = np.random.default_rng(11).integers(0, 512, 37).tolist()
    seen = {}
    eng = Engine(model_dir(name), dtype=dtype, ctx=128, parallel=1, page_size=4, probe_layer=layer,
                 probe=lambda n, t: seen.__setitem__(n, t.detach().float().cpu().numpy().copy()))
    eng.add_request(1)
    got_logits = eng.step([StepItem(1, toks, [len(toks) - 1])]).cpu().numpy()
    eng.end_request(1)
    ref = {}
    plain = plain_model(name)
    plain.hidden_states(toks, probe_layer=layer, probe=lambda n, a: ref.__setitem__(n, np.asarray(a, dtype=np.float64)))
    assert list(seen) == ["stream_in", "mixer_norm", "stream_mixer", "ff_norm", "stream_out"] == list(ref)
    tol = TOL[dtype]
    for n in ref:
        a, b = seen[n], ref[n]
        if a.shape[0] != b.shape[0]:                 # the model's last block shows the wanted rows only from its feed-forward on
            b = b[-a.shape[0]:]
        assert a.shape == b.shape, n
        assert np.abs(a - b).max() <= 4 * tol * max(1.0, np.abs(b).max()), n
    want = plain.logits(toks)[-1]
    assert np.abs(got_logits[0] - want).max() <= tol * np.abs(want).max()


def test_log_lines_per_step(capfd, monkeypatch):
    """IMPARO_LOG=1: one line per step on stderr and a summary at the end."""
    from imparo_b200.engine import Engine
    monkeypatch.setenv("IMPARO_LOG", "1")
    eng = Engine(model_dir("A"), dtype="bfloat16", ctx=128, parallel=2, page_size=16, max_step_tokens=16)
    out = eng.generate([[1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12, 13, 14, 15, 16, 17, 18, 19, 20], [5, 6, 7]], max_tokens=4)
    err = capfd.readouterr().err
    lines = [l for l in err.splitlines() if l.startswith("imparo step ")]
    assert len(lines) == eng.stats()["steps"] and all("prompt_tokens=" in l and "free_pages=" in l for l in lines)
    assert "imparo generate: 2 requests, 8 new tokens" in err
    assert [len(o) for o in out] == [4, 4]


@pytest.mark.parametrize("dtype,min_margin", [("float32", 1e-5), ("bfloat16", 2e-2)])
def test_stop_tokens_inside_a_running_batch(dtype, min_margin):
    """Six requests through three slots and a small pool; each has its own stop token, taken from what the plain
    implementation generates for it, so that requests end at different steps while others run: a stop token is
    found one step late (its request then has a wasted row in the step in flight), slots and pages are used
    again, greedy and seeded temperature rows mix.  Every output must be the plain run cut at its stop token."""
    from imparo_b200.engine import Engine
    lens = [9, 30, 17, 5, 26, 12]
    prompts = list(make_requests("B", lens, seed=21).values())
    temps = [0.0, 0.8, 0.0, 0.8, 0.0, 0.0]
    seeds = [0, 5, 0, 6, 0, 0]
    plain = [P.generate(plain_model("B"), p, 14, temps[i], seeds[i]) for i, p in enumerate(prompts)]
    # request i stops at the token the plain run produced at place cut[i] (first occurrence counts)
    cut = [3, 7, 1, 10, 5, 13]
    stops = {plain[i][0][cut[i]] for i in range(6)}
    want = []
    for toks, _ in plain:
        first = next((j for j, t in enumerate(toks) if t in stops), len(toks))
        want.append(toks[:first])
    assert len({len(w) for w in want}) >= 3                              # they do end at different steps
    eng = Engine(model_dir("B"), dtype=dtype, ctx=64, parallel=3, page_size=4, num_pages=26, max_step_tokens=16)
    seen = []
    got = eng.generate(prompts, max_tokens=14, temperature=temps, seed=seeds, stop_token_ids=sorted(stops),
                       on_step=lambda plan: seen.append(plan))
    for i in range(6):
        margins = plain[i][1]
        agree(got[i], want[i], margins, min_margin if temps[i] == 0 else 1e-4 if dtype == "float32" else 5e-3)
    assert any(any(e.count > 1 for e in plan) and any(e.count == 1 for e in plan) for plan in seen)
    assert eng.stats()["failed"] == []
    assert eng.cache.n_requests() == 0 and eng.cache.free_pages(0) == 26 and eng.cache.free_slots() == 3
    eng.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_logits_of_two_steps_of_the_same_shape_can_both_be_kept(dtype):
    """Engine.step hands out a tensor of the caller's own: the step function's logits buffer (a workspace view, or
    a captured graph's output) is written again by the next step of the same shape."""
    from imparo_b200.engine import Engine, StepItem
    toks = make_requests("A", [12], seed=3)["r0"]
    eng = Engine(model_dir("A"), dtype=dtype, ctx=64, parallel=1, page_size=16)
    eng.add_request(1)
    eng.step([StepItem(1, toks[:8], [])])
    kept = [eng.step([StepItem(1, [toks[8 + i]], [0])]) for i in range(4)]     # same shape four times: the third is a replay
    eng.end_request(1)
    ref = plain_model("A").logits(toks)
    scale = float(np.abs(ref).max())
    for i, t in enumerate(kept):
        assert np.abs(t.cpu().numpy()[0] - ref[8 + i]).max() <= TOL[dtype] * scale, i
    assert len({t.data_ptr() for t in kept}) == 4


@pytest.mark.parametrize("dtype,tol", [("float32", 2e-5), ("bfloat16", 2.5e-2)])
def test_padding_rows_change_the_shape_not_the_results(dtype, tol):
    """Three decoding requests beside a prompt portion: with padding the step runs four one-token rows (the
    fourth belongs to no request and writes to the spare page and slot); the real rows' logits are those of the
    step without padding and of the plain implementation, and nothing of the pool is taken."""
    from imparo_b200.engine import Engine, StepItem
    reqs = make_requests("B", [9, 14, 6, 30], seed=21)
    prompts = list(reqs.values())
    plain = plain_model("B")
    want = np.stack([plain.logits(prompts[3][:20])[19]] + [plain.logits(prompts[r])[-1] for r in range(3)])
    nxt = [int(np.argmax(want[i + 1])) for i in range(3)]
    outs = []
    for pad in (False, True):
        eng = Engine(model_dir("B"), dtype=dtype, ctx=64, parallel=4, page_size=4, num_pages=40, switches={})
        eng.step_fn.pad_rows = pad
        for r in range(4):
            eng.add_request(r)
        for r in range(3):                                   # three prompts but their last token, each alone
            eng.step([StepItem(r, prompts[r][:-1], [])])
        free = eng.cache.free_pages(0)
        items = [StepItem(3, prompts[3][:20], [19])] + [StepItem(r, prompts[r][-1:], [0]) for r in range(3)]
        logits = eng.step(items)
        key = eng.step_fn._graphs and list(eng.step_fn._graphs)[-1]
        assert key[1] == (5 if pad else 4) and key[0] == (24 if pad else 23)
        assert logits.shape[0] == 4
        outs.append(logits.float().cpu())
        # decode-only step of three rows: padded to four as well
        l2 = eng.step([StepItem(r, [nxt[r]], [0]) for r in range(3)])
        assert l2.shape[0] == 3
        outs.append(l2.float().cpu())
        eng.check_device_status()
        eng.cache.check()
        for r in range(4):
            eng.end_request(r)
        assert eng.cache.free_pages(0) == 40 and eng.cache.free_slots() == 4 and free < 40
    scale = float(np.abs(want).max())
    for got in (outs[0], outs[2]):
        assert np.abs(got.numpy() - want).max() <= tol * scale
    assert np.abs(outs[1].numpy() - outs[3].numpy()).max() <= tol * scale


@pytest.mark.parametrize("dtype,tol", [("float32", 2e-5), ("bfloat16", 2.5e-2)])
def test_a_new_shape_is_captured_at_first_sight_or_falls_back(dtype, tol):
    """With buffers made for the largest step a new shape is captured the first time it comes and replayed from then
    on.  When a buffer does have to grow under capture the recording is dropped, the step runs launch by launch, and
    the shape is captured the next time.  The logits are those of the plain implementation either way."""
    from imparo_b200.engine import Engine, StepItem
    prompt = make_requests("B", [24], seed=5)["r0"]
    want = plain_model("B").logits(prompt)
    scale = float(np.abs(want).max())
    for reserve in (True, False):
        eng = Engine(model_dir("B"), dtype=dtype, ctx=64, parallel=2, page_size=4, num_pages=40, capture_first=True)
        sf = eng.step_fn
        if not sf.use_graphs:
            pytest.skip("this model's steps are not captured")
        if not reserve:
            eng.rt.workspace.most = {"tokens": 0, "rows": 0, "context": 0}      # as if nothing were known beforehand
        eng.add_request(1)
        # the engine's very first step also makes the launchers' scratch, which cannot happen under capture: its
        # recording may be dropped; from then on only a buffer that is too small can do that
        got = [eng.step([StepItem(1, prompt[:12], [11])])[0].float().cpu().numpy()]
        first_failures = sf.capture_failures
        got.append(eng.step([StepItem(1, prompt[12:20], [7])])[0].float().cpu().numpy())      # a new shape
        if reserve:
            assert sf.capture_failures == first_failures, sf.last_capture_error
            assert sf.graph_captures >= 1 and sf.graph_replays >= 1
        for i in range(20, 24):                                                 # four steps of one more shape
            got.append(eng.step([StepItem(1, [prompt[i]], [0])])[0].float().cpu().numpy())
        if reserve:
            assert sf.capture_failures == first_failures, sf.last_capture_error
        assert sf.graph_replays >= 3
        eng.check_device_status()
        for g, pos in zip(got, (11, 19, 20, 21, 22, 23)):
            assert np.abs(g - want[pos]).max() <= tol * scale
        eng.end_request(1)
        eng.cache.check()
