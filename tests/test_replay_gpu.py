"""Replay families on the GPU, in 32-bit and in bfloat16, against the plain implementation:
each request whole; most of it in one step and the last 32 tokens one by one; portions of
changing size down to two tokens; and mixed, up to four live requests with so few pages
that they are used again."""
import numpy as np
import pytest

from tests import traces
from tests.gpu_helpers import check_trace, make_requests, model_dir
from tests.tiny_configs import ALL

pytestmark = pytest.mark.gpu

PAGE = {"A": 16, "B": 4, "C": 8, "D": 32, "E": 16, "F": 64}
LENGTHS = {"A": [70, 45, 96, 33, 64, 51, 80], "B": [5, 23, 40, 67, 90, 34], "C": [81, 40, 65, 97, 58], "D": [44, 71, 36, 60],
           "E": [150, 47, 96, 201, 64], "F": [130, 75, 40, 164]}


def engine_for(name, dtype, steps, parallel=4):
    from imparo_b200.engine import Engine
    page = PAGE[name]
    max_tokens = traces.max_live_tokens(steps, 64)
    return Engine(model_dir(name), dtype=dtype, ctx=max_tokens, parallel=parallel, page_size=page,
                  num_pages=(max_tokens + page - 1) // page, max_step_tokens=max(256, max_tokens))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E", "F"])
@pytest.mark.parametrize("family", ["whole", "tail", "portions", "mixed"])
def test_family(name, dtype, family):
    reqs = make_requests(name, LENGTHS[name])
    steps = {"whole": traces.whole, "tail": traces.tail_one_by_one, "portions": traces.portions,
             "mixed": lambda r: traces.mixed(r, seed=3)}[family](reqs)
    eng = engine_for(name, dtype, steps)
    check_trace(eng, steps, name, reqs, dtype)
    if family == "mixed":
        # the pool is smaller than everything the trace ever held: pages were used again
        total = sum(traces.round_up(len(t), 64) for t in reqs.values())
        assert traces.max_live_tokens(steps) < total


SWITCHED = [{"decode_from_qkv": False}, {"fuse_producers": False}, {"unfolded": False}, {"defer_adds": False},
            {"gemm": "library"}, {"prefill_gemm": "library"}, {"prefill_linear": True}, {"attn_prefill": "mma"},
            {"attn_prefill": "tcgen05_one_tile"}, {"attn_side_by_side": False}, {"pad_rows": False}, {"capture_first": False},
            {"use_graphs": False}]


@pytest.mark.parametrize("name", ["B", "F"])
@pytest.mark.parametrize("switched", SWITCHED, ids=lambda d: "-".join(f"{k}={v}" for k, v in d.items()))
def test_every_switch_leaves_a_path_that_gives_the_same_logits(name, switched):
    """The engine's switches choose between kernels and between ways of launching them; whichever way one is set,
    a mixed trace in bfloat16 gives the plain implementation's logits."""
    from imparo_b200.engine import Engine
    reqs = make_requests(name, LENGTHS[name])
    steps = traces.mixed(reqs, seed=5)
    page = PAGE[name]
    max_tokens = traces.max_live_tokens(steps, 64)
    top = {k: v for k, v in switched.items() if k in ("pad_rows", "capture_first", "use_graphs")}
    eng = Engine(model_dir(name), dtype="bfloat16", ctx=max_tokens, parallel=4, page_size=page,
                 num_pages=(max_tokens + page - 1) // page, max_step_tokens=max(256, max_tokens),
                 switches={k: v for k, v in switched.items() if k not in top}, **top)
    for k, v in switched.items():
        assert getattr(eng.engine_config if k in top else eng.engine_config.switches, k) == v
    check_trace(eng, steps, name, reqs, "bfloat16")


_WIDE = {}


def _wide_run(switched):
    """Two layers at LFM2-1.2B width: a prompt of 1,100 tokens, a second request's portion of 270 beside the first's
    decode row, then both decoding; every wanted row's logits."""
    import torch
    from imparo_b200.engine import Engine, StepItem
    cfg = {"architectures": ["Lfm2ForCausalLM"], "vocab_size": 8192, "hidden_size": 2048, "num_hidden_layers": 2,
           "layer_types": ["conv", "full_attention"], "num_attention_heads": 32, "num_key_value_heads": 8,
           "block_ff_dim": 12288, "block_auto_adjust_ff_dim": True, "block_multiple_of": 256, "conv_L_cache": 3,
           "conv_bias": False, "rope_theta": 1000000.0, "norm_eps": 1e-5, "tie_embedding": True}
    top = {k: v for k, v in switched.items() if k in ("pad_rows", "capture_first", "use_graphs")}
    eng = Engine(config=cfg, seed=11, dtype="bfloat16", ctx=2048, parallel=3, page_size=16, max_step_tokens=2048,
                 random_init={"norm_jitter": 0.1, "matrix_std": 0.02},
                 switches={k: v for k, v in switched.items() if k not in top}, **top)
    rng = np.random.default_rng(23)
    a, b = rng.integers(0, 8192, 1100 + 8).tolist(), rng.integers(0, 8192, 270 + 8).tolist()
    eng.add_request(1)
    eng.add_request(2)
    rows = [eng.step([StepItem(1, a[:1100], [0, 500, 1099])])]
    rows.append(eng.step([StepItem(1, [a[1100]], [0]), StepItem(2, b[:270], [0, 269])]))
    for i in range(1, 8):
        rows.append(eng.step([StepItem(1, [a[1100 + i]], [0]), StepItem(2, [b[269 + i]], [0])]))
    eng.check_device_status()
    eng.end_request(1); eng.end_request(2)
    eng.cache.check()
    out = np.concatenate([r.cpu().numpy() for r in rows])
    del eng
    torch.cuda.empty_cache()
    return out


@pytest.mark.parametrize("switched", SWITCHED, ids=lambda d: "-".join(f"{k}={v}" for k, v in d.items()))
def test_every_switch_at_full_width(switched):
    """The same at the width the tensor-core kernels are made for (the tiny models take few of these paths): each
    switch's other setting against the defaults, in bfloat16."""
    if "default" not in _WIDE:
        _WIDE["default"] = _wide_run({})
    ref = _WIDE["default"]
    got = _wide_run(switched)
    assert np.isfinite(ref).all() and np.isfinite(got).all()
    scale = float(np.abs(ref).max())
    assert scale > 0.1 and np.abs(ref[0] - ref[-1]).max() > 0.2 * scale
    err = float(np.abs(got - ref).max())
    assert err <= 2.5e-2 * scale, (switched, err, scale)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_cutting_does_not_change_logits_beyond_rounding(dtype):
    """The same positions through four ways of cutting: 32-bit results agree to ~1e-6."""
    from tests.gpu_helpers import run_trace
    name = "B"
    reqs = make_requests(name, [61, 47, 75], seed=5)
    outs = []
    for build in (traces.whole, traces.tail_one_by_one, traces.portions, lambda r: traces.mixed(r, seed=9)):
        steps = build(reqs)
        got = run_trace(engine_for(name, dtype, steps), steps)
        # gather by (request, position)
        by_pos, at = {}, {}
        for s in steps:
            r = 0
            for e in s["entries"]:
                start = at.get(e["id"], 0)
                for w in e["want"]:
                    by_pos[(e["id"], start + w)] = got[s["step"]][r]
                    r += 1
                at[e["id"]] = start + len(e["tokens"])
        outs.append(by_pos)
    keys = set(outs[1]) & set(outs[0])
    assert len(keys) > 90
    tol = 5e-6 if dtype == "float32" else 3e-2
    for k in keys:
        for o in outs[1:]:
            if k in o:
                assert np.abs(o[k] - outs[0][k]).max() <= tol, k


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(dtype):
    name = "A"
    reqs = make_requests(name, [400], seed=8)
    steps = traces.tail_one_by_one(reqs, tail=390)
    check_trace(engine_for(name, dtype, steps), steps, name, reqs, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_first_tokens_of_a_sequence(name, dtype):
    """Positions 0, 1, 2, ...: one-token prompts, a fresh state slot, the first page."""
    reqs = make_requests(name, [1, 2, 3, 6], seed=11)
    for build in (traces.whole, lambda r: traces.tail_one_by_one(r, tail=8)):
        steps = build(reqs)
        check_trace(engine_for(name, dtype, steps), steps, name, reqs, dtype)


def test_state_slots_and_pages_start_clean_when_used_again():
    """A request that takes over a slot and pages another one used sees none of it."""
    name = "B"
    a = make_requests(name, [50], seed=20)
    b = {"other": make_requests(name, [37], seed=21)["r0"]}
    steps = traces.whole(a) + [dict(s, step=s["step"] + 1) for s in traces.portions(b, sizes=(1, 2, 3))]
    reqs = dict(a, **b)
    eng = engine_for(name, "float32", steps, parallel=1)       # one slot: it must be reused
    check_trace(eng, steps, name, reqs, "float32")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "E"])
def test_a_captured_step_shape_serves_other_layouts(name, dtype):
    """Steps with the same totals (tokens, requests, wanted rows, longest portion) are captured
    once and replayed; which request brings how many tokens changes from step to step, and new
    requests start inside replayed steps."""
    lengths = {"a": 52, "b": 52, "c": 52, "d": 16, "e": 16}
    reqs = {k: v for k, v in zip(lengths, make_requests(name, list(lengths.values()), seed=31).values())}
    cuts = [{"a": 20, "b": 20, "c": 20},
            {"a": 1, "b": 5, "c": 10}, {"a": 1, "b": 10, "c": 5}, {"a": 10, "b": 1, "c": 5}, {"a": 5, "b": 10, "c": 1},
            {"a": 10, "b": 5, "c": 1}, {"a": 5, "b": 1, "c": 10},
            {"d": 16}, {"e": 16}]                                  # whole new requests, the same shape twice
    at = {k: 0 for k in reqs}
    steps = []
    for cut in cuts:
        entries = []
        for k, n in cut.items():
            entries.append({"id": k, "tokens": reqs[k][at[k]:at[k] + n], "want": [0, n - 1] if n > 1 else [0]})
            at[k] += n
        steps.append({"step": len(steps), "entries": entries, "end": [k for k in cut if at[k] == len(reqs[k])]})
    assert all(at[k] == len(reqs[k]) for k in reqs)
    # requests d and e: one step each, of one shape; the second is the capture, so add a third
    extra = make_requests(name, [16], seed=32)["r0"]
    reqs["f"] = extra
    steps.append({"step": len(steps), "entries": [{"id": "f", "tokens": extra, "want": [0, 15]}], "end": ["f"]})
    eng = engine_for(name, dtype, steps)
    check_trace(eng, steps, name, reqs, dtype)
    assert eng.step_fn.graph_replays >= 6


def test_full_width_layers_bfloat16_against_32_bit():
    """Four layers of LFM2-1.2B width (hidden 2048, 32 heads in 8 groups, head 64, ff 8192,
    vocabulary 65536): the sizes the tensor-core kernels are tuned for, which the tiny models
    never reach (split-K clusters, 128-row weight tiles, 64-key attention tiles, several key
    chunks).  The bfloat16 path (tensor cores) against the 32-bit path (FFMA product, scalar
    attention): different kernels, same weights up to rounding."""
    import torch
    from imparo_b200.engine import Engine, StepItem
    cfg = {"architectures": ["Lfm2ForCausalLM"], "vocab_size": 65536, "hidden_size": 2048, "num_hidden_layers": 4,
           "layer_types": ["conv", "full_attention", "conv", "full_attention"], "num_attention_heads": 32,
           "num_key_value_heads": 8, "block_ff_dim": 12288, "block_auto_adjust_ff_dim": True, "block_multiple_of": 256,
           "conv_L_cache": 3, "conv_bias": False, "rope_theta": 1000000.0, "norm_eps": 1e-5, "tie_embedding": True}
    rng = np.random.default_rng(3)
    prompt = rng.integers(0, 65536, 700).tolist()
    tail = rng.integers(0, 65536, 6).tolist()
    results = {}
    for dtype in ("float32", "bfloat16"):
        eng = Engine(config=cfg, seed=7, dtype=dtype, ctx=1024, parallel=2, page_size=16, max_step_tokens=1024,
                     random_init={"norm_jitter": 0.1, "matrix_std": 0.02})
        eng.add_request(1)
        rows = [eng.step([StepItem(1, prompt[:300], [0, 150, 299])]).cpu().numpy()]
        rows.append(eng.step([StepItem(1, prompt[300:], [0, 399])]).cpu().numpy())
        for t in tail:                                    # single tokens: the decode kernels
            rows.append(eng.step([StepItem(1, [t], [0])]).cpu().numpy())
        eng.check_device_status()
        eng.end_request(1)
        results[dtype] = np.concatenate(rows)
        del eng
        torch.cuda.empty_cache()
    ref, got = results["float32"], results["bfloat16"]
    assert np.isfinite(ref).all() and np.isfinite(got).all()
    scale = np.abs(ref).max()
    assert scale > 0.1
    err = np.abs(got - ref).max()
    assert err <= 4e-2 * scale, (err, scale)
    # and the rows are not all alike (a kernel that ignored its input would pass the bound above)
    assert np.abs(ref[0] - ref[-1]).max() > 0.2 * scale


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_full_width_layers_against_the_plain_implementation(dtype, tmp_path_factory):
    """One conv layer and one attention layer at LFM2-1.2B width (hidden 2048, 32 heads in 8 groups, head 64,
    ff 8192, vocabulary 65536) from a model folder, against the plain implementation in float64 on the same
    folder: a mistake that the bfloat16 and the 32-bit path share at width (a descriptor, a table stride) cannot
    pass here.  Three ways of cutting: the prompt whole and then single tokens; portions of 64 tokens (the
    tensor-core product at its widest token tile); a stretch of single tokens from the start."""
    import torch
    from imparo_b200.engine import Engine, StepItem
    from imparo_b200.weights import write_random_model
    from tests.plain.lfm2_plain import PlainLfm2
    cfg = {"architectures": ["Lfm2ForCausalLM"], "model_type": "lfm2", "vocab_size": 65536, "hidden_size": 2048,
           "num_hidden_layers": 2, "layer_types": ["conv", "full_attention"], "num_attention_heads": 32,
           "num_key_value_heads": 8, "block_ff_dim": 12288, "block_auto_adjust_ff_dim": True, "block_multiple_of": 256,
           "conv_L_cache": 3, "conv_bias": False, "rope_theta": 1000000.0, "norm_eps": 1e-5, "tie_embedding": True,
           "max_position_embeddings": 4096}
    d = _full_width_folder(cfg, tmp_path_factory)
    rng = np.random.default_rng(17)
    toks = rng.integers(0, 65536, 300 + 6).tolist()
    want_prompt = [0, 63, 64, 150, 299]
    ref = _full_width_reference(d, tuple(toks))
    scale = float(np.abs(ref).max())
    tol = (2.5e-2 if dtype == "bfloat16" else 2e-5) * scale
    eng = Engine(d, dtype=dtype, ctx=512, parallel=3, page_size=16, max_step_tokens=512)

    def check(got, places, what):
        for row, p in zip(got, places):
            err = float(np.abs(row - ref[p]).max())
            assert err <= tol, f"{what}: position {p}: error {err:.3e} > {tol:.3e}"

    # 1. the prompt whole, then its last six tokens one by one
    eng.add_request(1)
    check(eng.step([StepItem(1, toks[:300], want_prompt)]).cpu().numpy(), want_prompt, "whole")
    for i in range(300, 306):
        check(eng.step([StepItem(1, [toks[i]], [0])]).cpu().numpy(), [i], "single tokens after the prompt")
    eng.end_request(1)
    # 2. portions of 64 tokens
    eng.add_request(2)
    for a in range(0, 306, 64):
        part = toks[a:a + 64]
        places = [p for p in want_prompt + [305] if a <= p < a + len(part)]
        out = eng.step([StepItem(2, part, [p - a for p in places])])
        if places:
            check(out.cpu().numpy(), places, "portions of 64")
    eng.end_request(2)
    # 3. single tokens from the start (the decode kernels at short contexts), beside a second request's portion
    eng.add_request(3)
    eng.add_request(4)
    for i in range(40):
        items = [StepItem(3, [toks[i]], [0])]
        if i % 8 == 0:
            items.append(StepItem(4, toks[i * 4:i * 4 + 32], [31]))
        out = eng.step(items).cpu().numpy()
        check(out[:1], [i], "single tokens from the start")
        if i % 8 == 0:
            check(out[1:], [i * 4 + 31], "a portion beside a single token")
    eng.check_device_status()
    eng.end_request(3); eng.end_request(4)
    eng.cache.check()
    del eng
    torch.cuda.empty_cache()


_FULL_WIDTH = {}


def _full_width_folder(cfg, tmp_path_factory):
    from imparo_b200.weights import write_random_model
    if "dir" not in _FULL_WIDTH:
        _FULL_WIDTH["dir"] = write_random_model(str(tmp_path_factory.mktemp("full_width")), cfg, seed=5, dtype="bfloat16")
    return _FULL_WIDTH["dir"]


def _full_width_reference(folder, toks):
    from tests.plain.lfm2_plain import PlainLfm2
    if "ref" not in _FULL_WIDTH:
        _FULL_WIDTH["ref"] = PlainLfm2(folder, np.float64).logits(list(toks))
    return _FULL_WIDTH["ref"]


def test_long_context_whole_against_portions():
    """6,000 positions: hundreds of pages per request, table rows of several hundred blocks, key
    chunks and tiles far from position 0.  Whole prompt against 1,024-token portions and single
    tokens, at LFM2-350M width with two attention layers (bfloat16: the tensor-core kernels)."""
    import torch
    from imparo_b200.engine import Engine, StepItem
    cfg = {"architectures": ["Lfm2ForCausalLM"], "vocab_size": 4096, "hidden_size": 1024, "num_hidden_layers": 3,
           "layer_types": ["full_attention", "conv", "full_attention"], "num_attention_heads": 16,
           "num_key_value_heads": 8, "block_ff_dim": 6656, "block_auto_adjust_ff_dim": True, "block_multiple_of": 256,
           "conv_L_cache": 3, "conv_bias": False, "rope_theta": 1000000.0, "norm_eps": 1e-5, "tie_embedding": True}
    rng = np.random.default_rng(5)
    toks = rng.integers(0, 4096, 6000).tolist()
    tail = rng.integers(0, 4096, 5).tolist()
    want = [0, 1023, 1024, 3000, 5999]
    eng = Engine(config=cfg, seed=3, dtype="bfloat16", ctx=8192, parallel=2, page_size=16, max_step_tokens=6000,
                 random_init={"norm_jitter": 0.1})
    eng.add_request(1)
    whole = [eng.step([StepItem(1, toks, want)]).float().cpu().numpy()]
    for t in tail:
        whole.append(eng.step([StepItem(1, [t], [0])]).float().cpu().numpy())
    eng.add_request(2)
    parts = []
    for a in range(0, 6000, 1024):
        chunk = toks[a:a + 1024]
        w = [p - a for p in want if a <= p < a + len(chunk)]
        out = eng.step([StepItem(2, chunk, w)])
        if out is not None:
            parts.append(out.float().cpu().numpy())
    for t in tail:
        parts.append(eng.step([StepItem(2, [t], [0])]).float().cpu().numpy())
    eng.check_device_status()
    a, b = np.concatenate(whole), np.concatenate(parts)
    assert a.shape == b.shape == (10, 4096) and np.isfinite(a).all()
    scale = np.abs(a).max()
    assert np.abs(a - b).max() <= 3e-2 * scale, (np.abs(a - b).max(), scale)
    assert np.abs(a[0] - a[4]).max() > 0.1 * scale
    eng.end_request(1); eng.end_request(2)
    eng.cache.check()


def test_rows_of_one_token_come_first_and_wanted_rows_keep_their_order():
    """A step that holds portions and single tokens is laid out with the single tokens first; the
    logits still come in the order of the entries and of want."""
    from imparo_b200.engine import StepItem
    from tests.gpu_helpers import plain_logits
    name = "E"                                        # head size 64: the tensor-core kernels take this step
    reqs = make_requests(name, [40, 9, 33, 12], seed=41)
    all_live = [{"step": 0, "entries": [{"id": k, "tokens": v, "want": []} for k, v in reqs.items()], "end": []}]
    eng = engine_for(name, "bfloat16", all_live)
    ids = {k: i + 1 for i, k in enumerate(reqs)}
    for k in reqs:
        eng.add_request(ids[k])
    eng.step([StepItem(ids[k], v[:8], []) for k, v in reqs.items()])
    # r0: a portion, r1: its last token, r2: a portion, r3: one token (not its last)
    items = [StepItem(ids["r0"], reqs["r0"][8:30], [0, 21]), StepItem(ids["r1"], reqs["r1"][8:9], [0]),
             StepItem(ids["r2"], reqs["r2"][8:20], [5]), StepItem(ids["r3"], reqs["r3"][8:9], [0])]
    batch = eng.step_fn.build_batch(items, singles_first=True)
    assert batch.n_single == 2 and batch.item_row_start.cpu().tolist() == [0, 1, 2, 24, 36]
    assert batch.want_rows.cpu().tolist()[:5] == [2, 23, 0, 29, 1]
    got = eng.step(items).cpu().numpy()
    ref = plain_logits(name, reqs)
    want = np.stack([ref["r0"][8], ref["r0"][29], ref["r1"][8], ref["r2"][13], ref["r3"][8]])
    scale = max(float(np.abs(v).max()) for v in ref.values())
    assert np.abs(got - want).max() <= 2.5e-2 * scale
