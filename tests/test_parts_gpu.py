"""Each part alone, built from its parameters with random weights and run through the
framework's own batch and cache objects, against the plain function of the same part.
Sizes differ from the tiny models'."""
import math
from types import SimpleNamespace

import numpy as np
import pytest
import torch

from tests.plain import lfm2_plain as P

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def runtime(precision):
    from imparo_b200.kernels import ops
    from imparo_b200.parts.base import Runtime, Workspace
    return Runtime(precision=precision, device=DEV, status=ops.new_status(DEV), workspace=Workspace(DEV))


def build(kind, spec, prefix, rt, seed=0):
    """Make a part, draw its weights, bind them.  -> (part, {name: float64 numpy})"""
    from imparo_b200.parts.base import make_part
    from imparo_b200.weights.loader import target_dtype
    from imparo_b200.weights.random_init import draw_random_tensors
    part = make_part(kind, spec, prefix, rt)
    drawn = draw_random_tensors(part.weight_specs(), seed, "bfloat16", "cpu", matrix_std=0.1)
    part.bind({w.name: drawn[w.name].to(DEV, target_dtype(w.role, rt.precision)) for w in part.weight_specs() if w.name in drawn})
    return part, {k: v.double().numpy() for k, v in drawn.items()}


def batch_for(part, rt, portions, page=4, pages=64, slots=4):
    """A cache manager and step-batch builder for one part alone."""
    from imparo_b200.cache import CacheManager
    from imparo_b200.engine.step import StepFunction
    cache = CacheManager([(0, tuple(part.cache_specs()))] if part.cache_specs() else [], page, pages, slots,
                         kv_dtype=rt.act_dtype, device=DEV)
    fn = StepFunction(SimpleNamespace(rt=rt, schedule=[SimpleNamespace(cache_from=None)]), cache, 4096, slots)
    return cache, fn


def run_mixer(part, rt, x_by_req, cuts):
    """Feed each request's rows in the given cuts (same cut list for all requests, mixed in
    one batch per cut).  -> {req: [T, H] output}"""
    from imparo_b200.engine.step import StepItem
    cache, fn = batch_for(part, rt, cuts)
    out = {r: [] for r in x_by_req}
    at = {r: 0 for r in x_by_req}
    for r in x_by_req:
        cache.add(r)
    for cut in cuts:
        items, rows = [], []
        for r, x in x_by_req.items():
            n = min(cut, x.shape[0] - at[r])
            if n <= 0:
                continue
            items.append(StepItem(r, [0] * n))
            rows.append(x[at[r]:at[r] + n])
            cache.reserve(r, n)
        if not items:
            break
        batch = fn.build_batch(items)
        xin = torch.cat(rows).to(DEV, rt.act_dtype)
        residual = torch.zeros(xin.shape[0], x.shape[1], device=DEV)
        views = cache.views(0) if part.cache_specs() else ()
        if part.cache_specs() is not None and hasattr(part, "cache_specs") and part.cache_specs():
            part.forward(xin, batch, views, residual)
        else:
            part.forward(xin, batch, residual)
        t = 0
        for it in items:
            n = len(it.tokens)
            out[it.request].append(residual[t:t + n].cpu().double().numpy())
            cache.commit(it.request, n)
            at[it.request] += n
            t += n
    from imparo_b200.kernels import ops
    ops.read_status(rt.status)
    cache.check()
    return {r: np.concatenate(v) for r, v in out.items()}


def rounded(x, precision):
    t = torch.from_numpy(x).float()
    return (t.to(torch.bfloat16).float() if precision == "bfloat16" else t)


TOL = {"float32": 3e-6, "bfloat16": 2e-2}


@pytest.mark.parametrize("precision", ["float32", "bfloat16"])
@pytest.mark.parametrize("nh,nkv,hd,window", [(5, 5, 16, None), (8, 2, 48, None), (3, 1, 80, 11)])
def test_attention_mixer_alone(precision, nh, nkv, hd, window):
    from imparo_b200.parts.spec import PartSpec
    rt = runtime(precision)
    H = 104
    spec = PartSpec("attention", {"hidden": H, "n_heads": nh, "n_kv_heads": nkv, "head_dim": hd, "eps": 2e-6, "window": window,
                                  "position": PartSpec("rope_neox", {"head_dim": hd, "theta": 777.0})})
    part, w = build("mixer", spec, "L.", rt)
    rng = np.random.default_rng(0)
    xs = {1: rounded(rng.standard_normal((37, H)), precision), 2: rounded(rng.standard_normal((9, H)), precision)}
    got = run_mixer(part, rt, xs, cuts=[5, 1, 1, 13, 2, 40])
    cfg = SimpleNamespace(n_heads=nh, n_kv=nkv, head_dim=hd, eps=2e-6, theta=777.0)
    pw = {"q_proj": w["L.self_attn.q_proj.weight"], "k_proj": w["L.self_attn.k_proj.weight"],
          "v_proj": w["L.self_attn.v_proj.weight"], "out_proj": w["L.self_attn.out_proj.weight"],
          "q_layernorm": w["L.self_attn.q_layernorm.weight"], "k_layernorm": w["L.self_attn.k_layernorm.weight"]}
    if window:
        pw["window"] = window
    for r, x in xs.items():
        ref = P.attention_mixer(x.double().numpy(), pw, cfg, np.arange(x.shape[0]))
        assert np.abs(got[r] - ref).max() <= TOL[precision] * max(1.0, np.abs(ref).max())


@pytest.mark.parametrize("precision", ["float32", "bfloat16"])
@pytest.mark.parametrize("taps,bias", [(2, False), (5, True)])
def test_short_conv_mixer_alone(precision, taps, bias):
    from imparo_b200.parts.spec import PartSpec
    rt = runtime(precision)
    H = 88
    part, w = build("mixer", PartSpec("short_conv", {"hidden": H, "taps": taps, "bias": bias}), "L.", rt)
    rng = np.random.default_rng(1)
    xs = {1: rounded(rng.standard_normal((23, H)), precision), 2: rounded(rng.standard_normal((6, H)), precision)}
    got = run_mixer(part, rt, xs, cuts=[1, 2, 1, 7, 3, 30])
    pw = {"in_proj": w["L.conv.in_proj.weight"], "out_proj": w["L.conv.out_proj.weight"],
          "conv": w["L.conv.conv.weight"].reshape(H, taps)}
    if bias:
        pw["conv_bias"] = w["L.conv.conv.bias"]
    for r, x in xs.items():
        ref = P.conv_mixer(x.double().numpy(), pw, None)
        assert np.abs(got[r] - ref).max() <= TOL[precision] * max(1.0, np.abs(ref).max())


@pytest.mark.parametrize("precision", ["float32", "bfloat16"])
def test_swiglu_alone(precision):
    from imparo_b200.parts.spec import PartSpec
    rt = runtime(precision)
    H, F = 72, 200
    part, w = build("feed_forward", PartSpec("swiglu", {"hidden": H, "ff": F}), "L.", rt)
    x = rounded(np.random.default_rng(2).standard_normal((13, H)), precision)
    residual = torch.ones(13, H, device=DEV)
    part.forward(x.to(DEV, rt.act_dtype), None, residual)
    ref = 1.0 + P.swiglu(x.double().numpy(), {"w1": w["L.feed_forward.w1.weight"], "w2": w["L.feed_forward.w2.weight"],
                                              "w3": w["L.feed_forward.w3.weight"]})
    assert np.abs(residual.cpu().double().numpy() - ref).max() <= TOL[precision] * max(1.0, np.abs(ref).max())


@pytest.mark.parametrize("precision", ["float32", "bfloat16"])
def test_norm_embedding_and_head_alone(precision):
    from imparo_b200.parts.spec import PartSpec
    rt = runtime(precision)
    V, H = 333, 56
    emb, w = build("embedding", PartSpec("token_table", {"vocab": V, "width": H, "name": "E.weight"}), "", rt)
    ids = torch.tensor([5, 332, 0, 5], dtype=torch.int32, device=DEV)
    x = emb.forward(SimpleNamespace(token_ids=ids, n_tokens=4))          # an embedding part is given the step's batch
    assert np.array_equal(x.cpu().double().numpy(), w["E.weight"][[5, 332, 0, 5]])
    norm, wn = build("norm", PartSpec("rmsnorm", {"width": H, "eps": 1e-4, "name": "n.weight"}), "", rt, seed=3)
    y = norm.forward(x)
    ref = P.rms_norm(w["E.weight"][[5, 332, 0, 5]], wn["n.weight"], 1e-4)
    assert np.abs(y.float().cpu().double().numpy() - ref).max() <= (2e-6 if precision == "float32" else 8e-3) * np.abs(ref).max()
    head, wh = build("head", PartSpec("linear", {"vocab": V, "width": H, "name": "E.weight"}), "", rt)
    logits = head.forward(y)
    ref_logits = y.float().cpu().double().numpy() @ wh["E.weight"].T
    assert logits.dtype == torch.float32 and logits.shape == (4, V)
    assert np.abs(logits.cpu().double().numpy() - ref_logits).max() <= 1e-5 * max(1.0, np.abs(ref_logits).max())


def test_position_part_table():
    from imparo_b200.parts.base import make_part
    from imparo_b200.parts.spec import PartSpec
    rt = runtime("float32")
    pe = make_part("position", PartSpec("rope_neox", {"head_dim": 48, "theta": 123456.0, "n_rot": 32}), "", rt)
    inv, n_rot = pe.rotary()
    assert n_rot == 32 and np.array_equal(inv.cpu().numpy(), P.rope_inv_freq(32, 123456.0))
    assert make_part("position", PartSpec("none"), "", rt).rotary() is None


@pytest.mark.parametrize("precision", ["float32", "bfloat16"])
def test_block_alone(precision):
    """The arrangement: x += mixer(norm(x)); x += ffn(norm(x)), on the 32-bit stream."""
    from imparo_b200.engine.step import StepItem
    from imparo_b200.parts.spec import LayerSpec, PartSpec
    rt = runtime(precision)
    H, F, taps = 48, 112, 3
    layer = LayerSpec(prefix="B.", mixer=PartSpec("short_conv", {"hidden": H, "taps": taps, "bias": False}),
                      feed_forward=PartSpec("swiglu", {"hidden": H, "ff": F}),
                      mixer_norm=PartSpec("rmsnorm", {"width": H, "eps": 1e-5, "name": "operator_norm.weight"}),
                      feed_forward_norm=PartSpec("rmsnorm", {"width": H, "eps": 1e-5, "name": "ffn_norm.weight"}))
    block, w = build("block", PartSpec("prenorm_residual", {"layer": layer}), "B.", rt)
    cache, fn = batch_for(block, rt, None)
    cache.add(1)
    x0 = np.random.default_rng(4).standard_normal((10, H))
    outs = []
    for a, b in ((0, 4), (4, 5), (5, 10)):
        cache.reserve(1, b - a)
        batch = fn.build_batch([StepItem(1, [0] * (b - a))])
        x = torch.from_numpy(x0[a:b]).float().to(DEV)
        block.forward(x, batch, cache.views(0))
        cache.commit(1, b - a)
        outs.append(x.cpu().double().numpy())
    lw = {"kind": "conv", "operator_norm": w["B.operator_norm.weight"], "ffn_norm": w["B.ffn_norm.weight"],
          "in_proj": w["B.conv.in_proj.weight"], "out_proj": w["B.conv.out_proj.weight"],
          "conv": w["B.conv.conv.weight"].reshape(H, taps), "w1": w["B.feed_forward.w1.weight"],
          "w2": w["B.feed_forward.w2.weight"], "w3": w["B.feed_forward.w3.weight"]}
    ref = P.block(x0.astype(np.float32).astype(np.float64), lw, SimpleNamespace(eps=1e-5), np.arange(10))
    assert np.abs(np.concatenate(outs) - ref).max() <= TOL[precision] * max(1.0, np.abs(ref).max())


@pytest.mark.parametrize("precision", ["float32", "bfloat16"])
@pytest.mark.parametrize("qk_norm,bias", [(False, False), (True, True), (False, True)])
def test_attention_mixer_without_head_norms_and_with_biases(precision, qk_norm, bias):
    """The attention part's options: qk_norm=False declares no norm tensors and rotates q and k as they are;
    bias=True adds q/k/v and output biases.  Against the plain functions put together the same way."""
    from imparo_b200.parts.spec import PartSpec
    rt = runtime(precision)
    H, nh, nkv, hd = 88, 4, 2, 32
    spec = PartSpec("attention", {"hidden": H, "n_heads": nh, "n_kv_heads": nkv, "head_dim": hd, "eps": 1e-5, "window": None,
                                  "qk_norm": qk_norm, "bias": bias,
                                  "position": PartSpec("rope_neox", {"head_dim": hd, "theta": 5000.0})})
    part, w = build("mixer", spec, "L.", rt)
    names = set(w)
    assert ("L.self_attn.q_layernorm.weight" in names) == qk_norm and ("L.self_attn.q_proj.bias" in names) == bias
    rng = np.random.default_rng(1)
    xs = {1: rounded(rng.standard_normal((29, H)), precision), 2: rounded(rng.standard_normal((6, H)), precision)}
    got = run_mixer(part, rt, xs, cuts=[4, 1, 1, 9, 30])
    for r, xt in xs.items():
        x = xt.double().numpy()
        T = x.shape[0]
        pos = np.arange(T)
        q = x @ w["L.self_attn.q_proj.weight"].T
        k = x @ w["L.self_attn.k_proj.weight"].T
        v = x @ w["L.self_attn.v_proj.weight"].T
        if bias:
            q, k, v = q + w["L.self_attn.q_proj.bias"], k + w["L.self_attn.k_proj.bias"], v + w["L.self_attn.v_proj.bias"]
        q, k, v = q.reshape(T, nh, hd), k.reshape(T, nkv, hd), v.reshape(T, nkv, hd)
        if qk_norm:
            q = P.rms_norm(q, w["L.self_attn.q_layernorm.weight"], 1e-5)
            k = P.rms_norm(k, w["L.self_attn.k_layernorm.weight"], 1e-5)
        q, k = P.rope_neox(q, pos, hd, 5000.0), P.rope_neox(k, pos, hd, 5000.0)
        ref = P.attend(q, k, v, 1 / math.sqrt(hd)).reshape(T, nh * hd) @ w["L.self_attn.out_proj.weight"].T
        if bias:
            ref = ref + w["L.self_attn.out_proj.bias"]
        assert np.abs(got[r] - ref).max() <= TOL[precision] * max(1.0, np.abs(ref).max()), (r, np.abs(got[r] - ref).max())


def test_two_engines_in_one_process_do_not_share_launch_state():
    """Two engines of different configurations stepped in turn: each keeps its own launcher bookkeeping and
    scratch (pending split partials, captured graphs), and gives what it gives alone."""
    from imparo_b200.engine import Engine, StepItem
    from tests.gpu_helpers import make_requests, model_dir, plain_model
    engines, toks, refs = {}, {}, {}
    for name, page in (("E", 16), ("F", 64)):
        engines[name] = Engine(model_dir(name), dtype="bfloat16", ctx=128, parallel=2, page_size=page)
        toks[name] = make_requests(name, [40], seed=7)["r0"]
        refs[name] = plain_model(name).logits(toks[name])
        engines[name].add_request(1)
    assert engines["E"].rt.launch_state is not engines["F"].rt.launch_state
    at = {"E": 0, "F": 0}
    for cut in (8, 1, 1, 1, 5, 1, 1, 1, 1, 20):
        for name, eng in engines.items():
            n = min(cut, 40 - at[name])
            if n <= 0:
                continue
            got = eng.step([StepItem(1, toks[name][at[name]:at[name] + n], [n - 1])]).cpu().numpy()[0]
            ref = refs[name][at[name] + n - 1]
            assert np.abs(got - ref).max() <= 2.5e-2 * np.abs(refs[name]).max(), (name, at[name], n)
            at[name] += n
    for eng in engines.values():
        eng.check_device_status()
        eng.end_request(1)
        assert eng.step_fn.graph_replays >= 1
