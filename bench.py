#!/usr/bin/env python3
"""Headline measurement: LFM2-1.2B layer sizes, random bfloat16 weights, one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A "step" is one decode step of a batch of 8 requests, each with a 2,048-token prompt in
the cache (context length 4,096, pages of 16 tokens).  `value` is decoded tokens per
second over exactly K steps, timed on the device with CUDA events after W warm-up steps;
the step's inputs are larger than L2 (2.3 GB of weights are read every step), so no
flush is needed between iterations.  `e2e` is the same metric through Engine.generate:
host token lists in, host token lists out, with the per-step host-to-device copy of the
batch descriptor and device-to-host copy of the sampled ids inside the timed region.
One JSON line is printed.  For --gpus N > 1 one line says that this engine is a
one-GPU engine and the exit code is 2.

`prefill` times one 2,048-token prompt per repetition (a new request each time, CUDA events
around the step); from its third run on the step is replayed from the graph the engine
captured for its shape, as every step whose shape repeats is.

--workload continuous | long run the baseline's two other workloads (LFM2-700M sizes under
continuous batching; LFM2-350M sizes with 32,768-token prompts in bfloat16 and 32-bit) and
print one JSON line each; --workload sizes runs the headline's model at further prompt lengths
and decode contexts; the default is the headline above.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# the config.json of LFM2-1.2B (the sizes the headline is quoted on); weights are random
with open(os.path.join(ROOT, "imparo_b200", "config", "presets", "lfm2_1.2b.json")) as _f:
    LFM2_1_2B = json.load(_f)
PROMPT = 2048
CTX = 4096
PAGE = 16
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d.get("bf16_tflops_sustained") or d["bf16_tflops"]),
                "bf16_tflops_burst": float(d["bf16_tflops"]), "source": "measured"}
    except Exception:
        return dict(FALLBACK_PEAKS, bf16_tflops_burst=FALLBACK_PEAKS["bf16_tflops"], source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index=0):
        self.rows, self.proc, self.index = [], None, index

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-i", str(self.index), "-lms", "100"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 7:
                self.rows.append(parts)

    def __exit__(self, *a):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[0])); mx.append(float(r[1]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def model_numbers(engine):
    """Bytes a decode step must read for its weights, KV bytes per cached token, and the
    flops of a prompt of T tokens, from the model's own parts."""
    cfg = engine.config
    H, F, V = cfg.hidden_size, cfg.ff_dim, cfg.vocab_size
    nh, nkv, hd = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    n_attn = sum(1 for e in engine.model.schedule if cfg.layer_types[e.layer] != "conv")
    n_conv = len(engine.model.schedule) - n_attn
    per_layer_ffn = 3 * H * F
    conv = 3 * H * H + H * H
    attn = (nh + 2 * nkv) * hd * H + H * nh * hd
    matrix_params = len(engine.model.schedule) * per_layer_ffn + n_conv * conv + n_attn * attn
    elt = 2 if engine.precision == "bfloat16" else 4
    weight_bytes = (matrix_params + V * H) * elt          # every matrix once; the tied table is the head
    kv_per_token = n_attn * 2 * nkv * hd * elt

    def prefill_flops(T, wanted=1):
        # what the step executes: the last layer's feed-forward runs on the wanted rows only (as
        # in the reference), every other product on all T tokens; causal attention; the head on the wanted rows
        return 2.0 * T * (matrix_params - per_layer_ffn) + 2.0 * wanted * per_layer_ffn + 2.0 * wanted * V * H \
            + n_attn * 4.0 * nh * hd * T * (T + 1) / 2
    return weight_bytes, kv_per_token, prefill_flops, matrix_params + V * H


def measure_decode(engine, batch, steps, warmup, rng, sampler=None, prompt=None):
    """-> (ms per step, launches per step, h2d bytes per step, mean context) with `batch`
    requests holding `prompt` (default PROMPT) tokens each."""
    PROMPT = prompt or globals()["PROMPT"]
    import torch
    from imparo_b200.engine import StepItem
    from imparo_b200.kernels import ops
    ids = list(range(1000 * batch, 1000 * batch + batch))
    V = engine.vocab_size
    for r in ids:
        engine.add_request(r)
        engine.step([StepItem(r, rng.integers(0, V, PROMPT).tolist(), [PROMPT - 1])])
    out_ids = torch.empty(batch, dtype=torch.int32, device=engine.device)

    def one():
        logits = engine.step_fn([StepItem(r, [int(t)], [0]) for r, t in zip(ids, rng.integers(0, V, batch))])
        ops.sample_rows(logits, None, None, out_ids)
    for _ in range(max(warmup, 3)):
        one()
    torch.cuda.synchronize()
    before = dict(ops.COUNTS)
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        one()
    end.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(end) / steps
    launches = (ops.COUNTS["own"] - before["own"]) / steps
    library = (ops.COUNTS["library"] - before["library"]) / steps
    ctx = PROMPT + max(warmup, 3) + steps / 2.0
    engine.check_device_status()
    for r in ids:
        engine.end_request(r)
    return ms, launches, library, ctx


def measure_prefill(engine, reps, warmup, rng, prompt=None):
    import torch
    PROMPT = prompt or globals()["PROMPT"]
    from imparo_b200.engine import StepItem
    V = engine.vocab_size
    times = []
    for i in range(warmup + reps):
        toks = rng.integers(0, V, PROMPT).tolist()
        engine.add_request(77000 + i)
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        engine.step_fn([StepItem(77000 + i, toks, [PROMPT - 1])])
        end.record()
        torch.cuda.synchronize()
        engine.end_request(77000 + i)
        if i >= warmup:
            times.append(start.elapsed_time(end))
    return statistics.median(times)


def measure_e2e(engine, batch, steps, warmup, rng):
    """Decode tokens per second through Engine.generate: wall clock from the end of decode
    step `warmup` to the end of decode step `warmup + steps`, host lists in and out."""
    V = engine.vocab_size
    prompts = [rng.integers(0, V, PROMPT).tolist() for _ in range(batch)]
    stamps, h2d = [], []

    def on_step(plan):
        if all(e.count == 1 for e in plan) and len(plan) == batch:
            stamps.append(time.perf_counter())
            h2d.append(engine.step_fn.last_h2d_bytes)       # this step's batch description, as uploaded
    n_new = warmup + steps + 2 + 2 * batch      # requests start decoding up to ~batch steps apart
    out = engine.generate(prompts, max_tokens=n_new, on_step=on_step, stop_token_ids=[])
    assert all(len(o) == n_new for o in out) and len(stamps) > warmup + steps, (len(stamps), warmup + steps)
    dt = stamps[warmup + steps] - stamps[warmup]
    return batch * steps / dt, max(h2d[warmup:warmup + steps + 1])


def workload_sizes(args):
    """LFM2-1.2B layer sizes (all 16 layers, random bfloat16 weights) at further sizes than the headline: one prompt
    of 512, 2,048, 8,192 and 32,768 tokens (tokens per second; flops over time against the measured bfloat16 peak), and
    decode steps of 8 requests at contexts of 2,048, 16,384 and 32,768 tokens (tokens per second; bytes the step has
    to read over its time against the measured HBM peak)."""
    import numpy as np
    import torch
    from imparo_b200.engine import Engine
    rng = np.random.default_rng(0)
    pk = peaks()
    longest = 32768
    engine = Engine(config=dict(LFM2_1_2B), seed=0, dtype="bfloat16", ctx=longest + 256, parallel=8, page_size=PAGE,
                    max_step_tokens=longest, random_init={"norm_jitter": 0.0})
    weight_bytes, kv_per_token, prefill_flops, n_params = model_numbers(engine)
    out = {"metric": "LFM2-1.2B at further sizes: prefill of one prompt, decode at batch 8", "unit": "tokens/s", "dtype": "bf16",
           "data": "synthetic (random weights, uniform-random token ids)", "prefill": {}, "decode_b8": {}}
    with ClockSampler() as clocks:
        for T in (512, 2048, 8192, 32768):
            ms = measure_prefill(engine, reps=3 if T > 8192 else 5, warmup=3, rng=rng, prompt=T)
            out["prefill"][str(T)] = {"value": round(T * 1000.0 / ms, 1), "ms": round(ms, 3),
                                      "frac": round(prefill_flops(T) / (ms * 1e-3) / (pk["bf16_tflops_burst"] * 1e12), 4)}
        for ctx_len in (2048, 16384, 32768):
            ms, _, _, ctx = measure_decode(engine, 8, 30, 5, rng, prompt=ctx_len)
            nbytes = weight_bytes + 8 * ctx * kv_per_token
            out["decode_b8"][str(ctx_len)] = {"value": round(8 * 1000.0 / ms, 1), "ms_per_step": round(ms, 4),
                                              "roofline": {"bound": "hbm", "achieved": round(nbytes / (ms * 1e-3) / 1e9, 1),
                                                           "peak": pk["hbm_gbs"], "unit": "GB/s",
                                                           "frac": round(nbytes / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], 4)}}
    out["peaks"] = pk["source"]
    out["config"] = {"model": "LFM2-1.2B", "layers": 16, "layers_of_config": 16, "page_size": PAGE, "params": n_params}
    out["clocks"] = clocks.summary()
    print(json.dumps(out))
    return 0


def _preset(name):
    with open(os.path.join(ROOT, "imparo_b200", "config", "presets", name + ".json")) as f:
        return json.load(f)


def workload_continuous(args):
    """LFM2-700M sizes: a continuous batch of requests (32 unless --requests says otherwise) with prompt lengths
    uniform in [64, 4096] through 32 slots, prompts in portions under a 512-token step budget beside the running
    decode rows, temperature 0.7 (seeded), 128 new tokens each; requests join and leave mid-run, and with more
    requests than slots, slots and pages are used again.  Besides tokens per second: the step-time split (the
    reference prints step / gpu / gap medians for its loop, imparo-server/src/sched.rs:572-649): per class of step
    (decode rows only; portions beside decode rows; portions only) the device time between the events recorded after
    consecutive steps, the host time between their launches, and, for steps of decode rows only, the bytes they have
    to read (weights once, the cache of their rows) over that time against the measured HBM peak."""
    import numpy as np
    import torch
    from imparo_b200.engine import Engine
    from imparo_b200.kernels import ops
    rng = np.random.default_rng(1)
    n, slots, new = args.requests, 32, 128
    engine = Engine(config=_preset("lfm2_700m"), seed=0, dtype="bfloat16", ctx=4096 + new, parallel=slots, page_size=PAGE,
                    max_step_tokens=512, random_init={"norm_jitter": 0.0})
    pk = peaks()
    weight_bytes, kv_per_token, prefill_flops, n_params = model_numbers(engine)
    V = engine.vocab_size
    lens = [int(x) for x in rng.integers(64, 4097, n)]
    prompts = [rng.integers(0, V, k).tolist() for k in lens]
    engine.generate(prompts[:4], max_tokens=8, temperature=0.7, seed=list(range(4)))       # warm-up: buffers, first graphs
    steps = []                # per step: (class, event after it, host time, bytes of a decode-only step, tokens)

    def on_step(plan):
        portions = any(e.count > 1 or e.start == 0 for e in plan)
        rows = any(e.count == 1 and e.start > 0 for e in plan)
        kind = "portions_beside_decode_rows" if portions and rows else ("portions_only" if portions else "decode_rows_only")
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        nbytes = weight_bytes + kv_per_token * sum(e.start + e.count for e in plan)
        steps.append((kind, ev, time.perf_counter(), nbytes, sum(e.count for e in plan), len(plan)))
    # Two passes over the same requests with the same engine.  The first meets every step shape for the first time
    # (a new shape runs launch by launch once and is captured the second time it comes); the second is the timed
    # one: a server in its steady state, whose shapes have come before.  Both are reported.
    first = {}
    for timed in (False, True):
        steps.clear()
        before, replays, captures = dict(ops.COUNTS), engine.step_fn.graph_replays, engine.step_fn.graph_captures
        with ClockSampler() as clocks:
            t0 = time.perf_counter()
            out = engine.generate(prompts, max_tokens=new, temperature=0.7, seed=list(range(n)), on_step=on_step, stop_token_ids=[])
            torch.cuda.synchronize()
            dt = time.perf_counter() - t0
        assert all(len(o) == new for o in out)
        if not timed:
            first = {"value": round((sum(lens) + n * new) / dt, 1), "seconds": round(dt, 3), "steps": len(steps),
                     "graph_replays": engine.step_fn.graph_replays - replays,
                     "graph_captures": engine.step_fn.graph_captures - captures}
    st = engine.stats()
    split = {}
    for kind in ("decode_rows_only", "portions_beside_decode_rows", "portions_only"):
        dev, host, gbs, toks = [], [], [], []
        for i in range(1, len(steps)):
            if steps[i][0] != kind:
                continue
            d_ms = steps[i - 1][1].elapsed_time(steps[i][1])
            dev.append(d_ms)
            host.append((steps[i][2] - steps[i - 1][2]) * 1e3)
            toks.append(steps[i][4])
            if kind == "decode_rows_only" and d_ms > 0:
                gbs.append(steps[i][3] / (d_ms * 1e-3) / 1e9)
        if dev:
            split[kind] = {"steps": len(dev), "device_ms_median": round(statistics.median(dev), 4),
                           "host_ms_between_launches_median": round(statistics.median(host), 4),
                           "tokens_per_step_mean": round(sum(toks) / len(toks), 1)}
            if gbs:
                split[kind]["roofline"] = {"bound": "hbm", "achieved": round(statistics.median(gbs), 1), "peak": pk["hbm_gbs"],
                                           "unit": "GB/s", "frac": round(statistics.median(gbs) / pk["hbm_gbs"], 4),
                                           "peaks": pk["source"]}
    device_total = steps[0][1].elapsed_time(steps[-1][1]) * 1e-3 if len(steps) > 1 else 0.0
    flops = sum(prefill_flops(k) for k in lens)
    print(json.dumps({
        "metric": "LFM2-700M continuous batching, prompt + generated tokens per second (wall clock, through Engine.generate)",
        "value": round((sum(lens) + n * new) / dt, 1), "unit": "tokens/s", "generated_per_s": round(n * new / dt, 1),
        "seconds": round(dt, 3), "device_seconds_first_to_last_step": round(device_total, 3),
        "requests": n, "slots": slots, "prompt_tokens": sum(lens), "new_tokens": n * new,
        "first_pass": first, "step_budget": 512, "steps": len(steps), "mean_rows_per_step": round(sum(s_[5] for s_ in steps) / max(len(steps), 1), 1),
        "step_time_split": split,
        "prompt_flops_over_time_frac_of_bf16_peak": round(flops / max(dt, 1e-9) / (pk["bf16_tflops"] * 1e12), 4),
        "graph_replays": engine.step_fn.graph_replays - replays, "graph_captures": engine.step_fn.graph_captures - captures,
        "graph_resets": engine.step_fn.graph_resets, "preemptions": st["preemptions"], "failed": st["failed"],
        "own_kernel_launches": ops.COUNTS["own"] - before["own"], "library_gemms": ops.COUNTS["library"] - before["library"],
        "dtype": "bf16", "data": "synthetic (random weights, uniform-random token ids)", "clocks": clocks.summary()}))
    return 0


def workload_long(args):
    """LFM2-350M sizes: 4 requests with 32,768-token prompts and 512 greedy tokens each, in bfloat16 (all 16 layers:
    throughput, with the prefill's flops over its time against the measured bfloat16 peak and the decode step's bytes
    over its time against the measured HBM peak).  Then the 32-bit check: the logits at sampled positions of one
    32,768-token prompt, through the engine whole and in portions of 1,024 tokens, against the plain implementation
    (tests/plain, numpy, whole sequence, no cache).  The plain forward over 32,768 tokens is slow, so the check runs
    on the first --long-check-layers layers of the configuration (4 by default: two convolution blocks and two
    attention blocks, every width as configured); `config` names both numbers."""
    import tempfile
    import numpy as np
    import torch
    from imparo_b200.engine import Engine, StepItem
    from imparo_b200.weights import write_random_model
    cfg = _preset("lfm2_350m")
    pk = peaks()
    rng = np.random.default_rng(2)
    P, new, B = 32768, 512, 4
    out = {"metric": "LFM2-350M long context: 4 x 32,768-token prompts + 512 greedy tokens", "unit": "tokens/s",
           "data": "synthetic (random weights, uniform-random token ids)", "dtype": "bf16 (throughput), fp32 (check)"}
    engine = Engine(config=cfg, seed=0, dtype="bfloat16", ctx=P + new, parallel=B, page_size=PAGE, max_step_tokens=P,
                    random_init={"norm_jitter": 0.0})
    weight_bytes, kv_per_token, prefill_flops, n_params = model_numbers(engine)
    prompts = [rng.integers(0, engine.vocab_size, P).tolist() for _ in range(B)]
    stamps = []

    def on_step(plan):
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        stamps.append((time.perf_counter(), sum(e.count for e in plan), ev))
    # a first pass of the same shapes (buffers sized, the prompt step and the decode step captured), timed apart
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    engine.generate(prompts, max_tokens=16, stop_token_ids=[], on_step=on_step)
    torch.cuda.synchronize()
    first_decode = next(i for i, (_, c, _) in enumerate(stamps) if c == B)
    out["first_pass"] = {"prefill_tokens_per_s": round(B * P / (stamps[first_decode][0] - t0), 1),
                         "prefill_ms": round((stamps[first_decode][0] - t0) * 1e3, 1)}
    stamps.clear()
    with ClockSampler() as clocks:
        t0 = time.perf_counter()
        got = engine.generate(prompts, max_tokens=new, stop_token_ids=[], on_step=on_step)
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
    assert all(len(g) == new for g in got)
    first_decode = next(i for i, (_, c, _) in enumerate(stamps) if c == B)
    prefill_s = stamps[first_decode][0] - t0
    decode = [stamps[i - 1][2].elapsed_time(stamps[i][2]) for i in range(first_decode + 1, len(stamps)) if stamps[i][1] == B]
    dec_ms = statistics.median(decode)
    step_bytes = weight_bytes + B * (P + new / 2) * kv_per_token
    out["value"] = round(B * P / prefill_s, 1)
    out["bf16"] = {"seconds": round(dt, 3), "prefill_tokens_per_s": round(B * P / prefill_s, 1),
                   "prefill": {"tokens": B * P, "ms": round(prefill_s * 1e3, 1),
                               "frac": round(B * prefill_flops(P) / prefill_s / (pk["bf16_tflops"] * 1e12), 4)},
                   "decode_tokens_per_s": round(B * 1000.0 / dec_ms, 1), "decode_ms_per_step": round(dec_ms, 4),
                   "roofline": {"bound": "hbm", "achieved": round(step_bytes / (dec_ms * 1e-3) / 1e9, 1), "peak": pk["hbm_gbs"],
                                "unit": "GB/s", "frac": round(step_bytes / (dec_ms * 1e-3) / 1e9 / pk["hbm_gbs"], 4),
                                "peaks": pk["source"], "bytes_per_step": int(step_bytes)},
                   "new_tokens_each": new, "layers": cfg["num_hidden_layers"]}
    del engine
    torch.cuda.empty_cache()

    # ---- the 32-bit check against the plain implementation ----
    from tests.plain.lfm2_plain import PlainLfm2
    n_layers = args.long_check_layers
    small = dict(cfg)
    # the configuration's first blocks up to and including its second attention block, cut to n_layers by keeping the
    # last n_layers of them: two convolution and two attention blocks at the default of 4
    types = list(cfg["layer_types"])
    second_attn = [i for i, t_ in enumerate(types) if t_ != "conv"][1]
    small["layer_types"] = types[max(0, second_attn + 1 - n_layers):second_attn + 1] if n_layers < len(types) else types
    small["num_hidden_layers"] = len(small["layer_types"])
    places = [0, 1023, 1024, 16384, P - 1]
    toks = prompts[0]
    with tempfile.TemporaryDirectory(prefix="imparo_b200_long_") as d:
        write_random_model(d, small, seed=0, dtype="float32", norm_jitter=0.1)
        t1 = time.perf_counter()
        ref = PlainLfm2(d, np.float32).logits_at(toks, places, attend_block=256).astype(np.float64)
        plain_s = time.perf_counter() - t1
        engine = Engine(d, dtype="float32", ctx=P, parallel=1, page_size=PAGE, max_step_tokens=P)
        rows = {}
        for name, cut in (("whole", P), ("portions_of_1024", 1024)):
            engine.add_request(900 + cut)
            got_rows, at = [], 0
            t2 = time.perf_counter()
            while at < P:
                k = min(cut, P - at)
                want = [p_ - at for p_ in places if at <= p_ < at + k]
                lg = engine.step([StepItem(900 + cut, toks[at:at + k], want)])
                if want:
                    got_rows.append(lg.double().cpu().numpy())
                at += k
            torch.cuda.synchronize()
            rows[name] = (np.concatenate(got_rows), time.perf_counter() - t2)
            engine.end_request(900 + cut)
        engine.check_device_status()
    scale = float(np.abs(ref).max())
    out["fp32"] = {"layers": small["num_hidden_layers"], "layers_of_config": cfg["num_hidden_layers"],
                   "layer_types": small["layer_types"], "positions": places, "logit_scale": round(scale, 4),
                   "vs_plain_max_abs_diff": {k: float(np.abs(v[0] - ref).max()) for k, v in rows.items()},
                   "vs_plain_max_abs_diff_over_scale": {k: float(np.abs(v[0] - ref).max() / scale) for k, v in rows.items()},
                   "whole_vs_portions_max_abs_diff": float(np.abs(rows["whole"][0] - rows["portions_of_1024"][0]).max()),
                   "same_argmax_as_plain": {k: bool((v[0].argmax(-1) == ref.argmax(-1)).all()) for k, v in rows.items()},
                   "engine_seconds": {k: round(v[1], 2) for k, v in rows.items()}, "plain_seconds": round(plain_s, 1),
                   "plain": "tests/plain/lfm2_plain.py, numpy float32, whole sequence, attention a block of 256 queries at a time"}
    out["vs_plain_max_abs_diff"] = max(out["fp32"]["vs_plain_max_abs_diff"].values())
    out["config"] = {"model": "LFM2-350M", "global_batch": B, "prompt_len": P, "new_tokens": new, "layers": cfg["num_hidden_layers"],
                     "layers_of_config": cfg["num_hidden_layers"], "check_layers": small["num_hidden_layers"],
                     "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
                     "vocab": cfg["vocab_size"], "page_size": PAGE, "params": n_params}
    out["clocks"] = clocks.summary()
    print(json.dumps(out))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=None, help="run fewer layers than the configuration has (named in config)")
    ap.add_argument("--skip-points", action="store_true", help="skip the batch-1 and batch-64 points")
    ap.add_argument("--only-decode", action="store_true", help="time the decode steps only (for profiler captures)")
    ap.add_argument("--only-prefill", action="store_true", help="time the 2,048-token prompt only (for profiler captures)")
    ap.add_argument("--workload", default="headline", choices=["headline", "continuous", "long", "sizes"],
                    help="headline (default): the line the contract names.  continuous: LFM2-700M sizes, requests with prompts "
                         "of 64 to 4,096 tokens through 32 slots in 512-token portions beside decode rows, temperature 0.7, 128 new "
                         "tokens each.  long: LFM2-350M sizes, 4 prompts of 32,768 tokens and 512 greedy tokens each, bfloat16 and 32-bit")
    ap.add_argument("--requests", type=int, default=32, help="continuous: requests in all (the baseline's workload has 32)")
    ap.add_argument("--long-check-layers", type=int, default=4, help="long: layers of the 32-bit check against the plain implementation")
    args = ap.parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": "zeraix/imparo is a Rust workspace (no setup.py or pyproject.toml: "
                          "pip reports 'not installable') and this image has no cargo/rustc, so it cannot be built or run here"}))
        return 0
    if args.gpus != 1:
        print("bench.py: this engine runs on ONE GPU; --gpus > 1 is not supported (nothing was measured)")
        return 2
    import numpy as np
    import torch
    from imparo_b200.engine import Engine
    from imparo_b200.kernels import ops

    if args.workload == "continuous":
        return workload_continuous(args)
    if args.workload == "long":
        return workload_long(args)
    if args.workload == "sizes":
        return workload_sizes(args)
    cfg = dict(LFM2_1_2B)
    if args.layers is not None and args.layers < cfg["num_hidden_layers"]:
        cfg["layer_types"] = cfg["layer_types"][:args.layers]
        cfg["num_hidden_layers"] = args.layers
    steps, warmup = args.steps, max(args.warmup, 3)
    rng = np.random.default_rng(0)
    max_batch = args.batch if (args.skip_points or args.only_decode or args.only_prefill) else max(64, args.batch)
    engine = Engine(config=cfg, seed=0, dtype="bfloat16", ctx=CTX, parallel=max_batch, page_size=PAGE,
                    max_step_tokens=PROMPT, random_init={"norm_jitter": 0.0})
    pk = peaks()
    weight_bytes, kv_per_token, prefill_flops, n_params = model_numbers(engine)

    if args.only_prefill:
        pre_ms = measure_prefill(engine, reps=max(1, steps), warmup=warmup, rng=rng)
        print(json.dumps({"metric": "prefill only", "tokens": PROMPT, "ms": round(pre_ms, 3),
                          "value": round(PROMPT * 1000.0 / pre_ms, 1),
                          "frac": round(prefill_flops(PROMPT) / (pre_ms * 1e-3) / (pk["bf16_tflops_burst"] * 1e12), 4)}))
        return 0
    with ClockSampler() as clocks:
        ms, launches, library, ctx = measure_decode(engine, args.batch, steps, warmup, rng)
    value = args.batch * 1000.0 / ms
    step_bytes = weight_bytes + args.batch * ctx * kv_per_token
    achieved = step_bytes / (ms * 1e-3) / 1e9

    if args.only_decode:
        print(json.dumps({"metric": "decode only", "batch": args.batch, "ms_per_step": round(ms, 4), "value": round(value, 1),
                          "achieved_gbs": round(achieved, 1), "own_kernels_per_step": launches, "library_gemms_per_step": library}))
        return 0
    pre_ms = measure_prefill(engine, reps=5, warmup=3, rng=rng)
    pre_flops = prefill_flops(PROMPT)
    prefill = {"value": round(PROMPT * 1000.0 / pre_ms, 1), "tokens": PROMPT, "ms": round(pre_ms, 3),
               "frac": round(pre_flops / (pre_ms * 1e-3) / (pk["bf16_tflops_burst"] * 1e12), 4)}

    points = {}
    if not args.skip_points:
        for b in (1, 64):
            pms, _, _, _ = measure_decode(engine, b, max(20, steps // 4), warmup, rng)
            points[f"decode_b{b}"] = round(b * 1000.0 / pms, 1)

    # h2d: the step's descriptor (tokens, positions, request index, row starts, slots, start
    # positions, wanted rows, one block-table row per request), counted from the copied tensor
    e2e_value, h2d = measure_e2e(engine, args.batch, steps, warmup, rng)

    line = {
        "metric": "LFM2-1.2B decode tok/s @ batch 8 (2,048-token prompts, ctx 4,096)", "value": round(value, 1), "unit": "tokens/s",
        "n_gpus": 1, "steps": steps, "warmup": warmup, "ms_per_step": round(ms, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic (random weights, uniform-random token ids)",
        "impl": "ours",
        "config": {"model": "LFM2-1.2B", "global_batch": args.batch, "seq_len": CTX, "prompt_len": PROMPT, "parallelism": "1gpu",
                   "layers": cfg["num_hidden_layers"], "layers_of_config": LFM2_1_2B["num_hidden_layers"],
                   "hidden": cfg["hidden_size"], "heads": 32, "kv_heads": 8, "head_dim": 64, "ff_dim": engine.config.ff_dim,
                   "vocab": cfg["vocab_size"], "conv_L_cache": 3, "page_size": PAGE, "params": n_params,
                   "l2": "inputs larger than L2 (2.3 GB of weights read per step)", "cuda_graph": True,
                   "last_ffn": "wanted rows only"},
        "e2e": {"value": round(e2e_value, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4 * args.batch},
        "gpu_launches": int(round(launches * steps)), "own_kernels_per_step": round(launches, 1),
        "library_gemms_per_step": round(library, 1),
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "peaks": pk["source"], "bytes_per_step": int(step_bytes)},
        "points": points,
        "clocks": clocks.summary(),
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
