"""The Python entry point: load (or draw) a model, own its cache, run steps, generate.

    engine = Engine("model_dir", dtype="bfloat16", ctx=4096, parallel=8)
    out = engine.generate([[1, 2, 3], [4, 5]], max_tokens=16, temperature=0.0)

Option names follow the reference where it has them: model (-m/--model), ctx (-c/--ctx,
the context length, default 4096), parallel (-np/--parallel, requests that decode at
once), the request fields max_tokens and temperature (imparo-server/src/main.rs:178-240,
1811 ff.).  Page size, page count and the step's token budget are this engine's own.
"""
from __future__ import annotations

import sys

import time
from typing import Dict, List, Optional, Sequence, Union

import torch

from ..cache import CacheManager
from ..config.engine import EngineConfig
from ..config.registry import load_config
from ..kernels import lib as _lib
from ..kernels import ops
from ..parts.base import Runtime, Workspace
from ..parts.model import Model
from ..sampling import Sampler
from ..weights.loader import load_weights, target_dtype
from ..weights.random_init import draw_random_tensors
from .scheduler import Scheduler, padded_rows
from .step import StepFunction, StepItem

_PRECISIONS = {"bfloat16": "bfloat16", "bf16": "bfloat16", "float32": "float32", "fp32": "float32", "f32": "float32"}


class Engine:
    def __init__(self, model: Optional[str] = None, *, config: Optional[dict] = None, seed: int = 0,
                 dtype: Optional[str] = None, device: Union[str, torch.device, None] = None, ctx: Optional[int] = None,
                 parallel: Optional[int] = None, page_size: Optional[int] = None, num_pages: Optional[int] = None,
                 max_step_tokens: Optional[int] = None, random_init: Optional[dict] = None,
                 probe_layer: Optional[int] = None, probe=None, switches: Optional[dict] = None,
                 config_file: Optional[str] = None, engine_config: Optional[EngineConfig] = None,
                 use_graphs: Optional[bool] = None, pad_rows: Optional[bool] = None, capture_first: Optional[bool] = None):
        """model: a folder with config.json and model.safetensors.  Or config (a config.json
        dictionary) with seed: random weights drawn on the device (random_init may give
        matrix_std, conv_std, norm_jitter).

        The engine's own settings are one typed EngineConfig (config/engine.py), resolved here once: a keyword
        given to this constructor wins over the environment (IMPARO_CTX, IMPARO_PARALLEL, IMPARO_GEMM, ...), which
        wins over the JSON file config_file (or the one IMPARO_CONFIG names), which wins over the defaults; or
        pass a resolved engine_config.  dtype: "bfloat16" | "float32".  ctx: the most positions one request may
        reach.  parallel: the most requests live at once.  num_pages: pages in each pool (default: enough for
        parallel requests of ctx positions).  switches: kernel-path switches by name (KernelSwitches).
        use_graphs: replay captured steps; capture_first: capture a shape the first time it comes; pad_rows: fill
        the one-token rows of a step up to few sizes (StepFunction).
        probe_layer: a schedule entry whose block shows its stages (stream in, mixer norm, stream after the mixer,
        feed-forward norm, stream out) to probe(name, tensor); the default probe prints rms, sum and the first
        five values of each to stderr, as the reference's stage probes do (imparo-model/src/cpu_support.rs:26-46).
        Probing evaluates every stage on its own and switches graph replay off: for comparing engines, not for timing."""
        if engine_config is None:
            engine_config = EngineConfig.resolve(
                flags={"dtype": dtype, "device": None if device is None else str(device), "ctx": ctx, "parallel": parallel,
                       "page_size": page_size, "num_pages": num_pages, "max_step_tokens": max_step_tokens,
                       "probe_layer": probe_layer, "switches": switches, "use_graphs": use_graphs, "pad_rows": pad_rows,
                       "capture_first": capture_first}, file=config_file)
        self.engine_config = cfg = engine_config
        if cfg.dtype not in _PRECISIONS:
            raise ValueError(f"dtype must be one of {sorted(_PRECISIONS)}")
        self.precision = _PRECISIONS[cfg.dtype]
        self.device = torch.device(cfg.device)
        if self.device.type != "cuda" or not torch.cuda.is_available():
            raise RuntimeError("imparo_b200 runs on a CUDA device (sm_100a); there is no CPU path")
        _lib.kernels()      # build/load now: fail loudly if the extension is missing
        torch.cuda.set_device(self.device)
        ctx, parallel, page_size, num_pages = cfg.ctx, cfg.parallel, cfg.page_size, cfg.num_pages
        max_step_tokens, probe_layer = cfg.max_step_tokens, cfg.probe_layer
        self.arch, self.config = load_config(model if model is not None else config)
        self.status = ops.new_status(self.device)
        self.rt = Runtime(precision=self.precision, device=self.device, status=self.status,
                          workspace=Workspace(self.device), launch_state=ops.LaunchState(cfg.switches))
        self.model = Model(self.arch.model_spec(self.config), self.rt)
        specs = self.model.weight_specs()
        if model is not None:
            tensors = load_weights(model, specs, self.precision, self.device,
                                   duplicates=dict(self.model.spec.duplicate_tensors))
        else:
            if config is None:
                raise ValueError("give a model folder or a config dictionary")
            drawn = draw_random_tensors(specs, seed, self.precision, self.device, **(random_init or {}))
            tensors = {w.name: drawn[w.name].to(target_dtype(w.role, self.precision)) for w in specs if w.name in drawn}
        self.weight_bytes = sum(t.numel() * t.element_size() for t in tensors.values())
        self.model.bind(tensors)
        del tensors
        self.ctx = min(int(ctx), self.model.spec.max_positions)
        self.parallel = int(parallel)
        self.page_size = int(page_size)
        if num_pages is None:
            num_pages = self.parallel * ((self.ctx + self.page_size - 1) // self.page_size)
        self.cache = CacheManager(self.model.cache_requirements(), self.page_size, int(num_pages), self.parallel,
                                  kv_dtype=self.rt.act_dtype, device=self.device)
        self.max_step_tokens = int(max_step_tokens)
        self.step_fn = StepFunction(self.model, self.cache, self.max_step_tokens, self.parallel, use_graphs=cfg.use_graphs,
                                    pad_rows=cfg.pad_rows, capture_first=cfg.capture_first)
        if probe_layer is not None:
            if not 0 <= int(probe_layer) < len(self.model.schedule):
                raise ValueError(f"probe_layer {probe_layer} is not one of the model's {len(self.model.schedule)} schedule entries")
            self.rt.probe_entry = int(probe_layer)
            self.rt.probe = probe if probe is not None else self._print_probe
            self.step_fn.use_graphs = False
        # what the largest step holds, for buffers that are then made once (a moved buffer voids the captured graphs)
        rows = padded_rows(self.parallel) + 2 if cfg.pad_rows else self.parallel + 2
        self.rt.workspace.expect(tokens=min(self.max_step_tokens + rows, 8192), rows=min(rows, 512), context=self.ctx)
        previous = ops.use_state(self.rt.launch_state)
        try:
            ops.prepare(self.device, rows=rows)         # nothing is left to be made at a first use, i.e. under capture
        finally:
            ops.use_state(previous)
        self.step_fn.reserve(min(self.max_step_tokens + rows, 8192), min(rows, 512), -(-self.ctx // self.page_size))
        self.sampler = Sampler(self.device, max_rows=max(rows, 8))
        self.vocab_size = self.model.spec.vocab_size
        self._stats = {"steps": 0, "prompt_tokens": 0, "decode_tokens": 0, "preemptions": 0, "seconds": 0.0}

    def _print_probe(self, name: str, t: torch.Tensor) -> None:
        v = t.detach().float()
        head = ", ".join(f"{x:.6g}" for x in v.reshape(-1)[:5].tolist())
        print(f"probe entry {self.rt.probe_entry} {name} {tuple(t.shape)}: rms {float(v.pow(2).mean().sqrt()):.6g} "
              f"sum {float(v.sum()):.6g} first [{head}]", file=sys.stderr, flush=True)

    # -- the step function, for callers that schedule themselves ---------------------------
    def add_request(self, request: int) -> None:
        self.cache.add(request)

    def end_request(self, request: int) -> None:
        self.cache.release(request)

    def step(self, items: Sequence[StepItem]) -> Optional[torch.Tensor]:
        """items: StepItem(request, tokens, want).  Returns float32 logits [wanted, vocab]
        on the device, or None.  The result is the caller's own tensor: the step function writes
        its logits into a buffer that the next step of the same shape overwrites (a workspace view,
        or a captured graph's output), so what is handed out here is a copy of it."""
        self._check_tokens(items)
        out = self.step_fn(items)
        return None if out is None else out.clone()

    def check_device_status(self) -> None:
        ops.read_status(self.status)

    def _check_tokens(self, items) -> None:
        for it in items:
            toks = it.tokens
            if len(toks) and (min(toks) < 0 or max(toks) >= self.vocab_size):
                raise ValueError(f"request {it.request}: token id out of range [0, {self.vocab_size})")
            if self.cache.has(it.request) and self.cache.cached(it.request) + len(toks) > self.ctx:
                raise ValueError(f"request {it.request}: {self.cache.cached(it.request)} + {len(toks)} tokens "
                                 f"exceed the context length {self.ctx}")

    # -- generation --------------------------------------------------------------------------
    def generate(self, prompts: Sequence[Sequence[int]], max_tokens: Union[int, Sequence[int]] = 16,
                 temperature: Union[float, Sequence[float]] = 0.0, seed: Union[int, Sequence[int]] = 0,
                 stop_token_ids: Optional[Sequence[int]] = None, on_step=None) -> List[List[int]]:
        """Continuous batching over the prompts (lists of token ids).  Returns the generated
        ids per prompt.  temperature 0 is greedy; seed keys the per-request random stream.
        A stop token ends its request and is not part of the output.  A request that cannot
        fit the cache even alone ends with what it has (see failed in stats())."""
        previous = ops.use_state(self.rt.launch_state)       # the sampler's launches use this engine's scratch too
        try:
            return self._generate(prompts, max_tokens, temperature, seed, stop_token_ids, on_step)
        finally:
            ops.use_state(previous)

    def _generate(self, prompts, max_tokens, temperature, seed, stop_token_ids, on_step):
        n = len(prompts)
        as_list = lambda v: list(v) if isinstance(v, (list, tuple)) else [v] * n
        max_new, temps, seeds = as_list(max_tokens), as_list(temperature), as_list(seed)
        stops = set(self.model.spec.eos_token_ids if stop_token_ids is None else stop_token_ids)
        sched = Scheduler(self.cache, self.max_step_tokens, self.parallel, self.ctx, count_padded_rows=self.step_fn.pad_rows)
        tokens: Dict[int, List[int]] = {}
        index: Dict[int, int] = {}
        out: List[List[int]] = [[] for _ in range(n)]
        for i, p in enumerate(prompts):
            p = list(p)
            if not p:
                raise ValueError(f"prompt {i} is empty")
            if min(p) < 0 or max(p) >= self.vocab_size:
                raise ValueError(f"prompt {i}: token id out of range [0, {self.vocab_size})")
            if max_new[i] <= 0:
                continue            # ends before taking a token (imparo-server/src/sched.rs:427-431)
            rid = sched.submit(len(p), max_new[i])
            tokens[rid] = p
            index[rid] = i
        failed: List[int] = []
        t0 = time.perf_counter()
        log = self.engine_config.log
        t_log = t0
        gen = {rid: 0 for rid in tokens}        # tokens sampled so far per request (values may still be on the device)
        dead = set()                            # ended by a stop token
        carry = None                            # (wanting entries, PendingSample): sampled, values not read yet

        def settle(c) -> None:
            """Read a step's sampled ids and book them.  The scheduler was already told that
            these requests go on; one that hit a stop token is ended now.  This runs between
            step_done and the next plan, so the request is in no planned step; if the step in
            flight holds a row of it, that row is wasted work whose pages nobody reads."""
            entries, pending = c
            for e, tok in zip(entries, pending.result()):
                r = e.request
                if r in dead:
                    continue
                if tok in stops:
                    dead.add(r)
                    if sched.abort(r) == -2:
                        raise RuntimeError("a request ended by a stop token is part of a planned step")
                else:
                    out[index[r]].append(tok)
                    tokens[r].append(tok)

        idle = 0
        while carry is not None or sched.has_work():
            plan = sched.plan() if sched.has_work() else []
            for rid in sched.take_failed():
                failed.append(index[rid])
            if not plan:
                if carry is not None:
                    settle(carry)
                    carry = None
                    continue
                idle += 1
                if idle > 2:
                    raise RuntimeError("the scheduler has requests but plans no step")
                continue
            idle = 0
            # Rows whose token is the id the step in flight is sampling take it from that step's output
            # on the device; prompt portions bring tokens the host knows.  Nothing else occurs: the
            # pending ids are read right after the next step is issued, so the only values the host
            # lacks when it plans are those of the step in flight, each wanted by a request whose next
            # row is that one token; and a request preempted in a plan call is not admitted again in
            # the same call, so its recomputation starts with every token on the host
            # (tests/test_scheduler.py checks this over random runs).
            pending_at = {e.request: i for i, e in enumerate(carry[0])} if carry is not None else {}
            unknown = [e for e in plan if e.start + e.count > len(tokens[e.request])]
            for e in unknown:
                if not (e.count == 1 and e.start == len(tokens[e.request]) and e.request in pending_at):
                    sched.step_done(False)
                    raise RuntimeError(f"request {e.request}: the plan needs a token that is neither on the host "
                                       "nor being sampled by the step in flight")
            fed = carry is not None
            items, token_src = [], []
            for e in plan:
                want = [e.count - 1] if e.want else []
                if e.start + e.count > len(tokens[e.request]):
                    items.append(StepItem(e.request, [0], want))
                    token_src.append(pending_at[e.request])
                else:
                    items.append(StepItem(e.request, tokens[e.request][e.start:e.start + e.count], want))
                    token_src.extend([-1] * e.count)
            device_tokens = (carry[1].dev_ids, token_src) if fed and unknown else None
            try:
                logits = self.step_fn(items, manage_cache=False, device_tokens=device_tokens)
            except Exception:
                sched.step_done(False)
                raise
            sched.step_done(True)
            if fed:
                settle(carry)                   # while the step just launched runs
                carry = None
            wanting = [e for e in plan if e.want and e.request not in dead]
            all_wanting = [e for e in plan if e.want]
            if all_wanting:
                pending = self.sampler.sample_async(logits, [temps[index[e.request]] for e in all_wanting],
                                                    [seeds[index[e.request]] for e in all_wanting],
                                                    [gen[e.request] for e in all_wanting])
                for e in wanting:
                    gen[e.request] += 1
                    sched.on_token(e.request, False)          # optimistic: a stop token is booked when it is read
                carry = (all_wanting, pending)
            self._stats["steps"] += 1
            n_prompt = sum(e.count for e in plan if e.count > 1 or e.start == 0)
            self._stats["prompt_tokens"] += n_prompt
            self._stats["decode_tokens"] += len(wanting)
            if log:
                # one line per step, as the reference's IMPARO_LOG does for its forward calls
                # (imparo-model/src/lib.rs:938-946); host time since the previous step was issued,
                # not GPU time: steps are issued ahead of the device
                now = time.perf_counter()
                print(f"imparo step {self._stats['steps']} rows={len(plan)} prompt_tokens={n_prompt} "
                      f"decode_tokens={len(wanting)} free_pages={[self.cache.free_pages(g) for g in range(self.cache.n_groups)]} "
                      f"free_slots={self.cache.free_slots()} host_ms={1e3 * (now - t_log):.3f}", file=sys.stderr, flush=True)
                t_log = now
            if on_step is not None:
                on_step(plan)
        ops.read_status(self.status)
        if log:
            dt = time.perf_counter() - t0
            n_new = sum(gen.values())
            print(f"imparo generate: {len(prompts)} requests, {n_new} new tokens in {dt:.3f} s ({n_new / max(dt, 1e-9):.1f} tok/s), "
                  f"{self._stats['preemptions'] + sched.n_preemptions} preemptions so far", file=sys.stderr, flush=True)
        self._stats["seconds"] += time.perf_counter() - t0
        self._stats["preemptions"] += sched.n_preemptions
        self._stats["failed"] = failed
        return out

    def stats(self) -> dict:
        s = dict(self._stats)
        s.update(weight_bytes=self.weight_bytes, cache_bytes=self.cache.bytes(), workspace_bytes=self.rt.workspace.bytes(),
                 free_pages=[self.cache.free_pages(g) for g in range(self.cache.n_groups)],
                 free_slots=self.cache.free_slots(), precision=self.precision)
        return s
