"""Device timeline of a step: when each kernel's first block started, when its wait on the
previous kernel returned, and up to two marks of its own, in nanoseconds of the GPU's global timer.

It needs the kernels' timeline build (IMPARO_TIMELINE=1 in the environment before the library is
first used; a library of its own beside the normal one).  The stamps cost an atomic and a few
stores per launch, so the numbers are for finding where a step's time goes, never a benchmark.
The reference has per-category GPU times behind IMPARO_PROF (imparo-model/src/host.rs:9-95); a
chain of kernels that overlap through programmatic dependent launch needs stamps taken on the
device instead of events around launches.

    IMPARO_TIMELINE=1 python -m imparo_b200.kernels.timeline --config lfm2_1.2b --batch 8 --prompt-len 2048

prints, for the last decode step, one line per kernel: name, how long its first block was resident
before its wait returned, and its share of the chain (from its wait's return to the next
kernel's), which is what the kernel costs the step.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import re
from typing import List, Optional

import torch

from . import build, lib as _lib


PRESETS = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "config", "presets")


class Timeline:
    def __init__(self, capacity: int = 1 << 16, device="cuda:0"):
        if not build.timeline_build():
            raise RuntimeError("the device timeline needs IMPARO_TIMELINE=1 in the environment before the kernels are loaded")
        self.capacity = int(capacity)
        self.buffer = torch.zeros(2 + 4 * self.capacity, dtype=torch.int64, device=device)
        torch.cuda.synchronize()
        rc = _lib.kernels().imparo_timeline_start(self.buffer.data_ptr(), self.capacity)
        if rc != 0:
            raise RuntimeError(f"imparo_timeline_start returned {rc} (was the library built with IMPARO_TIMELINE?)")

    def host_launches(self) -> int:
        """Launches the host has issued (or captured) since the start."""
        return int(_lib.kernels().imparo_timeline_launches())

    def names(self, first: int, last: int) -> List[str]:
        out = []
        buf = ctypes.create_string_buffer(512)
        for i in range(first, last):
            rc = _lib.kernels().imparo_timeline_name(i, buf, 512)
            out.append(_short(buf.value.decode()) if rc == 0 else "?")
        return out

    def records(self):
        """-> int64 tensor [n, 4] on the host: start, wait returned, mark 0, mark 1 (0 = not stamped)."""
        torch.cuda.synchronize()
        h = self.buffer.cpu()
        n = min(int(h[0]), self.capacity)
        return h[2:2 + 4 * n].view(n, 4)

    def stop(self) -> None:
        torch.cuda.synchronize()
        _lib.kernels().imparo_timeline_start(None, 0)


def _short(mangled: str) -> str:
    """A readable name out of a mangled one without a demangler: the last length-prefixed
    identifier of the nested name, and the template arguments that are integers or types."""
    m = re.match(r"_ZN?", mangled)
    if not m:
        return mangled[:48]
    i, name = m.end(), None
    while i < len(mangled) and mangled[i].isdigit():
        j = i
        while mangled[j].isdigit():
            j += 1
        n = int(mangled[i:j])
        name, i = mangled[j:j + n], j + n
    if name is None:
        return mangled[:48]
    args = ""
    if i < len(mangled) and mangled[i] == "I":
        k = mangled.find("EEv", i)
        args = mangled[i + 1:k if k > 0 else i + 1]
        args = args.replace("13__nv_bfloat16", "bf16,").replace("Lb0E", "0,").replace("Lb1E", "1,")
        args = re.sub(r"Li(\d+)E", lambda g: g.group(1) + ",", args)
        args = "f32" if args == "f" else args.rstrip(",")
    return name + (f"<{args}>" if args else "")


def step_table(names: List[str], rec: torch.Tensor) -> List[dict]:
    """rec: the step's records in launch order [n, 4].  Chain share of kernel k = wait[k+1] - wait[k]."""
    rows = []
    n = rec.shape[0]
    t0 = int(rec[0, 1])
    for k in range(n):
        start, wait, m0, m1 = (int(v) for v in rec[k])
        nxt = int(rec[k + 1, 1]) if k + 1 < n else None
        rows.append({"kernel": names[k], "at_us": (wait - t0) / 1e3, "resident_before_us": (wait - start) / 1e3,
                     "chain_us": None if nxt is None else (nxt - wait) / 1e3,
                     "mark0_us": None if m0 == 0 else (m0 - wait) / 1e3, "mark1_us": None if m1 == 0 else (m1 - wait) / 1e3})
    return rows


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("-m", "--model", help="model folder (config.json, model.safetensors)")
    ap.add_argument("--config", help="a config.json, or the name of one under config/presets: random weights of that shape")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--prompt-len", type=int, default=2048)
    ap.add_argument("--steps", type=int, default=12, help="decode steps to run (the last one is printed)")
    ap.add_argument("--layers", type=int, default=None)
    ap.add_argument("--prefill", action="store_true", help="print the step of a whole prompt instead of a decode step "
                    "(library products are not stamped: their time shows in the share of the kernel before them)")
    ap.add_argument("--mixed", type=int, default=0, help="print a step of one prompt portion of --prompt-len tokens beside "
                    "this many decode rows, each with --context positions in the cache")
    ap.add_argument("--context", type=int, default=2048)
    ap.add_argument("--json", action="store_true")
    args = ap.parse_args(argv)
    import numpy as np
    from ..engine import Engine, StepItem
    from . import ops
    if args.model:
        engine = Engine(model=args.model, dtype="bfloat16", capture_first=False, ctx=max(args.prompt_len, args.context if args.mixed else 0) + 64,
                        parallel=max(args.batch, args.mixed + 1), max_step_tokens=max(args.prompt_len, args.context) + args.mixed)
    else:
        if not args.config:
            ap.error("give a model folder (-m) or a configuration (--config)")
        path = args.config if os.path.isfile(args.config) else os.path.join(PRESETS, args.config + ".json")
        with open(path) as f:
            cfg = json.load(f)
        if args.layers:
            cfg["layer_types"] = cfg["layer_types"][:args.layers]
            cfg["num_hidden_layers"] = args.layers
        engine = Engine(config=cfg, seed=0, dtype="bfloat16", capture_first=False, ctx=max(args.prompt_len, args.context if args.mixed else 0) + 64,
                        parallel=max(args.batch, args.mixed + 1), max_step_tokens=max(args.prompt_len, args.context) + args.mixed,
                        random_init={"norm_jitter": 0.0})
    tl = Timeline()
    rng = np.random.default_rng(0)
    V = engine.vocab_size
    if args.mixed:
        ids = list(range(args.mixed))
        for r in ids:
            engine.add_request(r)
            engine.step([StepItem(r, rng.integers(0, V, args.context).tolist(), [])])
        rows = None
        for rep in range(3):                     # the third time the step's shape is replayed from its graph
            engine.add_request(900 + rep)
            before, n_before = tl.host_launches(), tl.records().shape[0]
            engine.step([StepItem(r, [int(t)], [0]) for r, t in zip(ids, rng.integers(0, V, args.mixed))]
                        + [StepItem(900 + rep, rng.integers(0, V, args.prompt_len).tolist(), [args.prompt_len - 1])])
            rec = tl.records()[n_before:]
            if tl.host_launches() > before:
                names = tl.names(before, tl.host_launches())
            engine.end_request(900 + rep)
            rows = step_table(names[-rec.shape[0]:], rec)
        tl.stop()
        _print_table(rows, f"portion of {args.prompt_len} tokens beside {args.mixed} decode rows at {args.context} positions", args.json)
        return 0
    if args.prefill:
        rows = None
        for rep in range(3):
            engine.add_request(900 + rep)
            before = tl.host_launches()
            n_before = tl.records().shape[0]
            engine.step([StepItem(900 + rep, rng.integers(0, V, args.prompt_len).tolist(), [args.prompt_len - 1])])
            rec = tl.records()[n_before:]
            if tl.host_launches() > before:      # a replayed graph launches nothing from the host: the names are the last ones
                names = tl.names(before, tl.host_launches())
            engine.end_request(900 + rep)
            rows = step_table(names[-rec.shape[0]:], rec)
        tl.stop()
        _print_table(rows, f"prompt of {args.prompt_len} tokens", args.json)
        return 0
    ids = list(range(args.batch))
    for r in ids:
        engine.add_request(r)
        engine.step([StepItem(r, rng.integers(0, V, args.prompt_len).tolist(), [args.prompt_len - 1])])
    out_ids = torch.empty(args.batch, dtype=torch.int32, device=engine.device)
    marks = []
    for _ in range(max(args.steps, 4)):
        before = tl.host_launches()
        logits = engine.step_fn([StepItem(r, [int(t)], [0]) for r, t in zip(ids, rng.integers(0, V, args.batch))])
        ops.sample_rows(logits, None, None, out_ids)
        marks.append((before, tl.host_launches()))
    rec = tl.records()
    tl.stop()
    # replayed steps launch nothing on the host: the last step that was issued (or captured) whole
    # names the kernels of every later step
    most = max(b - a for a, b in marks)
    first, last = [m for m in marks if m[1] - m[0] == most][-1]
    names = tl.names(first, last)
    n = len(names)
    rows = step_table(names, rec[-n:])
    _print_table(rows, "last decode step", args.json)
    return 0


def _print_table(rows, what: str, as_json: bool) -> None:
    if as_json:
        print(json.dumps(rows))
        return
    n = len(rows)
    total = rows[-1]["at_us"] - rows[0]["at_us"]
    print(f"{what}: {n} kernels, {total:.1f} us from the first wait to the last")
    print(f"{'at us':>9} {'resident':>9} {'chain us':>9} {'mark0':>7} {'mark1':>7}  kernel")
    for r in rows:
        f = lambda v: "      -" if v is None else f"{v:7.2f}"
        print(f"{r['at_us']:9.2f} {r['resident_before_us']:9.2f} {f(r['chain_us']):>9} {f(r['mark0_us'])} {f(r['mark1_us'])}  {r['kernel']}")
    agg = {}
    for r in rows:
        if r["chain_us"] is not None:
            a = agg.setdefault(r["kernel"], [0, 0.0])
            a[0] += 1
            a[1] += r["chain_us"]
    print("\nchain time by kernel:")
    for k, (c, us) in sorted(agg.items(), key=lambda kv: -kv[1][1]):
        print(f"{us:9.1f} us {100 * us / total:5.1f}%  x{c:<3d} {us / c:6.2f} each  {k}")


if __name__ == "__main__":
    raise SystemExit(main())
