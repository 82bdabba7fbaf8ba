"""A toy mixer with state of its own, defined here, is registered, built and stepped
without a change to the framework's files; and the layer schedule is data (a layer run
twice, a layer reading another entry's cache).  The toys are test fixtures, not models."""
import numpy as np
import pytest
import torch

from tests.gpu_helpers import run_trace
from tests import traces

pytestmark = pytest.mark.gpu


def register_toy():
    from imparo_b200.config.base import KeyReader
    from imparo_b200.config.registry import Architecture, register_architecture
    from imparo_b200.parts.base import Part, register_part
    from imparo_b200.parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, SlotState, WeightSpec

    class RunningMeanMixer(Part):
        """out[t] = W * mean(x[0..t]) per request.  Its state: the running sum [H] and the
        count [1], one slot per request."""
        graph_safe = False      # forward() reads batch.host: not for capture and replay

        def __init__(self, params, prefix, rt):
            super().__init__(params, prefix, rt)
            self.H = int(params["hidden"])
            self.name = prefix + "toy.proj.weight"
            self.w = None

        def weight_specs(self):
            return [WeightSpec(self.name, ((self.H, self.H),))]

        def bind(self, tensors):
            self.w = tensors[self.name]

        def cache_specs(self):
            return (SlotState((self.H,)), SlotState((1,)))

        def forward(self, x, batch, caches, residual):
            total, count = caches[0].state, caches[1].state
            rows, slots = batch.host["row_start"], batch.host["slots"]
            for i, slot in enumerate(slots):
                a, b = int(rows[i]), int(rows[i + 1])
                xs = x[a:b].float()
                run = torch.cumsum(xs, 0) + total[slot]
                n = torch.arange(1, b - a + 1, device=x.device, dtype=torch.float32)[:, None] + count[slot]
                mean = (run / n).to(x.dtype)
                residual[a:b] += (mean.float() @ self.w.float().T)
                total[slot] = run[-1]
                count[slot] += b - a

    register_part("mixer", "toy_running_mean", RunningMeanMixer, replace=True)

    class PositionalTable(Part):
        """An embedding that reads more of the batch than the token ids: row of the token table plus a learned
        row per absolute position (out = E[token] + P[position])."""
        graph_safe = False      # it indexes with torch, which allocates: not for capture and replay

        def __init__(self, params, prefix, rt):
            super().__init__(params, prefix, rt)
            self.vocab, self.width, self.n_pos = int(params["vocab"]), int(params["width"]), int(params["positions"])
            self.names = (prefix + params["name"], prefix + "toy.positions.weight")
            self.table = self.pos = None

        def weight_specs(self):
            return [WeightSpec(self.names[0], ((self.vocab, self.width),)), WeightSpec(self.names[1], ((self.n_pos, self.width),))]

        def bind(self, tensors):
            self.table, self.pos = tensors[self.names[0]], tensors[self.names[1]]

        def forward(self, batch):
            out = self.rt.workspace.get("residual", (batch.n_tokens, self.width), torch.float32)
            out.copy_(self.table[batch.token_ids.long()].float() + self.pos[batch.positions.long()].float())
            return out

    register_part("embedding", "toy_positional_table", PositionalTable, replace=True)

    def parse(values):
        r = KeyReader(values)
        return {"vocab": r.integer("vocab_size"), "hidden": r.integer("hidden_size"), "layers": r.strings("layer_types"),
                "heads": r.integer("num_attention_heads"), "ff": r.integer("ff"), "eps": r.number("norm_eps"),
                "schedule": values.get("layer_schedule"), "embedding": values.get("embedding", "token_table")}

    def spec(c):
        H = c["hidden"]
        layers = []
        for i, kind in enumerate(c["layers"]):
            mixer = (PartSpec("toy_running_mean", {"hidden": H}) if kind == "toy" else
                     PartSpec("attention", {"hidden": H, "n_heads": c["heads"], "n_kv_heads": 1, "head_dim": H // c["heads"],
                                            "eps": c["eps"], "window": None,
                                            "position": PartSpec("rope_neox", {"head_dim": H // c["heads"], "theta": 100.0})}))
            layers.append(LayerSpec(prefix=f"toy.layers.{i}.", mixer=mixer,
                                    feed_forward=PartSpec("swiglu", {"hidden": H, "ff": c["ff"]}),
                                    mixer_norm=PartSpec("rmsnorm", {"width": H, "eps": c["eps"], "name": "n1.weight"}),
                                    feed_forward_norm=PartSpec("rmsnorm", {"width": H, "eps": c["eps"], "name": "n2.weight"})))
        sched = c["schedule"] or list(range(len(layers)))
        sched = tuple(ScheduleEntry(*e) if isinstance(e, (list, tuple)) else ScheduleEntry(e) for e in sched)
        return ModelSpec(architecture="ToyForCausalLM", vocab_size=c["vocab"], hidden_size=H,
                         embedding=PartSpec(c["embedding"], {"vocab": c["vocab"], "width": H, "name": "toy.embed.weight",
                                                              "positions": 128}),
                         layers=tuple(layers), schedule=sched,
                         final_norm=PartSpec("rmsnorm", {"width": H, "eps": c["eps"], "name": "toy.norm.weight"}),
                         head=PartSpec("linear", {"vocab": c["vocab"], "width": H, "name": "toy.embed.weight"}),
                         max_positions=4096)

    register_architecture(Architecture("ToyForCausalLM", ("toy",), parse, spec), replace=True)


TOY = {"architectures": ["ToyForCausalLM"], "vocab_size": 97, "hidden_size": 64, "layer_types": ["toy", "attn", "toy"],
       "num_attention_heads": 2, "ff": 80, "norm_eps": 1e-5}


def logits_by_position(steps, got):
    out, at = {}, {}
    for s in steps:
        r = 0
        for e in s["entries"]:
            start = at.get(e["id"], 0)
            for w in e["want"]:
                out[(e["id"], start + w)] = got[s["step"]][r]
                r += 1
            at[e["id"]] = start + len(e["tokens"])
    return out


@pytest.mark.parametrize("schedule", [None, [0, 1, 2, 0, [1, 1]]])
def test_toy_mixer_is_registered_built_and_stepped(schedule):
    from imparo_b200.engine import Engine
    register_toy()
    cfg = dict(TOY, layer_schedule=schedule) if schedule else dict(TOY)
    rng = np.random.default_rng(0)
    reqs = {f"r{i}": rng.integers(0, 97, n).tolist() for i, n in enumerate([40, 23, 31])}
    results = []
    for build in (traces.whole, traces.portions, lambda r: traces.mixed(r, seed=2, tail=5, max_portion=9)):
        steps = build(reqs)
        eng = Engine(config=cfg, seed=5, dtype="float32", ctx=64, parallel=3, page_size=4, num_pages=40,
                     random_init={"matrix_std": 0.1})
        if schedule:
            # entry 3 runs layer 0 a second time with a state slot of its own; entry 4 runs layer 1
            # again and reads the keys and values entry 1 wrote
            assert len(eng.cache.state) == 2 * 3 and eng.cache.group_entries == [[1]]
        results.append(logits_by_position(steps, run_trace(eng, steps)))
    keys = set(results[0])
    assert len(keys) == 94
    for other in results[1:]:
        for k in keys:
            assert np.abs(other[k] - results[0][k]).max() <= 1e-5, k
    # and the state matters: the same token at another position gives other logits
    assert np.abs(results[0][("r0", 5)] - results[0][("r0", 6)]).max() > 1e-3


def test_toy_embedding_that_reads_positions():
    """An embedding part gets the step's batch, so one that adds learned absolute positions is a new part and
    nothing else: registered here, built by the engine, stepped whole, in portions and mixed."""
    from imparo_b200.engine import Engine, StepItem
    register_toy()
    cfg = dict(TOY, embedding="toy_positional_table", layer_types=["toy", "toy"])       # no mixer knows positions
    rng = np.random.default_rng(3)
    reqs = {f"r{i}": rng.integers(0, 97, n).tolist() for i, n in enumerate([30, 17])}
    results = []
    for build in (traces.whole, traces.portions, lambda r: traces.mixed(r, seed=4, tail=4, max_portion=7)):
        steps = build(reqs)
        eng = Engine(config=cfg, seed=9, dtype="float32", ctx=64, parallel=2, page_size=4, num_pages=8,
                     random_init={"matrix_std": 0.1})
        results.append(logits_by_position(steps, run_trace(eng, steps)))
    for other in results[1:]:
        for k in results[0]:
            assert np.abs(other[k] - results[0][k]).max() <= 1e-5, k
    # the part alone: rows of the two tables, added
    emb = eng.model.embedding
    eng.add_request(7)
    eng.cache.reserve(7, 3)
    batch = eng.step_fn.build_batch([StepItem(7, [5, 5, 9])])
    x = emb.forward(batch).cpu()
    eng.cache.rollback(7)
    eng.end_request(7)
    want = emb.table[[5, 5, 9]].float().cpu() + emb.pos[[0, 1, 2]].float().cpu()
    assert torch.allclose(x, want, atol=1e-6) and not torch.allclose(x[0], x[1])


# ---------------------------------------------------------------------------------------------
# A feed-forward with routing and another position encoding, as toy parts
# ---------------------------------------------------------------------------------------------

def register_routed_toy():
    from imparo_b200.config.base import KeyReader
    from imparo_b200.config.registry import Architecture, register_architecture
    from imparo_b200.kernels import ops
    from imparo_b200.parts.base import Part, register_part
    from imparo_b200.parts.position import PositionEncoding
    from imparo_b200.parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, WeightSpec

    class RoutedFeedForward(Part):
        """Top-1 of E small SwiGLU experts per token; router logits and the choice in 32-bit."""
        graph_safe = False       # the shapes it launches depend on the routing: not for capture and replay

        def __init__(self, params, prefix, rt):
            super().__init__(params, prefix, rt)
            self.H, self.F, self.E = int(params["hidden"]), int(params["ff"]), int(params["experts"])
            self.names = {"router": prefix + "moe.router.weight",
                          **{f"w{k}_{e}": prefix + f"moe.experts.{e}.w{k}.weight" for e in range(self.E) for k in (1, 2, 3)}}

        def weight_specs(self):
            specs = [WeightSpec(self.names["router"], ((self.E, self.H),), role="vector", init=("bias",))]
            for e in range(self.E):
                specs += [WeightSpec(self.names[f"w1_{e}"], ((self.F, self.H),)), WeightSpec(self.names[f"w3_{e}"], ((self.F, self.H),)),
                          WeightSpec(self.names[f"w2_{e}"], ((self.H, self.F),))]
            return specs

        def bind(self, tensors):
            self.router = tensors[self.names["router"]]
            self.w13 = [torch.cat([tensors[self.names[f"w1_{e}"]], tensors[self.names[f"w3_{e}"]]]).contiguous() for e in range(self.E)]
            self.w2 = [tensors[self.names[f"w2_{e}"]] for e in range(self.E)]

        def forward(self, x, batch, residual):
            choice = (x.float() @ self.router.T).argmax(-1)              # router in 32-bit
            for e in range(self.E):
                idx = (choice == e).nonzero().flatten()
                if idx.numel() == 0:
                    continue
                xe = x[idx].contiguous()
                gu = torch.empty(idx.numel(), 2 * self.F, dtype=x.dtype, device=x.device)
                ops.linear(xe, self.w13[e], gu)                          # the framework's own product and activation kernels
                h = torch.empty(idx.numel(), self.F, dtype=x.dtype, device=x.device)
                ops.swiglu_act(gu, h)
                out = torch.zeros(idx.numel(), self.H, device=x.device)
                ops.linear(h, self.w2[e], out, accumulate=True)
                residual.index_add_(0, idx, out)

    class ScaledRotary(PositionEncoding):
        """Half-split rotation of the first n_rot dimensions with frequencies divided by a factor
        that grows with the pair index (another table, same kernel)."""

        def __init__(self, params, prefix, rt):
            super().__init__(params, prefix, rt)
            n_rot, theta, factor = int(params["n_rot"]), float(params["theta"]), float(params["factor"])
            i = torch.arange(n_rot // 2, dtype=torch.float64)
            inv = theta ** (-2.0 * i / n_rot) / (1.0 + factor * i)
            self.inv, self.n_rot = inv.to(torch.float32).to(rt.device), n_rot

        def rotary(self):
            return self.inv, self.n_rot

    register_part("feed_forward", "toy_routed", RoutedFeedForward, replace=True)
    register_part("position", "toy_scaled_rotary", ScaledRotary, replace=True)

    def parse(values):
        r = KeyReader(values)
        return {k: values[k] for k in ("vocab_size", "hidden_size", "n_layers", "heads", "kv_heads", "ff", "experts", "n_rot", "theta", "factor", "eps")}

    def spec(c):
        H, hd = c["hidden_size"], c["hidden_size"] // c["heads"]
        pos = PartSpec("toy_scaled_rotary", {"n_rot": c["n_rot"], "theta": c["theta"], "factor": c["factor"]})
        layers = tuple(LayerSpec(
            prefix=f"m.layers.{i}.",
            mixer=PartSpec("attention", {"hidden": H, "n_heads": c["heads"], "n_kv_heads": c["kv_heads"], "head_dim": hd,
                                         "eps": c["eps"], "window": None, "position": pos}),
            feed_forward=PartSpec("toy_routed", {"hidden": H, "ff": c["ff"], "experts": c["experts"]}),
            mixer_norm=PartSpec("rmsnorm", {"width": H, "eps": c["eps"], "name": "n1.weight"}),
            feed_forward_norm=PartSpec("rmsnorm", {"width": H, "eps": c["eps"], "name": "n2.weight"})) for i in range(c["n_layers"]))
        return ModelSpec(architecture="RoutedToyForCausalLM", vocab_size=c["vocab_size"], hidden_size=H,
                         embedding=PartSpec("token_table", {"vocab": c["vocab_size"], "width": H, "name": "m.embed.weight"}),
                         layers=layers, schedule=tuple(ScheduleEntry(i) for i in range(c["n_layers"])),
                         final_norm=PartSpec("rmsnorm", {"width": H, "eps": c["eps"], "name": "m.norm.weight"}),
                         head=PartSpec("linear", {"vocab": c["vocab_size"], "width": H, "name": "m.embed.weight"}), max_positions=4096)

    register_architecture(Architecture("RoutedToyForCausalLM", ("routed_toy",), parse, spec), replace=True)


ROUTED = {"architectures": ["RoutedToyForCausalLM"], "vocab_size": 211, "hidden_size": 96, "n_layers": 3, "heads": 3, "kv_heads": 1,
          "ff": 72, "experts": 4, "n_rot": 16, "theta": 5000.0, "factor": 0.25, "eps": 1e-5}


def plain_routed_logits(folder, toks):
    """The routed toy in numpy float64, whole sequence, with the plain implementation's parts."""
    from tests.plain import lfm2_plain as P
    t = {k: v.astype(np.float64) for k, v in P.read_safetensors(folder + "/model.safetensors").items()}
    c = ROUTED
    H, nh, nkv = c["hidden_size"], c["heads"], c["kv_heads"]
    hd = H // nh
    T = len(toks)
    pos = np.arange(T)
    i = np.arange(c["n_rot"] // 2, dtype=np.float64)
    inv = (c["theta"] ** (-2.0 * i / c["n_rot"]) / (1.0 + c["factor"] * i)).astype(np.float32)
    ang = (pos[:, None].astype(np.float64) * inv[None, :].astype(np.float64)).astype(np.float32).astype(np.float64)

    def rope(x):                                    # x [T, heads, hd]; first n_rot dims, half-split
        half = c["n_rot"] // 2
        out = x.copy()
        x0, x1 = x[..., :half], x[..., half:c["n_rot"]]
        out[..., :half] = x0 * np.cos(ang)[:, None] - x1 * np.sin(ang)[:, None]
        out[..., half:c["n_rot"]] = x0 * np.sin(ang)[:, None] + x1 * np.cos(ang)[:, None]
        return out
    x = t["m.embed.weight"][np.asarray(toks)]
    for l in range(c["n_layers"]):
        p = f"m.layers.{l}."
        cur = P.rms_norm(x, t[p + "n1.weight"], c["eps"])
        q = P.rms_norm((cur @ t[p + "self_attn.q_proj.weight"].T).reshape(T, nh, hd), t[p + "self_attn.q_layernorm.weight"], c["eps"])
        k = P.rms_norm((cur @ t[p + "self_attn.k_proj.weight"].T).reshape(T, nkv, hd), t[p + "self_attn.k_layernorm.weight"], c["eps"])
        v = (cur @ t[p + "self_attn.v_proj.weight"].T).reshape(T, nkv, hd)
        o = P.attend(rope(q), rope(k), v, 1.0 / np.sqrt(hd))
        x = x + o.reshape(T, H) @ t[p + "self_attn.out_proj.weight"].T
        n = P.rms_norm(x, t[p + "n2.weight"], c["eps"])
        choice = (n @ t[p + "moe.router.weight"].T).argmax(-1)
        ff = np.zeros_like(x)
        for tok in range(T):
            e = choice[tok]
            ff[tok] = P.swiglu(n[tok:tok + 1], {"w1": t[p + f"moe.experts.{e}.w1.weight"], "w2": t[p + f"moe.experts.{e}.w2.weight"],
                                                "w3": t[p + f"moe.experts.{e}.w3.weight"]})[0]
        x = x + ff
    return P.rms_norm(x, t["m.norm.weight"], c["eps"]) @ t["m.embed.weight"].T


def test_routed_feed_forward_and_another_position_encoding(tmp_path):
    """A feed-forward that routes each token to one of four experts and a rotary table of its own,
    both defined in this test, in a registered toy architecture: written to a model folder by the
    random-weights mode, loaded, stepped whole / in portions / mixed, and compared with numpy."""
    from imparo_b200.engine import Engine
    from imparo_b200.weights import write_random_model
    register_routed_toy()
    folder = str(tmp_path / "routed")
    write_random_model(folder, ROUTED, seed=4, dtype="float32", matrix_std=0.15)
    rng = np.random.default_rng(1)
    reqs = {f"r{i}": rng.integers(0, ROUTED["vocab_size"], n).tolist() for i, n in enumerate([37, 20, 29])}
    ref = {k: plain_routed_logits(folder, v) for k, v in reqs.items()}
    scale = max(np.abs(v).max() for v in ref.values())
    for build in (traces.whole, traces.portions, lambda r: traces.mixed(r, seed=5, tail=6, max_portion=8)):
        steps = build(reqs)
        eng = Engine(folder, dtype="float32", ctx=64, parallel=3, page_size=8, num_pages=24)
        got = logits_by_position(steps, run_trace(eng, steps))
        for (rid, pos), row in got.items():
            assert np.abs(row - ref[rid][pos]).max() <= 5e-5 * scale, (rid, pos)
    # the routing is real: tokens go to different experts
    assert len({int(x) for x in np.argmax(np.random.default_rng(0).standard_normal((50, 4)), -1)}) > 1
