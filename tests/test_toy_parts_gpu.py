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

    def parse(values):
        r = KeyReader(values)
        return {"vocab": r.integer("vocab_size"), "hidden": r.integer("hidden_size"), "layers": r.strings("layer_types"),
                "heads": r.integer("num_attention_heads"), "ff": r.integer("ff"), "eps": r.number("norm_eps"),
                "schedule": values.get("layer_schedule")}

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
                         embedding=PartSpec("token_table", {"vocab": c["vocab"], "width": H, "name": "toy.embed.weight"}),
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
