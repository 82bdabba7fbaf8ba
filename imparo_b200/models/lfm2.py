"""LFM2 (Lfm2ForCausalLM): which parts each layer has, from its typed config.

Per layer: an operator norm, a mixer — gated short convolution or grouped-query
attention with per-head q/k norms and NeoX rotation — then an ffn norm and a SwiGLU
feed-forward; embedding unscaled, final norm "embedding_norm", head tied to the embedding
unless tie_embedding is false (imparo-model/src/lfm2/plan.rs:86-170; tensor roles
lfm2/workflow_cpu.rs:84-122).  Tensor names are the HF names of this architecture.
"""
from __future__ import annotations

from ..config.lfm2 import Lfm2Config, parse_lfm2_config
from ..config.registry import Architecture, register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

MODEL_PREFIX = "model."


def lfm2_model_spec(cfg: Lfm2Config) -> ModelSpec:
    H = cfg.hidden_size
    position = PartSpec("rope_neox", {"head_dim": cfg.head_dim, "theta": cfg.rope_theta})
    layers = []
    for i, kind in enumerate(cfg.layer_types):
        prefix = f"{MODEL_PREFIX}layers.{i}."
        if kind == "conv":
            mixer = PartSpec("short_conv", {"hidden": H, "taps": cfg.conv_L_cache, "bias": cfg.conv_bias})
        else:
            mixer = PartSpec("attention", {
                "hidden": H, "n_heads": cfg.num_attention_heads, "n_kv_heads": cfg.num_key_value_heads,
                "head_dim": cfg.head_dim, "eps": cfg.norm_eps, "position": position,
                "window": cfg.sliding_window if kind == "sliding_attention" else None})
        layers.append(LayerSpec(
            prefix=prefix, mixer=mixer,
            feed_forward=PartSpec("swiglu", {"hidden": H, "ff": cfg.ff_dim}),
            mixer_norm=PartSpec("rmsnorm", {"width": H, "eps": cfg.norm_eps, "name": "operator_norm.weight"}),
            feed_forward_norm=PartSpec("rmsnorm", {"width": H, "eps": cfg.norm_eps, "name": "ffn_norm.weight"})))
    if cfg.layer_schedule is None:
        schedule = tuple(ScheduleEntry(i) for i in range(cfg.num_hidden_layers))
    else:
        schedule = tuple(ScheduleEntry(l, c) for l, c in cfg.layer_schedule)
    embed_name = MODEL_PREFIX + "embed_tokens.weight"
    return ModelSpec(
        architecture="Lfm2ForCausalLM", vocab_size=cfg.vocab_size, hidden_size=H,
        embedding=PartSpec("token_table", {"vocab": cfg.vocab_size, "width": H, "name": embed_name}),
        layers=tuple(layers), schedule=schedule,
        final_norm=PartSpec("rmsnorm", {"width": H, "eps": cfg.norm_eps, "name": MODEL_PREFIX + "embedding_norm.weight"}),
        head=PartSpec("linear", {"vocab": cfg.vocab_size, "width": H,
                                 "name": embed_name if cfg.tie_embedding else "lm_head.weight"}),
        max_positions=cfg.max_position_embeddings, eos_token_ids=cfg.eos_token_ids,
        duplicate_tensors=(("lm_head.weight", embed_name),) if cfg.tie_embedding else ())


register_architecture(Architecture(name="Lfm2ForCausalLM", model_types=("lfm2",),
                                   parse_config=parse_lfm2_config, model_spec=lfm2_model_spec), replace=True)
