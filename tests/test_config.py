import copy

import pytest

from imparo_b200.config import ConfigError, known_architectures, load_config, register_architecture, Architecture
from imparo_b200.config.lfm2 import parse_lfm2_config
from tests.tiny_configs import ALL, TINY_A, TINY_B, TINY_C


def test_registry_resolves_by_architecture_and_model_type():
    arch, cfg = load_config(TINY_A)
    assert arch.name == "Lfm2ForCausalLM"
    d = dict(TINY_A)
    d.pop("architectures")
    assert load_config(d)[0].name == "Lfm2ForCausalLM"
    assert "Lfm2ForCausalLM" in known_architectures()


def test_unknown_architecture_lists_known():
    d = dict(TINY_A, architectures=["NopeForCausalLM"], model_type="nope")
    with pytest.raises(ConfigError) as e:
        load_config(d)
    assert "NopeForCausalLM" in str(e.value) and "Lfm2ForCausalLM" in str(e.value)


def test_sizes_come_from_the_keys():
    a, b, c = (parse_lfm2_config(x) for x in (TINY_A, TINY_B, TINY_C))
    assert (a.head_dim, a.ff_dim, a.conv_L_cache, a.tie_embedding) == (16, 192, 3, True)
    # 768 -> int(2*768/3) = 512 -> *1.0 -> multiple of 64 -> 512
    assert (b.head_dim, b.ff_dim, b.conv_L_cache, b.tie_embedding, b.conv_bias) == (32, 512, 4, False, True)
    assert (c.head_dim, c.ff_dim, c.sliding_window) == (48, 200, 24)
    assert a.norm_eps == 1e-5 and b.norm_eps == 1e-6 and b.rope_theta == 1e6


@pytest.mark.parametrize("ff,mult,mo,want", [(12288, None, 256, 8192), (10240, None, 256, 6912), (6656, None, 256, 4608),
                                             (768, 1.0, 64, 512), (1000, 1.5, 32, 1024)])
def test_ff_auto_adjust(ff, mult, mo, want):
    d = dict(TINY_A, block_ff_dim=ff, block_auto_adjust_ff_dim=True, block_multiple_of=mo)
    if mult is not None:
        d["block_ffn_dim_multiplier"] = mult
    assert parse_lfm2_config(d).ff_dim == want


def test_full_attn_idxs_alias_and_intermediate_size():
    d = dict(TINY_A)
    d.pop("layer_types")
    d["full_attn_idxs"] = [2]
    d["intermediate_size"] = d.pop("block_ff_dim")
    cfg = parse_lfm2_config(d)
    assert cfg.layer_types == ("conv", "conv", "full_attention", "conv") and cfg.ff_dim == 192


@pytest.mark.parametrize("change,needle", [
    ({"hidden_size": None}, "hidden_size"),
    ({"vocab_size": "many"}, "vocab_size"),
    ({"conv_L_cache": 1}, "conv_L_cache"),
    ({"layer_types": ["conv"]}, "layer_types"),
    ({"layer_types": ["conv", "conv", "banana", "conv"]}, "banana"),
    ({"num_key_value_heads": 3}, "num_key_value_heads"),
    ({"hidden_size": 66}, "multiple"),
    ({"layer_types": ["conv", "conv", "sliding_attention", "conv"]}, "sliding_window"),
    ({"conv_bias": "yes"}, "conv_bias"),
    ({"block_auto_adjust_ff_dim": None}, "block_auto_adjust_ff_dim"),      # no default: the width follows from it
])
def test_bad_config_names_the_key(change, needle):
    d = copy.deepcopy(TINY_A)
    for k, v in change.items():
        if v is None:
            d.pop(k)
        else:
            d[k] = v
    with pytest.raises(ConfigError) as e:
        parse_lfm2_config(d)
    assert needle in str(e.value)


def test_model_spec_layers_and_schedule():
    arch, cfg = load_config(TINY_B)
    spec = arch.model_spec(cfg)
    kinds = [l.mixer.kind for l in spec.layers]
    assert kinds == ["attention", "short_conv", "short_conv", "attention", "short_conv", "attention"]
    assert [e.layer for e in spec.schedule] == list(range(6))
    assert spec.head.params["name"] == "lm_head.weight"
    arch, cfg = load_config(TINY_A)
    assert arch.model_spec(cfg).head.params["name"] == "model.embed_tokens.weight"
    assert spec.layers[0].mixer.params["window"] is None
    arch, cfg = load_config(TINY_C)
    assert arch.model_spec(cfg).layers[0].mixer.params["window"] == 24


def test_schedule_is_data():
    d = dict(TINY_A, layer_schedule=[0, 1, 2, [2, 2], 3, 0])
    arch, cfg = load_config(d)
    spec = arch.model_spec(cfg)
    assert [(e.layer, e.cache_from) for e in spec.schedule] == [(0, None), (1, None), (2, None), (2, 2), (3, None), (0, None)]
    with pytest.raises(ValueError):
        arch.model_spec(load_config(dict(TINY_A, layer_schedule=[0, [2, 3]]))[1])   # cache_from must be earlier


def test_config_round_trip():
    for cfg in ALL.values():
        typed = parse_lfm2_config(cfg)
        assert parse_lfm2_config(typed.to_json_dict()) == typed
