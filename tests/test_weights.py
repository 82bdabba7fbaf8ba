import json
import os

import pytest
import torch

from imparo_b200.weights import SafetensorsFile, WeightError, load_weights, write_random_model, write_safetensors
from imparo_b200.weights.random_init import model_on_cpu
from tests.tiny_configs import TINY_A, TINY_B


def _folder(tmp_path, cfg, **kw):
    d = str(tmp_path / "m")
    write_random_model(d, cfg, seed=3, **kw)
    return d


def test_random_model_folder(tmp_path):
    d = _folder(tmp_path, TINY_B)
    assert sorted(os.listdir(d)) == ["config.json", "model.safetensors"]
    with open(os.path.join(d, "config.json")) as f:
        assert json.load(f)["hidden_size"] == 192
    with SafetensorsFile(os.path.join(d, "model.safetensors")) as f:
        names = set(f.names())
        assert "lm_head.weight" in names and "model.layers.1.conv.conv.bias" in names
        assert f.info("model.layers.1.conv.conv.weight") == ("F32", (192, 1, 4))
        assert f.info("model.layers.0.self_attn.q_proj.weight") == ("BF16", (192, 192))
        assert f.info("model.layers.0.self_attn.k_proj.weight") == ("BF16", (64, 192))
        assert f.info("model.layers.0.feed_forward.w1.weight") == ("BF16", (512, 192))
        assert f.info("model.embedding_norm.weight")[0] == "F32"
        n = f.tensor("model.layers.0.operator_norm.weight")
        assert (n - 1).abs().max() <= 0.1 + 1e-6 and (n - 1).abs().max() > 0


def test_same_seed_same_bytes(tmp_path):
    a = write_random_model(str(tmp_path / "a"), TINY_A, seed=5)
    b = write_random_model(str(tmp_path / "b"), TINY_A, seed=5)
    c = write_random_model(str(tmp_path / "c"), TINY_A, seed=6)
    read = lambda d: open(os.path.join(d, "model.safetensors"), "rb").read()
    assert read(a) == read(b) and read(a) != read(c)


def test_load_dtypes(tmp_path):
    d = _folder(tmp_path, TINY_A)
    _, _, model = model_on_cpu(TINY_A)
    bf = load_weights(d, model.weight_specs(), "bfloat16", "cpu")
    fp = load_weights(d, model.weight_specs(), "float32", "cpu")
    assert bf["model.embed_tokens.weight"].dtype == torch.bfloat16
    assert fp["model.embed_tokens.weight"].dtype == torch.float32
    assert bf["model.layers.0.operator_norm.weight"].dtype == torch.float32
    assert bf["model.layers.0.conv.conv.weight"].dtype == torch.float32
    assert torch.equal(bf["model.embed_tokens.weight"].float(), fp["model.embed_tokens.weight"])


def test_one_error_lists_everything(tmp_path):
    d = _folder(tmp_path, TINY_A)
    path = os.path.join(d, "model.safetensors")
    with SafetensorsFile(path) as f:
        tensors = {n: f.tensor(n) for n in f.names()}
    del tensors["model.layers.2.self_attn.k_proj.weight"]
    del tensors["model.embedding_norm.weight"]
    tensors["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(4, 4)
    tensors["model.layers.1.feed_forward.w2.weight"] = torch.zeros(64, 100)
    tensors["model.layers.3.ffn_norm.weight"] = torch.zeros(64, dtype=torch.int32)
    write_safetensors(path, tensors)
    _, _, model = model_on_cpu(TINY_A)
    with pytest.raises(WeightError) as e:
        load_weights(d, model.weight_specs(), "bfloat16", "cpu")
    err = e.value
    assert sorted(err.missing) == ["model.embedding_norm.weight", "model.layers.2.self_attn.k_proj.weight"]
    assert err.unexpected == ["model.layers.0.self_attn.q_proj.weight"]
    assert [w[0] for w in err.wrong_shape] == ["model.layers.1.feed_forward.w2.weight"]
    assert [w[0] for w in err.bad_dtype] == ["model.layers.3.ffn_norm.weight"]
    text = str(err)
    for needle in ("missing (2)", "unexpected (1)", "wrong shape", "[64, 100]", "[64, 192]", "unreadable dtype"):
        assert needle in text


def test_names_without_model_prefix_and_flat_conv_kernel(tmp_path):
    d = _folder(tmp_path, TINY_A)
    path = os.path.join(d, "model.safetensors")
    with SafetensorsFile(path) as f:
        tensors = {}
        for n in f.names():
            t = f.tensor(n)
            if n.endswith("conv.conv.weight"):
                t = t.reshape(t.shape[0], t.shape[2])
            tensors[n[len("model."):] if n.startswith("model.") else n] = t
    write_safetensors(path, tensors)
    _, _, model = model_on_cpu(TINY_A)
    out = load_weights(d, model.weight_specs(), "float32", "cpu")
    assert out["model.layers.0.conv.conv.weight"].shape == (64, 3)


def test_safetensors_round_trip(tmp_path):
    p = str(tmp_path / "x.safetensors")
    t = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16), "c": torch.arange(6, dtype=torch.int32).reshape(2, 3)}
    write_safetensors(p, t)
    with SafetensorsFile(p) as f:
        for k, v in t.items():
            assert torch.equal(f.tensor(k), v)


def test_a_tied_head_stored_beside_the_embedding_is_accepted_when_equal(tmp_path):
    """TINY_A ties its head to the embedding table.  A file that also carries lm_head.weight loads when the
    copy equals the table; when it differs the model would ignore it silently, so the load fails and says so."""
    d = _folder(tmp_path, TINY_A)
    path = os.path.join(d, "model.safetensors")
    with SafetensorsFile(path) as f:
        tensors = {n: f.tensor(n) for n in f.names()}
    _, _, model = model_on_cpu(TINY_A)
    dup = dict(model.spec.duplicate_tensors)
    assert dup == {"lm_head.weight": "model.embed_tokens.weight"}
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()
    write_safetensors(path, tensors)
    out = load_weights(d, model.weight_specs(), "float32", "cpu", duplicates=dup)
    assert "lm_head.weight" not in out
    with pytest.raises(WeightError) as e:                       # without the declaration it stays unexpected
        load_weights(d, model.weight_specs(), "float32", "cpu")
    assert e.value.unexpected == ["lm_head.weight"]
    tensors["lm_head.weight"] = tensors["lm_head.weight"] + 1
    write_safetensors(path, tensors)
    with pytest.raises(WeightError, match="the two differ"):
        load_weights(d, model.weight_specs(), "float32", "cpu", duplicates=dup)


def test_a_sharded_checkpoint_is_refused_by_name(tmp_path):
    d = _folder(tmp_path, TINY_A)
    os.remove(os.path.join(d, "model.safetensors"))
    with open(os.path.join(d, "model.safetensors.index.json"), "w") as f:
        f.write("{}")
    _, _, model = model_on_cpu(TINY_A)
    with pytest.raises(FileNotFoundError, match="sharded"):
        load_weights(d, model.weight_specs(), "float32", "cpu")
