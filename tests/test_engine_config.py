"""The engine's typed configuration: every field resolved once, an explicit argument over the environment over an
optional JSON file over the default (the reference's order: imparo-host/src/lib.rs:236-275,909-1010)."""
import json

import pytest

from imparo_b200.config import ConfigError, EngineConfig, KernelSwitches


def test_defaults():
    c = EngineConfig.resolve(env={})
    assert (c.dtype, c.ctx, c.parallel, c.page_size, c.num_pages, c.max_step_tokens, c.log) == \
        ("bfloat16", 4096, 8, 16, None, 2048, False)
    s = c.switches
    assert (s.gemm, s.tc_max_tokens, s.unfolded, s.defer_adds, s.fuse_producers, s.attn_prefill) == \
        ("tcgen05", 64, True, True, True, "auto")


def test_flag_over_environment_over_file_over_default(tmp_path):
    f = tmp_path / "engine.json"
    f.write_text(json.dumps({"ctx": 1000, "parallel": 3, "page_size": 32, "log": True,
                             "switches": {"gemm": "library", "tc_max_tokens": 8}, "fuse_producers": False}))
    env = {"IMPARO_CTX": "2000", "IMPARO_PARALLEL": "5", "IMPARO_TC_MAX_TOKENS": "16", "IMPARO_DEFER_ADDS": "0"}
    c = EngineConfig.resolve(flags={"ctx": 3000, "dtype": None, "switches": {"attn_prefill": "mma"}}, env=env, file=str(f))
    assert c.ctx == 3000                 # flag over environment and file
    assert c.parallel == 5               # environment over file
    assert c.page_size == 32             # file over default
    assert c.max_step_tokens == 2048     # default
    assert c.dtype == "bfloat16"         # a flag that is None was not given
    assert c.log is True
    s = c.switches
    assert s.attn_prefill == "mma"       # flag
    assert s.tc_max_tokens == 16         # environment over file
    assert s.defer_adds is False         # environment
    assert s.gemm == "library"           # file (nested)
    assert s.fuse_producers is False     # file (flat)
    assert s.unfolded is True            # default
    # the file may also be named by the environment
    c2 = EngineConfig.resolve(env={"IMPARO_CONFIG": str(f)})
    assert c2.ctx == 1000 and c2.switches.gemm == "library"


def test_bad_values_name_their_source(tmp_path):
    with pytest.raises(ConfigError, match="IMPARO_CTX"):
        EngineConfig.resolve(env={"IMPARO_CTX": "many"})
    with pytest.raises(ConfigError, match="IMPARO_DEFER_ADDS"):
        EngineConfig.resolve(env={"IMPARO_DEFER_ADDS": "perhaps"})
    with pytest.raises(ConfigError, match="unknown"):
        EngineConfig.resolve(flags={"context": 5}, env={})
    with pytest.raises(ConfigError, match="gemm"):
        EngineConfig.resolve(flags={"switches": {"gemm": "magic"}}, env={})
    with pytest.raises(ConfigError, match="at least 1"):
        EngineConfig.resolve(flags={"ctx": 0}, env={})
    f = tmp_path / "bad.json"
    f.write_text("[1, 2]")
    with pytest.raises(ConfigError, match="object"):
        EngineConfig.resolve(env={}, file=str(f))
    with pytest.raises(ConfigError, match="nothere"):
        EngineConfig.resolve(env={}, file=str(tmp_path / "nothere.json"))


def test_the_launchers_read_the_resolved_switches_not_the_environment(monkeypatch):
    """ops works on the switches of the state that is current; setting a variable after the state was made changes
    nothing, and an engine's state carries the engine's own switches."""
    from imparo_b200.kernels import ops
    base = ops.switches()
    monkeypatch.setenv("IMPARO_GEMM", "library")
    monkeypatch.setenv("IMPARO_TC_MAX_TOKENS", "7")
    assert ops.gemm_backend() == base.gemm and ops.tc_max_tokens() == base.tc_max_tokens
    mine = ops.LaunchState(KernelSwitches(gemm="library", tc_max_tokens=7, defer_adds=False))
    old = ops.use_state(mine)
    try:
        assert ops.gemm_backend() == "library" and ops.tc_max_tokens() == 7 and not ops.defer_adds()
    finally:
        ops.use_state(old)
    assert ops.gemm_backend() == base.gemm
    # a state made now resolves the environment as it is now
    assert ops.LaunchState().switches.gemm == "library" and ops.LaunchState().switches.tc_max_tokens == 7
