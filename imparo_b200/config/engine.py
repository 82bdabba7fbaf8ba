"""Typed configuration of the engine itself (not of a model): how much it may hold, how it cuts
steps, and which kernel paths it takes.

Every value is resolved once, when an engine is built, in the reference's order: an explicit
argument (a command-line flag, a keyword of Engine) wins over the environment (IMPARO_* names),
which wins over an optional JSON file, which wins over the default
(imparo-host/src/lib.rs:236-275 flags and IMPARO_* variables, :909-1010 the tuned-configuration
file).  The launchers read the resolved KernelSwitches object; nothing on the launch path looks
at the environment.

    cfg = EngineConfig.resolve(flags={"ctx": 8192}, env=os.environ, file="engine.json")
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field, fields
from typing import Any, Mapping, Optional

from .base import ConfigError

_TRUE, _FALSE = ("1", "true", "yes", "on"), ("0", "false", "no", "off", "")


def _parse(name: str, kind: type, raw: Any, where: str):
    """A value from the environment (a string) or from a JSON file, as the field's type."""
    try:
        if kind is bool:
            if isinstance(raw, bool):
                return raw
            s = str(raw).strip().lower()
            if s in _TRUE:
                return True
            if s in _FALSE:
                return False
            raise ValueError(raw)
        if kind is int:
            if isinstance(raw, bool):
                raise ValueError(raw)
            return int(raw)
        if kind is float:
            return float(raw)
        return str(raw)
    except (TypeError, ValueError):
        raise ConfigError(f"{where}: '{name}' must be {kind.__name__}, found {raw!r}") from None


@dataclass
class KernelSwitches:
    """Which kernel path the launchers take.  The defaults are what measured fastest on B200."""
    gemm: str = "tcgen05"                 # IMPARO_GEMM: "tcgen05" | "library" (which product bfloat16 uses)
    tc_max_tokens: int = 64               # IMPARO_TC_MAX_TOKENS: most tokens the weight-streaming product takes
    prefill_gemm: str = "tcgen05"         # IMPARO_PREFILL_GEMM: "tcgen05" | "library" for prompt-sized products
    prefill_tc_min_tokens: int = 256      # IMPARO_PREFILL_TC_MIN_TOKENS: fewest tokens of the persistent tile product
    prefill_linear: bool = False          # IMPARO_PREFILL_LINEAR: the tile product also for plain products (not only SwiGLU)
    unfolded: bool = True                 # IMPARO_UNFOLDED: in_proj / qkv leave split partials to their consumer
    defer_adds: bool = True               # IMPARO_DEFER_ADDS: products into the stream leave partials to the next norm
    fuse_producers: bool = True           # IMPARO_FUSE_PRODUCERS: the attention combine inside the output product (decode rows)
    decode_from_qkv: bool = True          # IMPARO_DECODE_FROM_QKV: decode rows' q/k norm, rotation and cache write inside the attention kernel
    attn_side_by_side: bool = True        # IMPARO_ATTN_SIDE_BY_SIDE: a step's prompt-portion attention and decode-row attention run at the same time
    attn_prefill: str = "auto"            # IMPARO_ATTN_PREFILL: "auto" | "mma" | "tcgen05" | "tcgen05_one_tile"

    ENV_PREFIX = "IMPARO_"

    def __post_init__(self):
        self.gemm = {"lib": "library", "cublas": "library"}.get(self.gemm.lower(), self.gemm.lower())
        self.prefill_gemm = {"lib": "library", "cublas": "library"}.get(self.prefill_gemm.lower(), self.prefill_gemm.lower())
        if self.gemm not in ("tcgen05", "library") or self.prefill_gemm not in ("tcgen05", "library"):
            raise ConfigError("gemm and prefill_gemm must be 'tcgen05' or 'library'")
        if self.attn_prefill not in ("auto", "mma", "tcgen05", "tcgen05_one_tile"):
            raise ConfigError("attn_prefill must be 'auto', 'mma', 'tcgen05' or 'tcgen05_one_tile'")
        if self.tc_max_tokens < 0 or self.prefill_tc_min_tokens < 1:
            raise ConfigError("tc_max_tokens must be >= 0 and prefill_tc_min_tokens >= 1")


@dataclass
class EngineConfig:
    dtype: str = "bfloat16"               # --dtype / IMPARO_DTYPE
    device: str = "cuda:0"                # IMPARO_DEVICE
    ctx: int = 4096                       # -c/--ctx / IMPARO_CTX: most positions one request may reach
    parallel: int = 8                     # -np/--parallel / IMPARO_PARALLEL: most requests live at once
    page_size: int = 16                   # --page-size / IMPARO_PAGE_SIZE: positions per cache page
    num_pages: Optional[int] = None       # --num-pages / IMPARO_NUM_PAGES: pages per pool (default: parallel * ctx worth)
    max_step_tokens: int = 2048           # --max-step-tokens / IMPARO_MAX_STEP_TOKENS (the reference's IMPARO_BATCH)
    use_graphs: bool = True               # IMPARO_USE_GRAPHS: replay captured steps
    capture_first: bool = True            # IMPARO_CAPTURE_FIRST: capture a step's graph the first time its shape comes
    pad_rows: bool = True                 # IMPARO_PAD_ROWS: one-token rows of a step filled up to 1, 2, 4, 8, 16, 24, ... rows
    probe_layer: Optional[int] = None     # --probe-layer / IMPARO_PROBE_LAYER
    log: bool = False                     # IMPARO_LOG: one line per generation step on stderr
    switches: KernelSwitches = field(default_factory=KernelSwitches)

    ENV_PREFIX = "IMPARO_"
    FILE_ENV = "IMPARO_CONFIG"            # path of the optional JSON file, when no explicit one is given

    def __post_init__(self):
        for name in ("ctx", "parallel", "page_size", "max_step_tokens"):
            if int(getattr(self, name)) < 1:
                raise ConfigError(f"engine configuration: '{name}' must be at least 1")
        if self.num_pages is not None and self.num_pages < 1:
            raise ConfigError("engine configuration: 'num_pages' must be at least 1")

    @classmethod
    def resolve(cls, flags: Optional[Mapping[str, Any]] = None, env: Optional[Mapping[str, str]] = None,
                file: Optional[str] = None) -> "EngineConfig":
        """flags: explicit values by field name (None = not given; the switches' fields may be given flat or
        under "switches").  env: the environment (default os.environ).  file: a JSON object with the same field
        names (switches flat or under "switches"); default: the path in IMPARO_CONFIG, if set.
        Precedence per field: flag > environment > file > default."""
        env = os.environ if env is None else env
        flags = dict(flags or {})
        flag_switches = dict(flags.pop("switches", None) or {})
        path = file or env.get(cls.FILE_ENV) or None
        from_file: dict = {}
        if path:
            try:
                with open(path) as f:
                    from_file = json.load(f)
            except (OSError, json.JSONDecodeError) as e:
                raise ConfigError(f"engine configuration file {path}: {e}") from None
            if not isinstance(from_file, dict):
                raise ConfigError(f"engine configuration file {path}: top level must be an object")
        file_switches = dict(from_file.pop("switches", None) or {})

        def pick(owner, name, kind, optional, flag_maps, file_maps):
            for m in flag_maps:
                if m.get(name) is not None:
                    return m[name] if isinstance(m[name], kind) and not (kind is int and isinstance(m[name], bool)) \
                        else _parse(name, kind, m[name], "argument")
            raw = env.get(owner.ENV_PREFIX + name.upper())
            if raw is not None and not (optional and raw == ""):
                return _parse(name, kind, raw, f"environment variable {owner.ENV_PREFIX}{name.upper()}")
            for m in file_maps:
                if m.get(name) is not None:
                    return _parse(name, kind, m[name], f"engine configuration file {path}")
            return None

        known = {f.name for f in fields(cls)} | {f.name for f in fields(KernelSwitches)}
        for src, what in ((flags, "argument"), (flag_switches, "argument"), (from_file, f"file {path}"), (file_switches, f"file {path}")):
            for k in src:
                if k not in known:
                    raise ConfigError(f"engine configuration: unknown {what} '{k}'")
        sw = {}
        for f in fields(KernelSwitches):
            v = pick(KernelSwitches, f.name, type(f.default), False, (flag_switches, flags), (file_switches, from_file))
            if v is not None:
                sw[f.name] = v
        top = {}
        for f in fields(cls):
            if f.name == "switches":
                continue
            optional = f.name in ("num_pages", "probe_layer")
            kind = int if optional else type(f.default)
            v = pick(cls, f.name, kind, optional, (flags,), (from_file,))
            if v is not None:
                top[f.name] = v
        return cls(switches=KernelSwitches(**sw), **top)
