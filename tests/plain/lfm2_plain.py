"""Plain LFM2 forward: whole sequences, no cache, one function per part.

Written from the formulas of zeraix/imparo's CPU oracle; every function names the
file and lines (paths inside that project) it restates.  It shares no code with
the engine: it has its own config reading, its own safetensors reader and plain
numpy arithmetic.  It rests on the formulas alone for everything except the
gated convolution, whose core is also compared once with the reference's own
host C++ (tests/golden/).

All arithmetic runs in the numpy dtype given (float32 by default, float64 as a
ground truth for judging rounding).
"""
from __future__ import annotations

import json
import math
import os
import struct

import numpy as np

# ----------------------------------------------------------------------------
# files
# ----------------------------------------------------------------------------

_ST_DTYPES = {"F32": np.float32, "F16": np.float16, "I32": np.int32, "I64": np.int64,
              "F64": np.float64}


def read_safetensors(path):
    """name -> float32/int ndarray.  BF16 is widened by shifting into the high half."""
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        blob = f.read()
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        a, b = info["data_offsets"]
        raw = blob[a:b]
        if info["dtype"] == "BF16":
            u = np.frombuffer(raw, dtype=np.uint16).astype(np.uint32) << 16
            arr = u.view(np.float32)
        else:
            arr = np.frombuffer(raw, dtype=_ST_DTYPES[info["dtype"]])
        out[name] = arr.reshape(info["shape"]).copy()
    return out


class PlainConfig:
    """The sizes and constants of one LFM2 model, read from config.json keys."""

    def __init__(self, d):
        self.vocab = int(d["vocab_size"])
        self.hidden = int(d["hidden_size"])
        self.n_layers = int(d["num_hidden_layers"])
        if "layer_types" in d:
            self.layer_types = list(d["layer_types"])
        else:
            full = set(d["full_attn_idxs"])
            self.layer_types = ["full_attention" if i in full else "conv"
                                for i in range(self.n_layers)]
        self.n_heads = int(d["num_attention_heads"])
        self.n_kv = int(d["num_key_value_heads"])
        # imparo-model/src/lfm2/plan.rs:54-63: the head size is hidden / heads.
        self.head_dim = int(d.get("head_dim", self.hidden // self.n_heads))
        self.taps = int(d["conv_L_cache"])
        self.conv_bias = bool(d.get("conv_bias", False))
        ff = int(d["block_ff_dim"] if "block_ff_dim" in d else d["intermediate_size"])
        if d["block_auto_adjust_ff_dim"]:
            ff = int(2 * ff / 3)
            mult = d.get("block_ffn_dim_multiplier")
            if mult is not None:
                ff = int(mult * ff)
            mo = int(d.get("block_multiple_of", 256))
            ff = mo * ((ff + mo - 1) // mo)
        self.ff = ff
        self.theta = float(d.get("rope_theta", 10000.0))       # plan.rs:41
        self.eps = float(d.get("norm_eps", 1e-5))              # plan.rs:39-40
        self.tied = bool(d.get("tie_embedding", d.get("tie_word_embeddings", True)))
        self.window = d.get("sliding_window")                  # plan.rs:82-84

    @classmethod
    def from_dir(cls, folder):
        with open(os.path.join(folder, "config.json")) as f:
            return cls(json.load(f))


# ----------------------------------------------------------------------------
# parts
# ----------------------------------------------------------------------------

def rms_norm(x, w, eps):
    """imparo-cpu/src/ops.rs:6-22 — mean of squares over the row, 1/sqrt(mean+eps),
    then x * scale * w in that order."""
    mean = (x * x).sum(axis=-1, keepdims=True) / x.shape[-1]
    scale = 1.0 / np.sqrt(mean + x.dtype.type(eps))
    return x * scale * w


def rope_inv_freq(n_rot, theta):
    """imparo-cpu/src/ops.rs:558-560 — inv[i] = base^(-2i/n_rot), a 32-bit value."""
    i = np.arange(n_rot // 2, dtype=np.float64)
    return (float(theta) ** (-2.0 * i / n_rot)).astype(np.float32)


def rope_neox(x, positions, n_rot, theta):
    """imparo-cpu/src/ops.rs:551-569 — half-split pairs (i, i+n_rot/2); the angle is
    the product position*inv rounded to 32 bits, then sin and cos of that.
    x: [T, heads, head_dim]; positions: [T]."""
    half = n_rot // 2
    inv = rope_inv_freq(n_rot, theta)
    ang = (positions.astype(np.float64)[:, None] * inv.astype(np.float64)[None, :]).astype(np.float32)
    cos = np.cos(ang).astype(x.dtype)[:, None, :]
    sin = np.sin(ang).astype(x.dtype)[:, None, :]
    out = x.copy()
    x0 = x[..., :half]
    x1 = x[..., half:n_rot]
    out[..., :half] = x0 * cos - x1 * sin
    out[..., half:n_rot] = x0 * sin + x1 * cos
    return out


def head_norm_rope(x, w, eps, positions, n_rot, theta):
    """imparo-model/src/cpu_support.rs:361-376 — per (token, head): RMS norm over the
    head, then NeoX rotation at the token's absolute position."""
    return rope_neox(rms_norm(x, w, eps), positions, n_rot, theta)


def softmax(s):
    """imparo-cpu/src/ops.rs:572-583 — subtract the max, exp, sum, times 1/sum."""
    e = np.exp(s - s.max())
    return e * (s.dtype.type(1.0) / e.sum())


def attend(q, k, v, scale, window=None):
    """imparo-model/src/cpu_support.rs:402-445 — token t sees keys lo..=t, lo = 0 or
    (t+1-window); head h reads kv head h // (heads / kv_heads); no mask tensor.
    q: [T, nh, hd]; k, v: [T, nkv, hd] (position == row)."""
    T, nh, hd = q.shape
    nkv = k.shape[1]
    per_kv = nh // nkv
    out = np.zeros_like(q)
    for t in range(T):
        lo = 0 if not window else max(0, t + 1 - int(window))
        for h in range(nh):
            kvh = h // per_kv
            s = (k[lo:t + 1, kvh, :] @ q[t, h, :]) * q.dtype.type(scale)
            p = softmax(s)
            out[t, h, :] = p @ v[lo:t + 1, kvh, :]
    return out


def attend_blocked(q, k, v, scale, window=None, block=256):
    """The same formula as attend() (imparo-model/src/cpu_support.rs:402-445: token t sees keys lo..=t, head h
    reads kv head h // (heads / kv_heads), softmax of the scaled scores, times the values), evaluated for a
    block of query tokens at a time so that long sequences finish: scores of a block against keys 0..end of the
    block, positions a query must not see set to -inf before the softmax."""
    T, nh, hd = q.shape
    nkv = k.shape[1]
    per_kv = nh // nkv
    out = np.zeros_like(q)
    neg = q.dtype.type(-np.inf)
    for a in range(0, T, block):
        b = min(T, a + block)
        lo_blk = 0 if not window else max(0, a + 1 - int(window))
        kpos = np.arange(lo_blk, b)[None, :]
        qpos = np.arange(a, b)[:, None]
        dead = kpos > qpos
        if window:
            dead = dead | (kpos < qpos + 1 - int(window))
        for kvh in range(nkv):
            kk = k[lo_blk:b, kvh, :]                                  # [keys, hd]
            vv = v[lo_blk:b, kvh, :]
            qq = q[a:b, kvh * per_kv:(kvh + 1) * per_kv, :]           # [block, per_kv, hd]
            s = (qq.reshape(-1, hd) @ kk.T).reshape(b - a, per_kv, -1) * q.dtype.type(scale)     # one matrix product per block
            s[np.broadcast_to(dead[:, None, :], s.shape)] = neg
            s -= s.max(axis=-1, keepdims=True)
            np.exp(s, out=s)
            s *= q.dtype.type(1.0) / s.sum(axis=-1, keepdims=True)
            out[a:b, kvh * per_kv:(kvh + 1) * per_kv, :] = (s.reshape(-1, s.shape[-1]) @ vv).reshape(b - a, per_kv, hd)
    return out


def attention_mixer(cur, w, cfg, positions, attend_block=None):
    """imparo-model/src/lfm2/workflow_cpu.rs:203-250 — q/k/v projections, per-head
    norm and rotation of q and k, causal attention scaled by 1/sqrt(head_dim),
    output projection.  attend_block: evaluate the attention a block of queries at a time (long sequences)."""
    T = cur.shape[0]
    hd = cfg.head_dim
    q = (cur @ w["q_proj"].T).reshape(T, cfg.n_heads, hd)
    k = (cur @ w["k_proj"].T).reshape(T, cfg.n_kv, hd)
    v = (cur @ w["v_proj"].T).reshape(T, cfg.n_kv, hd)
    q = head_norm_rope(q, w["q_layernorm"], cfg.eps, positions, hd, cfg.theta)
    k = head_norm_rope(k, w["k_layernorm"], cfg.eps, positions, hd, cfg.theta)
    if attend_block:
        o = attend_blocked(q, k, v, 1.0 / math.sqrt(hd), window=w.get("window"), block=int(attend_block))
    else:
        o = attend(q, k, v, 1.0 / math.sqrt(hd), window=w.get("window"))
    return o.reshape(T, cfg.n_heads * hd) @ w["out_proj"].T


def gated_conv(bcx, conv_w, conv_b=None):
    """imparo-cpu/src/ops.rs:109-167 with an all-zero starting state — rows are
    [b | c | x]; v = b*x; sum[t] = sum_k w[ch,k] * seq[t+k] where seq is taps-1 zeros
    followed by v (tap 0 meets the oldest value); y = c * sum.  A bias, which the
    reference does not have, is added to sum before the gate.
    bcx: [T, 3H]; conv_w: [H, taps]."""
    T = bcx.shape[0]
    H, taps = conv_w.shape
    b, c, x = bcx[:, :H], bcx[:, H:2 * H], bcx[:, 2 * H:]
    seq = np.concatenate([np.zeros((taps - 1, H), dtype=bcx.dtype), b * x], axis=0)
    acc = np.zeros((T, H), dtype=bcx.dtype)
    for k in range(taps):
        acc = acc + conv_w[:, k][None, :] * seq[k:k + T, :]
    if conv_b is not None:
        acc = acc + conv_b[None, :]
    return c * acc


def conv_mixer(cur, w, cfg):
    """imparo-model/src/lfm2/workflow_cpu.rs:260-277 — in_proj to [b|c|x], the gated
    causal convolution, out_proj."""
    bcx = cur @ w["in_proj"].T
    if "in_proj_bias" in w:
        bcx = bcx + w["in_proj_bias"]
    y = gated_conv(bcx, w["conv"], w.get("conv_bias"))
    out = y @ w["out_proj"].T
    if "out_proj_bias" in w:
        out = out + w["out_proj_bias"]
    return out


def silu(x):
    """imparo-cpu/src/ops.rs:73-78 — t / (1 + exp(-t))."""
    return x / (x.dtype.type(1.0) + np.exp(-x))


def swiglu(n, w):
    """imparo-model/src/lfm2/workflow_cpu.rs:307-313 — down(silu(gate(n)) * up(n)),
    SiLU on the gate (w1), up is w3, down is w2."""
    return (silu(n @ w["w1"].T) * (n @ w["w3"].T)) @ w["w2"].T


def block(x, lw, cfg, positions, probe=None, attend_block=None):
    """imparo-model/src/lfm2/workflow_cpu.rs:172-319 — pre-norms only:
    x += mixer(rms(x, operator_norm)); x += ffn(rms(x, ffn_norm)).
    probe(name, array): shown the stages the reference's probe names
    (imparo-model/src/cpu_support.rs:26-46), for comparing with another engine."""
    show = probe if probe is not None else (lambda name, a: None)
    show("stream_in", x)
    cur = rms_norm(x, lw["operator_norm"], cfg.eps)
    show("mixer_norm", cur)
    if lw["kind"] == "conv":
        mix = conv_mixer(cur, lw, cfg)
    else:
        mix = attention_mixer(cur, lw, cfg, positions, attend_block)
    x = x + mix
    show("stream_mixer", x)
    h = rms_norm(x, lw["ffn_norm"], cfg.eps)
    show("ff_norm", h)
    x = x + swiglu(h, lw)
    show("stream_out", x)
    return x


# ----------------------------------------------------------------------------
# the model
# ----------------------------------------------------------------------------

class PlainLfm2:
    def __init__(self, folder, dtype=np.float32):
        self.cfg = PlainConfig.from_dir(folder)
        self.dtype = dtype
        raw = read_safetensors(os.path.join(folder, "model.safetensors"))
        t = {}
        for name, arr in raw.items():
            t[name[6:] if name.startswith("model.") else name] = arr.astype(dtype)
        cfg = self.cfg
        self.embed = t["embed_tokens.weight"]
        self.head = self.embed if cfg.tied else t["lm_head.weight"]
        self.out_norm = t["embedding_norm.weight"]
        self.layers = []
        for i, kind in enumerate(cfg.layer_types):
            p = f"layers.{i}."
            lw = {"operator_norm": t[p + "operator_norm.weight"],
                  "ffn_norm": t[p + "ffn_norm.weight"],
                  "w1": t[p + "feed_forward.w1.weight"],
                  "w2": t[p + "feed_forward.w2.weight"],
                  "w3": t[p + "feed_forward.w3.weight"]}
            if kind == "conv":
                lw["kind"] = "conv"
                lw["in_proj"] = t[p + "conv.in_proj.weight"]
                lw["out_proj"] = t[p + "conv.out_proj.weight"]
                lw["conv"] = t[p + "conv.conv.weight"].reshape(cfg.hidden, cfg.taps)
                if p + "conv.conv.bias" in t:
                    lw["conv_bias"] = t[p + "conv.conv.bias"]
                if p + "conv.in_proj.bias" in t:
                    lw["in_proj_bias"] = t[p + "conv.in_proj.bias"]
                if p + "conv.out_proj.bias" in t:
                    lw["out_proj_bias"] = t[p + "conv.out_proj.bias"]
            else:
                lw["kind"] = "attention"
                for nm in ("q_proj", "k_proj", "v_proj", "out_proj"):
                    lw[nm] = t[p + f"self_attn.{nm}.weight"]
                lw["q_layernorm"] = t[p + "self_attn.q_layernorm.weight"]
                lw["k_layernorm"] = t[p + "self_attn.k_layernorm.weight"]
                if kind == "sliding_attention":
                    lw["window"] = int(cfg.window)
            self.layers.append(lw)

    def hidden_states(self, tokens, probe_layer=None, probe=None, attend_block=None):
        """imparo-model/src/cpu_support.rs:327-342 (rows of the table, no scale), then
        every block in order.  probe_layer / probe: see block()."""
        tokens = np.asarray(tokens, dtype=np.int64)
        positions = np.arange(len(tokens))
        x = self.embed[tokens].astype(self.dtype)
        for i, lw in enumerate(self.layers):
            x = block(x, lw, self.cfg, positions, probe if i == probe_layer else None, attend_block)
        return x

    def logits_at(self, tokens, places, attend_block=256):
        """Logits at the given positions only, with the attention evaluated block by block: for sequences too
        long for logits().  [len(places), vocab]."""
        x = self.hidden_states(tokens, attend_block=attend_block)[np.asarray(places, dtype=np.int64)]
        h = rms_norm(x, self.out_norm, self.cfg.eps)
        return h @ self.head.T

    def logits(self, tokens):
        """imparo-model/src/cpu_support.rs:451-466 — final norm then the head, here at
        every position: [T, vocab]."""
        x = self.hidden_states(tokens)
        h = rms_norm(x, self.out_norm, self.cfg.eps)
        return h @ self.head.T


# ----------------------------------------------------------------------------
# sampling
# ----------------------------------------------------------------------------

def argmax_first(logits):
    """imparo-cpu/src/ops.rs:637-640 — the smallest index that attains the maximum;
    NaN never wins."""
    row = np.where(np.isnan(logits), -np.inf, logits)
    return int(np.argmax(row))


def greedy_generate(model, prompt, n_new):
    toks = list(prompt)
    for _ in range(n_new):
        toks.append(argmax_first(model.logits(toks)[-1]))
    return toks[len(prompt):]


_MASK64 = (1 << 64) - 1


def uniform_for(seed, step):
    """The engine's per-(seed, step) uniform number, restated: splitmix64 of
    seed * 0x9E3779B97F4A7C15 + step, top 24 bits.  (The reference has no temperature
    sampling: imparo-server/src/main.rs:3383-3390.)"""
    z = ((seed & _MASK64) * 0x9E3779B97F4A7C15 + (step & _MASK64) + 0x9E3779B97F4A7C15) & _MASK64
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK64
    z ^= z >> 31
    return (z >> 40) / float(1 << 24)


def sample_temperature(logits, temperature, u):
    """First index whose running sum of softmax(logits / T), in vocabulary order, exceeds u.
    Returns (index, distance of u to the nearest boundary of that index's interval)."""
    z = (logits.astype(np.float64) - logits.max()) / temperature
    p = np.exp(z)
    cdf = np.cumsum(p) / p.sum()
    i = int(np.searchsorted(cdf, u, side="right"))
    i = min(i, len(cdf) - 1)
    lo = cdf[i - 1] if i > 0 else 0.0
    return i, min(u - lo, cdf[i] - u)


def generate(model, prompt, n_new, temperature=0.0, seed=0):
    """Token by token from whole-sequence logits.  -> (tokens, margins): margin is how far
    each pick was from going another way (top-2 logit gap for greedy, distance of u to an
    interval boundary for temperature)."""
    toks, out, margins = list(prompt), [], []
    for step in range(n_new):
        row = model.logits(toks)[-1]
        if temperature > 0:
            t, margin = sample_temperature(row, temperature, uniform_for(seed, step))
        else:
            t = argmax_first(row)
            top2 = np.partition(row, -2)[-2:]
            margin = float(top2[1] - top2[0])
        out.append(t)
        margins.append(margin)
        toks.append(t)
    return out, margins
