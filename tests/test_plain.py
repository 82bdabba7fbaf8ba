"""The plain implementation itself: closed-form cases the reference tests its CPU oracle
with, and the gated convolution against the reference's own host C++ (tests/golden/)."""
import json
import os

import numpy as np
import pytest

from tests.plain import lfm2_plain as P
from tests.tiny_configs import TINY_A, TINY_B

HERE = os.path.dirname(os.path.abspath(__file__))


def test_rms_norm_by_hand():
    x = np.array([[3.0, 4.0]], dtype=np.float64)
    w = np.array([2.0, 0.5])
    got = P.rms_norm(x, w, 0.0)
    assert np.allclose(got, [[3 / np.sqrt(12.5) * 2, 4 / np.sqrt(12.5) * 0.5]])


def test_rope_pairs_are_half_split_and_position_zero_is_identity():
    x = np.arange(8, dtype=np.float64).reshape(1, 1, 8) + 1
    assert np.array_equal(P.rope_neox(x, np.array([0]), 8, 10000.0), x)
    y = P.rope_neox(x, np.array([3]), 8, 10000.0)[0, 0]
    inv = P.rope_inv_freq(8, 10000.0)
    for i in range(4):
        a = np.float32(3.0 * inv[i])
        assert np.isclose(y[i], x[0, 0, i] * np.cos(a) - x[0, 0, i + 4] * np.sin(a))
        assert np.isclose(y[i + 4], x[0, 0, i] * np.sin(a) + x[0, 0, i + 4] * np.cos(a))
    # norms are kept by a rotation
    assert np.isclose(np.linalg.norm(y), np.linalg.norm(x))


def test_attention_with_identity_values_is_a_causal_average():
    # imparo-model/src/cpu_support.rs:483-512: equal scores -> token t averages values 0..t
    T, hd = 5, 4
    q = np.zeros((T, 1, hd))
    k = np.ones((T, 1, hd))
    v = np.arange(T * hd, dtype=np.float64).reshape(T, 1, hd)
    out = P.attend(q, k, v, 0.5)
    for t in range(T):
        assert np.allclose(out[t, 0], v[:t + 1, 0].mean(axis=0))


def test_attention_window_and_contiguous_groups():
    # cpu_support.rs:537-557: head h reads kv head h // (heads / kv_heads)
    T, hd = 6, 2
    q = np.zeros((T, 4, hd))
    k = np.zeros((T, 2, hd))
    v = np.zeros((T, 2, hd))
    v[:, 0, :] = 1.0
    v[:, 1, :] = 7.0
    out = P.attend(q, k, v, 1.0)
    assert np.allclose(out[:, :2], 1.0) and np.allclose(out[:, 2:], 7.0)
    v2 = np.arange(T, dtype=np.float64)[:, None, None] * np.ones((T, 2, hd))
    out = P.attend(q, k, v2, 1.0, window=3)
    assert np.allclose(out[5, 0], np.mean([3, 4, 5])) and np.allclose(out[1, 0], np.mean([0, 1]))


def test_conv_tap_zero_is_the_oldest_and_c_gates_the_output():
    # imparo-cpu/src/ops.rs:1205-1285
    H, taps, T = 1, 3, 4
    bcx = np.zeros((T, 3 * H))
    bcx[:, 0] = 1.0                      # b
    bcx[:, 1] = 1.0                      # c
    bcx[:, 2] = [1.0, 10.0, 100.0, 1000.0]   # x
    w = np.array([[0.0, 0.0, 1.0]])      # only the newest tap
    assert np.allclose(P.gated_conv(bcx, w)[:, 0], [1, 10, 100, 1000])
    w = np.array([[1.0, 0.0, 0.0]])      # only the oldest tap: two tokens late
    assert np.allclose(P.gated_conv(bcx, w)[:, 0], [0, 0, 1, 10])
    bcx[:, 1] = 0.0
    assert np.allclose(P.gated_conv(bcx, w), 0.0)


def test_conv_matches_the_reference_host_code():
    """tests/golden/conv_golden.json was made by the reference's shortconv_reference /
    shortconv_state_reference.  A non-zero starting state is fed to the whole-sequence
    function as taps-1 earlier tokens whose b*x equal the state."""
    with open(os.path.join(HERE, "golden", "conv_golden.json")) as f:
        cases = json.load(f)["cases"]
    assert len(cases) >= 5
    for c in cases:
        H, taps, T = c["width"], c["kernel"], c["n_tok"]
        hist = taps - 1
        bcx = np.array(c["bcx"], dtype=np.float32).reshape(T, 3 * H)
        w = np.array(c["weights"], dtype=np.float32).reshape(H, taps)
        state = np.array(c["state"], dtype=np.float32).reshape(hist, H)
        pre = np.concatenate([state, np.zeros((hist, H), np.float32), np.ones((hist, H), np.float32)], axis=1)
        y = P.gated_conv(np.concatenate([pre, bcx]), w)[hist:]
        assert np.allclose(y.reshape(-1), np.array(c["output"], dtype=np.float32), rtol=1e-6, atol=1e-6)
        v = np.concatenate([state, bcx[:, :H] * bcx[:, 2 * H:]])
        assert np.allclose(v[-hist:].reshape(-1), np.array(c["next_state"], dtype=np.float32), rtol=1e-6, atol=1e-7)


def test_silu_and_argmax_rules():
    x = np.array([-2.0, 0.0, 3.0])
    assert np.allclose(P.silu(x), x / (1 + np.exp(-x)))
    assert P.argmax_first(np.array([1.0, 5.0, 5.0, np.nan, 2.0])) == 1
    assert P.argmax_first(np.array([np.nan, np.nan])) == 0


def test_whole_model_is_causal_and_prefix_stable(tmp_path):
    from imparo_b200.weights import write_random_model
    for name, cfg in (("a", TINY_A), ("b", TINY_B)):
        d = write_random_model(str(tmp_path / name), cfg, seed=2)
        m = P.PlainLfm2(d, np.float64)
        toks = np.random.default_rng(1).integers(0, cfg["vocab_size"], 23).tolist()
        full = m.logits(toks)
        assert full.shape == (23, cfg["vocab_size"])
        assert np.allclose(m.logits(toks[:9]), full[:9], atol=1e-12)
        assert P.PlainConfig(cfg).ff == (192 if name == "a" else 512)


def test_blocked_attention_is_the_same_formula():
    """attend_blocked (a block of queries at a time, for long sequences) against attend (token by token), with and
    without a window, block sizes that do and do not divide the length."""
    rng = np.random.default_rng(3)
    T, nh, nkv, hd = 45, 6, 2, 8
    q, k, v = rng.standard_normal((T, nh, hd)), rng.standard_normal((T, nkv, hd)), rng.standard_normal((T, nkv, hd))
    for window in (None, 7, 16):
        ref = P.attend(q, k, v, 0.3, window)
        for block in (1, 8, 16, 64):
            assert np.allclose(P.attend_blocked(q, k, v, 0.3, window, block), ref, atol=1e-12), (window, block)


def test_logits_at_places_equal_whole_logits(tmp_path):
    from imparo_b200.weights import write_random_model
    d = write_random_model(str(tmp_path / "b"), TINY_B, seed=4)
    m = P.PlainLfm2(d, np.float64)
    toks = np.random.default_rng(2).integers(0, TINY_B["vocab_size"], 37).tolist()
    full = m.logits(toks)
    assert np.allclose(m.logits_at(toks, [0, 5, 36], attend_block=8), full[[0, 5, 36]], atol=1e-10)
