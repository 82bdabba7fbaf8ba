"""Each CUDA kernel alone against a plain float32/float64 reference of the same operation,
at sizes other than the engine's test models: widths and vocabularies that are no power of
two, head sizes 16..256, several head/group counts, page sizes 1..64, scrambled page
tables, windows, ragged batches."""
import json
import math
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
HERE = os.path.dirname(os.path.abspath(__file__))


def ops():
    from imparo_b200.kernels import ops as o
    return o


def bf16_round(x):
    return x.to(torch.bfloat16).to(torch.float32)


# ---------------------------------------------------------------------------------------
@pytest.mark.parametrize("width,vocab", [(72, 1000), (2048, 65536), (100, 331)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embed_gather(width, vocab, dtype):
    o = ops()
    g = torch.Generator().manual_seed(0)
    table = torch.randn(vocab, width, generator=g).to(dtype).to(DEV)
    ids = torch.randint(0, vocab, (37,), generator=g, dtype=torch.int32).to(DEV)
    out = torch.empty(37, width, device=DEV)
    st = o.new_status(DEV)
    o.embed_gather(table, ids, out, st)
    assert torch.equal(out, table[ids.long()].float())
    o.read_status(st)
    ids[5] = vocab
    o.embed_gather(table, ids, out, st)
    with pytest.raises(o.KernelError, match="token id"):
        o.read_status(st)


@pytest.mark.parametrize("width", [100, 144, 2048, 3000, 101, 1026])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm(width, out_dtype):
    o = ops()
    g = torch.Generator().manual_seed(1)
    x = torch.randn(19, width, generator=g) * 3
    w = 1 + 0.1 * torch.randn(width, generator=g)
    eps = 3e-6
    ref = (x.double() * (1.0 / torch.sqrt((x.double() ** 2).mean(-1, keepdim=True) + eps)) * w.double())
    out = torch.empty(19, width, dtype=out_dtype, device=DEV)
    o.rmsnorm(x.to(DEV), w.to(DEV), eps, out)
    tol = 2e-6 if out_dtype == torch.float32 else 8e-3
    assert (out.float().cpu().double() - ref).abs().max() <= tol * ref.abs().max()
    rows = torch.tensor([18, 0, 7], dtype=torch.int32, device=DEV)
    out2 = torch.empty(3, width, dtype=out_dtype, device=DEV)
    o.rmsnorm(x.to(DEV), w.to(DEV), eps, out2, rows)
    assert torch.equal(out2, out[rows.long()])


@pytest.mark.parametrize("width", [128, 1024, 2048, 2176, 144])
def test_rmsnorm_many_rows(width):
    """A prompt portion's worth of rows (another kernel from 256 rows on, where the width allows it)."""
    o = ops()
    g = torch.Generator().manual_seed(width)
    n = 300
    x = torch.randn(n + 20, width, generator=g) * 3
    w = 1 + 0.1 * torch.randn(width, generator=g)
    eps = 1e-5
    rows = torch.randperm(n + 20, generator=g)[:n].to(torch.int32)
    xs = x[rows.long()].double()
    ref = xs * (1.0 / torch.sqrt((xs ** 2).mean(-1, keepdim=True) + eps)) * w.double()
    out = torch.full((n, width), float("nan"), dtype=torch.bfloat16, device=DEV)
    o.rmsnorm(x.to(DEV), w.to(DEV), eps, out, rows.to(DEV))
    assert (out.float().cpu().double() - ref).abs().max() <= 8e-3 * ref.abs().max()
    out2 = torch.full((n + 20, width), float("nan"), dtype=torch.bfloat16, device=DEV)
    o.rmsnorm(x.to(DEV), w.to(DEV), eps, out2)
    assert torch.equal(out2[rows.long().to(DEV)], out)


@pytest.mark.parametrize("M,N,K", [(1, 53, 71), (37, 130, 64), (64, 64, 16), (130, 1, 5), (7, 331, 144)])
def test_sgemm_is_true_float32(M, N, K):
    o = ops()
    g = torch.Generator().manual_seed(2)
    a, w = torch.randn(M, K, generator=g), torch.randn(N, K, generator=g)
    # values with mantissa bits below what a reduced-precision product keeps
    a = a * (1 + 2.0 ** -15)
    ref = a.double() @ w.double().T
    out = torch.empty(M, N, device=DEV)
    o.linear(a.to(DEV), w.to(DEV), out)
    assert (out.cpu().double() - ref).abs().max() <= 2e-6 * max(1.0, ref.abs().max())
    base = torch.randn(M, N, generator=g)
    out2 = base.to(DEV).clone()
    o.linear(a.to(DEV), w.to(DEV), out2, accumulate=True)
    assert (out2.cpu().double() - (ref + base.double())).abs().max() <= 3e-6 * max(1.0, ref.abs().max())


@pytest.mark.parametrize("M,N,K", [(1, 96, 64), (5, 200, 136), (77, 512, 192), (300, 1000, 264)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_gemm_bf16(M, N, K, out_dtype):
    o = ops()
    g = torch.Generator().manual_seed(3)
    a, w = bf16_round(torch.randn(M, K, generator=g)), bf16_round(torch.randn(N, K, generator=g))
    ref = a.double() @ w.double().T
    out = torch.empty(M, N, dtype=out_dtype, device=DEV)
    o.linear(a.to(torch.bfloat16).to(DEV), w.to(torch.bfloat16).to(DEV), out)
    tol = 1e-5 if out_dtype == torch.float32 else 8e-3
    assert (out.float().cpu().double() - ref).abs().max() <= tol * ref.abs().max()
    if out_dtype == torch.float32:
        base = torch.randn(M, N, generator=g)
        out2 = base.to(DEV).clone()
        o.linear(a.to(torch.bfloat16).to(DEV), w.to(torch.bfloat16).to(DEV), out2, accumulate=True)
        assert (out2.cpu().double() - (ref + base.double())).abs().max() <= 1e-5 * ref.abs().max()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,F", [(11, 200), (11, 204), (3, 77), (130, 1016)])     # 16-byte path and not
def test_swiglu_act(dtype, rows, F):
    o = ops()
    g = torch.Generator().manual_seed(4)
    gu = (torch.randn(rows, 2 * F, generator=g) * 4).to(dtype)
    out = torch.empty(rows, F, dtype=dtype, device=DEV)
    o.swiglu_act(gu.to(DEV), out)
    gate, up = gu[:, :F].double(), gu[:, F:].double()
    ref = gate / (1 + torch.exp(-gate)) * up
    tol = 1e-6 if dtype == torch.float32 else 8e-3
    assert (out.float().cpu().double() - ref).abs().max() <= tol * ref.abs().max()


# ---------------------------------------------------------------------------------------
def conv_reference(bcx, w, bias, state):
    """numpy restatement of imparo-cpu/src/ops.rs:109-167 for one request's portion."""
    T, H, taps = bcx.shape[0], w.shape[0], w.shape[1]
    v = bcx[:, :H] * bcx[:, 2 * H:]
    seq = np.concatenate([state, v])
    y = np.zeros((T, H))
    for t in range(T):
        acc = sum(w[:, k] * seq[t + k] for k in range(taps))
        if bias is not None:
            acc = acc + bias
        y[t] = bcx[t, H:2 * H] * acc
    return y, seq[-(taps - 1):]


@pytest.mark.parametrize("taps", [2, 3, 4, 7])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("bias", [False, True])
@pytest.mark.parametrize("H,lens", [(72, [1, 9, 2, 1, 5]),          # shorter than taps-1, equal, longer
                                    (72, [40, 1, 3, 57, 6]),        # enough tokens for the 16-byte kernel
                                    (76, [33, 2, 70, 1, 1]),        # a width it does not take
                                    (72, [131, 1, 2, 97, 66])])     # a few hundred tokens, portions of every length
def test_gated_conv_ragged_batch(taps, dtype, bias, H, lens):
    o = ops()
    n_slots = 5
    slots = [3, 0, 4, 1, 2]
    g = torch.Generator().manual_seed(taps)
    T = sum(lens)
    bcx = torch.randn(T, 3 * H, generator=g).to(dtype)
    w = torch.randn(H, taps, generator=g)
    b = torch.randn(H, generator=g) if bias else None
    state = torch.randn(n_slots, taps - 1, H, generator=g)
    row_start = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    item_of_token = np.repeat(np.arange(len(lens)), lens).astype(np.int32)
    y = torch.empty(T, H, dtype=dtype, device=DEV)
    st_dev = state.to(DEV).clone()
    status = o.new_status(DEV)
    o.gated_conv(bcx.to(DEV), w.to(DEV), None if b is None else b.to(DEV), st_dev,
                 torch.from_numpy(row_start).to(DEV), torch.from_numpy(item_of_token).to(DEV),
                 torch.tensor(slots, dtype=torch.int32, device=DEV), y, taps, status)
    o.read_status(status)
    tol = 2e-6 if dtype == torch.float32 else 1e-2
    for i, n in enumerate(lens):
        a = row_start[i]
        ref_y, ref_s = conv_reference(bcx[a:a + n].double().numpy(), w.double().numpy(),
                                      None if b is None else b.double().numpy(), state[slots[i]].double().numpy())
        assert np.abs(y[a:a + n].float().cpu().double().numpy() - ref_y).max() <= tol * max(1.0, np.abs(ref_y).max())
        assert np.abs(st_dev[slots[i]].cpu().double().numpy() - ref_s).max() <= 2e-6 * max(1.0, np.abs(ref_s).max())


def test_gated_conv_matches_the_reference_host_code():
    """Outputs and next state against tests/golden/conv_golden.json, which the reference's
    own shortconv_reference / shortconv_state_reference produced."""
    o = ops()
    with open(os.path.join(HERE, "golden", "conv_golden.json")) as f:
        cases = json.load(f)["cases"]
    for c in cases:
        H, taps, T = c["width"], c["kernel"], c["n_tok"]
        bcx = torch.tensor(c["bcx"]).reshape(T, 3 * H).to(DEV)
        w = torch.tensor(c["weights"]).reshape(H, taps).to(DEV)
        state = torch.tensor(c["state"]).reshape(1, taps - 1, H).to(DEV)
        y = torch.empty(T, H, device=DEV)
        status = o.new_status(DEV)
        o.gated_conv(bcx, w, None, state, torch.tensor([0, T], dtype=torch.int32, device=DEV),
                     torch.zeros(T, dtype=torch.int32, device=DEV), torch.zeros(1, dtype=torch.int32, device=DEV),
                     y, taps, status)
        o.read_status(status)
        assert np.allclose(y.cpu().numpy().reshape(-1), np.array(c["output"], np.float32), rtol=2e-6, atol=2e-6)
        assert np.allclose(state.cpu().numpy().reshape(-1), np.array(c["next_state"], np.float32), rtol=1e-6, atol=1e-7)


# ---------------------------------------------------------------------------------------
def make_paged(rng, lens, page, nkv, hd, dtype, extra_pages=3):
    """Random keys/values for requests of the given lengths, laid out in scrambled pages."""
    R = len(lens)
    blocks = [(n + page - 1) // page for n in lens]
    n_pages = sum(blocks) + extra_pages
    perm = rng.permutation(n_pages)
    stride = max(blocks) + 2
    table = -np.ones((R, stride), dtype=np.int32)
    k_cache = torch.zeros(n_pages, page, nkv * hd)
    v_cache = torch.zeros(n_pages, page, nkv * hd)
    ks, vs = [], []
    at = 0
    for r, n in enumerate(lens):
        table[r, :blocks[r]] = perm[at:at + blocks[r]]
        at += blocks[r]
        k = torch.from_numpy(rng.standard_normal((n, nkv * hd)).astype(np.float32)).to(dtype).float()
        v = torch.from_numpy(rng.standard_normal((n, nkv * hd)).astype(np.float32)).to(dtype).float()
        for p in range(n):
            k_cache[table[r, p // page], p % page] = k[p]
            v_cache[table[r, p // page], p % page] = v[p]
        ks.append(k)
        vs.append(v)
    return table, k_cache.to(dtype), v_cache.to(dtype), ks, vs, n_pages


def attention_reference(q, k, v, pos, nh, nkv, hd, scale, window):
    """imparo-model/src/cpu_support.rs:402-445 for one query row, in float64."""
    out = np.zeros((nh, hd))
    lo = max(0, pos + 1 - window) if window else 0
    for h in range(nh):
        kvh = h // (nh // nkv)
        kk = k[lo:pos + 1, kvh * hd:(kvh + 1) * hd]
        vv = v[lo:pos + 1, kvh * hd:(kvh + 1) * hd]
        s = kk @ q[h * hd:(h + 1) * hd] * scale
        p = np.exp(s - s.max())
        out[h] = (p / p.sum()) @ vv
    return out.reshape(-1)


def run_attention(kind, q, kc, vc, positions, items, table, page, n_pages, window, scale, out, nh, nkv, hd, status,
                  chunk=None):
    """kind: "general" (one warp per token and head) or "split" (key chunks + ordered combine)."""
    o = ops()
    if kind == "general":
        o.paged_attention(q, kc, vc, positions, items, table, page, n_pages, window, scale, out, nh, nkv, hd, status)
        return
    T = q.shape[0]
    upper = table.shape[1] * page
    if chunk is None:
        chunk, n_splits = o.split_plan(T, nkv, upper)
    else:
        n_splits = -(-upper // chunk)
    part_acc = torch.full((T * nh * n_splits * hd,), float("nan"), device=DEV)
    part_ml = torch.full((T * nh * n_splits * 2,), float("nan"), device=DEV)
    assert o.paged_attention_split(q, kc, vc, positions, items, table, page, n_pages, window, scale, out, part_acc, part_ml,
                                   chunk, n_splits, nh, nkv, hd, status, mma=kind.startswith("split_mma"),
                                   fresh=1 if kind == "split_mma_early" else 0)


# "split": the scalar split-key kernel; "split_mma": its tensor-core version where it applies
# (bfloat16, head 64 or 128), else the scalar one again
# "split_mma_early": the same, told that every cache row but a token's own was written before the
# launch's stream last synchronised (true here: the caches are copied to the device), so that it
# requests its first key tiles before waiting for the previous kernel
KINDS = [("general", None), ("split", None), ("split", 64), ("split", 512), ("split_mma", None), ("split_mma", 64),
         ("split_mma", 512), ("split_mma_early", None), ("split_mma_early", 64), ("split_mma_early", 128)]


# heads 144 and 192: in float32 a row has more vectors than a warp has lanes and not twice as many
@pytest.mark.parametrize("nh,nkv,hd", [(4, 2, 16), (6, 2, 32), (3, 1, 48), (5, 5, 64), (8, 2, 128), (2, 1, 256), (8, 1, 64),
                                       (2, 1, 192), (2, 1, 144), (4, 2, 240)])
@pytest.mark.parametrize("page,window", [(1, None), (4, None), (16, 13), (64, None), (8, 40)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("kind,chunk", KINDS)
def test_paged_attention(nh, nkv, hd, page, window, dtype, kind, chunk):
    o = ops()
    rng = np.random.default_rng(nh * 1000 + hd + page)
    lens = [70, 1, 33, 129]
    table, kc, vc, ks, vs, n_pages = make_paged(rng, lens, page, nkv, hd, dtype)
    # queries: a portion of request 0 (positions 50..69), the single token of request 1,
    # the last token of request 2, three scattered positions of request 3
    rows = [(0, p) for p in range(50, 70)] + [(1, 0), (2, 32)] + [(3, 0), (3, 64), (3, 128)]
    q = torch.from_numpy(rng.standard_normal((len(rows), nh * hd)).astype(np.float32)).to(dtype)
    out = torch.empty(len(rows), nh * hd, dtype=dtype, device=DEV)
    status = o.new_status(DEV)
    scale = 1 / math.sqrt(hd)
    run_attention(kind, q.to(DEV), kc.to(DEV), vc.to(DEV),
                  torch.tensor([p for _, p in rows], dtype=torch.int32, device=DEV),
                  torch.tensor([r for r, _ in rows], dtype=torch.int32, device=DEV),
                  torch.from_numpy(table).to(DEV), page, n_pages, window, scale, out, nh, nkv, hd, status, chunk)
    o.read_status(status)
    tol = 3e-6 if dtype == torch.float32 else 1e-2
    for i, (r, p) in enumerate(rows):
        ref = attention_reference(q[i].double().numpy(), ks[r].double().numpy(), vs[r].double().numpy(), p, nh, nkv, hd,
                                  scale, window)
        err = np.abs(out[i].float().cpu().double().numpy() - ref).max()
        assert err <= tol * max(1.0, np.abs(ref).max()), (r, p, err)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("far,window", [(3, None), (511, None), (512, None), (0, None), (700, 200), (701, 200), (899, 200),
                                        (63, None), (64, None), (127, None), (128, None)])
@pytest.mark.parametrize("kind,chunk", KINDS)
def test_one_far_key_stands_out(dtype, far, window, kind, chunk):
    _far_key(dtype, far, window, kind, chunk, 4, 2, 64)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("far,window", [(3, None), (512, None), (701, 200), (899, 200)])
@pytest.mark.parametrize("kind,chunk", [("general", None), ("split", None), ("split", 64)])
@pytest.mark.parametrize("nh,nkv,hd", [(2, 1, 192), (2, 1, 144), (3, 1, 208)])
def test_one_far_key_stands_out_wide_heads(dtype, far, window, kind, chunk, nh, nkv, hd):
    """Head sizes whose float32 rows have more 16-byte vectors than a warp has lanes, and not twice as many:
    every value dimension must reach the output (the far key's value is compared over the whole head)."""
    _far_key(dtype, far, window, kind, chunk, nh, nkv, hd)


def _far_key(dtype, far, window, kind, chunk, nh, nkv, hd):
    """Among 900 keys one is scaled so that its score dominates: the output must be that
    key's value (or must NOT be, when a window has passed it).  Random weights would hide
    a kernel that drops a far key, a page edge or a window edge."""
    o = ops()
    page = 16
    rng = np.random.default_rng(far)
    n = 900
    table, kc, vc, ks, vs, n_pages = make_paged(rng, [n], page, nkv, hd, dtype)
    q = torch.from_numpy(rng.standard_normal((1, nh * hd)).astype(np.float32))
    # key `far` of every kv head points along q of the group's first head, strongly
    for kvh in range(nkv):
        h = kvh * (nh // nkv)
        ks[0][far, kvh * hd:(kvh + 1) * hd] = (q[0, h * hd:(h + 1) * hd] * 12).to(dtype).float()
    kc = kc.clone()
    kc[table[0, far // page], far % page] = ks[0][far].to(dtype)
    out = torch.empty(1, nh * hd, dtype=dtype, device=DEV)
    status = o.new_status(DEV)
    run_attention(kind, q.to(dtype).to(DEV), kc.to(DEV), vc.to(DEV), torch.tensor([n - 1], dtype=torch.int32, device=DEV),
                  torch.zeros(1, dtype=torch.int32, device=DEV), torch.from_numpy(table).to(DEV), page, n_pages,
                  window, 1 / math.sqrt(hd), out, nh, nkv, hd, status, chunk)
    o.read_status(status)
    visible = window is None or far >= n - window
    for kvh in range(nkv):
        h = kvh * (nh // nkv)
        got = out[0, h * hd:(h + 1) * hd].float().cpu()
        target = vs[0][far, kvh * hd:(kvh + 1) * hd]
        close = (got - target).abs().max() < 0.05
        assert close == visible, (far, window, kvh)
    ref = attention_reference(q[0].to(dtype).double().numpy(), ks[0].double().numpy(), vs[0].double().numpy(), n - 1, nh, nkv,
                              hd, 1 / math.sqrt(hd), window)
    tol = 3e-6 if dtype == torch.float32 else 1e-2
    assert np.abs(out[0].float().cpu().double().numpy() - ref).max() <= tol * max(1.0, np.abs(ref).max())


@pytest.mark.parametrize("nh,nkv,hd,n_rot", [(4, 2, 16, 16), (6, 2, 32, 32), (3, 1, 48, 48), (2, 2, 64, 32), (1, 1, 256, 256),
                                             (4, 2, 64, 64), (3, 1, 128, 128), (5, 2, 128, 64), (6, 3, 96, 64)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("many", [False, True])
def test_qk_norm_rope_store(nh, nkv, hd, n_rot, dtype, many):
    o = ops()
    rng = np.random.default_rng(hd)
    page, n_pages, eps, theta = 4, 40 if not many else 120, 1e-6, 50000.0
    positions = np.array([0, 1, 2, 3, 4, 17, 900, 4095, 100000, 7], dtype=np.int32)
    items = np.array([0, 0, 0, 0, 0, 1, 2, 3, 4, 5], dtype=np.int32)
    if many:        # a prompt portion beside them: the launch then gives a warp several heads
        positions = np.concatenate([positions, np.arange(20, 320, dtype=np.int32)])
        items = np.concatenate([items, np.full(300, 5, dtype=np.int32)])
    T = len(positions)
    table = -np.ones((6, 100000 // page + 2), dtype=np.int32)
    perm = rng.permutation(n_pages)
    used = {}
    for t in range(T):
        key = (items[t], positions[t] // page)
        if key not in used:
            used[key] = perm[len(used)]
        table[key] = used[key]
    qkv = torch.from_numpy(rng.standard_normal((T, (nh + 2 * nkv) * hd)).astype(np.float32)).to(dtype)
    qw = torch.from_numpy(1 + 0.1 * rng.standard_normal(hd).astype(np.float32))
    kw = torch.from_numpy(1 + 0.1 * rng.standard_normal(hd).astype(np.float32))
    inv = (theta ** (-2.0 * np.arange(n_rot // 2) / n_rot)).astype(np.float32)
    q_out = torch.empty(T, nh * hd, dtype=dtype, device=DEV)
    kc = torch.zeros(n_pages, page, nkv * hd, dtype=dtype, device=DEV)
    vc = torch.zeros_like(kc)
    status = o.new_status(DEV)
    o.qk_norm_rope_store(qkv.to(DEV), torch.from_numpy(positions).to(DEV), torch.from_numpy(items).to(DEV), qw.to(DEV),
                         kw.to(DEV), torch.from_numpy(inv).to(DEV), n_rot, eps, q_out, kc, vc,
                         torch.from_numpy(table).to(DEV), page, n_pages, nh, nkv, hd, status)
    o.read_status(status)

    def ref_rows(x, w, pos):            # x [heads, hd] float64
        x = x * (1.0 / np.sqrt((x * x).mean(-1, keepdims=True) + eps)) * w
        ang = (np.float64(pos) * inv.astype(np.float64)).astype(np.float32).astype(np.float64)
        half = n_rot // 2
        out = x.copy()
        out[:, :half] = x[:, :half] * np.cos(ang) - x[:, half:n_rot] * np.sin(ang)
        out[:, half:n_rot] = x[:, :half] * np.sin(ang) + x[:, half:n_rot] * np.cos(ang)
        return out
    # float32 angles: position * inv_freq loses bits at large positions equally in both
    tol = 2e-5 if dtype == torch.float32 else 1e-2
    x = qkv.double().numpy()
    for t in range(T):
        qr = ref_rows(x[t, :nh * hd].reshape(nh, hd), qw.double().numpy(), positions[t]).reshape(-1)
        kr = ref_rows(x[t, nh * hd:(nh + nkv) * hd].reshape(nkv, hd), kw.double().numpy(), positions[t]).reshape(-1)
        vr = x[t, (nh + nkv) * hd:]
        pg, off = table[items[t], positions[t] // page], positions[t] % page
        assert np.abs(q_out[t].float().cpu().numpy() - qr).max() <= tol * np.abs(qr).max(), ("q", t)
        assert np.abs(kc[pg, off].float().cpu().numpy() - kr).max() <= tol * np.abs(kr).max(), ("k", t)
        assert np.abs(vc[pg, off].float().cpu().numpy() - vr).max() <= 1e-7, ("v", t)
    # a write to a page that is not mapped is refused and reported, not done
    table[0, 0] = -1
    o.qk_norm_rope_store(qkv.to(DEV), torch.from_numpy(positions).to(DEV), torch.from_numpy(items).to(DEV), qw.to(DEV),
                         kw.to(DEV), torch.from_numpy(inv).to(DEV), n_rot, eps, q_out, kc, vc,
                         torch.from_numpy(table).to(DEV), page, n_pages, nh, nkv, hd, status)
    with pytest.raises(o.KernelError, match="page"):
        o.read_status(status)


@pytest.mark.parametrize("splits", [2, 3, 6, 11])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_consumers_of_unfolded_products(splits, dtype):
    """gated_conv and qk_norm_rope_store on the split partials of a product give what they give on the
    folded tensor (sum in split order, rounded to the activations' dtype), bit for bit."""
    o = ops()
    g = torch.Generator().manual_seed(splits)
    # --- conv: lengths around taps - 1, a decode token among them
    H, taps, lens, slots = 40, 3, [1, 5, 2, 1], [2, 0, 3, 1]
    T = sum(lens)
    parts = torch.randn(splits, T, 3 * H, generator=g).to(DEV)
    folded = torch.zeros(T, 3 * H, device=DEV)
    for s_ in range(splits):
        folded += parts[s_]
    folded = folded.to(dtype)
    w = torch.randn(H, taps, generator=g).to(DEV)
    state0 = torch.randn(4, taps - 1, H, generator=g).to(DEV)
    row_start = torch.tensor(np.concatenate([[0], np.cumsum(lens)]).astype(np.int32), device=DEV)
    iot = torch.tensor(np.repeat(np.arange(len(lens)), lens).astype(np.int32), device=DEV)
    slot_t = torch.tensor(slots, dtype=torch.int32, device=DEV)
    status = o.new_status(DEV)
    outs = []
    for src in ("tensor", "parts"):
        y = torch.empty(T, H, dtype=dtype, device=DEV)
        st = state0.clone()
        bcx = folded if src == "tensor" else o.PartialProduct(parts.reshape(-1), splits, (T, 3 * H), torch.empty(T, 3 * H, dtype=dtype, device=DEV))
        o.gated_conv(bcx, w, None, st, row_start, iot, slot_t, y, taps, status)
        outs.append((y, st))
    o.read_status(status)
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])
    pp = o.PartialProduct(parts.reshape(-1), splits, (T, 3 * H), torch.empty(T, 3 * H, dtype=dtype, device=DEV))
    assert torch.equal(pp.tensor(), folded)                  # the fold kernel, for consumers that want a tensor
    # --- q/k norm, rotation, cache write
    nh, nkv, hd, page, n_pages = 3, 1, 32, 4, 8
    width = (nh + 2 * nkv) * hd
    parts = torch.randn(splits, T, width, generator=g).to(DEV)
    folded = torch.zeros(T, width, device=DEV)
    for s_ in range(splits):
        folded += parts[s_]
    folded = folded.to(dtype)
    positions = torch.arange(T, dtype=torch.int32, device=DEV)
    items = torch.zeros(T, dtype=torch.int32, device=DEV)
    table = torch.arange(n_pages, dtype=torch.int32, device=DEV).flip(0).reshape(1, n_pages).contiguous()
    qw = (1 + 0.1 * torch.randn(hd, generator=g)).to(DEV)
    kw = (1 + 0.1 * torch.randn(hd, generator=g)).to(DEV)
    inv = torch.tensor((10000.0 ** (-2.0 * np.arange(hd // 2) / hd)).astype(np.float32), device=DEV)
    res = []
    for src in ("tensor", "parts"):
        q_out = torch.empty(T, nh * hd, dtype=dtype, device=DEV)
        kc = torch.zeros(n_pages, page, nkv * hd, dtype=dtype, device=DEV)
        vc = torch.zeros_like(kc)
        qkv = folded if src == "tensor" else o.PartialProduct(parts.reshape(-1), splits, (T, width), torch.empty(T, width, dtype=dtype, device=DEV))
        o.qk_norm_rope_store(qkv, positions, items, qw, kw, inv, hd, 1e-5, q_out, kc, vc, table, page, n_pages, nh, nkv, hd, status)
        res.append((q_out, kc, vc))
    o.read_status(status)
    for a, b in zip(res[0], res[1]):
        assert torch.equal(a, b)


@pytest.mark.parametrize("T,N,K", [(8, 6144, 2048), (3, 3072, 2048), (16, 384, 512), (5, 200, 136)])
def test_linear_unfolded_sums_to_the_product(T, N, K):
    o = ops()
    g = torch.Generator().manual_seed(N + T)
    x = bf16_round(torch.randn(T, K, generator=g))
    w = bf16_round(torch.randn(N, K, generator=g) * 0.05)
    out = torch.empty(T, N, dtype=torch.bfloat16, device=DEV)
    status = o.new_status(DEV)
    r = o.linear_unfolded(x.to(torch.bfloat16).to(DEV), w.to(torch.bfloat16).to(DEV), out, status)
    o.read_status(status)
    if N >= 3072:
        assert isinstance(r, o.PartialProduct) and r.splits > 1        # the decode products of the model's sizes are cut
    got = (r.tensor() if isinstance(r, o.PartialProduct) else r).float().cpu().double()
    ref = x.double() @ w.double().T
    assert (got - ref).abs().max() <= 8e-3 * max(1.0, ref.abs().max())


def test_kernels_refuse_sizes_they_do_not_take():
    o = ops()
    st = o.new_status(DEV)
    z = lambda *s, dt=torch.float32: torch.zeros(*s, dtype=dt, device=DEV)
    zi = lambda *s: torch.zeros(*s, dtype=torch.int32, device=DEV)
    with pytest.raises(o.KernelError, match="head size"):
        o.paged_attention(z(1, 24), z(2, 4, 24), z(2, 4, 24), zi(1), zi(1), zi(1, 4), 4, 2, None, 1.0, z(1, 24), 1, 1, 24, st)
    with pytest.raises(o.KernelError, match="head size"):
        o.paged_attention(z(1, 512), z(2, 4, 512), z(2, 4, 512), zi(1), zi(1), zi(1, 4), 4, 2, None, 1.0, z(1, 512), 1, 1, 512, st)
    with pytest.raises(o.KernelError, match="taps"):
        o.gated_conv(z(1, 24), z(8, 17), None, z(1, 16, 8), zi(2), zi(1), zi(1), z(1, 8), 17, st)
    with pytest.raises(o.KernelError):
        o.rmsnorm(torch.zeros(2, 8), torch.zeros(8), 1e-5, torch.zeros(2, 8))      # CPU tensors: no CPU path
    # split-key attention: more key chunks than the combine kernel holds, or chunks that do not cover the
    # table, are refused by the launcher and by both entry points, before anything is launched
    q, kv, tab = z(1, 16), z(2, 16, 16), zi(1, 4096)
    with pytest.raises(o.KernelError, match="key chunks"):
        o.paged_attention_split(q, kv, kv, zi(1), zi(1), tab, 16, 2, None, 1.0, z(1, 16), z(16 * 4096), z(2 * 4096), 32, 4096,
                                1, 1, 16, st)
    with pytest.raises(o.KernelError, match="cover"):
        o.paged_attention_split(q, kv, kv, zi(1), zi(1), tab, 16, 2, None, 1.0, z(1, 16), z(16 * 8), z(2 * 8), 64, 8, 1, 1, 16, st)
    k = o._lib.kernels()
    stream = torch.cuda.current_stream().cuda_stream
    p = lambda t: t.data_ptr()
    assert k.imparo_paged_attention_split(p(q), p(kv), p(kv), 0, p(zi(1)), p(zi(1)), p(tab), 4096, 16, 2, 0, 1.0, p(z(1, 16)),
                                          p(z(16 * 4096)), p(z(2 * 4096)), 1, 1, 1, 16, 32, 4096, p(st), stream) == -2
    qb, kvb = z(1, 64, dt=torch.bfloat16), z(2, 16, 64, dt=torch.bfloat16)
    assert k.imparo_attention_decode_mma(p(qb), p(kvb), p(kvb), p(zi(1)), p(zi(1)), p(tab), 4096, 16, 2, 0, 1.0,
                                         p(z(1, 64, dt=torch.bfloat16)), p(z(64 * 4096)), p(z(2 * 4096)), 1, 1, 1, 64, 64, 4096, 0, 0,
                                         p(st), stream) == -2
    torch.cuda.synchronize()
    o.read_status(st)
    # the plan never asks for more chunks than that: very wide tables get longer chunks
    chunk, n = o.split_plan(1, 1, 3_000_000)
    assert n <= o.MAX_SPLITS and chunk * n >= 3_000_000


# ---------------------------------------------------------------------------------------
def test_greedy_pick_smallest_index_and_nan():
    o = ops()
    V = 70001
    logits = torch.full((4, V), -1.0)
    logits[0, 500] = 3.0; logits[0, 69999] = 3.0; logits[0, 123] = 3.0
    logits[1, :] = float("nan"); logits[1, 77] = -5.0
    logits[2, :] = float("nan")
    logits[3, V - 1] = 9.0
    out = torch.empty(4, dtype=torch.int32, device=DEV)
    o.sample_rows(logits.to(DEV), None, None, out)
    assert out.tolist() == [123, 77, 0, V - 1]


def test_temperature_sampling_skips_nan_and_empty_stretches():
    """Large vocabulary (the two-stage kernels): whole stretches of -inf or NaN carry no weight, a row of NaN gives 0,
    a row with one finite entry gives that entry whatever the uniform number."""
    o = ops()
    V = 70001
    logits = torch.full((5, V), float("-inf"))
    logits[0, 40000] = 1.0; logits[0, 40001] = 1.0                      # two equal entries: u picks between them
    logits[1, :] = float("nan"); logits[1, 69000] = -3.0
    logits[2, :] = float("nan")
    logits[3, :] = float("nan"); logits[3, 5] = 0.0; logits[3, V - 1] = 0.0
    logits[4, 123] = 2.0                                                # greedy row among sampled ones
    temps = torch.tensor([0.7, 1.0, 1.0, 2.0, 0.0])
    for us, want in (([0.25, 0.5, 0.5, 0.25, 0.9], [40000, 69000, 0, 5, 123]),
                     ([0.75, 0.0, 0.99, 0.75, 0.1], [40001, 69000, 0, V - 1, 123])):
        out = torch.empty(5, dtype=torch.int32, device=DEV)
        o.sample_rows(logits.to(DEV), temps.to(DEV), torch.tensor(us).to(DEV), out)
        assert out.tolist() == want


@pytest.mark.parametrize("V", [331, 65536, 70001])
def test_temperature_sampling_is_the_inverse_cdf(V):
    o = ops()
    rng = np.random.default_rng(V)
    n = 64
    logits = (rng.standard_normal((n, V)) * 3).astype(np.float32)
    temps = rng.choice([0.0, 0.5, 0.8, 1.3], size=n).astype(np.float32)
    us = rng.random(n).astype(np.float32)
    out = torch.empty(n, dtype=torch.int32, device=DEV)
    o.sample_rows(torch.from_numpy(logits).to(DEV), torch.from_numpy(temps).to(DEV), torch.from_numpy(us).to(DEV), out)
    got = out.tolist()
    for r in range(n):
        if temps[r] == 0:
            assert got[r] == int(np.argmax(logits[r]))
            continue
        p = np.exp((logits[r].astype(np.float64) - logits[r].max()) / temps[r])
        cdf = np.cumsum(p) / p.sum()
        want = int(np.searchsorted(cdf, us[r], side="right"))
        if got[r] != want:
            # only a target that sits within rounding of a boundary may fall either side
            edge = min(abs(cdf[min(got[r], want)] - us[r]), abs(cdf[max(got[r], want) - 1] - us[r]))
            assert abs(got[r] - want) == 1 and edge < 1e-5, (r, got[r], want)
    # the picks follow the distribution: a row sampled many times
    row = np.array([0.0, 1.0, 2.0, -1.0] + [-30.0] * (V - 4), dtype=np.float32)
    m = 4000
    us = ((np.arange(m) + 0.5) / m).astype(np.float32)
    out = torch.empty(m, dtype=torch.int32, device=DEV)
    o.sample_rows(torch.from_numpy(np.tile(row, (m, 1))).to(DEV), torch.full((m,), 1.0, device=DEV),
                  torch.from_numpy(us).to(DEV), out)
    freq = np.bincount(out.cpu().numpy(), minlength=4)[:4] / m
    p = np.exp(row[:4].astype(np.float64)); p /= np.exp(row.astype(np.float64)).sum()
    assert np.abs(freq - p).max() < 2e-3


@pytest.mark.parametrize("nh,nkv,hd", [(8, 2, 64), (4, 4, 64), (6, 2, 128), (3, 1, 64), (8, 1, 64), (2, 1, 128), (32, 8, 64), (4, 2, 64),
                                       (5, 1, 64), (6, 1, 128), (7, 1, 64)])
@pytest.mark.parametrize("page,window", [(4, None), (16, None), (16, 50), (64, 7), (32, 200), (128, None)])
@pytest.mark.parametrize("kernel", ["mma", "tcgen05", "tcgen05_one_tile"])
def test_attention_prefill_tensor_cores(nh, nkv, hd, page, window, kernel):
    """Prompt portions of several requests in one launch: a long portion that starts in the
    middle of its request, a single token, a whole short prompt, a short tail, and one long enough
    for several key steps with a window's edge inside them."""
    o = ops()
    dtype = torch.bfloat16
    rng = np.random.default_rng(nh * 100 + hd + page)
    portions = [(37, 130), (0, 1), (0, 70), (200, 9), (115, 300)]            # (start position, tokens)
    lens = [s + n for s, n in portions]
    table, kc, vc, ks, vs, n_pages = make_paged(rng, lens, page, nkv, hd, dtype)
    T = sum(n for _, n in portions)
    q = torch.from_numpy(rng.standard_normal((T, nh * hd)).astype(np.float32)).to(dtype)
    row_start = np.concatenate([[0], np.cumsum([n for _, n in portions])]).astype(np.int32)
    start_pos = np.array([s for s, _ in portions], dtype=np.int32)
    out = torch.full((T, nh * hd), float("nan"), dtype=dtype, device=DEV)
    status = o.new_status(DEV)
    scale = 1 / math.sqrt(hd)
    took = o.attention_prefill(q.to(DEV), kc.to(DEV), vc.to(DEV), torch.from_numpy(row_start).to(DEV),
                               torch.from_numpy(start_pos).to(DEV), len(portions), torch.from_numpy(table).to(DEV), page, n_pages,
                               window, scale, out, nh, nkv, hd, status, kernel=kernel)
    assert took == (kernel == "mma" or page >= 16)           # the tcgen05 kernel declines pages below 16 positions
    if not took:
        return
    o.read_status(status)
    got = out.float().cpu().double().numpy()
    assert np.isfinite(got).all()
    t = 0
    for r, (s, n) in enumerate(portions):
        for i in range(n):
            ref = attention_reference(q[t].double().numpy(), ks[r].double().numpy(), vs[r].double().numpy(), s + i, nh, nkv, hd,
                                      scale, window)
            err = np.abs(got[t] - ref).max()
            assert err <= 1.5e-2 * max(1.0, np.abs(ref).max()), (r, s + i, err)
            t += 1


@pytest.mark.parametrize("nh,nkv", [(6, 2), (8, 2), (5, 1)])
@pytest.mark.parametrize("start,n", [(3180, 488), (2017, 130), (1, 260)])
def test_attention_prefill_portion_far_into_its_request(nh, nkv, start, n):
    """A portion that starts thousands of keys in: the two query tiles of a CTA walk dozens of key steps in turn, and
    where the second tile's last position lies in a further block of 128 keys than the first's it has a step more.
    Launched repeatedly (the tiles' hand-over is a matter of timing), every launch must give the same rows, and those
    the reference's."""
    o = ops()
    hd, page, dtype = 64, 16, torch.bfloat16
    rng = np.random.default_rng(start + nh)
    table, kc, vc, ks, vs, n_pages = make_paged(rng, [start + n], page, nkv, hd, dtype)
    q = torch.from_numpy(rng.standard_normal((n, nh * hd)).astype(np.float32)).to(dtype)
    status = o.new_status(DEV)
    scale = 1 / math.sqrt(hd)
    args = (q.to(DEV), kc.to(DEV), vc.to(DEV), torch.tensor([0, n], dtype=torch.int32, device=DEV),
            torch.tensor([start], dtype=torch.int32, device=DEV), 1, torch.from_numpy(table).to(DEV), page, n_pages, None, scale)
    first = None
    for rep in range(30):
        out = torch.full((n, nh * hd), float("nan"), dtype=dtype, device=DEV)
        assert o.attention_prefill(*args, out, nh, nkv, hd, status, kernel="tcgen05")
        torch.cuda.synchronize()
        o.read_status(status)
        if first is None:
            first = out
        else:
            assert torch.equal(out, first), rep
    got = first.float().cpu().double().numpy()
    kd, vd = ks[0].double().numpy(), vs[0].double().numpy()
    for i in list(range(0, n, 37)) + [n - 1]:
        ref = attention_reference(q[i].double().numpy(), kd, vd, start + i, nh, nkv, hd, scale, None)
        err = np.abs(got[i] - ref).max()
        assert err <= 1.5e-2 * max(1.0, np.abs(ref).max()), (i, err)


@pytest.mark.parametrize("nh,nkv,hd", [(8, 2, 64), (6, 2, 64), (4, 2, 128)])
@pytest.mark.parametrize("kernel", ["tcgen05", "tcgen05_one_tile"])
def test_portion_attention_and_decode_row_attention_side_by_side(nh, nkv, hd, kernel):
    """A step's prompt portions go to the prompt kernel and its decode rows to the split-key kernel, which may run
    beside it: the first lets its dependents come after its own wait, the second does not wait at its start and
    completes after the first.  The pair, launched many times in a row behind a kernel that writes their queries, gives
    what the two give when each waits for the one before."""
    o = ops()
    dtype, page, window = torch.bfloat16, 16, None
    rng = np.random.default_rng(nh + hd)
    singles = [700, 33, 1, 520]                                   # decode rows: a request's last position + 1
    portions = [(300, 140), (0, 90)]                              # (start position, tokens)
    lens = singles + [s + n for s, n in portions]
    table, kc, vc, ks, vs, n_pages = make_paged(rng, lens, page, nkv, hd, dtype)
    n1, T = len(singles), len(singles) + sum(n for _, n in portions)
    q_host = torch.from_numpy(rng.standard_normal((T, nh * hd)).astype(np.float32)).to(dtype)
    positions = torch.tensor([L - 1 for L in singles], dtype=torch.int32, device=DEV)
    items = torch.arange(n1, dtype=torch.int32, device=DEV)
    row_start = torch.from_numpy(np.concatenate([[n1], n1 + np.cumsum([n for _, n in portions])]).astype(np.int32)).to(DEV)
    start_pos = torch.tensor([s for s, _ in portions], dtype=torch.int32, device=DEV)
    table_d, kc_d, vc_d = torch.from_numpy(table).to(DEV), kc.to(DEV), vc.to(DEV)
    scale = 1 / math.sqrt(hd)
    chunk, n_splits = 64, -(-table.shape[1] * page // 64)
    part_acc = torch.empty(n1 * nh * n_splits * hd, device=DEV)
    part_ml = torch.empty(n1 * nh * n_splits * 2, device=DEV)
    status = o.new_status(DEV)
    src = q_host.to(DEV)
    q = torch.empty_like(src)

    def pair(side_by_side, out):
        q.copy_(src)                                              # the kernel before the pair writes what both read
        took = o.attention_prefill(q, kc_d, vc_d, row_start, start_pos, len(portions), table_d[n1:], page, n_pages, window,
                                   scale, out, nh, nkv, hd, status, kernel=kernel, dependents_after_wait=side_by_side)
        assert took == (2 if side_by_side else True)
        assert o.paged_attention_split(q[:n1], kc_d, vc_d, positions, items, table_d, page, n_pages, window, scale, out[:n1],
                                       part_acc, part_ml, chunk, n_splits, nh, nkv, hd, status, fresh=1,
                                       overlap_prev=side_by_side)

    want = torch.full((T, nh * hd), float("nan"), dtype=dtype, device=DEV)
    pair(False, want)
    torch.cuda.synchronize()
    for _ in range(20):
        got = torch.full((T, nh * hd), float("nan"), dtype=dtype, device=DEV)
        pair(True, got)
        o.linear(got, torch.eye(nh * hd, dtype=dtype, device=DEV)[:8].contiguous(),
                 torch.empty(T, 8, dtype=dtype, device=DEV))      # a kernel behind the pair that reads all its rows
        torch.cuda.synchronize()
        assert torch.equal(got, want)
    o.read_status(status)
    ref = attention_reference(q_host[0].double().numpy(), ks[0].double().numpy(), vs[0].double().numpy(), singles[0] - 1, nh, nkv,
                              hd, scale, window)
    assert np.abs(want[0].float().cpu().double().numpy() - ref).max() <= 1.5e-2 * max(1.0, np.abs(ref).max())


@pytest.mark.parametrize("kernel", ["mma", "tcgen05", "tcgen05_one_tile"])
def test_attention_prefill_far_key_and_refusals(kernel):
    o = ops()
    nh, nkv, hd, page, n = 8, 2, 64, 16, 900
    rng = np.random.default_rng(5)
    for far in (0, 63, 64, 127, 128, 511, 512, 700, 899):
        table, kc, vc, ks, vs, n_pages = make_paged(rng, [n], page, nkv, hd, torch.bfloat16)
        q = torch.from_numpy(rng.standard_normal((n, nh * hd)).astype(np.float32)).to(torch.bfloat16)
        for kvh in range(nkv):
            h = kvh * (nh // nkv)
            ks[0][far, kvh * hd:(kvh + 1) * hd] = (q[n - 1, h * hd:(h + 1) * hd].float() * 12).to(torch.bfloat16).float()
        kc = kc.clone()
        kc[table[0, far // page], far % page] = ks[0][far].to(torch.bfloat16)
        out = torch.empty(n, nh * hd, dtype=torch.bfloat16, device=DEV)
        status = o.new_status(DEV)
        assert o.attention_prefill(q.to(DEV), kc.to(DEV), vc.to(DEV), torch.tensor([0, n], dtype=torch.int32, device=DEV),
                                   torch.zeros(1, dtype=torch.int32, device=DEV), 1, torch.from_numpy(table).to(DEV), page,
                                   n_pages, None, 1 / math.sqrt(hd), out, nh, nkv, hd, status, kernel=kernel)
        o.read_status(status)
        for kvh in range(nkv):
            h = kvh * (nh // nkv)
            got = out[n - 1, h * hd:(h + 1) * hd].float().cpu()
            assert (got - vs[0][far, kvh * hd:(kvh + 1) * hd]).abs().max() < 0.05, (far, kvh)
    # shapes the tensor-core kernel does not take are declined, not computed wrongly
    z = torch.zeros(4, 48, dtype=torch.bfloat16, device=DEV)
    assert not o.attention_prefill(z, z, z, None, None, 1, None, 4, 1, None, 1.0, z, 1, 1, 48, None)
    zf = torch.zeros(4, 64, device=DEV)
    assert not o.attention_prefill(zf, zf, zf, None, None, 1, None, 4, 1, None, 1.0, zf, 1, 1, 64, None)


@pytest.mark.parametrize("sized", [True, False])
def test_zero_state_slots_clears_the_named_slots_only(sized):
    """State tensors of very different sizes in one arena (5, 3,072 and 70,000 floats per slot: less than a block's
    share, a few blocks, more than the grid's 64 blocks cover in one pass), a padded list of fresh slots; with the
    largest per-slot size given (the engine's call) and without."""
    o = ops()
    slots_total, pers = 6, [5, 3072, 70000]
    segs, off = [], 0
    for per in pers:
        segs.append((off, per))
        off += slots_total * ((per + 3) // 4 * 4)
    arena = torch.ones(off, device=DEV)
    fresh = torch.tensor([1, -1, 4, -1], dtype=torch.int32, device=DEV)
    st = o.new_status(DEV)
    o.zero_state_slots(arena, torch.tensor(segs, dtype=torch.int64, device=DEV), len(segs), fresh, slots_total, st,
                       max_per_slot=max(pers) if sized else None)
    torch.cuda.synchronize()
    o.read_status(st)
    host = arena.cpu().numpy()
    for (start, per) in segs:
        for slot in range(slots_total):
            got = host[start + slot * per:start + (slot + 1) * per]
            assert (got == (0.0 if slot in (1, 4) else 1.0)).all(), (per, slot)


@pytest.mark.parametrize("n,n_prev", [(1, 1), (37, 8), (700, 64)])
def test_take_sampled_tokens(n, n_prev):
    """token_ids[i] = prev[src[i]] where src[i] >= 0; other rows keep what the host wrote."""
    from imparo_b200.kernels import ops as o
    rng = np.random.default_rng(n)
    ids = rng.integers(0, 60000, n).astype(np.int32)
    prev = rng.integers(0, 60000, n_prev).astype(np.int32)
    src = np.where(rng.random(n) < 0.5, rng.integers(0, n_prev, n), -1).astype(np.int32)
    d_ids = torch.from_numpy(ids).to(DEV)
    o.take_sampled_tokens(d_ids, torch.from_numpy(src).to(DEV), torch.from_numpy(prev).to(DEV))
    want = np.where(src >= 0, prev[np.clip(src, 0, None)], ids)
    assert np.array_equal(d_ids.cpu().numpy(), want)


# ---------------------------------------------------------------------------------------
# failure paths that hang and fault nothing
def test_a_bounded_wait_that_runs_out_reports_and_returns():
    """Every device wait has a poll limit.  A kernel waits on a barrier nothing completes: it must give up,
    record the wait-limit code in the status word and run to its end; the context stays usable."""
    o = ops()
    status = o.new_status(DEV)
    assert o.selftest_wait_limit(status, limit=2000) == 2
    with pytest.raises(o.KernelError, match="bounded device wait"):
        o.read_status(status)
    o.read_status(status)                                    # cleared by the read; later work runs
    x = torch.ones(2, 8, device=DEV)
    out = torch.empty(2, 8, device=DEV)
    o.rmsnorm(x, torch.ones(8, device=DEV), 1e-5, out)
    torch.cuda.synchronize()
    assert torch.allclose(out, torch.ones(2, 8, device=DEV), atol=1e-4)


@pytest.mark.parametrize("bad_slot", [5, -1, 1 << 20])
def test_gated_conv_reports_a_state_slot_out_of_range(bad_slot):
    """A slot index outside the state arena is reported through the status word; the request's state and
    output are not touched, the other requests' are computed."""
    o = ops()
    H, taps, n_slots, lens = 24, 3, 5, [1, 4, 1]
    g = torch.Generator().manual_seed(1)
    T = sum(lens)
    bcx = torch.randn(T, 3 * H, generator=g).to(DEV)
    w = torch.randn(H, taps, generator=g).to(DEV)
    state = torch.randn(n_slots, taps - 1, H, generator=g).to(DEV)
    before = state.clone()
    row_start = torch.tensor([0, 1, 5, 6], dtype=torch.int32, device=DEV)
    iot = torch.tensor([0, 1, 1, 1, 1, 2], dtype=torch.int32, device=DEV)
    slots = torch.tensor([2, bad_slot, 0], dtype=torch.int32, device=DEV)
    y = torch.full((T, H), 7.0, device=DEV)
    status = o.new_status(DEV)
    o.gated_conv(bcx, w, None, state, row_start, iot, slots, y, taps, status)
    with pytest.raises(o.KernelError, match="state slot"):
        o.read_status(status)
    assert torch.equal(state[[1, 3, 4]], before[[1, 3, 4]])          # untouched slots
    assert not torch.equal(state[2], before[2]) and not torch.equal(state[0], before[0])
    assert torch.equal(y[1:2], torch.full((1, H), 7.0, device=DEV))   # the bad request's first row was not written


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_cache_rows_are_addressed_as_the_reference_addresses_them(dtype):
    """tests/golden/kv_paging_golden.json: physical cache rows from the reference's own physical_row
    (imparo-cuda/native/kv_paging.cuh:25-30) for shuffled block tables, page size 64.  The store kernel must put a
    token's value row exactly there, and the attention kernels must find it there."""
    o = ops()
    with open(os.path.join(HERE, "golden", "kv_paging_golden.json")) as f:
        cases = json.load(f)["cases"]
    nh = nkv = 1
    hd = 64
    for c in cases:
        page, table = c["page"], np.array([c["table"]], dtype=np.int32)
        n_pages = table.shape[1]
        seen, logical, physical = set(), [], []
        for l, p in zip(c["logical"], c["physical"]):
            if l not in seen:
                seen.add(l); logical.append(l); physical.append(p)
        T = len(logical)
        qkv = torch.zeros(T, 3 * hd)
        qkv[:, :2 * hd] = 1.0
        for t in range(T):
            qkv[t, 2 * hd:] = float(t + 1)                        # the value row names its token
        kc = torch.zeros(n_pages, page, hd, dtype=dtype, device=DEV)
        vc = torch.zeros_like(kc)
        q_out = torch.empty(T, hd, dtype=dtype, device=DEV)
        status = o.new_status(DEV)
        ones = torch.ones(hd, device=DEV)
        o.qk_norm_rope_store(qkv.to(dtype).to(DEV), torch.tensor(logical, dtype=torch.int32, device=DEV),
                             torch.zeros(T, dtype=torch.int32, device=DEV), ones, ones, None, 0, 1e-6, q_out, kc, vc,
                             torch.from_numpy(table).to(DEV), page, n_pages, nh, nkv, hd, status)
        o.read_status(status)
        rows = vc.view(n_pages * page, hd).float().cpu()
        want = torch.zeros(n_pages * page)
        for t, p in enumerate(physical):
            want[p] = t + 1
        assert torch.equal(rows[:, 0], want) and torch.equal(rows[:, hd - 1], want)
        # reading: a query at the last position of the table, every stored key scores alike except one that is
        # scaled up; the output must be that token's value
        star = T // 2
        kc.view(n_pages * page, hd)[physical[star]] *= 30.0
        pos = n_pages * page - 1
        for kind in ("general", "split", "split_mma"):
            out = torch.empty(1, hd, dtype=dtype, device=DEV)
            run_attention(kind, torch.ones(1, hd, dtype=dtype, device=DEV), kc, vc, torch.tensor([pos], dtype=torch.int32, device=DEV),
                          torch.zeros(1, dtype=torch.int32, device=DEV), torch.from_numpy(table).to(DEV), page, n_pages, None,
                          1 / math.sqrt(hd), out, nh, nkv, hd, status)
            o.read_status(status)
            assert abs(float(out[0, 0]) - (star + 1)) < 0.05 * (star + 1), (kind, float(out[0, 0]), star + 1)


# ---------------------------------------------------------------------------------------
# the attention's output product that makes its own token operand (decode rows)
@pytest.mark.parametrize("T,nh,nkv,hd,N,ctx", [(8, 32, 8, 64, 2048, 2100), (1, 4, 2, 64, 256, 300), (16, 6, 2, 128, 512, 700),
                                                (3, 8, 8, 64, 384, 9000), (20, 4, 2, 64, 256, 150)])
@pytest.mark.parametrize("deferred", [False, True])
def test_output_product_with_the_attention_combine_inside(T, nh, nkv, hd, N, ctx, deferred):
    """The split-key attention leaves its partial results (out=None) and linear_of_attention_partials combines them
    inside the output product; against the combine kernel followed by linear."""
    o = ops()
    rng = np.random.default_rng(T + hd)
    page = 16
    lens = [int(x) for x in rng.integers(max(1, ctx // 3), ctx, T)]
    table, kc, vc, ks, vs, n_pages = make_paged(rng, lens, page, nkv, hd, torch.bfloat16)
    q = torch.from_numpy(rng.standard_normal((T, nh * hd)).astype(np.float32)).bfloat16().to(DEV)
    positions = torch.tensor([n - 1 for n in lens], dtype=torch.int32, device=DEV)
    items = torch.arange(T, dtype=torch.int32, device=DEV)
    tab = torch.from_numpy(table).to(DEV)
    kc, vc = kc.to(DEV), vc.to(DEV)
    w_o = torch.from_numpy((rng.standard_normal((N, nh * hd)) * 0.05).astype(np.float32)).bfloat16().to(DEV)
    base = torch.from_numpy(rng.standard_normal((T, N)).astype(np.float32)).to(DEV)
    chunk, n_splits = o.split_plan(T, nkv, tab.shape[1] * page)
    status = o.new_status(DEV)
    scale = 1 / math.sqrt(hd)
    outs = []
    for fused in (False, True):
        part_acc = torch.full((T * nh * n_splits * hd,), float("nan"), device=DEV)
        part_ml = torch.full((T * nh * n_splits * 2,), float("nan"), device=DEV)
        out = base.clone()
        if fused:
            assert o.paged_attention_split(q, kc, vc, positions, items, tab, page, n_pages, None, scale, None, part_acc, part_ml,
                                           chunk, n_splits, nh, nkv, hd, status)
            if deferred:
                o.allow_deferred_add(out)
            took = o.linear_of_attention_partials(part_acc, part_ml, T, nh, hd, n_splits, w_o, out, status)
            o.disallow_deferred_add(out)
            assert took == (T <= 16 and n_splits <= 64)
            if not took:
                return
            o.settle(out)
        else:
            att = torch.empty(T, nh * hd, dtype=torch.bfloat16, device=DEV)
            assert o.paged_attention_split(q, kc, vc, positions, items, tab, page, n_pages, None, scale, att, part_acc, part_ml,
                                           chunk, n_splits, nh, nkv, hd, status)
            o.linear(att, w_o, out, accumulate=True, status=status)
        outs.append(out)
    torch.cuda.synchronize()
    o.read_status(status)
    s_ = float(outs[0].abs().max())
    assert float((outs[0] - outs[1]).abs().max()) <= 2e-6 * s_
    ref = np.stack([attention_reference(q[t].double().cpu().numpy(), ks[t].double().numpy(), vs[t].double().numpy(), lens[t] - 1,
                                        nh, nkv, hd, scale, None) for t in range(T)])
    want = base.double().cpu().numpy() + ref @ w_o.double().cpu().numpy().T
    assert np.abs(outs[1].double().cpu().numpy() - want).max() <= 2e-2 * np.abs(want).max()


# ---------------------------------------------------------------------------------------
# the persistent tile product for prompt-sized batches (gemm_prefill.cu)
@pytest.mark.parametrize("T,N,K", [(128, 256, 64), (300, 520, 136), (129, 264, 72), (1000, 768, 1024), (2048, 2048, 2048), (257, 8, 8)])
@pytest.mark.parametrize("epi", ["store_bf16", "store_f32", "add_f32", "swiglu"])
def test_prefill_product_against_float64(T, N, K, epi):
    """Tokens, rows and depth that are no multiples of the tile (128 x 256 x 64), several tiles per CTA (the second
    accumulator in tensor memory, the ring running on across tiles), every epilogue; against float64 on the same
    bfloat16 inputs."""
    o = ops()
    g = torch.Generator().manual_seed(T + N + K)
    x = (torch.randn(T, K, generator=g) * 0.5).bfloat16()
    rows = 2 * N if epi == "swiglu" else N
    w = (torch.randn(rows, K, generator=g) * 0.1).bfloat16()
    xd, wd = x.double(), w.double()
    status = o.new_status(DEV)
    if epi == "swiglu":
        out = torch.full((T, N), float("nan"), dtype=torch.bfloat16, device=DEV)
        o.gemm_prefill(x.to(DEV), w.to(DEV), out, o.EPI_SWIGLU, status)
        gate, up = xd @ wd[:N].T, xd @ wd[N:].T
        ref = gate / (1 + torch.exp(-gate)) * up
        tol = 1e-2
    elif epi == "add_f32":
        base = torch.randn(T, N, generator=g)
        out = base.clone().to(DEV)
        o.gemm_prefill(x.to(DEV), w.to(DEV), out, o.EPI_ADD_F32, status)
        ref = base.double() + xd @ wd.T
        tol = 1e-5                              # 32-bit accumulation over up to 2,048 products
    else:
        dt = torch.bfloat16 if epi == "store_bf16" else torch.float32
        out = torch.full((T, N), float("nan"), dtype=dt, device=DEV)
        o.gemm_prefill(x.to(DEV), w.to(DEV), out, o.EPI_STORE_BF16 if epi == "store_bf16" else o.EPI_STORE_F32, status)
        ref = xd @ wd.T
        tol = 1e-2 if epi == "store_bf16" else 1e-5
    torch.cuda.synchronize()
    o.read_status(status)
    err = float((out.double().cpu() - ref).abs().max())
    assert err <= tol * max(1.0, float(ref.abs().max())), err


def test_prefill_product_refuses_what_it_cannot_address():
    o = ops()
    z = lambda *s, dt=torch.bfloat16: torch.zeros(*s, dtype=dt, device=DEV)
    with pytest.raises(o.KernelError, match="refused"):
        o.gemm_prefill(z(256, 12), z(64, 12), z(256, 64), o.EPI_STORE_BF16)            # K no multiple of 8: rows not 16 bytes
    with pytest.raises(o.KernelError, match="refused"):
        o.gemm_prefill(z(256, 16), z(12, 16), z(256, 12), o.EPI_STORE_BF16)            # N no multiple of 8
    assert not o.prefill_tc_usable(z(256, 12), z(64, 12), z(256, 64))
    assert not o.prefill_tc_usable(z(100, 16), z(64, 16), z(100, 64))                 # too few tokens for this kernel
    assert o.prefill_tc_usable(z(256, 16), z(64, 16), z(256, 64))


@pytest.mark.parametrize("nh,nkv,hd,n_rot", [(8, 2, 64, 64), (6, 6, 64, 32), (16, 2, 128, 128), (3, 1, 64, 64), (8, 2, 128, 0)])
@pytest.mark.parametrize("page,window,qk_norm", [(16, None, True), (4, 37, True), (64, None, False)])
def test_decode_attention_from_the_qkv_partials(nh, nkv, hd, n_rot, page, window, qk_norm):
    """Decode rows straight from the qkv product's split partials: the kernel makes its queries and the new key and
    value rows itself.  It must leave the same cache rows and the same outputs as the q/k kernel followed by the
    split-key attention (the same arithmetic in the same order), and both must agree with the float64 reference.
    Requests stand at a page's first and last row, at position 0, inside and beyond a window."""
    o = ops()
    dtype = torch.bfloat16
    rng = np.random.default_rng(nh * 7 + hd + page)
    pos = [0, page - 1, page, 5 * page + 3, 130, 259]                 # each request's new position = tokens it holds
    lens = [p + 1 for p in pos]
    T = len(pos)
    table, kc, vc, ks, vs, n_pages = make_paged(rng, lens, page, nkv, hd, dtype)
    width = (nh + 2 * nkv) * hd
    splits = 3
    parts = torch.from_numpy(rng.standard_normal((splits, T, width)).astype(np.float32) * 0.6).to(DEV)
    q_w = torch.from_numpy((1 + 0.1 * rng.standard_normal(hd)).astype(np.float32)).to(DEV) if qk_norm else None
    k_w = torch.from_numpy((1 + 0.1 * rng.standard_normal(hd)).astype(np.float32)).to(DEV) if qk_norm else None
    inv = (1e4 ** (-np.arange(n_rot // 2) * 2.0 / max(n_rot, 1))).astype(np.float32)
    inv_freq = torch.from_numpy(inv).to(DEV) if n_rot else None
    positions = torch.tensor(pos, dtype=torch.int32, device=DEV)
    items = torch.arange(T, dtype=torch.int32, device=DEV)
    tab = torch.from_numpy(table).to(DEV)
    scale = 1.0 / math.sqrt(hd)
    st = o.new_status(DEV)
    chunk, n_splits = o.split_plan(T, nkv, table.shape[1] * page)
    results = []
    for fused in (False, True):
        kcd, vcd = kc.clone().to(DEV), vc.clone().to(DEV)
        qkv = o.PartialProduct(parts.reshape(-1), splits, (T, width), torch.empty(T, width, dtype=dtype, device=DEV))
        out = torch.full((T, nh * hd), float("nan"), dtype=dtype, device=DEV)
        pa = torch.empty(T * nh * n_splits * hd, device=DEV)
        pm = torch.empty(T * nh * n_splits * 2, device=DEV)
        if fused:
            assert o.attention_decode_from_qkv(qkv, positions, items, q_w, k_w, inv_freq, n_rot, 1e-5, kcd, vcd, tab, page,
                                               n_pages, window, scale, out, pa, pm, chunk, n_splits, nh, nkv, hd, st)
        else:
            q = torch.empty(T, nh * hd, dtype=dtype, device=DEV)
            o.qk_norm_rope_store(qkv, positions, items, q_w, k_w, inv_freq, n_rot, 1e-5, q, kcd, vcd, tab, page, n_pages,
                                 nh, nkv, hd, st)
            assert o.paged_attention_split(q, kcd, vcd, positions, items, tab, page, n_pages, window, scale, out, pa, pm,
                                           chunk, n_splits, nh, nkv, hd, st, fresh=1)
        torch.cuda.synchronize()
        o.read_status(st)
        results.append((out.float().cpu(), kcd.float().cpu(), vcd.float().cpu()))
    (out_a, k_a, v_a), (out_b, k_b, v_b) = results
    assert torch.equal(k_a, k_b) and torch.equal(v_a, v_b)            # the same rows in the same pages, nothing else touched
    assert torch.equal(out_a, out_b)
    # and against float64: sum of the partials rounded to bfloat16, norm, rotation, attention over the request's rows
    x = parts.sum(0).to(dtype).float().cpu().numpy().astype(np.float64)
    for t in range(T):
        def head(col0, w):
            v = x[t, col0:col0 + hd].copy()
            if w is not None:
                v = v / np.sqrt((v * v).mean() + 1e-5) * w.cpu().numpy().astype(np.float64)
            if n_rot:
                ang = float(pos[t]) * inv.astype(np.float64)
                a, b = v[:n_rot // 2].copy(), v[n_rot // 2:n_rot].copy()
                v[:n_rot // 2] = a * np.cos(ang) - b * np.sin(ang)
                v[n_rot // 2:n_rot] = a * np.sin(ang) + b * np.cos(ang)
            return v
        qq = np.concatenate([head(h * hd, q_w) for h in range(nh)])
        kk = ks[t].numpy().astype(np.float64).copy()
        vv = vs[t].numpy().astype(np.float64).copy()
        kk[pos[t]] = np.concatenate([head((nh + g) * hd, k_w) for g in range(nkv)])
        vv[pos[t]] = x[t, (nh + nkv) * hd:]
        want = attention_reference(qq, kk, vv, pos[t], nh, nkv, hd, scale, window)
        assert np.abs(out_b[t].numpy() - want).max() < 4e-2 * max(1.0, np.abs(want).max())


@pytest.mark.parametrize("nh,nkv,hd", [(5, 2, 64), (3, 1, 128), (32, 8, 64)])
@pytest.mark.parametrize("normed,rotated,T", [(False, True, 300), (True, False, 300), (False, False, 300),
                                              (True, True, 600), (True, True, 1100), (True, True, 2050)])
def test_qk_kernel_of_prompt_portions_without_norm_or_rotation(nh, nkv, hd, normed, rotated, T):
    """The warp-per-token kernel (bfloat16, 256 tokens or more, heads of 64 / 128) with null norm weights (no per-head
    norm on that side) and with no rotation: what is left is a copy of the values into q and the pages.  And with both,
    at the token counts where a token's heads are shared among 8, 4 and 2 warps or belong to one."""
    o = ops()
    rng = np.random.default_rng(nh + hd)
    page, eps = 16, 1e-5
    n_pages = T // page + 2
    positions = np.arange(T, dtype=np.int32)
    items = np.zeros(T, dtype=np.int32)
    table = np.arange(n_pages, dtype=np.int32)[None, :].copy()
    qkv = torch.from_numpy(rng.standard_normal((T, (nh + 2 * nkv) * hd)).astype(np.float32)).bfloat16()
    qw = torch.from_numpy(1 + 0.1 * rng.standard_normal(hd).astype(np.float32)) if normed else None
    kw = torch.from_numpy(1 + 0.1 * rng.standard_normal(hd).astype(np.float32)) if normed else None
    inv = (1e4 ** (-2.0 * np.arange(hd // 2) / hd)).astype(np.float32)
    q_out = torch.empty(T, nh * hd, dtype=torch.bfloat16, device=DEV)
    kc = torch.zeros(n_pages, page, nkv * hd, dtype=torch.bfloat16, device=DEV)
    vc = torch.zeros_like(kc)
    st = o.new_status(DEV)
    o.qk_norm_rope_store(qkv.to(DEV), torch.from_numpy(positions).to(DEV), torch.from_numpy(items).to(DEV),
                         None if qw is None else qw.to(DEV), None if kw is None else kw.to(DEV),
                         torch.from_numpy(inv).to(DEV) if rotated else None, hd if rotated else 0, eps, q_out, kc, vc,
                         torch.from_numpy(table).to(DEV), page, n_pages, nh, nkv, hd, st)
    o.read_status(st)
    x = qkv.double().numpy()

    def ref(rows, w, pos):
        if w is not None:
            rows = rows / np.sqrt((rows * rows).mean(-1, keepdims=True) + eps) * w.double().numpy()
        if rotated:
            ang = (np.float64(pos) * inv.astype(np.float64))
            half = hd // 2
            out = rows.copy()
            out[:, :half] = rows[:, :half] * np.cos(ang) - rows[:, half:] * np.sin(ang)
            out[:, half:] = rows[:, :half] * np.sin(ang) + rows[:, half:] * np.cos(ang)
            rows = out
        return rows.reshape(-1)
    for t in (0, 1, 15, 16, 255, 299, T // 2 + 1, T - 1):
        qr = ref(x[t, :nh * hd].reshape(nh, hd), qw, t)
        kr = ref(x[t, nh * hd:(nh + nkv) * hd].reshape(nkv, hd), kw, t)
        assert np.abs(q_out[t].float().cpu().numpy() - qr).max() <= 1e-2 * np.abs(qr).max()
        assert np.abs(kc[t // page, t % page].float().cpu().numpy() - kr).max() <= 1e-2 * np.abs(kr).max()
        assert np.abs(vc[t // page, t % page].float().cpu().numpy() - x[t, (nh + nkv) * hd:]).max() <= 1e-7

