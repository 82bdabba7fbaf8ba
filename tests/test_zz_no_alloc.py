"""The entry point that allocates nothing (imparo_b200/csrc/kernels/no_alloc.h).

Some hosts of the attention kernel cannot give it scratch memory or let it allocate: code
inside a stream capture, latency-bound serving loops, programs whose device memory is all
handed out by their own allocator.  For them the library exports
imparo_paged_attention_split_static, which keeps its scratch in a fixed 8 MiB array inside
the library.  This test calls it through its exported C symbol, twice in a row with
different inputs (the array keeps the first call's contents), and compares each result
with the ordinary entry point's and with a plain reference; it also checks the refusal of
sizes beyond the array.  It is collected last so that a run that stops at the first
failure has already run every other test.
"""
import ctypes
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _lib():
    from imparo_b200.kernels import lib
    k = lib.kernels()
    P, I = ctypes.c_void_p, ctypes.c_int
    fn = k.imparo_paged_attention_split_static
    fn.argtypes = [P, P, P, I, P, P, P, I, I, I, I, ctypes.c_float, P, I, I, I, I, I, I, P, P]
    fn.restype = I
    need = k.imparo_paged_attention_split_static_need
    need.argtypes = [I, I, I, I]
    need.restype = ctypes.c_longlong
    return fn, need


def _case(seed, dtype, n_req=5, nh=8, nkv=2, hd=64, page=16):
    from tests.test_kernels_gpu import make_paged
    rng = np.random.default_rng(seed)
    lens = [int(x) for x in rng.integers(40, 700, n_req)]
    table, kc, vc, ks, vs, n_pages = make_paged(rng, lens, page, nkv, hd, dtype)
    q = torch.from_numpy(rng.standard_normal((n_req, nh * hd)).astype(np.float32)).to(dtype)
    positions = torch.tensor([n - 1 for n in lens], dtype=torch.int32)
    items = torch.arange(n_req, dtype=torch.int32)
    return dict(q=q.to(DEV), kc=kc.to(DEV), vc=vc.to(DEV), positions=positions.to(DEV), items=items.to(DEV),
                table=torch.from_numpy(table).to(DEV), page=page, n_pages=n_pages, nh=nh, nkv=nkv, hd=hd, lens=lens,
                ks=ks, vs=vs, q_host=q)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_static_scratch_entry_point_matches_the_ordinary_one(dtype):
    from imparo_b200.kernels import ops
    from tests.test_kernels_gpu import attention_reference
    fn, need = _lib()
    stream = torch.cuda.current_stream().cuda_stream
    status = ops.new_status(DEV)
    for call, seed in enumerate((11, 12)):                       # two calls in a row, sharing the array
        c = _case(seed, dtype)
        nh, nkv, hd = c["nh"], c["nkv"], c["hd"]
        T = c["q"].shape[0]
        scale = 1 / math.sqrt(hd)
        upper = c["table"].shape[1] * c["page"]
        chunk, n_splits = ops.split_plan(T, nkv, upper)
        assert need(T, nh, hd, n_splits) <= 2 * 1024 * 1024
        out_static = torch.full((T, nh * hd), float("nan"), dtype=dtype, device=DEV)
        rc = fn(c["q"].data_ptr(), c["kc"].data_ptr(), c["vc"].data_ptr(), 1 if dtype == torch.bfloat16 else 0,
                c["positions"].data_ptr(), c["items"].data_ptr(), c["table"].data_ptr(), c["table"].shape[1], c["page"],
                c["n_pages"], 0, scale, out_static.data_ptr(), T, nh, nkv, hd, chunk, n_splits, status.data_ptr(), stream)
        assert rc == 0, rc
        out_plain = torch.empty_like(out_static)
        part_acc = torch.empty(T * nh * n_splits * hd, device=DEV)
        part_ml = torch.empty(T * nh * n_splits * 2, device=DEV)
        assert ops.paged_attention_split(c["q"], c["kc"], c["vc"], c["positions"], c["items"], c["table"], c["page"],
                                         c["n_pages"], None, scale, out_plain, part_acc, part_ml, chunk, n_splits, nh, nkv, hd,
                                         status, mma=False)          # the same scalar kernel the static entry point runs
        torch.cuda.synchronize()
        ops.read_status(status)
        assert torch.equal(out_static, out_plain), f"call {call}: the two entry points disagree"
        tol = 3e-6 if dtype == torch.float32 else 1e-2
        got = out_static.float().cpu().double().numpy()
        for t in range(T):
            ref = attention_reference(c["q_host"][t].double().numpy(), c["ks"][t].double().numpy(), c["vs"][t].double().numpy(),
                                      c["lens"][t] - 1, nh, nkv, hd, scale, None)
            assert np.abs(got[t] - ref).max() <= tol * max(1.0, np.abs(ref).max()), (call, t)


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    from imparo_b200.kernels import ops
    fn, need = _lib()
    assert need(4096, 32, 64, 16) > 2 * 1024 * 1024
    z = torch.zeros(16, device=DEV)
    status = ops.new_status(DEV)
    rc = fn(z.data_ptr(), z.data_ptr(), z.data_ptr(), 0, z.data_ptr(), z.data_ptr(), z.data_ptr(), 1, 16, 1, 0, 1.0,
            z.data_ptr(), 4096, 32, 8, 64, 256, 16, status.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == -30                                           # IMPARO_ERR_STATIC_SCRATCH_TOO_SMALL, nothing launched
    # more key chunks than the combine kernel can hold, although the partials would fit the array: refused (-2)
    args = lambda n_tok, nh, nkv, hd, chunk, n_splits, max_blocks: (
        z.data_ptr(), z.data_ptr(), z.data_ptr(), 0, z.data_ptr(), z.data_ptr(), z.data_ptr(), max_blocks, 16, 1, 0, 1.0,
        z.data_ptr(), n_tok, nh, nkv, hd, chunk, n_splits, status.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert need(1, 1, 16, 4096) <= 2 * 1024 * 1024
    assert fn(*args(1, 1, 1, 16, 32, 4096, 1)) == -2
    # chunks that do not cover the block table (keys would be dropped silently): refused (-2)
    assert fn(*args(1, 1, 1, 16, 64, 2, 64)) == -2
    # a head size or head counts the kernel does not take, checked before the scratch need is computed
    assert fn(*args(1, 1, 1, 24, 64, 1, 1)) == -3
    assert fn(*args(1, 3, 2, 16, 64, 1, 1)) == -5
    torch.cuda.synchronize()
    ops.read_status(status)
