"""Launchers: check what the host can check, then call the CUDA entry points.

Every function works on CUDA tensors only and raises otherwise; there is no CPU or
library fallback for these operations.  The reference's launchers check layouts on
the host in the same spirit (imparo-cuda/native/lfm2_ops.cuh:28-42,
cobatch_rows.cuh:37-61).
"""
from __future__ import annotations

import os
from typing import Optional

import torch

from . import lib as _lib

F32, BF16 = 0, 1
_DT = {torch.float32: F32, torch.bfloat16: BF16}


class KernelError(RuntimeError):
    pass


def _code(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise KernelError(f"unsupported dtype {t.dtype}: kernels take float32 or bfloat16") from None


def _need(cond: bool, msg: str) -> None:
    if not cond:
        raise KernelError(msg)


def _cuda(*ts) -> None:
    for t in ts:
        if t is not None:
            if not t.is_cuda:
                raise KernelError("kernels run on CUDA tensors only (there is no CPU path)")
            if not t.is_contiguous():
                raise KernelError("kernel arguments must be contiguous")


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_current_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream():
    """The current stream's handle.  A step issues well over a hundred launches from Python, so the
    handle is asked of the runtime directly, not through a Stream object built per call."""
    if _raw_stream is not None and _current_device is not None:
        return _raw_stream(_current_device())
    return torch.cuda.current_stream().cuda_stream


# Launch counts since import: "own" = this engine's CUDA kernels, "library" = cuBLAS products.
COUNTS = {"own": 0, "library": 0}


class LaunchState:
    """What the launchers remember between calls: which streams have split partials pending and the
    scratch buffers behind them.  An engine owns one (its Runtime
    holds it and the step function makes it current for the length of a step), so two engines in
    one process neither share bookkeeping nor scratch; code that calls the launchers directly
    works on the module's default state."""

    def __init__(self, switches=None):
        # which kernel paths are taken (config/engine.py KernelSwitches): resolved once, never read from the
        # environment on the launch path
        self.switches = switches if switches is not None else _default_switches()
        self.deferrable = set()      # data_ptr of streams whose next accumulate-product may stay pending
        self.pending = {}            # data_ptr -> (scratch, n_splits, rows, width)
        self.partials = {}           # device index -> scratch of products into the stream
        self.consumer_parts = {}     # device index -> scratch of products a consumer kernel folds
        self.tc_scratch = {}         # device index -> (floats, counters) of the cluster-folded products
        self.argmax_scratch = {}
        self.sample_scratch = {}
        self.status_fallback = {}
        self.generation = 0          # bumped when a scratch buffer moves: captured graphs that used it are stale


def _default_switches():
    from ..config.engine import EngineConfig
    return EngineConfig.resolve().switches


_S = LaunchState()


def switches():
    """The kernel switches of the state that is current (an engine's, during its steps; else the module's own,
    resolved from the environment and the optional configuration file when the module was imported)."""
    return _S.switches


def use_state(state: "LaunchState") -> "LaunchState":
    """Makes `state` the one the launchers work on; returns the one it replaces."""
    global _S
    old, _S = _S, state
    return old


def generation() -> int:
    return _S.generation


def _cuda_error_text(rc: int) -> str:
    try:
        rt = torch.cuda.cudart()
        return rt.cudaGetErrorString(rt.cudaError(rc))
    except Exception:                    # noqa: BLE001 - the text is a courtesy
        return ""


def _check(rc: int, what: str, kind: str = "own") -> None:
    if rc == 0:
        COUNTS[kind] += 1
        return
    reasons = {-1: "unsupported dtype code or missing library handle", -2: "bad accumulate/grid",
               -3: "head size must be a multiple of 16 between 16 and 256",
               -4: "rotated dimensions must be even and at most the head size",
               -5: "kv heads must divide heads", -6: "conv taps must be between 2 and 16",
               -7: "temperature sampling needs uniform numbers",
               -23: "rows must be 16 bytes wide and 16-byte aligned (K and the row stride multiples of 8 elements; an output "
                    "of 8 bfloat16 or 4 float32 per group)",
               -22: "unknown epilogue", -24: "scratch missing", -25: "the kernel does not take this case"}
    if rc < 0:
        raise KernelError(f"{what}: refused: {reasons.get(rc, rc)}")
    if rc >= 1000:
        raise KernelError(f"{what}: cuBLAS status {rc - 1000}")
    raise KernelError(f"{what}: CUDA error {rc} ({_cuda_error_text(rc)})")


# --------------------------------------------------------------------------------------

def new_status(device) -> torch.Tensor:
    return torch.zeros(4, dtype=torch.int32, device=device)


_STATUS_TEXT = {1: "token id out of the vocabulary", 2: "cache page out of range (unmapped block or bad table)",
                3: "state slot out of range", 4: "a bounded device wait gave up (tensor-core product)"}


def read_status(status: torch.Tensor) -> None:
    """Raise if a kernel recorded a bad index since the word was last cleared (synchronizes)."""
    s = status.tolist()
    if s[0] != 0:
        status.zero_()
        raise KernelError(f"device check failed: {_STATUS_TEXT.get(s[0], s[0])} "
                          f"(kernel {s[1]}, index {s[2]}, value {s[3]})")


def selftest_wait_limit(status: torch.Tensor, limit: int = 1000) -> int:
    """Runs a kernel whose bounded wait cannot complete (csrc/kernels/selftest.cu).  Returns 2 when the kernel
    gave up, recorded the wait-limit code in `status` and ran to its end; 1 if the wait completed (it cannot)."""
    _cuda(status)
    outcome = torch.zeros(1, dtype=torch.int32, device=status.device)
    _check(_lib.kernels().imparo_selftest_wait_limit(_ptr(status), int(limit), _ptr(outcome), _stream()), "selftest_wait_limit")
    return int(outcome.item())


def embed_gather(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, status: torch.Tensor) -> None:
    _cuda(table, ids, out, status)
    _S.pending.pop(out.data_ptr(), None)       # the stream starts afresh: partials of an unfinished step are void
    n, width = out.shape
    _need(ids.dtype == torch.int32 and ids.numel() >= n, "ids must be int32, one per output row")
    _need(out.dtype == torch.float32 and table.shape[1] == width, "embedding output is float32 [tokens, width]")
    _check(_lib.kernels().imparo_embed_gather(_ptr(table), _code(table), _ptr(ids), _ptr(out), n, width,
                                              table.shape[0], _ptr(status), _stream()), "embed_gather")


# ---- adds into the 32-bit stream that are still split partials ---------------------------------
# A decode-sized product into the stream is cut along K over many CTAs.  Instead of folding the
# splits itself it may leave them in scratch ("pending"); the next reader of the stream — nearly
# always the RMS norm — adds them in split order and goes on in the same kernel.


def _grown(floats: int, old) -> int:
    """Size of a scratch buffer that must hold `floats`: at least 4 MB, and twice the old size while that stays
    under 256 MB, because every move of a scratch buffer makes the captured graphs that used it stale and a
    serving loop meets slightly larger steps for a long while."""
    had = old.numel() if old is not None else 0
    return max(floats, 1 << 20, 2 * had if had <= (32 << 20) else 0)


def prepare(device, rows: int = 8) -> None:
    """Make, for the launch state that is current, what the launchers would otherwise make at their first use: the
    library product's handle and workspace, the split partials' scratch and the samplers' scratch for `rows` rows.
    A step recorded into a graph must not allocate, so an engine calls this before its first step."""
    device = torch.device(device)
    key = device.index or 0
    _gemm_lib_ready(device)
    global _tc_configured
    if not _tc_configured:
        # shared-memory attributes and the cluster plan's occupancy table (a query the runtime refuses under capture)
        with torch.cuda.device(device):
            _check(_lib.kernels().imparo_gemm_tc_configure(), "gemm_tc_configure")
        COUNTS["own"] -= 1           # nothing was launched
        _tc_configured = True
    if key not in _S.partials:
        _S.partials[key] = torch.empty(_grown(0, None), dtype=torch.float32, device=device)
    if key not in _S.consumer_parts:
        _S.consumer_parts[key] = torch.empty(_grown(0, None), dtype=torch.float32, device=device)
    if key not in _S.tc_scratch:
        _S.tc_scratch[key] = (torch.empty(1 << 20, dtype=torch.float32, device=device),
                              torch.zeros(4096, dtype=torch.int32, device=device))
    n = max(int(rows), 256)
    if key not in _S.argmax_scratch:
        _S.argmax_scratch[key] = (torch.empty(n * 32, dtype=torch.float32, device=device),
                                  torch.empty(n * 32, dtype=torch.int32, device=device))
    if key not in _S.sample_scratch:
        _S.sample_scratch[key] = (torch.empty(n * 64, dtype=torch.float32, device=device),
                                  torch.empty(n * 32, dtype=torch.int32, device=device))


def defer_adds() -> bool:
    return _S.switches.defer_adds


def allow_deferred_add(stream: torch.Tensor) -> None:
    """The caller promises that whatever reads `stream` next goes through ops.rmsnorm, ops.settle, ops.add_bias,
    ops.gather_rows or another ops.linear(accumulate=True)."""
    if defer_adds():
        _S.deferrable.add(stream.data_ptr())


def disallow_deferred_add(stream: torch.Tensor) -> None:
    _S.deferrable.discard(stream.data_ptr())


def settle(stream: torch.Tensor) -> None:
    """Fold pending partials into the stream (no-op when there are none)."""
    p = _S.pending.pop(stream.data_ptr(), None)
    if p is not None:
        scratch, S, T, N = p
        _check(_lib.kernels().imparo_add_partials_rmsnorm(_ptr(stream), _ptr(scratch), S, T * N, None, 0.0, None, 0, T, N,
                                                          _stream()), "add_partials")


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float, out: torch.Tensor,
            rows: Optional[torch.Tensor] = None) -> None:
    _cuda(x, w, out, rows)
    pend = _S.pending.get(x.data_ptr())
    if pend is not None:
        scratch, S, T, N = pend
        if rows is None and out.shape == (T, N) and x.shape[1] == N and w.numel() == N and w.dtype == torch.float32:
            # the stream's pending partials are added and the updated rows normed in one kernel
            _S.pending.pop(x.data_ptr())
            _check(_lib.kernels().imparo_add_partials_rmsnorm(_ptr(x), _ptr(scratch), S, T * N, _ptr(w), float(eps), _ptr(out),
                                                              _code(out), T, N, _stream()), "add_partials_rmsnorm")
            return
        settle(x)
    n, width = out.shape
    _need(x.dtype == torch.float32 and w.dtype == torch.float32, "rmsnorm reads a float32 stream and float32 weights")
    _need(x.shape[1] == width and w.numel() == width, "rmsnorm width mismatch")
    if rows is None:
        _need(x.shape[0] >= n, "rmsnorm: fewer input rows than output rows")
    else:
        _need(rows.dtype == torch.int32 and rows.numel() >= n, "rmsnorm: rows must be int32, one per output row")
    _check(_lib.kernels().imparo_rmsnorm(_ptr(x), _ptr(rows), _ptr(w), float(eps), _ptr(out), _code(out), n, width,
                                         _stream()), "rmsnorm")


def swiglu_act(gu: torch.Tensor, out: torch.Tensor) -> None:
    _cuda(gu, out)
    n, F = out.shape
    _need(gu.shape == (n, 2 * F) and gu.dtype == out.dtype, "swiglu_act: gu must be [tokens, 2F] of the output dtype")
    _check(_lib.kernels().imparo_swiglu_act(_ptr(gu), _ptr(out), _code(out), n, F, _stream()), "swiglu_act")


def add_bias(out: torch.Tensor, bias: torch.Tensor) -> None:
    _cuda(out, bias)
    settle(out)
    n, width = out.shape
    _need(bias.dtype == torch.float32 and bias.numel() == width, "bias must be float32 [width]")
    _check(_lib.kernels().imparo_add_bias(_ptr(out), _code(out), _ptr(bias), n, width, _stream()), "add_bias")


_gemm_ws = {}
_tc_configured = False


def _gemm_lib_ready(device) -> None:
    key = torch.device(device).index or 0
    if key not in _gemm_ws:
        _need(not torch.cuda.is_current_stream_capturing(), "the library product's first use would allocate during graph capture")
        ws = torch.empty(64 << 20, dtype=torch.uint8, device=device)
        _check(_lib.kernels().imparo_gemm_lib_init(_ptr(ws), ws.numel()), "gemm_lib_init")
        _gemm_ws[key] = ws


# ---- tcgen05 product ---------------------------------------------------------------------
EPI_STORE_BF16, EPI_STORE_F32, EPI_ADD_F32, EPI_SWIGLU, EPI_PARTIAL = 0, 1, 2, 3, 4
_tc_plans = {}


def gemm_backend() -> str:
    """"tcgen05" (default) or "library" (cuBLAS): the switch `gemm`."""
    return _S.switches.gemm


def _tc_plan(T, N, K, epi):
    key = (T, N, K, epi)
    plan = _tc_plans.get(key)
    if plan is None:
        import ctypes
        nt, sp, sf, nc = ctypes.c_int(), ctypes.c_int(), ctypes.c_int64(), ctypes.c_int()
        rc = _lib.kernels().imparo_gemm_tc_plan(T, N, K, epi, ctypes.byref(nt), ctypes.byref(sp), ctypes.byref(sf), ctypes.byref(nc))
        if rc != 0:
            raise KernelError(f"gemm_tc_plan({T}, {N}, {K}) refused: {rc}")
        plan = _tc_plans[key] = (nt.value, sp.value, sf.value, nc.value)
    return plan


def _tc_buffers(device, floats: int, counters: int):
    """Split-K scratch and tile counters, shared by all products of a device (they run one
    after the other on the stream).  Grown outside graph capture only."""
    key = torch.device(device).index or 0
    buf = _S.tc_scratch.get(key)
    if buf is None or buf[0].numel() < floats or buf[1].numel() < counters:
        if torch.cuda.is_current_stream_capturing():
            raise KernelError("split-K scratch would grow during graph capture")
        old_f = buf[0].numel() if buf else 0
        old_c = buf[1].numel() if buf else 0
        buf = (torch.empty(max(floats, old_f, 1 << 20), dtype=torch.float32, device=device),
               torch.zeros(max(counters, old_c, 4096), dtype=torch.int32, device=device))
        _S.tc_scratch[key] = buf
        _S.generation += 1 if old_f else 0          # a buffer that did not exist is in no captured graph
    return buf


# Above this many tokens the library product is faster than the hand-written kernel as it
# stands (one token tile per CTA, no overlap of epilogue and main loop).  Measured on B200, whole
# decode steps of LFM2-1.2B shapes in their CUDA graph, ms per step (own kernel / library product):
# batch 32: 1.058 / 1.107; batch 64: 1.381 / 1.421 (the own kernels stay in the chain of
# programmatic dependent launches and prefetch their weights; a library product breaks it).  At
# 2,048 tokens the library is ahead: down 66 / 50 us, gate+up 275 / 160 us per product.


def tc_max_tokens() -> int:
    return _S.switches.tc_max_tokens


def tc_usable(x: torch.Tensor, w: torch.Tensor, any_size: bool = False) -> bool:
    K = x.shape[1]
    if not any_size and x.shape[0] > tc_max_tokens():
        return False
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and K % 8 == 0 and x.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and w.is_contiguous())


def gemm_tc(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int, status: Optional[torch.Tensor] = None,
            scratch: Optional[torch.Tensor] = None) -> None:
    """The hand-written tensor-core product (csrc/kernels/gemm_tcgen05.cu).
    epilogue: EPI_STORE_BF16 | EPI_STORE_F32 | EPI_ADD_F32 (out += x w^T) | EPI_SWIGLU
    (w = [gate rows; up rows] of shape [2F, K], out = silu(x gate^T) * (x up^T), [T, F])."""
    _need(x.is_cuda and w.is_cuda and out.is_cuda, "kernels run on CUDA tensors only (there is no CPU path)")
    _need(tc_usable(x, w, any_size=True), "gemm_tc: bfloat16 operands, K a multiple of 8, 16-byte aligned rows")
    T, K = x.shape
    N = w.shape[0] // 2 if epilogue == EPI_SWIGLU else w.shape[0]
    _need(w.shape[1] == K and (epilogue != EPI_SWIGLU or w.shape[0] % 2 == 0), "gemm_tc: weight shape")
    if not (out.shape == (T, N) and out.stride(1) == 1):
        raise KernelError(f"gemm_tc: out must be [{T}, {N}]")
    want_dtype = torch.bfloat16 if epilogue in (EPI_STORE_BF16, EPI_SWIGLU) else torch.float32
    if not (epilogue == EPI_PARTIAL or out.dtype == want_dtype):
        raise KernelError(f"gemm_tc: this epilogue writes {want_dtype}")
    nt, splits, floats, counters = _tc_plan(T, N, K, epilogue)
    if epilogue == EPI_PARTIAL:
        _need(scratch is not None and scratch.dtype == torch.float32 and scratch.numel() >= floats, "gemm_tc: partials scratch")
        cnt = scratch
    else:
        scratch, cnt = _tc_buffers(x.device, floats, counters)
    if status is None:
        key = torch.device(x.device).index or 0
        status = _S.status_fallback.get(key)
        if status is None:
            status = _S.status_fallback[key] = new_status(x.device)
    rows_alloc = (x.untyped_storage().nbytes() // x.element_size() - x.storage_offset()) // x.stride(0) if x.stride(0) else T
    rows_alloc = max(T, min(rows_alloc, 1 << 30))
    _check(_lib.kernels().imparo_gemm_tc(_ptr(x), x.stride(0), rows_alloc, _ptr(w), _ptr(out), out.stride(0), T, N, K, epilogue,
                                         _ptr(scratch), _ptr(cnt), _ptr(status), _stream()), "gemm_tc")


# ---- tcgen05 product for prompt-sized batches (csrc/kernels/gemm_prefill.cu) ---------------------
# From this many tokens on the persistent 128 x 256-tile kernel takes the product (below it, down to
# TC_MAX_TOKENS, the library does): a tile holds 128 tokens, and its SwiGLU epilogue saves the
# [T, 2F] intermediate only where the kernel also keeps up with the library on the product itself.


def prefill_tc_min_tokens() -> int:
    return _S.switches.prefill_tc_min_tokens


def prefill_tc_usable(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, swiglu: bool = False) -> bool:
    """Whether gemm_prefill takes out (+)= x w^T: bfloat16 operands with 16-byte rows, an output whose rows
    are 16-byte aligned groups, enough tokens, and the own product not switched off."""
    if gemm_backend() != "tcgen05" or _S.switches.prefill_gemm != "tcgen05":
        return False
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or x.shape[0] < prefill_tc_min_tokens():
        return False
    K = x.shape[1]
    N = w.shape[0] // 2 if swiglu else w.shape[0]
    group = 4 if out.dtype == torch.float32 else 8
    return (K % 8 == 0 and x.stride(0) % 8 == 0 and x.stride(1) == 1 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
            and w.is_contiguous() and out.stride(1) == 1 and N % group == 0 and out.stride(0) % group == 0
            and out.data_ptr() % 16 == 0 and out.dtype in (torch.float32, torch.bfloat16))


def gemm_prefill(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int, status: Optional[torch.Tensor] = None) -> None:
    """The persistent tensor-core product for many tokens.  epilogue: EPI_STORE_BF16 | EPI_STORE_F32 |
    EPI_ADD_F32 (out += x w^T) | EPI_SWIGLU (w = [gate rows; up rows], out = silu(x gate^T) * (x up^T))."""
    _need(x.is_cuda and w.is_cuda and out.is_cuda, "kernels run on CUDA tensors only (there is no CPU path)")
    _need(epilogue in (EPI_STORE_BF16, EPI_STORE_F32, EPI_ADD_F32, EPI_SWIGLU), "gemm_prefill: unknown epilogue")
    T, K = x.shape
    N = w.shape[0] // 2 if epilogue == EPI_SWIGLU else w.shape[0]
    _need(w.shape[1] == K and (epilogue != EPI_SWIGLU or w.shape[0] % 2 == 0), "gemm_prefill: weight shape")
    _need(tuple(out.shape) == (T, N), f"gemm_prefill: out must be [{T}, {N}]")
    want_dtype = torch.bfloat16 if epilogue in (EPI_STORE_BF16, EPI_SWIGLU) else torch.float32
    _need(out.dtype == want_dtype, f"gemm_prefill: this epilogue writes {want_dtype}")
    if status is None:
        key = torch.device(x.device).index or 0
        status = _S.status_fallback.get(key)
        if status is None:
            status = _S.status_fallback[key] = new_status(x.device)
    rows_alloc = (x.untyped_storage().nbytes() // x.element_size() - x.storage_offset()) // x.stride(0) if x.stride(0) else T
    rows_alloc = max(T, min(rows_alloc, 1 << 30))
    _check(_lib.kernels().imparo_gemm_prefill(_ptr(x), x.stride(0), rows_alloc, _ptr(w), _ptr(out), out.stride(0), T, N, K,
                                              epilogue, _ptr(status), _stream()), "gemm_prefill")


def linear_swiglu(x, w_gu: torch.Tensor, out: torch.Tensor, status: Optional[torch.Tensor] = None,
                  tmp: Optional[torch.Tensor] = None) -> None:
    """out[T, F] = silu(x gate^T) * (x up^T) with w_gu = [gate; up] of shape [2F, K].
    bfloat16 on the tensor-core kernels (the weight streamer for few tokens, the persistent tile kernel for
    many): one launch, the activation in the epilogue.  Otherwise: the product into tmp [T, 2F] (a tensor,
    or a function that makes it, called only on this path), then the activation kernel."""
    if x.dtype == torch.bfloat16 and gemm_backend() == "tcgen05" and tc_usable(x, w_gu):
        gemm_tc(x, w_gu, out, EPI_SWIGLU, status)
        return
    if prefill_tc_usable(x, w_gu, out, swiglu=True):
        gemm_prefill(x, w_gu, out, EPI_SWIGLU, status)
        return
    if callable(tmp):
        tmp = tmp()
    _need(tmp is not None and tmp.shape == (x.shape[0], w_gu.shape[0]), "linear_swiglu: tmp [T, 2F] needed on this path")
    linear(x, w_gu, tmp)
    swiglu_act(tmp, out)


def linear(x, w: torch.Tensor, out: torch.Tensor, accumulate: bool = False,
           status: Optional[torch.Tensor] = None) -> None:
    """out[M,N] (+)= x[M,K] @ w[N,K]^T.  float32 x/w -> the FFMA kernel (true 32-bit);
    bfloat16 x/w -> tensor cores with 32-bit accumulation, out float32 or bfloat16."""
    _need(x.is_cuda and w.is_cuda and out.is_cuda, "kernels run on CUDA tensors only (there is no CPU path)")
    M, K = x.shape
    N = w.shape[0]
    if not (w.shape[1] == K and out.shape == (M, N)):
        raise KernelError(f"linear: shapes x{tuple(x.shape)} w{tuple(w.shape)} out{tuple(out.shape)}")
    _need(x.stride(1) == 1 and out.is_contiguous() and w.is_contiguous(), "linear: rows must be dense")
    _need(x.dtype == w.dtype, "linear: x and w must share a dtype")
    if x.dtype == torch.float32:
        _need(out.dtype == torch.float32, "linear: float32 product writes float32")
        if accumulate:
            settle(out)
        _check(_lib.kernels().imparo_sgemm_nt(_ptr(x), _ptr(w), _ptr(out), M, N, K, x.stride(0), N, int(accumulate),
                                              _stream()), "sgemm_nt")
    elif x.dtype == torch.bfloat16:
        _need(not accumulate or out.dtype == torch.float32, "linear: accumulate needs a float32 output")
        if gemm_backend() == "tcgen05" and tc_usable(x, w):
            epi = EPI_ADD_F32 if accumulate else (EPI_STORE_F32 if out.dtype == torch.float32 else EPI_STORE_BF16)
            if accumulate and out.data_ptr() in _S.deferrable and out.is_contiguous():
                settle(out)                                       # one set of partials at a time
                nt, splits, floats, _ = _tc_plan(M, N, K, EPI_PARTIAL)
                if splits > 1:
                    key = torch.device(x.device).index or 0
                    buf = _S.partials.get(key)
                    if buf is None or buf.numel() < floats:
                        _need(not torch.cuda.is_current_stream_capturing(), "partials scratch would grow during graph capture")
                        _S.generation += 0 if buf is None else 1      # a buffer that did not exist is in no captured graph
                        buf = _S.partials[key] = torch.empty(_grown(floats, buf), dtype=torch.float32, device=x.device)
                    gemm_tc(x, w, out, EPI_PARTIAL, status, scratch=buf)
                    _S.pending[out.data_ptr()] = (buf, splits, M, N)
                    return
            if accumulate:
                settle(out)
            gemm_tc(x, w, out, epi, status)
            return
        if accumulate:
            settle(out)
        if _S.switches.prefill_linear and prefill_tc_usable(x, w, out):
            gemm_prefill(x, w, out, EPI_ADD_F32 if accumulate else (EPI_STORE_F32 if out.dtype == torch.float32 else EPI_STORE_BF16),
                         status)
            return
        _gemm_lib_ready(x.device)
        _check(_lib.kernels().imparo_gemm_bf16_nt(_ptr(x), _ptr(w), _ptr(out), _code(out), M, N, K, x.stride(0), N,
                                                  int(accumulate), _stream()), "gemm_bf16_nt", "library")
    else:
        raise KernelError(f"linear: unsupported dtype {x.dtype}")


def gather_rows(x: torch.Tensor, rows: torch.Tensor, out: torch.Tensor) -> None:
    """out[r, :] = x[rows[r], :] for a 32-bit stream (folds split partials pending on x first)."""
    _cuda(x, rows, out)
    settle(x)
    n, width = out.shape
    _need(x.dtype == torch.float32 and out.dtype == torch.float32 and x.shape[1] == width and x.stride(1) == 1
          and x.stride(0) == width and out.is_contiguous(), "gather_rows: dense float32 [rows, width]")
    _need(rows.dtype == torch.int32 and rows.numel() >= n, "gather_rows: rows must be int32, one per output row")
    _check(_lib.kernels().imparo_gather_rows_f32(_ptr(x), _ptr(rows), _ptr(out), n, width, _stream()), "gather_rows")
    COUNTS["own"] += 1


class PartialProduct:
    """A product x w^T that was cut along K and not folded: parts[s] (float32 [T, N], split s at
    offset s * stride floats) sum to the result.  gated_conv and qk_norm_rope_store read it as it is
    (they sum in split order and round to `dtype`, what the product's own fold would have stored);
    anything else calls tensor(), which folds it into the buffer the product would have written."""

    def __init__(self, parts: torch.Tensor, splits: int, shape, out: torch.Tensor):
        self.parts, self.splits, self.shape, self._out = parts, int(splits), tuple(shape), out
        self.stride = self.shape[0] * self.shape[1]
        self.dtype, self.device = out.dtype, out.device
        self._done = False

    def tensor(self) -> torch.Tensor:
        if not self._done:
            _check(_lib.kernels().imparo_fold_partials(_ptr(self.parts), self.splits, self.stride, _ptr(self._out),
                                                       _code(self._out), self.stride, _stream()), "fold_partials")
            self._done = True
        return self._out


def unfolded_products() -> bool:
    """Whether linear_unfolded may leave split partials to its consumer (the switch `unfolded`)."""
    return _S.switches.unfolded


def linear_unfolded(x, w: torch.Tensor, out: torch.Tensor, status: Optional[torch.Tensor] = None):
    """out = x w^T for a consumer that can read split partials (gated_conv, qk_norm_rope_store).
    Returns `out`, filled; or, when the tensor-core product is cut along K (few tokens), a
    PartialProduct: each split's CTAs store their tile and are done, with no fold across CTAs inside
    the product, and the consumer adds the splits while it reads."""
    if unfolded_products() and x.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and out.is_contiguous() \
            and gemm_backend() == "tcgen05" and tc_usable(x, w):
        M, K = x.shape
        N = w.shape[0]
        nt, splits, floats, _ = _tc_plan(M, N, K, EPI_PARTIAL)
        if splits > 1:
            key = torch.device(x.device).index or 0
            buf = _S.consumer_parts.get(key)
            if buf is None or buf.numel() < floats:
                _need(not torch.cuda.is_current_stream_capturing(), "partials scratch would grow during graph capture")
                _S.generation += 0 if buf is None else 1
                buf = _S.consumer_parts[key] = torch.empty(_grown(floats, buf), dtype=torch.float32, device=x.device)
            gemm_tc(x, w, out, EPI_PARTIAL, status, scratch=buf)
            return PartialProduct(buf, splits, (M, N), out)
    linear(x, w, out, status=status)
    return out


# ---- the attention's output product with the combine of the split partials inside (decode rows) ----------
def fuse_producers() -> bool:
    """Whether the attention combine of decode rows runs inside the output product that follows it (the switch
    `fuse_producers`; off: as a kernel of its own)."""
    return _S.switches.fuse_producers


def _into_stream(out: torch.Tensor, M: int, N: int, K: int):
    """How a tensor-core product into the 32-bit stream `out` is issued: (EPI_PARTIAL, scratch, splits) when its add
    may stay split partials for the next reader of the stream, else (EPI_ADD_F32, None, 1) with the stream made whole."""
    if out.data_ptr() in _S.deferrable and out.is_contiguous():
        settle(out)                                           # one set of partials at a time
        nt, splits, floats, _ = _tc_plan(M, N, K, EPI_PARTIAL)
        if splits > 1:
            key = torch.device(out.device).index or 0
            buf = _S.partials.get(key)
            if buf is None or buf.numel() < floats:
                _need(not torch.cuda.is_current_stream_capturing(), "partials scratch would grow during graph capture")
                _S.generation += 0 if buf is None else 1
                buf = _S.partials[key] = torch.empty(_grown(floats, buf), dtype=torch.float32, device=out.device)
            return EPI_PARTIAL, buf, splits
    settle(out)
    return EPI_ADD_F32, None, 1


def _produced_usable(T: int, w: torch.Tensor, out: torch.Tensor) -> bool:
    K = w.shape[1]
    return (fuse_producers() and gemm_backend() == "tcgen05" and T <= min(16, tc_max_tokens()) and w.dtype == torch.bfloat16
            and w.is_contiguous() and w.data_ptr() % 16 == 0 and K % 8 == 0 and out.dtype == torch.float32
            and out.dim() == 2 and out.stride(1) == 1 and out.shape[1] == w.shape[0])


def _after_stream_product(out, epi, buf, splits, M, N) -> None:
    if epi == EPI_PARTIAL:
        _S.pending[out.data_ptr()] = (buf, splits, M, N)


def linear_of_attention_partials(part_acc, part_ml, n_tok, nh, hd, n_splits, w_out, out, status) -> bool:
    """out += combine(partials) w_out^T: the ordered combine of the split-key attention's partial results (as
    paged_attention_split(out=None) leaves them) computed inside the output product.  Returns False, having launched
    nothing, when the kernel does not take the case; the caller then combines with attention_split_combine."""
    if not (_produced_usable(n_tok, w_out, out) and w_out.shape[1] == nh * hd and hd % 8 == 0 and n_splits <= 64):
        return False
    _cuda(part_acc, part_ml, w_out, out, status)
    N, K = w_out.shape
    epi, buf, splits = _into_stream(out, n_tok, N, K)
    rc = _lib.kernels().imparo_gemm_tc_combine(_ptr(part_acc), _ptr(part_ml), nh, hd, n_splits, _ptr(w_out), _ptr(out),
                                               out.stride(0), n_tok, N, K, epi, _ptr(buf), _ptr(status), _stream())
    if rc == -25:
        return False
    _check(rc, "gemm_tc_combine")
    _after_stream_product(out, epi, buf, splits, n_tok, N)
    return True


def attention_split_combine(part_acc, part_ml, out, n_rows, hd, n_splits) -> None:
    """The ordered combine alone: out[row, :] from the partials of paged_attention_split(out=None)."""
    _cuda(part_acc, part_ml, out)
    _check(_lib.kernels().imparo_attention_split_combine(_ptr(part_acc), _ptr(part_ml), _ptr(out), _code(out), n_rows, hd,
                                                         n_splits, _stream()), "attention_split_combine")


def _parts_of(x):
    """(pointer tensor, parts, stride) of a kernel input that is a tensor or a PartialProduct."""
    if isinstance(x, PartialProduct):
        return x.parts, x.splits, x.stride
    return x, 0, 0


def qk_norm_rope_store(qkv, positions, item_of_token, q_w, k_w, inv_freq, n_rot, eps, q_out,
                       k_cache, v_cache, table, page_size, n_pages, nh, nkv, hd, status) -> None:
    """qkv [T, (nh+2*nkv)*hd] (a tensor or a PartialProduct) -> q_out [T, nh*hd] normed and rotated;
    k (normed, rotated) and v written into their pages.  nkv == 0: q only (a layer that reads
    another's cache).  q_w / k_w None: no per-head norm on that side (rotation only)."""
    src, parts, part_stride = _parts_of(qkv)
    _cuda(src, positions, item_of_token, q_w, k_w, inv_freq, q_out, k_cache, v_cache, table, status)
    T = q_out.shape[0]
    _need(tuple(qkv.shape) == (T, (nh + 2 * nkv) * hd) and q_out.shape[1] == nh * hd, "qk_norm_rope_store: widths")
    _need(qkv.dtype == q_out.dtype, "qk_norm_rope_store: q_out must have the activations' dtype")
    _need(positions.dtype == torch.int32 and item_of_token.dtype == torch.int32 and positions.numel() >= T
          and item_of_token.numel() >= T, "positions / item_of_token must be int32 per token")
    _need(q_w is None or (q_w.dtype == torch.float32 and q_w.numel() == hd), "q norm weight must be float32 [head]")
    if nkv:
        _need(k_w is None or (k_w.dtype == torch.float32 and k_w.numel() == hd), "k norm weight must be float32 [head]")
        _need(k_cache.dtype == qkv.dtype and v_cache.dtype == qkv.dtype, "cache dtype must match activations")
        _need(k_cache.numel() >= n_pages * page_size * nkv * hd and v_cache.numel() >= n_pages * page_size * nkv * hd,
              "cache arena smaller than n_pages")
        _need(table.dtype == torch.int32 and table.dim() == 2, "block table must be int32 [items, blocks]")
    if inv_freq is not None:
        _need(inv_freq.dtype == torch.float32 and inv_freq.numel() >= n_rot // 2, "inv_freq must be float32 [n_rot/2]")
    max_blocks = table.shape[1] if table is not None else 0
    _check(_lib.kernels().imparo_qk_norm_rope_store(
        _ptr(src), _code(q_out), _ptr(positions), _ptr(item_of_token), _ptr(q_w), _ptr(k_w), _ptr(inv_freq), n_rot,
        float(eps), _ptr(q_out), _ptr(k_cache), _ptr(v_cache), _ptr(table), max_blocks, page_size, n_pages,
        T, nh, nkv, hd, parts, part_stride, _ptr(status), _stream()), "qk_norm_rope_store")


def paged_attention(q, k_cache, v_cache, positions, item_of_token, table, page_size, n_pages, window, scale,
                    out, nh, nkv, hd, status) -> None:
    _cuda(q, k_cache, v_cache, positions, item_of_token, table, out, status)
    T = q.shape[0]
    _need(q.shape == (T, nh * hd) and out.shape == (T, nh * hd) and out.dtype == q.dtype, "paged_attention: q/out shapes")
    _need(k_cache.dtype == q.dtype and v_cache.dtype == q.dtype, "cache dtype must match q")
    _need(k_cache.numel() >= n_pages * page_size * nkv * hd, "cache arena smaller than n_pages")
    _need(table.dtype == torch.int32 and table.dim() == 2, "block table must be int32 [items, blocks]")
    _check(_lib.kernels().imparo_paged_attention(
        _ptr(q), _ptr(k_cache), _ptr(v_cache), _code(q), _ptr(positions), _ptr(item_of_token), _ptr(table),
        table.shape[1], page_size, n_pages, int(window or 0), float(scale), _ptr(out), T, nh, nkv, hd,
        _ptr(status), _stream()), "paged_attention")


MAX_SPLITS = 2048        # the ordered combine keeps one (max, sum) pair per key chunk in shared memory


_sm_count = {}


def sm_count(device=None) -> int:
    """Multiprocessors of the device (the current one by default), asked once."""
    key = torch.cuda.current_device() if device is None else (torch.device(device).index or 0)
    n = _sm_count.get(key)
    if n is None:
        n = _sm_count[key] = int(torch.cuda.get_device_properties(key).multi_processor_count)
    return n


def split_plan(n_tok: int, nkv: int, upper_context: int, sms: Optional[int] = None):
    """(chunk, n_splits) for the split-key attention kernel: the largest chunk of 512, 256, 128
    or 64 keys that still gives about four CTAs per SM; when even the smallest does not (a step of
    one or two tokens), the largest of 256, 128, 64 that gives 64 CTAs, since fewer and longer CTAs
    with fewer partials to combine then measured faster (batch 1: 0.735 ms per step with 256, 0.743
    with 64).  A function of the launch's shape only."""
    chunk = None
    full = 4 * (sms if sms is not None else sm_count())
    for c in (512, 256, 128, 64):
        if n_tok * nkv * -(-upper_context // c) >= full:
            chunk = c
            break
    if chunk is None:
        chunk = 64
        for c in (256, 128):
            if n_tok * nkv * -(-upper_context // c) >= 64:
                chunk = c
                break
    while -(-upper_context // chunk) > MAX_SPLITS:       # tables wider than 2048 * 512 positions: longer chunks
        chunk *= 2
    return chunk, max(1, -(-upper_context // chunk))


def paged_attention_split(q, k_cache, v_cache, positions, item_of_token, table, page_size, n_pages, window, scale,
                          out, part_acc, part_ml, chunk, n_splits, nh, nkv, hd, status, mma: bool = True,
                          fresh: int = 0, overlap_prev: bool = False) -> bool:
    """Split-key attention (one CTA per key chunk, kv head and query token, then an ordered
    combine).  Returns False, having launched nothing, when the group size is above 8.

    out None: the partial results stay in part_acc / part_ml, uncombined, for a consumer that combines them itself
    (linear_of_attention_partials).

    fresh: the most tokens one request brings to this step, when the caller knows that cache rows
    below `position + 1 - fresh` were written before the stream's last copy or foreign kernel (the
    engine's steps start with such a copy).  The tensor-core kernel then requests its first key
    tiles while the kernels before it still run.  0: nothing is assumed.

    overlap_prev: the kernel launched just before this one was attention_prefill with dependents_after_wait and
    returned 2, and it neither writes what this launch reads nor reads what it writes: the tensor-core kernel then
    runs beside it instead of after it (and completes after it)."""
    if nh // nkv > 8:
        return False
    _cuda(q, k_cache, v_cache, positions, item_of_token, table, out, part_acc, part_ml, status)
    use_mma = mma and q.dtype == torch.bfloat16 and hd in (64, 128) and chunk >= 64
    T = q.shape[0]
    _need(q.shape == (T, nh * hd) and (out is None or (out.shape == (T, nh * hd) and out.dtype == q.dtype)),
          "paged_attention_split: q/out shapes")
    _need(k_cache.dtype == q.dtype and v_cache.dtype == q.dtype, "cache dtype must match q")
    _need(k_cache.numel() >= n_pages * page_size * nkv * hd, "cache arena smaller than n_pages")
    _need(table.dtype == torch.int32 and table.dim() == 2, "block table must be int32 [items, blocks]")
    _need(part_acc.dtype == torch.float32 and part_acc.numel() >= T * nh * n_splits * hd
          and part_ml.dtype == torch.float32 and part_ml.numel() >= T * nh * n_splits * 2, "split scratch too small")
    _need(T <= 65535, "paged_attention_split: at most 65535 query tokens per launch")
    _need(1 <= n_splits <= MAX_SPLITS, f"paged_attention_split: 1 to {MAX_SPLITS} key chunks per request, found {n_splits}")
    _need(chunk * n_splits >= table.shape[1] * page_size,
          "paged_attention_split: chunk * n_splits must cover every position the block table can hold")
    if use_mma:
        # bfloat16, head 64/128: the tensor-core version (the scalar one is bound by instruction issue)
        rc = _lib.kernels().imparo_attention_decode_mma(
            _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(positions), _ptr(item_of_token), _ptr(table),
            table.shape[1], page_size, n_pages, int(window or 0), float(scale), _ptr(out), _ptr(part_acc), _ptr(part_ml),
            T, nh, nkv, hd, int(chunk), int(n_splits), int(fresh), int(bool(overlap_prev)), _ptr(status), _stream())
    else:
        rc = _lib.kernels().imparo_paged_attention_split(
            _ptr(q), _ptr(k_cache), _ptr(v_cache), _code(q), _ptr(positions), _ptr(item_of_token), _ptr(table),
            table.shape[1], page_size, n_pages, int(window or 0), float(scale), _ptr(out), _ptr(part_acc), _ptr(part_ml),
            T, nh, nkv, hd, int(chunk), int(n_splits), _ptr(status), _stream())
    _check(rc, "paged_attention_split")
    if out is not None:
        COUNTS["own"] += 1      # partial + combine
    return True


def attention_decode_from_qkv(qkv, positions, item_of_token, q_w, k_w, inv_freq, n_rot, eps, k_cache, v_cache, table,
                              page_size, n_pages, window, scale, out, part_acc, part_ml, chunk, n_splits, nh, nkv, hd,
                              status) -> bool:
    """The split-key attention of a step in which every request brings ONE token, straight from the qkv product's
    split partials: the kernel makes its queries itself (sum in split order, per-head norm, rotation) and writes the
    new key and value rows into their pages, so no q/k kernel runs before it.  Returns False, having launched
    nothing, unless qkv is a PartialProduct in bfloat16 with head size 64 or 128 and at most 8 query heads per kv
    head.  out None: the partial results stay uncombined (linear_of_attention_partials)."""
    if not isinstance(qkv, PartialProduct) or qkv.dtype != torch.bfloat16 or hd not in (64, 128) or nkv < 1 \
            or nh % nkv or nh // nkv > 8 or chunk < 64:
        return False
    T = qkv.shape[0]
    _cuda(qkv.parts, positions, item_of_token, q_w, k_w, inv_freq, k_cache, v_cache, table, out, part_acc, part_ml, status)
    _need(tuple(qkv.shape) == (T, (nh + 2 * nkv) * hd), "attention_decode_from_qkv: the product's width is (heads + 2 kv heads) * head size")
    _need(positions.dtype == torch.int32 and item_of_token.dtype == torch.int32 and positions.numel() >= T
          and item_of_token.numel() >= T, "positions / item_of_token must be int32 per token")
    _need(q_w is None or (q_w.dtype == torch.float32 and q_w.numel() == hd), "q norm weight must be float32 [head]")
    _need(k_w is None or (k_w.dtype == torch.float32 and k_w.numel() == hd), "k norm weight must be float32 [head]")
    _need(inv_freq is None or (inv_freq.dtype == torch.float32 and inv_freq.numel() >= n_rot // 2 and n_rot % 2 == 0
                               and n_rot <= hd), "inv_freq must be float32 [n_rot/2], n_rot even and at most the head size")
    _need(k_cache.dtype == torch.bfloat16 and v_cache.dtype == torch.bfloat16, "cache dtype must match activations")
    _need(k_cache.numel() >= n_pages * page_size * nkv * hd and v_cache.numel() >= n_pages * page_size * nkv * hd,
          "cache arena smaller than n_pages")
    _need(table.dtype == torch.int32 and table.dim() == 2, "block table must be int32 [items, blocks]")
    _need(out is None or (out.shape == (T, nh * hd) and out.dtype == torch.bfloat16), "attention_decode_from_qkv: out shape")
    _need(part_acc.dtype == torch.float32 and part_acc.numel() >= T * nh * n_splits * hd
          and part_ml.dtype == torch.float32 and part_ml.numel() >= T * nh * n_splits * 2, "split scratch too small")
    _need(T <= 65535 and 1 <= n_splits <= MAX_SPLITS, f"at most 65535 tokens and {MAX_SPLITS} key chunks")
    _need(chunk * n_splits >= table.shape[1] * page_size, "chunk * n_splits must cover every position the block table can hold")
    _check(_lib.kernels().imparo_attention_decode_mma_qkv(
        _ptr(qkv.parts), qkv.splits, qkv.stride, _ptr(q_w), _ptr(k_w), _ptr(inv_freq), int(n_rot), float(eps),
        _ptr(k_cache), _ptr(v_cache), _ptr(positions), _ptr(item_of_token), _ptr(table), table.shape[1], page_size, n_pages,
        int(window or 0), float(scale), _ptr(out), _ptr(part_acc), _ptr(part_ml), T, nh, nkv, hd, int(chunk), int(n_splits),
        _ptr(status), _stream()), "attention_decode_from_qkv")
    if out is not None:
        COUNTS["own"] += 1      # partial + combine
    return True


def attention_prefill(q, k_cache, v_cache, item_row_start, item_start_pos, n_items, table, page_size, n_pages, window,
                      scale, out, nh, nkv, hd, status, kernel: str = "auto", dependents_after_wait: bool = False):
    """Tensor-core attention for prompt portions (bfloat16, head size 64 or 128, at most 8
    query heads per kv head).  Returns False, having launched nothing, for other shapes.

    dependents_after_wait: the caller's next kernel works on other rows and may run beside this one
    (paged_attention_split with overlap_prev).  Where the kernel that ran honours it the result is 2 instead of True.

    kernel: "tcgen05" (TMA + tcgen05.mma with the scores in tensor memory; pages of 16, 32, 64 or
    128 positions; at head size 64 a CTA takes two query tiles in turn), "tcgen05_one_tile" (the same with one tile
    per CTA at every head size), "mma" (mma.sync, any page size), or "auto": the first where it takes the shape
    (IMPARO_ATTN_PREFILL=mma in the environment makes "auto" skip it)."""
    if q.dtype != torch.bfloat16 or hd not in (64, 128) or nh // nkv > 8:
        return False
    _cuda(q, k_cache, v_cache, item_row_start, item_start_pos, table, out, status)
    T = q.shape[0]
    _need(q.shape == (T, nh * hd) and out.shape == (T, nh * hd) and out.dtype == q.dtype, "attention_prefill: q/out shapes")
    _need(q.is_contiguous() and out.is_contiguous(), "attention_prefill: q and out must be dense")
    _need(k_cache.dtype == q.dtype and v_cache.dtype == q.dtype, "cache dtype must match q")
    _need(k_cache.numel() >= n_pages * page_size * nkv * hd, "cache arena smaller than n_pages")
    _need(table.dtype == torch.int32 and table.dim() == 2 and table.shape[0] >= n_items, "block table must be int32 [items, blocks]")
    _need(item_row_start.numel() >= n_items + 1 and item_start_pos.numel() >= n_items, "attention_prefill: item arrays")
    _need(kernel in ("auto", "tcgen05", "tcgen05_one_tile", "mma"), "attention_prefill: kernel is auto, tcgen05, tcgen05_one_tile or mma")
    args = (_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(item_row_start), _ptr(item_start_pos), n_items, _ptr(table),
            table.shape[1], page_size, n_pages, int(window or 0), float(scale), _ptr(out), T, nh, nkv, hd, _ptr(status),
            _stream())
    if kernel == "auto":
        kernel = _S.switches.attn_prefill
    if kernel in ("auto", "tcgen05", "tcgen05_one_tile"):
        # two tiles per CTA pay once a request has a thousand keys or so to walk (measured: 4 x 512 tokens 41.8 us with
        # one tile, 45.6 with two; 2,048 tokens 71 against 63.5): "auto" decides by the width of the block table, which is
        # part of the step's shape
        two_tiles = kernel == "tcgen05" or (kernel == "auto" and table.shape[1] * page_size >= 1024)
        late = bool(dependents_after_wait)      # without programmatic launches the two kernels simply run in stream order
        rc = _lib.kernels().imparo_attention_prefill_tc(*args[:-2], (1 if two_tiles else 0) | (2 if late else 0), *args[-2:])
        if rc != -8:
            _check(rc, "attention_prefill_tc")
            return 2 if late else True
        if kernel != "auto":
            return False
    _check(_lib.kernels().imparo_attention_prefill(*args), "attention_prefill")
    return True


def gated_conv(bcx, w, bias, state, item_row_start, item_of_token, item_slot, y, taps, status) -> None:
    """bcx: [tokens, 3*width] rows [b | c | x], a tensor of y's dtype or a PartialProduct."""
    src, parts, part_stride = _parts_of(bcx)
    _cuda(src, w, bias, state, item_row_start, item_of_token, item_slot, y, status)
    T, width = y.shape
    _need(tuple(bcx.shape) == (T, 3 * width) and bcx.dtype == y.dtype, "gated_conv: bcx must be [tokens, 3*width]")
    _need(w.dtype == torch.float32 and w.shape == (width, taps), "gated_conv: taps must be float32 [width, taps]")
    _need(state.dtype == torch.float32 and state.dim() == 3 and state.shape[1:] == (taps - 1, width),
          "gated_conv: state must be float32 [slots, taps-1, width]")
    if bias is not None:
        _need(bias.dtype == torch.float32 and bias.numel() == width, "gated_conv: bias must be float32 [width]")
    _check(_lib.kernels().imparo_gated_conv(
        _ptr(src), _code(y), _ptr(w), _ptr(bias), _ptr(state), _ptr(item_row_start), _ptr(item_of_token),
        _ptr(item_slot), _ptr(y), T, width, taps, state.shape[0], parts, part_stride, _ptr(status), _stream()), "gated_conv")


def zero_state_slots(arena: torch.Tensor, segments: torch.Tensor, n_segments: int, slots: torch.Tensor, n_slots_total: int,
                     status: torch.Tensor, max_per_slot: Optional[int] = None) -> None:
    """Zero, in every state tensor of the arena, the slots named in `slots` (int32 on the device; entries below 0
    are skipped).  segments: int64 [n_segments, 2] on the device: (offset in the arena, floats per slot).
    max_per_slot: the largest of those sizes, which the host knows (it sizes the grid: 1,024 floats per block; without
    it the launch takes the most blocks per tensor and slot, 64, and a step of 32 requests waits 20 us for 20,000
    blocks of which a handful have work)."""
    _cuda(arena, segments, slots, status)
    _need(arena.dtype == torch.float32 and segments.dtype == torch.int64 and slots.dtype == torch.int32, "zero_state_slots: dtypes")
    if n_segments == 0 or slots.numel() == 0:
        return
    _check(_lib.kernels().imparo_zero_state_slots(_ptr(arena), _ptr(segments), int(n_segments),
                                                  int(arena.numel() if max_per_slot is None else max_per_slot), _ptr(slots),
                                                  slots.numel(), int(n_slots_total), _ptr(status), _stream()), "zero_state_slots")


def take_sampled_tokens(token_ids: torch.Tensor, src: torch.Tensor, prev: torch.Tensor) -> None:
    """token_ids[i] = prev[src[i]] where src[i] >= 0 (all int32): rows whose token is the id an
    earlier step sampled take it from that step's output on the device."""
    _cuda(token_ids, src, prev)
    n = token_ids.numel()
    _need(token_ids.dtype == torch.int32 and src.dtype == torch.int32 and prev.dtype == torch.int32 and src.numel() >= n,
          "take_sampled_tokens: int32 ids, one source index per token")
    _check(_lib.kernels().imparo_take_sampled_tokens(_ptr(token_ids), _ptr(src), _ptr(prev), n, prev.numel(), _stream()),
           "take_sampled_tokens")


def sample_rows(logits, temperature, uniform, out) -> None:
    """out[r] = greedy pick where temperature[r] <= 0 (or temperature is None), else the
    inverse-CDF pick of softmax(logits[r] / temperature[r]) at uniform[r]."""
    _cuda(logits, temperature, uniform, out)
    n, vocab = logits.shape
    _need(logits.dtype == torch.float32 and out.dtype == torch.int32 and out.numel() >= n, "sample_rows: dtypes")
    if temperature is None and vocab >= 4096 and n <= 65535:
        # greedy over a large vocabulary: 32 blocks per row, then one warp per row
        key = torch.device(logits.device).index or 0
        buf = _S.argmax_scratch.get(key)
        if buf is None or buf[0].numel() < n * 32:
            _need(not torch.cuda.is_current_stream_capturing(), "argmax scratch would grow during graph capture")
            buf = _S.argmax_scratch[key] = (torch.empty(max(n, 256) * 32, dtype=torch.float32, device=logits.device),
                                          torch.empty(max(n, 256) * 32, dtype=torch.int32, device=logits.device))
        _check(_lib.kernels().imparo_argmax_rows(_ptr(logits), _ptr(out), _ptr(buf[0]), _ptr(buf[1]), n, vocab,
                                                 logits.stride(0), _stream()), "argmax_rows")
        COUNTS["own"] += 1
        return
    if temperature is not None:
        _need(temperature.dtype == torch.float32 and uniform is not None and uniform.dtype == torch.float32
              and temperature.numel() >= n and uniform.numel() >= n, "sample_rows: temperature/uniform float32 per row")
        if vocab >= 4096 and n <= 65535:
            # a large vocabulary: 32 blocks per row take a stretch each, then a block per row picks
            key = torch.device(logits.device).index or 0
            buf = _S.sample_scratch.get(key)
            if buf is None or buf[1].numel() < n * 32:
                _need(not torch.cuda.is_current_stream_capturing(), "sampling scratch would grow during graph capture")
                buf = _S.sample_scratch[key] = (torch.empty(max(n, 256) * 64, dtype=torch.float32, device=logits.device),
                                                torch.empty(max(n, 256) * 32, dtype=torch.int32, device=logits.device))
            _check(_lib.kernels().imparo_sample_rows_parts(_ptr(logits), _ptr(temperature), _ptr(uniform), _ptr(out),
                                                           _ptr(buf[0]), _ptr(buf[1]), n, vocab, logits.stride(0), _stream()),
                   "sample_rows_parts")
            COUNTS["own"] += 1
            return
    _check(_lib.kernels().imparo_sample_rows(_ptr(logits), _ptr(temperature), _ptr(uniform), _ptr(out), n, vocab,
                                             logits.stride(0), _stream()), "sample_rows")
