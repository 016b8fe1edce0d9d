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
        self.pending_mean = {}       # data_ptr -> arguments of a norm_mean_add the next reader of the stream carries out
        self.pending_mix = {}        # data_ptr -> arguments of a streams_mix_add the next reader of the stream carries out
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
    _S.pending_mean.pop(out.data_ptr(), None)
    _S.pending_mix.pop(out.data_ptr(), None)
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
    """Fold pending partials into the stream, carry out a pending norm_mean_add (no-op when there is none)."""
    pm = _S.pending_mean.pop(stream.data_ptr(), None)
    if pm is not None:
        norm_mean_add(stream, *pm)
    px = _S.pending_mix.pop(stream.data_ptr(), None)
    if px is not None:
        streams_mix_add(stream, *px)
    p = _S.pending.pop(stream.data_ptr(), None)
    if p is not None:
        scratch, S, T, N = p
        _check(_lib.kernels().imparo_add_partials_rmsnorm(_ptr(stream), _ptr(scratch), S, T * N, None, 0.0, None, 0, T, N,
                                                          _stream()), "add_partials")


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float, out: torch.Tensor,
            rows: Optional[torch.Tensor] = None) -> None:
    _cuda(x, w, out, rows)
    pm = _S.pending_mean.get(x.data_ptr())
    if pm is not None:
        if rows is None and out.shape == x.shape and w.numel() == x.shape[1] and w.dtype == torch.float32:
            # the add that was left pending and the norm of the updated rows in one pass over the stream
            import ctypes
            _S.pending_mean.pop(x.data_ptr())
            branches, weights, b_eps, coef, extra, extra_coef = pm
            bp = (ctypes.c_void_p * 4)(*[b.data_ptr() for b in branches])
            wp = (ctypes.c_void_p * 4)(*[t.data_ptr() for t in weights])
            _check(_lib.kernels().imparo_norm_mean_add_rmsnorm(_ptr(x), len(branches), bp, wp, float(b_eps), float(coef), _ptr(extra),
                                                               float(extra_coef), _ptr(w), float(eps), _ptr(out), _code(out),
                                                               x.shape[0], x.shape[1], _stream()), "norm_mean_add_rmsnorm")
            return
        settle(x)
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


GATED_ACTIVATIONS = {"silu": 0, "gelu_tanh": 1, "clamped_swish": 2}


def gated_act(gu: torch.Tensor, out: torch.Tensor, kind: str = "silu", limit: float = 0.0, bias: Optional[torch.Tensor] = None) -> None:
    """out[T, F] = act(gate, up) of gu = [gate | up] rows ([T, 2F]), after adding bias (float32 [2F]) when given.
    kind: "silu" silu(g) u; "gelu_tanh" gelu(g) u; "clamped_swish" with g' = min(g, limit), u' = clamp(u, -limit, limit):
    g' sigmoid(1.702 g') (u' + 1)."""
    _cuda(gu, out)
    _need(kind in GATED_ACTIVATIONS, f"gated_act: unknown kind '{kind}' (known: {', '.join(sorted(GATED_ACTIVATIONS))})")
    n, F = out.shape
    _need(gu.shape == (n, 2 * F) and gu.dtype == out.dtype, "gated_act: gu must be [tokens, 2F] of the output dtype")
    if bias is not None:
        _cuda(bias)
        _need(bias.dtype == torch.float32 and bias.numel() == 2 * F, "gated_act: bias float32 [2F]")
    _check(_lib.kernels().imparo_gated_act(_ptr(gu), _ptr(bias), _ptr(out), _code(out), n, F, GATED_ACTIVATIONS[kind], float(limit),
                                           _stream()), "gated_act")


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
            scratch: Optional[torch.Tensor] = None, act: str = "silu", limit: float = 0.0, bias: Optional[torch.Tensor] = None) -> None:
    """The hand-written tensor-core product (csrc/kernels/gemm_tcgen05.cu).
    epilogue: EPI_STORE_BF16 | EPI_STORE_F32 | EPI_ADD_F32 (out += x w^T) | EPI_SWIGLU
    (w = [gate rows; up rows] of shape [2F, K], out = act(x gate^T + b_g, x up^T + b_u), [T, F]; act one of gated_act's kinds,
    "silu" by default; bias float32 [2F] or None)."""
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
    if epilogue == EPI_SWIGLU and (act != "silu" or bias is not None):
        if bias is not None:
            _cuda(bias)
            _need(bias.dtype == torch.float32 and bias.numel() == 2 * N and bias.is_contiguous(), "gemm_tc: bias float32 [2N]")
        _check(_lib.kernels().imparo_gemm_tc_gated(_ptr(x), x.stride(0), rows_alloc, _ptr(w), _ptr(out), out.stride(0), T, N, K,
                                                   GATED_ACTIVATIONS[act], float(limit), _ptr(bias), _ptr(scratch), _ptr(cnt),
                                                   _ptr(status), _stream()), "gemm_tc_gated")
        return
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


def gemm_prefill(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int, status: Optional[torch.Tensor] = None,
                 act: str = "silu", limit: float = 0.0, bias: Optional[torch.Tensor] = None) -> None:
    """The persistent tensor-core product for many tokens.  epilogue: EPI_STORE_BF16 | EPI_STORE_F32 |
    EPI_ADD_F32 (out += x w^T) | EPI_SWIGLU (w = [gate rows; up rows], out = act(x gate^T + b_g, x up^T + b_u) with act one of
    gated_act's kinds, "silu" by default, and bias float32 [2N] or None)."""
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
    if bias is not None:
        _cuda(bias)
        _need(epilogue == EPI_SWIGLU and bias.dtype == torch.float32 and bias.numel() == 2 * N and bias.is_contiguous(),
              "gemm_prefill: bias float32 [2N] with the gated epilogue")
    _check(_lib.kernels().imparo_gemm_prefill(_ptr(x), x.stride(0), rows_alloc, _ptr(w), _ptr(out), out.stride(0), T, N, K,
                                              epilogue, GATED_ACTIVATIONS[act], float(limit), _ptr(bias), _ptr(status), _stream()),
           "gemm_prefill")


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


def linear_gated(x, w_gu: torch.Tensor, out: torch.Tensor, kind: str, limit: float = 0.0, bias: Optional[torch.Tensor] = None,
                 status: Optional[torch.Tensor] = None, tmp=None) -> None:
    """out[T, F] = act(x gate^T + b_g, x up^T + b_u) with w_gu = [gate; up] ([2F, K]), bias float32 [2F] or None, for the
    gated activations of gated_act: the product into tmp [T, 2F] (a tensor, or a function that makes it), then one kernel
    that adds the biases and applies the activation.  For many bfloat16 tokens: the persistent tensor-core product with the
    biases and the activation in its epilogue (one launch, no [T, 2F] tensor); for few: the weight-streaming tensor-core
    product with the same epilogue."""
    if x.dtype == torch.bfloat16 and gemm_backend() == "tcgen05" and tc_usable(x, w_gu):
        gemm_tc(x, w_gu, out, EPI_SWIGLU, status, act=kind, limit=limit, bias=bias)
        return
    if prefill_tc_usable(x, w_gu, out, swiglu=True):
        gemm_prefill(x, w_gu, out, EPI_SWIGLU, status, act=kind, limit=limit, bias=bias)
        return
    if callable(tmp):
        tmp = tmp()
    _need(tmp is not None and tmp.shape == (x.shape[0], w_gu.shape[0]), "linear_gated: tmp [T, 2F] needed")
    linear(x, w_gu, tmp, status=status)
    gated_act(tmp, out, kind, limit, bias)


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


def attention_split_combine(part_acc, part_ml, out, n_rows, hd, n_splits, sink: bool = False) -> None:
    """The ordered combine alone: out[row, :] from the partials of paged_attention_split(out=None).  sink: the softmax's
    denominator counts one more term of score 0 that has no value."""
    _cuda(part_acc, part_ml, out)
    _check(_lib.kernels().imparo_attention_split_combine(_ptr(part_acc), _ptr(part_ml), _ptr(out), _code(out), n_rows, hd,
                                                         n_splits, int(bool(sink)), _stream()), "attention_split_combine")


def head_groups(nh: int, nkv: int, most: int = 8) -> int:
    """Into how many groups the query heads of one kv head are cut so that a group has at most `most` heads: the fewest
    that divide them evenly (1 when they fit as they are)."""
    per = nh // nkv
    for g in range(1, per + 1):
        if per % g == 0 and per // g <= most:
            return g
    return per


def paged_attention_split_shared(q, k_cache, v_cache, positions, item_of_token, table, page_size, n_pages, window, scale,
                                 out, part_acc, part_ml, chunk, n_splits, nh, nkv, hd, status, fresh: int = 0,
                                 softcap: float = 0.0, sink_values: Optional[torch.Tensor] = None) -> bool:
    """Split-key attention on tensor cores for any number of query heads per kv head: the heads of a kv head are cut into
    groups of at most 8 (head_groups), each group a CTA row of its own over the same cached head, so an attention whose
    heads all share one cached row per position (nkv = 1) still spreads over heads x key chunks CTAs.  Then the ordered
    combine, with one more term per head in the denominator when sink_values (float32 [nh], unscaled scores) is given.
    bfloat16, head size 64 or 128, chunk >= 64; returns False, having launched nothing, for other shapes."""
    if not (q.dtype == torch.bfloat16 and hd in (64, 128) and chunk >= 64):
        return False
    _cuda(q, k_cache, v_cache, positions, item_of_token, table, out, part_acc, part_ml, status, sink_values)
    T = q.shape[0]
    groups = head_groups(nh, nkv)
    _need(q.shape == (T, nh * hd) and out.shape == (T, nh * hd) and out.dtype == q.dtype, "paged_attention_split_shared: q/out shapes")
    _need(k_cache.dtype == q.dtype and v_cache.dtype == q.dtype, "cache dtype must match q")
    _need(k_cache.numel() >= n_pages * page_size * nkv * hd, "cache arena smaller than n_pages")
    _need(table.dtype == torch.int32 and table.dim() == 2, "block table must be int32 [items, blocks]")
    _need(part_acc.dtype == torch.float32 and part_acc.numel() >= T * nh * n_splits * hd
          and part_ml.dtype == torch.float32 and part_ml.numel() >= T * nh * n_splits * 2, "split scratch too small")
    _need(T <= 65535 and 1 <= n_splits <= MAX_SPLITS and chunk * n_splits >= table.shape[1] * page_size,
          "paged_attention_split_shared: tokens, chunks and their cover of the block table")
    _need(sink_values is None or (sink_values.dtype == torch.float32 and sink_values.numel() == nh), "sink values float32 [heads]")
    _check(_lib.kernels().imparo_attention_decode_mma_grouped(
        _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(positions), _ptr(item_of_token), _ptr(table), table.shape[1], page_size,
        n_pages, int(window or 0), float(scale), _ptr(part_acc), _ptr(part_ml), T, nh, nkv * groups, groups, hd, int(chunk),
        int(n_splits), int(fresh), float(softcap or 0.0), _ptr(status), _stream()), "attention_decode_mma_grouped")
    if sink_values is not None:
        _check(_lib.kernels().imparo_attention_split_combine_sinks(_ptr(part_acc), _ptr(part_ml), _ptr(out), _code(out), T * nh, hd,
                                                                   n_splits, _ptr(sink_values), nh, _stream()),
               "attention_split_combine_sinks")
    else:
        attention_split_combine(part_acc, part_ml, out, T * nh, hd, n_splits)
    return True


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
                          fresh: int = 0, overlap_prev: bool = False, sink: bool = False, softcap: float = 0.0) -> bool:
    """Split-key attention (one CTA per key chunk, kv head and query token, then an ordered
    combine).  Returns False, having launched nothing, when the group size is above 8, or when a soft cap on the scores
    (softcap c > 0: c * tanh(score / c)) is asked of the kernel without tensor cores, which has none.

    out None: the partial results stay in part_acc / part_ml, uncombined, for a consumer that combines them itself
    (linear_of_attention_partials).

    fresh: the most tokens one request brings to this step, when the caller knows that cache rows
    below `position + 1 - fresh` were written before the stream's last copy or foreign kernel (the
    engine's steps start with such a copy).  The tensor-core kernel then requests its first key
    tiles while the kernels before it still run.  0: nothing is assumed.

    overlap_prev: the kernel launched just before this one was attention_prefill with dependents_after_wait and
    returned 2, and it neither writes what this launch reads nor reads what it writes: the tensor-core kernel then
    runs beside it instead of after it (and completes after it).

    sink: the softmax's denominator counts one more term of score 0 that has no value; it enters in the combine, so
    the partials are left uncombined by the first kernel and the combine runs as a launch of its own (out is needed)."""
    if nh // nkv > 8:
        return False
    if softcap and not (mma and q.dtype == torch.bfloat16 and hd in (64, 128) and chunk >= 64):
        return False
    if sink:
        _need(out is not None, "paged_attention_split: a sink is added by the combine, which needs out")
        ok = paged_attention_split(q, k_cache, v_cache, positions, item_of_token, table, page_size, n_pages, window, scale,
                                   None, part_acc, part_ml, chunk, n_splits, nh, nkv, hd, status, mma=mma, fresh=fresh,
                                   overlap_prev=overlap_prev, softcap=softcap)
        if ok:
            attention_split_combine(part_acc, part_ml, out, q.shape[0] * nh, hd, n_splits, sink=True)
        return ok
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
        rc = _lib.kernels().imparo_attention_decode_mma_capped(
            _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(positions), _ptr(item_of_token), _ptr(table),
            table.shape[1], page_size, n_pages, int(window or 0), float(scale), _ptr(out), _ptr(part_acc), _ptr(part_ml),
            T, nh, nkv, hd, int(chunk), int(n_splits), int(fresh), int(bool(overlap_prev)), float(softcap or 0.0), _ptr(status),
            _stream())
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
                      scale, out, nh, nkv, hd, status, kernel: str = "auto", dependents_after_wait: bool = False,
                      sink: bool = False, softcap: float = 0.0, sink_values: Optional[torch.Tensor] = None, max_group: int = 8):
    """Tensor-core attention for prompt portions (bfloat16, head size 64 or 128, at most 8
    query heads per kv head).  Returns False, having launched nothing, for other shapes.

    dependents_after_wait: the caller's next kernel works on other rows and may run beside this one
    (paged_attention_split with overlap_prev).  Where the kernel that ran honours it the result is 2 instead of True.

    kernel: "tcgen05" (TMA + tcgen05.mma with the scores in tensor memory; pages of 16, 32, 64 or
    128 positions; at head size 64 a CTA takes two query tiles in turn), "tcgen05_one_tile" (the same with one tile
    per CTA at every head size), "mma" (mma.sync, any page size), or "auto": the first where it takes the shape
    (IMPARO_ATTN_PREFILL=mma in the environment makes "auto" skip it).

    sink: the softmax's denominator counts one more term of score 0 that has no value (the tcgen05 kernels only;
    where they decline the result is False).  softcap c > 0: the scaled score becomes c * tanh(score / c) (the tcgen05
    kernels only, likewise).  sink_values: float32 [nh], the extra term's score per head, unscaled (implies sink).

    max_group: the most query heads per kv head the caller wants on this kernel (the tcgen05 kernels take up to 128: a tile
    is 128 / group tokens of the group's heads, which pays when all heads share one cached row; the mma kernel takes 8)."""
    if q.dtype != torch.bfloat16 or hd not in (64, 128) or nh // nkv > min(max_group, 128):
        return False
    sink = bool(sink) or sink_values is not None
    only_tc = sink or bool(softcap) or nh // nkv > 8      # variants that only the tcgen05 kernels have
    if only_tc and kernel == "auto" and _S.switches.attn_prefill == "mma":
        return False
    _cuda(q, k_cache, v_cache, item_row_start, item_start_pos, table, out, status, sink_values)
    T = q.shape[0]
    _need(sink_values is None or (sink_values.dtype == torch.float32 and sink_values.numel() == nh), "attention_prefill: sink values float32 [heads]")
    _need(q.shape == (T, nh * hd) and out.shape == (T, nh * hd) and out.dtype == q.dtype, "attention_prefill: q/out shapes")
    _need(q.is_contiguous() and out.is_contiguous(), "attention_prefill: q and out must be dense")
    _need(k_cache.dtype == q.dtype and v_cache.dtype == q.dtype, "cache dtype must match q")
    _need(k_cache.numel() >= n_pages * page_size * nkv * hd, "cache arena smaller than n_pages")
    _need(table.dtype == torch.int32 and table.dim() == 2 and table.shape[0] >= n_items, "block table must be int32 [items, blocks]")
    _need(item_row_start.numel() >= n_items + 1 and item_start_pos.numel() >= n_items, "attention_prefill: item arrays")
    _need(kernel in ("auto", "tcgen05", "tcgen05_one_tile", "mma"), "attention_prefill: kernel is auto, tcgen05, tcgen05_one_tile or mma")
    head = (_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(item_row_start), _ptr(item_start_pos), n_items, _ptr(table),
            table.shape[1], page_size, n_pages, int(window or 0), float(scale))
    tail = (_ptr(out), T, nh, nkv, hd, _ptr(status), _stream())
    args = head + tail
    if kernel == "auto":
        kernel = _S.switches.attn_prefill
    if kernel in ("auto", "tcgen05", "tcgen05_one_tile"):
        # two tiles per CTA pay once a request has a thousand keys or so to walk (measured: 4 x 512 tokens 41.8 us with
        # one tile, 45.6 with two; 2,048 tokens 71 against 63.5): "auto" decides by the width of the block table, which is
        # part of the step's shape
        two_tiles = kernel == "tcgen05" or (kernel == "auto" and table.shape[1] * page_size >= 1024)
        late = bool(dependents_after_wait)      # without programmatic launches the two kernels simply run in stream order
        rc = _lib.kernels().imparo_attention_prefill_tc_sinks(*head, float(softcap or 0.0), _ptr(sink_values), *tail[:-2],
                                                              (1 if two_tiles else 0) | (2 if late else 0) | (4 if sink else 0), *tail[-2:])
        if rc != -8:
            _check(rc, "attention_prefill_tc")
            return 2 if late else True
        if kernel != "auto" or only_tc:
            return False
    if only_tc:
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


# ---- stream operations of arrangements other than the pre-norm block (csrc/kernels/stream_ops.cu) ----------
ACTIVATIONS = {"relu2": 0, "gelu_tanh": 1, "silu": 2}


def activation(x: torch.Tensor, out: torch.Tensor, kind: str) -> None:
    """out = act(x) elementwise (relu2: relu(x)^2, gelu_tanh, silu); out may be x.  x may be a [rows, width] stretch of
    wider rows (a column range of a product that several consumers share); out is then dense [rows, width]."""
    _need(kind in ACTIVATIONS, f"activation: unknown kind '{kind}' (known: {', '.join(sorted(ACTIVATIONS))})")
    _need(x.shape == out.shape and x.dtype == out.dtype, "activation: out must match x")
    if x.dim() == 2 and not x.is_contiguous():
        _need(x.is_cuda and out.is_cuda and out.is_contiguous() and x.stride(1) == 1, "activation: rows of x must be dense")
        _check(_lib.kernels().imparo_act_rows_strided(_ptr(x), x.stride(0), _ptr(out), _code(x), x.shape[0], x.shape[1],
                                                      ACTIVATIONS[kind], _stream()), "activation")
        return
    _cuda(x, out)
    _check(_lib.kernels().imparo_act_rows(_ptr(x), _ptr(out), _code(x), x.numel(), ACTIVATIONS[kind], _stream()), "activation")


def gated_rmsnorm(o: torch.Tensor, w: torch.Tensor, eps: float, gate: torch.Tensor, out: torch.Tensor) -> None:
    """out[r] = o[r] / rms(o[r]) * w * sigmoid(gate[r]).  o: float32 [rows, width]; gate: [rows, width] of out's
    dtype, rows may be strided (a stretch of a wider product)."""
    _need(o.is_cuda and gate.is_cuda and out.is_cuda and w.is_cuda, "kernels run on CUDA tensors only (there is no CPU path)")
    n, width = out.shape
    _need(o.dtype == torch.float32 and o.shape == (n, width) and o.is_contiguous() and out.is_contiguous(), "gated_rmsnorm: o float32 [rows, width]")
    _need(w.dtype == torch.float32 and w.numel() == width, "gated_rmsnorm: weight float32 [width]")
    _need(gate.shape == (n, width) and gate.dtype == out.dtype and gate.stride(1) == 1, "gated_rmsnorm: gate [rows, width] of the output dtype")
    _check(_lib.kernels().imparo_gated_rmsnorm(_ptr(o), _ptr(w), float(eps), _ptr(gate), gate.stride(0), _ptr(out), _code(out),
                                               n, width, _stream()), "gated_rmsnorm")


def norm_mean_add(x: torch.Tensor, branches, weights, eps: float, coef: float, extra: Optional[torch.Tensor] = None,
                  extra_coef: float = 0.0, defer: bool = False) -> None:
    """x += coef * sum_b rms(branches[b]) * weights[b] + extra_coef * extra, row by row; all float32 [rows, width],
    up to four branches.

    defer: when the caller of this part has promised (allow_deferred_add) that whatever reads x next goes through
    ops.rmsnorm, ops.settle or another launcher that settles, the add is only noted; ops.rmsnorm then carries it out and
    norms the updated rows in the same kernel.  The branches and extra must stay untouched until then."""
    import ctypes
    settle(x)
    if defer and x.data_ptr() in _S.deferrable and x.is_contiguous():
        _S.pending_mean[x.data_ptr()] = (list(branches), list(weights), eps, coef, extra, extra_coef)
        return
    _cuda(x, extra, *branches, *weights)
    n, width = x.shape
    _need(1 <= len(branches) <= 4 and len(weights) == len(branches), "norm_mean_add: one to four branches, a weight each")
    for b, w in zip(branches, weights):
        _need(b.dtype == torch.float32 and b.shape == (n, width) and w.dtype == torch.float32 and w.numel() == width,
              "norm_mean_add: branches float32 [rows, width], weights float32 [width]")
    _need(x.dtype == torch.float32 and (extra is None or (extra.dtype == torch.float32 and extra.shape == (n, width))),
          "norm_mean_add: stream and extra are float32 [rows, width]")
    bp = (ctypes.c_void_p * 4)(*[b.data_ptr() for b in branches])
    wp = (ctypes.c_void_p * 4)(*[w.data_ptr() for w in weights])
    _check(_lib.kernels().imparo_norm_mean_add(_ptr(x), len(branches), bp, wp, float(eps), float(coef), _ptr(extra),
                                               float(extra_coef), n, width, _stream()), "norm_mean_add")


def add_scaled(x: torch.Tensor, y: torch.Tensor, coef: float) -> None:
    """x += coef * y (float32, same shape)."""
    settle(x)
    _cuda(x, y)
    _need(x.dtype == torch.float32 and y.dtype == torch.float32 and x.shape == y.shape, "add_scaled: float32 tensors of one shape")
    _check(_lib.kernels().imparo_add_scaled(_ptr(x), _ptr(y), float(coef), x.numel(), _stream()), "add_scaled")


def add_weighted(x: torch.Tensor, ys, coefs) -> None:
    """x += sum_b coefs[b] * ys[b] for one to four float32 tensors of x's shape, in one pass over x."""
    settle(x)
    _cuda(x, *ys)
    _need(1 <= len(ys) <= 4 and len(coefs) == len(ys), "add_weighted: one to four sources, a factor each")
    _need(x.dtype == torch.float32 and x.is_contiguous() and all(y.dtype == torch.float32 and y.shape == x.shape and y.is_contiguous() for y in ys),
          "add_weighted: float32 tensors of one shape")
    p = [_ptr(y) for y in ys] + [None] * (4 - len(ys))
    c = [float(v) for v in coefs] + [0.0] * (4 - len(ys))
    _check(_lib.kernels().imparo_add_weighted(_ptr(x), p[0], p[1], p[2], p[3], len(ys), c[0], c[1], c[2], c[3], x.numel(), _stream()),
           "add_weighted")


def stream_inject(x: torch.Tensor, table: Optional[torch.Tensor], ids: Optional[torch.Tensor], vec: Optional[torch.Tensor],
                  status: torch.Tensor) -> None:
    """x[t] += table[ids[t]] (when table is given) + vec (when given).  x: float32 [tokens, width]."""
    settle(x)
    _cuda(x, table, ids, vec, status)
    n, width = x.shape
    _need(x.dtype == torch.float32, "stream_inject: the stream is float32")
    if table is not None:
        _need(table.shape[1] == width and ids is not None and ids.dtype == torch.int32 and ids.numel() >= n,
              "stream_inject: table [vocab, width], int32 ids per row")
    _need(vec is None or (vec.dtype == torch.float32 and vec.numel() == width), "stream_inject: vec float32 [width]")
    _check(_lib.kernels().imparo_stream_inject(_ptr(x), _ptr(table), _code(table) if table is not None else F32, _ptr(ids),
                                               _ptr(vec), n, width, table.shape[0] if table is not None else 0, _ptr(status),
                                               _stream()), "stream_inject")


def softcap(x: torch.Tensor, cap: float) -> None:
    """x = cap * tanh(x / cap) in place (float32)."""
    _cuda(x)
    _need(x.dtype == torch.float32, "softcap: float32 logits")
    _check(_lib.kernels().imparo_softcap(_ptr(x), x.numel(), float(cap), _stream()), "softcap")


# ---- attention of any shape and variant (csrc/kernels/attention_any.cu) ------------------------------------
def qkv_rotate_store(qkv, positions, item_of_token, inv_freq, n_rot, interleaved, magnitude, q_out, k_cache, v_cache,
                     table, page_size, n_pages, nh, nkv, hd, vd, status) -> None:
    """qkv [T, nh*hd + nkv*hd + nkv*vd] -> q_out [T, nh*hd] rotated; k rotated and v written into their pages
    (K rows nkv*hd wide, V rows nkv*vd wide).  Rotation over the first n_rot dims: pairs (2i, 2i+1) when interleaved,
    else (i, i + n_rot/2); sines and cosines times magnitude.  nkv == 0: queries only.  qkv may be a column range of a
    wider product (rows dense, any row stride)."""
    _need(qkv.is_cuda and qkv.stride(1) == 1, "qkv_rotate_store: rows of qkv must be dense CUDA memory")
    _cuda(positions, item_of_token, inv_freq, q_out, k_cache, v_cache, table, status)
    T = q_out.shape[0]
    _need(tuple(qkv.shape) == (T, nh * hd + nkv * (hd + vd)) and q_out.shape[1] == nh * hd and qkv.dtype == q_out.dtype,
          "qkv_rotate_store: widths")
    _need(positions.dtype == torch.int32 and item_of_token.dtype == torch.int32 and positions.numel() >= T
          and item_of_token.numel() >= T, "positions / item_of_token must be int32 per token")
    if nkv:
        _need(k_cache.dtype == qkv.dtype and v_cache.dtype == qkv.dtype, "cache dtype must match activations")
        _need(k_cache.numel() >= n_pages * page_size * nkv * hd and v_cache.numel() >= n_pages * page_size * nkv * vd,
              "cache arena smaller than n_pages")
        _need(table.dtype == torch.int32 and table.dim() == 2, "block table must be int32 [items, blocks]")
    if inv_freq is not None:
        _need(inv_freq.dtype == torch.float32 and inv_freq.numel() >= n_rot // 2, "inv_freq must be float32 [n_rot/2]")
    _check(_lib.kernels().imparo_qkv_rotate_store(
        _ptr(qkv), _code(q_out), _ptr(positions), _ptr(item_of_token), _ptr(inv_freq), int(n_rot), int(bool(interleaved)),
        float(magnitude), _ptr(q_out), _ptr(k_cache), _ptr(v_cache), _ptr(table), table.shape[1] if table is not None else 0,
        page_size, n_pages, T, nh, nkv, hd, vd, qkv.stride(0), _ptr(status), _stream()), "qkv_rotate_store")


def attention_any(q, k_cache, v_cache, positions, item_of_token, table, page_size, n_pages, window, scale, sink,
                  out, nh, nkv, hd, vd, status, softcap: float = 0.0, sink_values: Optional[torch.Tensor] = None) -> None:
    """General attention: any head size hd and value size vd up to 640, optional window, optional sink (one more
    term in the softmax's denominator that has no value: of score 0, or with sink_values, float32 [nh], of the head's
    own number, exp(value)), optional soft cap c > 0 on the scaled scores (c * tanh(score / c)).  out [T, nh*vd].
    k_cache and v_cache may be the same tensor (keys that are their own values)."""
    _cuda(q, k_cache, v_cache, positions, item_of_token, table, out, status, sink_values)
    _need(sink_values is None or (sink_values.dtype == torch.float32 and sink_values.numel() == nh), "attention_any: sink values float32 [heads]")
    T = q.shape[0]
    _need(q.shape == (T, nh * hd) and out.shape == (T, nh * vd) and out.dtype == q.dtype, "attention_any: q/out shapes")
    _need(k_cache.dtype == q.dtype and v_cache.dtype == q.dtype, "cache dtype must match q")
    _need(k_cache.numel() >= n_pages * page_size * nkv * hd and v_cache.numel() >= n_pages * page_size * nkv * vd,
          "cache arena smaller than n_pages")
    _need(table.dtype == torch.int32 and table.dim() == 2, "block table must be int32 [items, blocks]")
    _check(_lib.kernels().imparo_attention_any(
        _ptr(q), _ptr(k_cache), _ptr(v_cache), _code(q), _ptr(positions), _ptr(item_of_token), _ptr(table),
        table.shape[1], page_size, n_pages, int(window or 0), float(scale), int(bool(sink) or sink_values is not None),
        _ptr(sink_values), float(softcap or 0.0), _ptr(out), T, nh, nkv, hd, vd, _ptr(status), _stream()), "attention_any")


def qkv_prepare_store(qkv, bias, positions, item_of_token, inv_freq, n_rot, unit_eps, v_other, v_lambda, v_save, q_out,
                      k_cache, v_cache, table, page_size, n_pages, nh, nkv, hd, vd, status, v_from_k: bool = False) -> None:
    """qkv: float32 [T, nh*hd + nkv*hd + nkv*vd] (a 32-bit product; rows dense, any row stride).  Per head, in 32-bit:
    + bias (float32 over the same columns, or None), half-split rotation of the first n_rot dimensions of q and k, then
    q and k divided by sqrt(mean(square) + unit_eps) (unit_eps None: kept as they are); q -> q_out [T, nh*hd], k and v
    into their pages.  v_other ([T, nkv*vd], the cache's dtype) with v_lambda (a float32 scalar on the device) blends
    the values: v = (1 - lambda) v + lambda v_other; v_save ([T, nkv*vd]) receives the values before blending.
    v_from_k: qkv is [T, nh*hd + nkv*hd] and the values are the keys as they stand before the rotation (vd == hd)."""
    _need(qkv.is_cuda and qkv.stride(1) == 1 and qkv.dtype == torch.float32, "qkv_prepare_store: a float32 product with dense rows")
    _cuda(bias, positions, item_of_token, inv_freq, v_other, v_lambda, v_save, q_out, k_cache, v_cache, table, status)
    T = q_out.shape[0]
    width = nh * hd + nkv * (hd + (0 if v_from_k else vd))
    _need(not v_from_k or vd == hd, "qkv_prepare_store: keys as values need equal sizes")
    _need(tuple(qkv.shape) == (T, width) and q_out.shape[1] == nh * hd, "qkv_prepare_store: widths")
    _need(bias is None or (bias.dtype == torch.float32 and bias.numel() == width), "qkv_prepare_store: bias float32 over the product's columns")
    _need(positions.dtype == torch.int32 and item_of_token.dtype == torch.int32 and positions.numel() >= T
          and item_of_token.numel() >= T, "positions / item_of_token must be int32 per token")
    _need(k_cache.dtype == q_out.dtype and v_cache.dtype == q_out.dtype, "cache dtype must match activations")
    _need(k_cache.numel() >= n_pages * page_size * nkv * hd and v_cache.numel() >= n_pages * page_size * nkv * vd,
          "cache arena smaller than n_pages")
    _need(table.dtype == torch.int32 and table.dim() == 2, "block table must be int32 [items, blocks]")
    for t in (v_other, v_save):
        _need(t is None or (t.dtype == q_out.dtype and t.numel() >= T * nkv * vd), "qkv_prepare_store: v_other / v_save [T, nkv*vd]")
    _need(v_other is None or (v_lambda is not None and v_lambda.dtype == torch.float32 and v_lambda.numel() >= 1),
          "qkv_prepare_store: blending needs a float32 scalar on the device")
    if inv_freq is not None:
        _need(inv_freq.dtype == torch.float32 and inv_freq.numel() >= n_rot // 2, "inv_freq must be float32 [n_rot/2]")
    _check(_lib.kernels().imparo_qkv_prepare_store(
        _ptr(qkv), qkv.stride(0), _ptr(bias), _code(q_out), _ptr(positions), _ptr(item_of_token), _ptr(inv_freq), int(n_rot),
        -1.0 if unit_eps is None else float(unit_eps), _ptr(v_other), _ptr(v_lambda), _ptr(v_save), _ptr(q_out), _ptr(k_cache),
        _ptr(v_cache), _ptr(table), table.shape[1], page_size, n_pages, T, nh, nkv, hd, vd, int(bool(v_from_k)), _ptr(status),
        _stream()), "qkv_prepare_store")


# ---- linear attention with decay (csrc/kernels/linear_attention.cu) -------------------------------------------
def linear_attention(qkv: torch.Tensor, q_off: int, k_off: int, v_off: int, decay: torch.Tensor, state: torch.Tensor,
                     item_row_start, item_slot, n_items: int, out: torch.Tensor, heads: int, dim: int, vdim: int,
                     status: torch.Tensor, act: Optional[str] = "silu", chunk: int = 0,
                     chunk_state: Optional[torch.Tensor] = None) -> None:
    """Per request and head: S = decay * S + k v^T, o = S^T q over the request's rows in order, from and into
    state[slot].  qkv: [T, width] rows holding q (heads*dim) at column q_off, k at k_off, v (heads*vdim) at v_off;
    act: "silu" or None, applied to q, k and v.  state: float32 [slots, heads, dim, vdim]; out: float32 [T, heads*vdim].

    chunk > 0 (batches with long portions): the rows of a request are cut into chunks of that many rows which run side by
    side (three launches: every chunk's own sum, a scan over each request's chunks, every chunk's outputs); chunk_state is
    float32 scratch for (T // chunk + n_items) * heads * dim * vdim values.  The result differs from the row-by-row walk
    by the order of 32-bit additions only."""
    _need(qkv.is_cuda and qkv.stride(1) == 1, "kernels run on CUDA tensors only (there is no CPU path)")
    _cuda(decay, state, item_row_start, item_slot, out, status)
    T = qkv.shape[0]
    _need(act in ("silu", None), "linear_attention: act is 'silu' or None")
    _need(decay.dtype == torch.float32 and decay.numel() == heads, "linear_attention: decay float32 [heads]")
    _need(state.dtype == torch.float32 and tuple(state.shape[1:]) == (heads, dim, vdim), "linear_attention: state float32 [slots, heads, dim, vdim]")
    _need(out.dtype == torch.float32 and out.shape == (T, heads * vdim), "linear_attention: out float32 [tokens, heads*vdim]")
    _need(max(q_off, k_off) + heads * dim <= qkv.shape[1] and v_off + heads * vdim <= qkv.shape[1], "linear_attention: offsets")
    _need(item_row_start.numel() >= n_items + 1 and item_slot.numel() >= n_items, "linear_attention: item arrays")
    es = qkv.element_size()
    base = qkv.data_ptr()
    if chunk > 0:
        max_chunks = T // chunk + n_items
        _cuda(chunk_state)
        _need(chunk_state is not None and chunk_state.dtype == torch.float32
              and chunk_state.numel() >= max_chunks * heads * dim * vdim, "linear_attention: chunk_state scratch too small")
        _check(_lib.kernels().imparo_linear_attention_chunked(
            base + q_off * es, base + k_off * es, base + v_off * es, qkv.stride(0), _code(qkv), int(act == "silu"), _ptr(decay),
            _ptr(state), _ptr(chunk_state), int(chunk), int(max_chunks), _ptr(item_row_start), _ptr(item_slot), int(n_items),
            state.shape[0], _ptr(out), heads, dim, vdim, _ptr(status), _stream()), "linear_attention_chunked")
        COUNTS["own"] += 2
        return
    _check(_lib.kernels().imparo_linear_attention_recurrent(
        base + q_off * es, base + k_off * es, base + v_off * es, qkv.stride(0), _code(qkv), int(act == "silu"), _ptr(decay),
        _ptr(state), _ptr(item_row_start), _ptr(item_slot), int(n_items), state.shape[0], _ptr(out), heads, dim, vdim,
        _ptr(status), _stream()), "linear_attention")


# ---- a norm on a sublayer's output, casts, scaling (csrc/kernels/stream_ops.cu) --------------------------------
def out_norm_add(x: torch.Tensor, y: torch.Tensor, w: torch.Tensor, eps: float, copy: Optional[torch.Tensor] = None) -> None:
    """x += y / rms(y) * w row by row (x, y float32 [rows, width]; w float32 [width]).  copy ([rows, width], float32 or
    bfloat16): also receives the updated rows, for products that read the stream itself."""
    settle(x)
    _cuda(x, y, w, copy)
    n, width = x.shape
    _need(x.dtype == torch.float32 and y.dtype == torch.float32 and y.shape == x.shape, "out_norm_add: float32 [rows, width]")
    _need(w.dtype == torch.float32 and w.numel() == width, "out_norm_add: weight float32 [width]")
    _need(copy is None or copy.shape == x.shape, "out_norm_add: copy must have the stream's shape")
    _check(_lib.kernels().imparo_out_norm_add(_ptr(x), _ptr(y), _ptr(w), float(eps), _ptr(copy), _code(copy) if copy is not None else F32,
                                              n, width, _stream()), "out_norm_add")


def cast_rows(x: torch.Tensor, out: torch.Tensor) -> None:
    """out = x in out's dtype (x float32)."""
    settle(x)
    _cuda(x, out)
    _need(x.dtype == torch.float32 and x.numel() == out.numel(), "cast_rows: a float32 source of the same size")
    _check(_lib.kernels().imparo_cast_rows(_ptr(x), _ptr(out), _code(out), x.numel(), _stream()), "cast_rows")


def scale_rows(x: torch.Tensor, factor: float) -> None:
    """x *= factor in place (float32)."""
    _cuda(x)
    _need(x.dtype == torch.float32, "scale_rows: float32")
    _check(_lib.kernels().imparo_scale_rows(_ptr(x), x.numel(), float(factor), _stream()), "scale_rows")


# ---- selective state-space mixer (csrc/kernels/mamba2.cu) --------------------------------------------------------
def mamba2_conv(proj: torch.Tensor, x_off: int, dt_off: int, channels: int, heads: int, taps: int, w: torch.Tensor,
                bias: Optional[torch.Tensor], dt_bias: torch.Tensor, state: torch.Tensor, item_row_start, item_of_token,
                item_slot, n_items: int, xbc: torch.Tensor, dt: torch.Tensor, status: torch.Tensor) -> None:
    """Causal conv + silu over columns [x_off, x_off + channels) of proj with the slot's conv state (float32
    [slots, taps-1, channels], moved on afterwards) -> xbc float32 [T, channels]; dt = softplus(proj[:, dt_off + h] +
    dt_bias[h]) -> float32 [T, heads]."""
    _need(proj.is_cuda and proj.stride(1) == 1, "mamba2_conv: rows of proj must be dense CUDA memory")
    _cuda(w, bias, dt_bias, state, item_row_start, item_of_token, item_slot, xbc, dt, status)
    T = proj.shape[0]
    _need(x_off + channels <= proj.shape[1] and dt_off + heads <= proj.shape[1], "mamba2_conv: offsets")
    _need(w.dtype == torch.float32 and tuple(w.shape) == (channels, taps), "mamba2_conv: taps float32 [channels, taps]")
    _need(bias is None or (bias.dtype == torch.float32 and bias.numel() == channels), "mamba2_conv: bias float32 [channels]")
    _need(dt_bias.dtype == torch.float32 and dt_bias.numel() == heads, "mamba2_conv: dt_bias float32 [heads]")
    _need(state.dtype == torch.float32 and tuple(state.shape[1:]) == (max(taps - 1, 1), channels), "mamba2_conv: state float32 [slots, taps-1, channels]")
    _need(xbc.dtype == torch.float32 and tuple(xbc.shape) == (T, channels) and dt.dtype == torch.float32 and tuple(dt.shape) == (T, heads),
          "mamba2_conv: outputs float32 [T, channels] and [T, heads]")
    _need(item_row_start.numel() >= n_items + 1 and item_slot.numel() >= n_items and item_of_token.numel() >= T, "mamba2_conv: item arrays")
    _check(_lib.kernels().imparo_mamba2_conv(_ptr(proj), _code(proj), proj.stride(0), int(x_off), int(dt_off), int(channels), int(heads),
                                             int(taps), _ptr(w), _ptr(bias), _ptr(dt_bias), _ptr(state), _ptr(item_row_start),
                                             _ptr(item_of_token), _ptr(item_slot), int(n_items), state.shape[0], T, _ptr(xbc), _ptr(dt),
                                             _ptr(status), _stream()), "mamba2_conv")
    if taps > 1:
        COUNTS["own"] += 1


def mamba2_scan(xbc: torch.Tensor, dt: torch.Tensor, A_log: torch.Tensor, D: torch.Tensor, state: torch.Tensor, item_row_start,
                item_slot, n_items: int, y: torch.Tensor, heads: int, vdim: int, n_state: int, groups: int, status: torch.Tensor,
                chunk: int = 0, scratch=None) -> None:
    """Per request and head, over the request's rows in order, from and into state[slot] (float32 [slots, heads, N, vdim]):
    S = exp(-exp(A_log) dt) S + dt B x^T;  y = S^T C + D x.  xbc float32 [T, heads*vdim + 2*groups*N] = [x | B | C].
    chunk > 0 (steps with long portions): the rows of a request are cut into chunks of that many rows that run side by
    side; scratch = (int32 [3*max_chunks + n_items + 1], float32 [max_chunks*heads*N*vdim], float32 [max_chunks*heads])
    with max_chunks = T // chunk + n_items.  The result differs from the row-by-row walk by 32-bit rounding only."""
    _cuda(xbc, dt, A_log, D, state, item_row_start, item_slot, y, status)
    T = xbc.shape[0]
    inner = heads * vdim
    _need(xbc.dtype == torch.float32 and xbc.shape[1] == inner + 2 * groups * n_state, "mamba2_scan: xbc float32 [T, inner + 2 groups N]")
    _need(dt.dtype == torch.float32 and tuple(dt.shape) == (T, heads), "mamba2_scan: dt float32 [T, heads]")
    _need(A_log.dtype == torch.float32 and A_log.numel() == heads and D.dtype == torch.float32 and D.numel() == heads,
          "mamba2_scan: A_log and D float32 [heads]")
    _need(state.dtype == torch.float32 and tuple(state.shape[1:]) == (heads, n_state, vdim), "mamba2_scan: state float32 [slots, heads, N, vdim]")
    _need(y.dtype == torch.float32 and tuple(y.shape) == (T, inner), "mamba2_scan: y float32 [T, heads*vdim]")
    _need(item_row_start.numel() >= n_items + 1 and item_slot.numel() >= n_items, "mamba2_scan: item arrays")
    if chunk > 0:
        max_chunks = T // chunk + n_items
        si, cs, cd = scratch
        _cuda(si, cs, cd)
        _need(si.dtype == torch.int32 and si.numel() >= 3 * max_chunks + n_items + 1 and cs.dtype == torch.float32
              and cs.numel() >= max_chunks * heads * n_state * vdim and cd.dtype == torch.float32 and cd.numel() >= max_chunks * heads,
              "mamba2_scan: chunk scratch too small")
        _check(_lib.kernels().imparo_mamba2_scan_chunked(_ptr(xbc), _ptr(dt), _ptr(A_log), _ptr(D), _ptr(state), _ptr(item_row_start),
                                                         _ptr(item_slot), int(n_items), state.shape[0], _ptr(y), heads, vdim, n_state,
                                                         groups, int(chunk), int(max_chunks), _ptr(si), _ptr(cs), _ptr(cd), _ptr(status),
                                                         _stream()), "mamba2_scan_chunked")
        COUNTS["own"] += 3
        return
    _check(_lib.kernels().imparo_mamba2_scan(_ptr(xbc), _ptr(dt), _ptr(A_log), _ptr(D), _ptr(state), _ptr(item_row_start), _ptr(item_slot),
                                             int(n_items), state.shape[0], _ptr(y), heads, vdim, n_state, groups, _ptr(status),
                                             _stream()), "mamba2_scan")


def gate_group_rmsnorm(y: torch.Tensor, z: torch.Tensor, w: torch.Tensor, eps: float, groups: int, out: torch.Tensor) -> None:
    """out = (y * silu(z)) normed in `groups` equal stretches of the row (each by its own root mean square), times w.
    y float32 [rows, width]; z [rows, width], rows may be strided (a stretch of a wider product); out [rows, width]."""
    _need(y.is_cuda and z.is_cuda and out.is_cuda and w.is_cuda, "kernels run on CUDA tensors only (there is no CPU path)")
    n, width = out.shape
    _need(y.dtype == torch.float32 and tuple(y.shape) == (n, width) and y.is_contiguous() and out.is_contiguous(), "gate_group_rmsnorm: y float32 [rows, width]")
    _need(w.dtype == torch.float32 and w.numel() == width and width % groups == 0, "gate_group_rmsnorm: weight float32 [width], groups divide width")
    _need(tuple(z.shape) == (n, width) and z.stride(1) == 1, "gate_group_rmsnorm: z [rows, width] with dense rows")
    _check(_lib.kernels().imparo_gate_group_rmsnorm(_ptr(y), _ptr(z), _code(z), z.stride(0), _ptr(w), float(eps), _ptr(out), _code(out),
                                                    n, width, int(groups), _stream()), "gate_group_rmsnorm")


# ---- routed feed-forward (csrc/kernels/moe.cu) -------------------------------------------------------------------
def _pick_args(top, ids, wts, n, groups, keep, always):
    stride = int(top) + int(always)
    _need(ids.dtype == torch.int32 and wts.dtype == torch.float32 and ids.numel() >= n * stride and wts.numel() >= n * stride,
          "moe: ids int32 and wts float32 [rows, top + always]")
    return int(groups), int(keep if keep else groups), stride


def moe_route(h: torch.Tensor, w_router: torch.Tensor, top: int, ids: torch.Tensor, wts: torch.Tensor, softmax: bool = False,
              renormalise: bool = False, logits: Optional[torch.Tensor] = None, groups: int = 1, keep: int = 0,
              renorm_eps: float = 0.0, weight_scale: float = 1.0, always: int = 0) -> None:
    """Router logits W_r h in 32-bit, sigmoid (or softmax) scores, the `top` largest per row: ids int32 [rows, top],
    wts float32 [rows, top].  logits: float32 scratch [rows, experts] (made here when not given).
    groups, keep: the experts form `groups` equal groups of neighbours, a group's score is its largest, and only the `keep`
    best groups' experts can be chosen.  renormalise divides the chosen scores by their sum + renorm_eps; weight_scale
    multiplies the weights.  always = a: ids and wts are [rows, top + a], the last a entries name experts number
    experts, experts + 1, ... with weight 1 (experts every row uses, stacked behind the routed ones)."""
    n, width = h.shape
    E = w_router.shape[0]
    if logits is None:
        logits = torch.empty(n, E, dtype=torch.float32, device=h.device)
    _cuda(h, w_router, ids, wts, logits)
    _need(logits.dtype == torch.float32 and logits.numel() >= n * E, "moe_route: logits float32 [rows, experts]")
    _need(w_router.dtype == torch.float32 and w_router.shape[1] == width, "moe_route: router float32 [experts, width]")
    groups, keep, stride = _pick_args(top, ids, wts, n, groups, keep, always)
    _check(_lib.kernels().imparo_moe_route(_ptr(h), _code(h), _ptr(w_router), n, width, E, int(top), int(bool(softmax)),
                                           int(bool(renormalise)), groups, keep, float(renorm_eps), float(weight_scale), stride,
                                           _ptr(logits), _ptr(ids), _ptr(wts), _stream()), "moe_route")
    COUNTS["own"] += 1


def moe_pick(logits: torch.Tensor, experts: int, parts: int, top: int, ids: torch.Tensor, wts: torch.Tensor, softmax: bool = False,
             renormalise: bool = False, groups: int = 1, keep: int = 0, renorm_eps: float = 0.0, weight_scale: float = 1.0,
             always: int = 0) -> None:
    """The router's choice from logits a product has made: logits float32 [rows, parts * experts], a logit being the sum of
    its `parts` entries `experts` apart (a 32-bit router matrix cut into bfloat16 pieces that add up to it to its last bit).
    groups, keep, renorm_eps, weight_scale, always: as for moe_route."""
    _cuda(logits, ids, wts)
    n = logits.shape[0]
    _need(logits.dtype == torch.float32 and logits.shape[1] == parts * experts, "moe_pick: logits float32 [rows, parts * experts]")
    groups, keep, stride = _pick_args(top, ids, wts, n, groups, keep, always)
    _check(_lib.kernels().imparo_moe_pick(_ptr(logits), n, int(experts), int(parts), int(top), int(bool(softmax)),
                                          int(bool(renormalise)), groups, keep, float(renorm_eps), float(weight_scale), stride,
                                          _ptr(ids), _ptr(wts), _stream()), "moe_pick")


MOE_GROUP_FROM = 32          # steps with at least this many (row, choice) pairs per expert on average run grouped by expert


def moe_tiles_usable(h: torch.Tensor, w_gu: torch.Tensor) -> bool:
    """Whether moe_experts_tiles takes these sizes: bfloat16, width and features in multiples of 8, at most 256 experts."""
    return (h.dtype == torch.bfloat16 and h.shape[1] % 8 == 0 and (w_gu.shape[1] // 2) % 8 == 0 and w_gu.shape[0] <= 256
            and gemm_backend() == "tcgen05")


def moe_experts_tiles(h: torch.Tensor, w_gu: torch.Tensor, w_down: torch.Tensor, ids: torch.Tensor, wts: torch.Tensor, top: int,
                      weight_input: bool, xg: torch.Tensor, mid_g: torch.Tensor, out_g: torch.Tensor, scratch_i: torch.Tensor,
                      out: torch.Tensor, status: torch.Tensor, act: str = "silu", limit: float = 0.0) -> None:
    """The same result as moe_experts for steps of many rows in bfloat16: the (row, choice) pairs are sorted by expert into
    a buffer in which every expert's rows start at a multiple of 128 (xg, inputs already weighted), and both products run
    on the persistent tensor-memory kernel in its grouped form (silu(gate) * up in the first one's epilogue).  With
    m_tiles = rows * top // 128 + experts: xg bfloat16 [m_tiles * 128, width], mid_g bfloat16 [m_tiles * 128, ff], out_g
    float32 [m_tiles * 128, width], scratch_i int32 [rows * top + m_tiles]."""
    _cuda(h, w_gu, w_down, ids, wts, xg, mid_g, out_g, scratch_i, out, status)
    n, width = h.shape
    E, ff2, _ = w_gu.shape
    ff = ff2 // 2
    m_tiles = n * top // 128 + E
    _need(moe_tiles_usable(h, w_gu), "moe_experts_tiles: bfloat16, width and features multiples of 8, at most 256 experts")
    _need(w_gu.dtype == h.dtype and w_down.dtype == h.dtype and xg.dtype == h.dtype and mid_g.dtype == h.dtype,
          "moe_experts_tiles: one dtype for h, the experts and the sorted buffers")
    _need(xg.numel() >= m_tiles * 128 * width and mid_g.numel() >= m_tiles * 128 * ff and out_g.dtype == torch.float32
          and out_g.numel() >= m_tiles * 128 * width and scratch_i.dtype == torch.int32 and scratch_i.numel() >= n * top + m_tiles,
          "moe_experts_tiles: scratch too small")
    _need(out.dtype == torch.float32 and tuple(out.shape) == (n, width), "moe_experts_tiles: out float32 [rows, width]")
    _check(_lib.kernels().imparo_moe_tiles(_ptr(h), _ptr(w_gu), _ptr(w_down), _ptr(ids), _ptr(wts), n, width, ff, int(top), E,
                                           int(bool(weight_input)), GATED_ACTIVATIONS[act], float(limit), _ptr(xg), _ptr(mid_g),
                                           _ptr(out_g), _ptr(scratch_i), _ptr(out), _ptr(status), _stream()), "moe_tiles")
    COUNTS["own"] += 4


def moe_experts(h: torch.Tensor, w_gu: torch.Tensor, w_down: torch.Tensor, ids: torch.Tensor, wts: torch.Tensor, top: int,
                weight_input: bool, mid: torch.Tensor, out: torch.Tensor, scratch=None, act: str = "silu", limit: float = 0.0) -> None:
    """out[r] = sum_k expert_{ids[r,k]}(wts[r,k] * h[r])  (weight_input) or sum_k wts[r,k] * expert(h[r]).
    act, limit: the experts' gated activation (gated_act's kinds).
    w_gu [experts, 2 ff, width] = [gate; up], w_down [experts, width, ff]; mid [rows*top, ff] in h's dtype; out float32
    [rows, width], overwritten.  scratch = (float32 [rows*top, width], int32 [rows*top + experts + 2 + 3*(rows*top//32 + experts)]):
    when given, pairs are sorted by expert and run as tiles (steps of many rows); else each pair on its own."""
    _cuda(h, w_gu, w_down, ids, wts, mid, out)
    n, width = h.shape
    E, ff2, _ = w_gu.shape
    ff = ff2 // 2
    _need(w_gu.dtype == h.dtype and w_down.dtype == h.dtype and mid.dtype == h.dtype, "moe_experts: one dtype for h, the experts and mid")
    _need(w_gu.shape[2] == width and tuple(w_down.shape) == (E, width, ff), "moe_experts: expert shapes")
    _need(mid.numel() >= n * top * ff and out.dtype == torch.float32 and tuple(out.shape) == (n, width), "moe_experts: mid / out sizes")
    if scratch is not None:
        pair_out, si = scratch
        _cuda(pair_out, si)
        _need(pair_out.dtype == torch.float32 and pair_out.numel() >= n * top * width and si.dtype == torch.int32
              and si.numel() >= n * top + E + 2 + 3 * (n * top // 32 + E), "moe_experts: grouped scratch too small")
        _check(_lib.kernels().imparo_moe_grouped(_ptr(h), _ptr(w_gu), _ptr(w_down), _code(h), _ptr(ids), _ptr(wts), n, width, ff, int(top),
                                                 E, int(bool(weight_input)), GATED_ACTIVATIONS[act], float(limit), _ptr(mid), _ptr(pair_out),
                                                 _ptr(si), _ptr(out), _stream()),
               "moe_grouped")
        COUNTS["own"] += 3
        return
    _check(_lib.kernels().imparo_moe_rows(_ptr(h), _ptr(w_gu), _ptr(w_down), _code(h), _ptr(ids), _ptr(wts), n, width, ff, int(top), E,
                                          int(bool(weight_input)), GATED_ACTIVATIONS[act], float(limit), _ptr(mid), _ptr(out), _stream()),
           "moe_rows")
    COUNTS["own"] += 1


# ---- a stream kept as n copies per token (csrc/kernels/hyper_connections.cu) -----------------------------------
def embed_copies(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, status: torch.Tensor, scale: float = 1.0,
                 copies: int = 1, pos_table: Optional[torch.Tensor] = None, positions: Optional[torch.Tensor] = None) -> None:
    """out [T, copies * width] float32: the embedding row times scale, plus (with pos_table [n, width] and positions
    int32 [T]) the unscaled row of the token's position, written into every copy."""
    _cuda(table, ids, out, status)
    if pos_table is not None:
        _cuda(pos_table, positions)
        _need(pos_table.dtype == table.dtype and pos_table.is_contiguous() and pos_table.shape[1] == table.shape[1],
              "position table: the embedding table's dtype and width")
        _need(positions.dtype == torch.int32 and positions.numel() >= out.shape[0], "positions must be int32, one per output row")
    for d in (_S.pending, _S.pending_mean, _S.pending_mix):      # the stream starts afresh
        d.pop(out.data_ptr(), None)
    n = out.shape[0]
    width = table.shape[1]
    _need(ids.dtype == torch.int32 and ids.numel() >= n, "ids must be int32, one per output row")
    _need(out.dtype == torch.float32 and out.shape[1] == copies * width and out.is_contiguous(),
          "embedding output is float32 [tokens, copies * width]")
    _check(_lib.kernels().imparo_embed_copies(_ptr(table), _code(table), _ptr(ids), float(scale), int(copies), _ptr(pos_table),
                                              _ptr(positions), pos_table.shape[0] if pos_table is not None else 0, _ptr(out), n, width,
                                              table.shape[0], _ptr(status), _stream()), "embed_copies")


def streams_norm(x: torch.Tensor, n: int, coef: Optional[torch.Tensor], w: torch.Tensor, eps: float, out: torch.Tensor,
                 rows: Optional[torch.Tensor] = None) -> None:
    """out[r] = u / rms(u) * w with u = sum_s coef[s] x[row, s] (coef None: the plain sum of the n copies).
    x: float32 [*, n * width]; rows (int32) picks input rows.  A streams_mix_add left pending on x is carried out
    by the same kernel when the norm reads every row in place."""
    _cuda(x, coef, w, out, rows)
    n_rows, width = out.shape
    _need(x.dtype == torch.float32 and x.is_contiguous() and x.shape[1] == n * width, "streams_norm: x float32 [rows, n * width]")
    _need(w.dtype == torch.float32 and w.numel() == width, "streams_norm: weight float32 [width]")
    _need(coef is None or (coef.dtype == torch.float32 and coef.numel() == n), "streams_norm: coefficients float32 [n]")
    px = _S.pending_mix.get(x.data_ptr())
    if px is not None and rows is None and x.shape[0] == n_rows and px[0] == n and x.data_ptr() not in _S.pending:
        _S.pending_mix.pop(x.data_ptr())
        _, mix, b, y = px
        _check(_lib.kernels().imparo_streams_mix_add(_ptr(x), n, _ptr(mix), _ptr(b), _ptr(y), _ptr(coef), _ptr(w), float(eps),
                                                     _ptr(out), _code(out), n_rows, width, _stream()), "streams_mix_add_norm")
        return
    settle(x)
    if rows is None:
        _need(x.shape[0] >= n_rows, "streams_norm: fewer input rows than output rows")
    else:
        _need(rows.dtype == torch.int32 and rows.numel() >= n_rows, "streams_norm: rows must be int32, one per output row")
    _check(_lib.kernels().imparo_streams_norm(_ptr(x), _ptr(rows), n, _ptr(coef), _ptr(w), float(eps), _ptr(out), _code(out),
                                              n_rows, width, _stream()), "streams_norm")


def streams_mix_add(x: torch.Tensor, n: int, mix: torch.Tensor, b: torch.Tensor, y: torch.Tensor, defer: bool = False) -> None:
    """x'[r, t] = sum_s mix[s, t] x[r, s] + b[t] y[r] for all n copies at once.  x: float32 [rows, n * width] in place;
    mix float32 [n, n] ([from, to]); b float32 [n]; y float32 [rows, width].  defer: the update is left to the next
    reader of x (streams_norm does it in its own pass; settle() does it alone); y must stay as it is until then."""
    _cuda(x, mix, b, y)
    rows, width = y.shape
    _need(x.dtype == torch.float32 and x.is_contiguous() and tuple(x.shape) == (rows, n * width), "streams_mix_add: x float32 [rows, n * width]")
    _need(y.dtype == torch.float32 and y.is_contiguous(), "streams_mix_add: y float32 [rows, width]")
    _need(mix.dtype == torch.float32 and mix.numel() == n * n and b.dtype == torch.float32 and b.numel() == n,
          "streams_mix_add: mix float32 [n, n], b float32 [n]")
    settle(x)
    settle(y)
    if defer:
        _S.pending_mix[x.data_ptr()] = (n, mix, b, y)
        return
    _check(_lib.kernels().imparo_streams_mix_add(_ptr(x), n, _ptr(mix), _ptr(b), _ptr(y), None, None, 0.0, None, 0, rows, width,
                                                 _stream()), "streams_mix_add")


# ---- short convolution over time on the channels of a 32-bit product (csrc/kernels/channel_conv.cu) --------------
def channel_conv(proj: torch.Tensor, col0: int, channels: int, taps: int, w: torch.Tensor, bias: Optional[torch.Tensor],
                 state: torch.Tensor, item_row_start, item_of_token, item_slot, n_items: int, out: torch.Tensor,
                 status: torch.Tensor, act: Optional[str] = None) -> None:
    """out[t, c] = act(sum_j w[c, j] * u[t - taps + 1 + j, c]), u = proj[:, col0 + c] (+ bias[c]); inputs before a portion's
    first row come from the request's slot of state (float32 [slots, taps - 1, channels], the last inputs, oldest first),
    which is then moved on by the portion's rows.  proj, out: float32, rows dense.  act: None | "silu"."""
    _cuda(w, bias, state, item_row_start, item_of_token, item_slot, status)
    _need(proj.is_cuda and out.is_cuda, "kernels run on CUDA tensors only (there is no CPU path)")
    T = out.shape[0]
    _need(proj.dtype == torch.float32 and proj.stride(1) == 1 and proj.shape[0] == T and proj.shape[1] >= col0 + channels,
          "channel_conv: a float32 product with dense rows")
    _need(out.dtype == torch.float32 and out.stride(1) == 1 and out.shape[1] == channels, "channel_conv: out float32 [T, channels]")
    _need(w.dtype == torch.float32 and tuple(w.shape) == (channels, taps) and w.is_contiguous(), "channel_conv: taps float32 [channels, taps]")
    _need(bias is None or (bias.dtype == torch.float32 and bias.numel() == channels), "channel_conv: bias float32 [channels]")
    _need(act in (None, "silu"), "channel_conv: act is None or 'silu'")
    _need(state.dtype == torch.float32 and state.is_contiguous() and state.dim() == 3 and state.shape[2] == channels
          and state.shape[1] >= max(taps - 1, 1), "channel_conv: state float32 [slots, taps - 1, channels]")
    _need(state.shape[1] == taps - 1 or taps == 1, "channel_conv: state holds taps - 1 rows")
    _check(_lib.kernels().imparo_channel_conv(_ptr(proj), proj.stride(0), int(col0), channels, taps, _ptr(w), _ptr(bias), _ptr(state),
                                              _ptr(item_row_start), _ptr(item_of_token), _ptr(item_slot), state.shape[0],
                                              1 if act == "silu" else 0, _ptr(out), out.stride(0), T, _ptr(status), _stream()),
           "channel_conv")
    if taps > 1:
        _check(_lib.kernels().imparo_channel_conv_state(_ptr(proj), proj.stride(0), int(col0), channels, taps, _ptr(bias), _ptr(state),
                                                        _ptr(item_row_start), _ptr(item_slot), state.shape[0], n_items, _stream()),
               "channel_conv_state")


# ---- gated delta rule with a decay per key channel (csrc/kernels/delta_rule.cu) ----------------------------------
def delta_prepare(qkv: torch.Tensor, q_off: int, k_off: int, bproj: torch.Tensor, b_off: int, a: torch.Tensor, A_log: torch.Tensor,
                  dt_bias: torch.Tensor, beta: torch.Tensor, heads: int, kv_heads: int, dim: int, unit_eps: float,
                  q_scale: float) -> None:
    """In 32-bit, per row: the kv_heads query heads (at q_off) and key heads (at k_off) of qkv divided by
    sqrt(sum of squares + unit_eps), queries also times q_scale; beta[t, h] = sigmoid(bproj[t, b_off + h]);
    a [T, heads * dim] becomes exp(-exp(A_log[h]) * softplus(a + dt_bias))."""
    _cuda(a, A_log, dt_bias, beta)
    _need(qkv.is_cuda and bproj.is_cuda, "kernels run on CUDA tensors only (there is no CPU path)")
    T = qkv.shape[0]
    for t in (qkv, bproj, a, A_log, dt_bias, beta):
        _need(t.dtype == torch.float32, "delta_prepare: float32 tensors")
    _need(qkv.stride(1) == 1 and bproj.stride(1) == 1 and a.is_contiguous() and beta.is_contiguous(), "delta_prepare: dense rows")
    _need(tuple(a.shape) == (T, heads * dim) and tuple(beta.shape) == (T, heads) and A_log.numel() == heads
          and dt_bias.numel() == heads * dim, "delta_prepare: shapes")
    _need(qkv.shape[1] >= max(q_off, k_off) + kv_heads * dim and bproj.shape[1] >= b_off + heads and bproj.shape[0] == T,
          "delta_prepare: column ranges")
    _check(_lib.kernels().imparo_delta_prepare(_ptr(qkv), qkv.stride(0), int(q_off), int(k_off), _ptr(bproj), bproj.stride(0), int(b_off),
                                               _ptr(a), _ptr(A_log), _ptr(dt_bias), _ptr(beta), T, heads, kv_heads, dim, float(unit_eps),
                                               float(q_scale), _stream()), "delta_prepare")


def delta_scan(qkv: torch.Tensor, q_off: int, k_off: int, v_off: int, g: torch.Tensor, beta: torch.Tensor, state: torch.Tensor,
               item_row_start, item_slot, n_items: int, out: torch.Tensor, heads: int, kv_heads: int, dim: int, vdim: int,
               status: torch.Tensor) -> None:
    """Per request and value head, rows in order: S = g * S; u = beta (v - S^T k); S += k u^T; out = S^T q.
    qkv float32 rows (query / key heads kv_heads * dim at q_off / k_off, values heads * vdim at v_off); g float32
    [T, heads * dim]; beta float32 [T, heads]; state float32 [slots, heads, dim, vdim]; out float32 [T, heads * vdim]."""
    _cuda(g, beta, state, item_row_start, item_slot, out, status)
    _need(qkv.is_cuda, "kernels run on CUDA tensors only (there is no CPU path)")
    T = qkv.shape[0]
    for t in (qkv, g, beta, state, out):
        _need(t.dtype == torch.float32, "delta_scan: float32 tensors")
    _need(qkv.stride(1) == 1 and g.is_contiguous() and beta.is_contiguous() and out.is_contiguous() and state.is_contiguous(),
          "delta_scan: dense rows")
    _need(tuple(g.shape) == (T, heads * dim) and tuple(beta.shape) == (T, heads) and tuple(out.shape) == (T, heads * vdim),
          "delta_scan: shapes")
    _need(tuple(state.shape[1:]) == (heads, dim, vdim), "delta_scan: state [slots, heads, dim, vdim]")
    _need(1 <= dim <= 256, "delta_scan: key size 1 to 256")
    _need(qkv.shape[1] >= max(q_off + kv_heads * dim, k_off + kv_heads * dim, v_off + heads * vdim), "delta_scan: column ranges")
    _check(_lib.kernels().imparo_delta_scan(_ptr(qkv), qkv.stride(0), int(q_off), int(k_off), int(v_off), _ptr(g), _ptr(beta), _ptr(state),
                                            _ptr(item_row_start), _ptr(item_slot), state.shape[0], n_items, _ptr(out), heads, kv_heads,
                                            dim, vdim, _ptr(status), _stream()), "delta_scan")


def head_norm_gate(o: torch.Tensor, w: torch.Tensor, eps: float, gate: torch.Tensor, out: torch.Tensor, heads: int, vdim: int) -> None:
    """out[t, h] = o[t, h] / rms(o[t, h]) * w * sigmoid(gate[t, h]) per head.  o float32 [T, heads * vdim]; w float32 [vdim]
    (one weight shared by the heads) or [heads * vdim] (each head's own); gate float32 rows (dense, any row stride)."""
    _cuda(o, w, out)
    _need(gate.is_cuda, "kernels run on CUDA tensors only (there is no CPU path)")
    T = o.shape[0]
    _need(o.dtype == torch.float32 and o.is_contiguous() and tuple(o.shape) == (T, heads * vdim), "head_norm_gate: o float32 [T, heads * vdim]")
    _need(w.dtype == torch.float32 and w.numel() in (vdim, heads * vdim), "head_norm_gate: weight float32 [vdim] or [heads * vdim]")
    _need(gate.dtype == torch.float32 and gate.stride(1) == 1 and tuple(gate.shape) == (T, heads * vdim), "head_norm_gate: gate float32")
    _need(out.is_contiguous() and tuple(out.shape) == (T, heads * vdim), "head_norm_gate: out [T, heads * vdim]")
    _check(_lib.kernels().imparo_head_norm_gate(_ptr(o), _ptr(w), float(eps), _ptr(gate), gate.stride(0), _ptr(out), _code(out), T,
                                                heads, vdim, vdim if w.numel() == heads * vdim and heads > 1 else 0, _stream()),
           "head_norm_gate")


# ---- a matrix memory with exponential gates (csrc/kernels/mlstm.cu) ---------------------------------------------
def mlstm_value_blocks(vdim: int) -> int:
    """How many copies of n and m a head keeps in its slot: one per 32 value columns (one per warp of the recurrence)."""
    return (int(vdim) + 31) // 32


def mlstm_scan(proj: torch.Tensor, q_off: int, k_off: int, v_off: int, i_off: int, f_off: int, i_bias: torch.Tensor,
               f_bias: torch.Tensor, cap: float, q_scale: float, state_S: torch.Tensor, state_n: torch.Tensor, state_m: torch.Tensor,
               item_row_start, item_slot, n_items: int, out: torch.Tensor, heads: int, dim: int, vdim: int, status: torch.Tensor,
               chunk: int = 0, scratch=None) -> None:
    """Per request and head, over the request's rows in order, from and into its slot:
    a = cap tanh((x_i + b_i) / cap), f = log sigmoid(cap tanh((x_f + b_f) / cap)), m' = max(f + m, a),
    S' = exp(f + m - m') S + exp(a - m') k v^T, n' alike with k alone, o = S'^T q / (max(|n' . q|, exp(-m')) + 1e-6), q times
    q_scale.  proj: float32 rows holding q, k (heads * dim each), v (heads * vdim) and the gates' inputs (heads each) at the
    given column offsets; biases float32 [heads].  With vb = mlstm_value_blocks(vdim): state_S float32 [slots, heads, dim,
    vdim], state_n [slots, heads, vb, dim], state_m [slots, heads, vb]; out float32 [T, heads * vdim].

    chunk > 0 (batches with long portions): a request's rows are cut into chunks of that many rows which run side by side
    (three launches); scratch = (S, n, mb) float32 for (T // chunk + n_items) chunks: heads * dim * vdim, heads * vb * dim and
    heads * vb * 3 values per chunk.  The result differs from the row-by-row walk by the order of 32-bit additions only."""
    _need(proj.is_cuda and proj.stride(1) == 1 and proj.dtype == torch.float32, "mlstm_scan: a float32 product with dense rows")
    _cuda(i_bias, f_bias, state_S, state_n, state_m, item_row_start, item_slot, out, status)
    T = proj.shape[0]
    vb = mlstm_value_blocks(vdim)
    _need(1 <= dim <= 256 and heads >= 1 and vdim >= 1 and cap > 0.0, "mlstm_scan: key size 1 to 256, a positive gate cap")
    _need(max(q_off, k_off) + heads * dim <= proj.shape[1] and v_off + heads * vdim <= proj.shape[1]
          and max(i_off, f_off) + heads <= proj.shape[1], "mlstm_scan: column ranges")
    _need(i_bias.dtype == torch.float32 and f_bias.dtype == torch.float32 and i_bias.numel() == heads and f_bias.numel() == heads,
          "mlstm_scan: gate biases float32 [heads]")
    n_slots = state_S.shape[0]
    _need(state_S.dtype == torch.float32 and state_S.is_contiguous() and tuple(state_S.shape[1:]) == (heads, dim, vdim)
          and state_n.dtype == torch.float32 and state_n.is_contiguous() and tuple(state_n.shape) == (n_slots, heads, vb, dim)
          and state_m.dtype == torch.float32 and state_m.is_contiguous() and tuple(state_m.shape) == (n_slots, heads, vb),
          "mlstm_scan: state tensors float32 [slots, heads, dim, vdim], [slots, heads, vb, dim], [slots, heads, vb]")
    _need(out.dtype == torch.float32 and out.is_contiguous() and tuple(out.shape) == (T, heads * vdim), "mlstm_scan: out float32 [T, heads * vdim]")
    _need(item_row_start.dtype == torch.int32 and item_slot.dtype == torch.int32 and item_row_start.numel() >= n_items + 1
          and item_slot.numel() >= n_items and n_items <= 65535, "mlstm_scan: item arrays int32")
    cS = cn = cmb = None
    if chunk > 0:
        cS, cn, cmb = scratch
        _cuda(cS, cn, cmb)
        most = T // chunk + n_items
        _need(cS.dtype == cn.dtype == cmb.dtype == torch.float32 and cS.numel() >= most * heads * dim * vdim
              and cn.numel() >= most * heads * vb * dim and cmb.numel() >= most * heads * vb * 3, "mlstm_scan: chunk scratch too small")
    _check(_lib.kernels().imparo_mlstm_scan(_ptr(proj), proj.stride(0), int(q_off), int(k_off), int(v_off), int(i_off), int(f_off),
                                            _ptr(i_bias), _ptr(f_bias), float(cap), float(q_scale), _ptr(state_S), _ptr(state_n),
                                            _ptr(state_m), _ptr(item_row_start), _ptr(item_slot), n_slots, int(n_items), T, _ptr(out),
                                            heads, dim, vdim, int(chunk), _ptr(cS), _ptr(cn), _ptr(cmb), _ptr(status), _stream()),
           "mlstm_scan")


# ---- attention over cached latent vectors (csrc/kernels/latent.cu) ----------------------------------------------
def latent_norm_store(proj: torch.Tensor, q_off: int, q_rank: int, c_off: int, c_rank: int, wq: torch.Tensor, wc: torch.Tensor,
                      eps: float, positions, item_of_token, q_out: torch.Tensor, cache: torch.Tensor, table, page_size: int,
                      n_pages: int, status: torch.Tensor) -> None:
    """Two stretches of a 32-bit product row, each divided by its root mean square times a weight: the query latent
    -> q_out [T, q_rank], the key/value latent -> the row's place in the paged cache (rows of c_rank)."""
    _cuda(wq, wc, positions, item_of_token, q_out, cache, table, status)
    _need(proj.is_cuda, "kernels run on CUDA tensors only (there is no CPU path)")
    T = q_out.shape[0]
    _need(proj.dtype == torch.float32 and proj.stride(1) == 1 and proj.shape[0] == T, "latent_norm_store: a float32 product with dense rows")
    _need(proj.shape[1] >= max(q_off + q_rank, c_off + c_rank), "latent_norm_store: column ranges")
    _need(wq.dtype == torch.float32 and wq.numel() == q_rank and wc.dtype == torch.float32 and wc.numel() == c_rank,
          "latent_norm_store: weights float32")
    _need(q_out.is_contiguous() and q_out.shape[1] == q_rank and cache.dtype == q_out.dtype, "latent_norm_store: q_out / cache dtype")
    _need(cache.numel() >= n_pages * page_size * c_rank, "cache arena smaller than n_pages")
    _need(table.dtype == torch.int32 and table.dim() == 2, "block table must be int32 [items, blocks]")
    _check(_lib.kernels().imparo_latent_norm_store(_ptr(proj), proj.stride(0), int(q_off), q_rank, int(c_off), c_rank, _ptr(wq), _ptr(wc),
                                                   float(eps), _ptr(positions), _ptr(item_of_token), _ptr(q_out), _ptr(cache),
                                                   _code(q_out), _ptr(table), table.shape[1], page_size, n_pages, T, _ptr(status),
                                                   _stream()), "latent_norm_store")


def latent_rot_store(proj: torch.Tensor, heads: int, dim: int, rot: int, rank: int, wc: torch.Tensor, eps: float,
                     inv_freq: Optional[torch.Tensor], n_rot: int, positions, item_of_token, q_plain: torch.Tensor,
                     q_lat: torch.Tensor, cache: torch.Tensor, table, page_size: int, n_pages: int, status: torch.Tensor) -> None:
    """The latent attention's row preparation when a rotated part stands beside the latent.  proj: a 32-bit product's rows
    [heads x (dim | rot) | rank | rot | ...].  The page row becomes [rms(latent) * wc | turned key part] (rank + rot wide);
    q_plain [T, heads * dim] gets every head's plain query dimensions, q_lat [T, heads * (rank + rot)] the turned ones in each
    head's last rot entries.  The turn is the half-split rotation of the first n_rot of the rot dimensions by
    position * inv_freq (float32 [n_rot / 2])."""
    _cuda(wc, positions, item_of_token, q_plain, q_lat, cache, table, status)
    _need(proj.is_cuda, "kernels run on CUDA tensors only (there is no CPU path)")
    T = q_plain.shape[0]
    _need(proj.dtype == torch.float32 and proj.stride(1) == 1 and proj.shape[0] == T and proj.shape[1] >= heads * (dim + rot) + rank + rot,
          "latent_rot_store: a float32 product with dense rows [heads * (dim + rot) + rank + rot]")
    _need(wc.dtype == torch.float32 and wc.numel() == rank, "latent_rot_store: norm weight float32 [rank]")
    _need(q_plain.is_contiguous() and tuple(q_plain.shape) == (T, heads * dim) and q_lat.is_contiguous()
          and tuple(q_lat.shape) == (T, heads * (rank + rot)) and q_plain.dtype == q_lat.dtype == cache.dtype, "latent_rot_store: outputs")
    _need(n_rot == 0 or (inv_freq is not None and inv_freq.is_cuda and inv_freq.dtype == torch.float32 and inv_freq.numel() == n_rot // 2
                         and n_rot % 2 == 0 and n_rot <= rot), "latent_rot_store: rotation table float32 [n_rot / 2]")
    _need(cache.numel() >= n_pages * page_size * (rank + rot), "cache arena smaller than n_pages")
    _need(table.dtype == torch.int32 and table.dim() == 2, "block table must be int32 [items, blocks]")
    _check(_lib.kernels().imparo_latent_rot_store(_ptr(proj), proj.stride(0), heads, dim, rot, rank, _ptr(wc), float(eps),
                                                  _ptr(inv_freq) if n_rot else None, int(n_rot), _ptr(positions), _ptr(item_of_token),
                                                  _ptr(q_plain), _ptr(q_lat), _ptr(cache), _code(q_plain), _ptr(table), table.shape[1],
                                                  page_size, n_pages, T, _ptr(status), _stream()), "latent_rot_store")


def sigmoid_gate(x: torch.Tensor, gate: torch.Tensor, group: int = 1) -> None:
    """x[t, c] *= sigmoid(gate[t, c // group]) in place.  x [T, width] (rows dense, bfloat16 or float32); gate float32
    [T, width // group] (rows dense, any row stride: columns of a 32-bit product)."""
    _need(x.is_cuda and gate.is_cuda, "kernels run on CUDA tensors only (there is no CPU path)")
    T, width = x.shape
    _need(x.stride(1) == 1 and gate.dtype == torch.float32 and gate.stride(1) == 1 and group >= 1 and width % group == 0
          and tuple(gate.shape) == (T, width // group), "sigmoid_gate: gate float32 [T, width / group]")
    _check(_lib.kernels().imparo_sigmoid_gate(_ptr(x), x.stride(0), _ptr(gate), gate.stride(0), _code(x), T, width, int(group),
                                              _stream()), "sigmoid_gate")


HEADS_LINEAR_LIBRARY_ROWS = 64          # from this many rows on the per-head products go to the library in one batched call


def heads_linear(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, gate: Optional[torch.Tensor] = None,
                 x_head: Optional[int] = None, out_head: Optional[int] = None) -> None:
    """out[t, h, :] = w[h] x[t, h, :] for every head (w [heads, n_out, n_in]; rows dense), optionally times a sigmoid gate:
    gate float32 [T, heads * n_out] (an own gate per output) or [T, heads] (one per head), rows dense.  Head h's inputs start
    at column h * x_head of x (default n_in: x is [T, heads * n_in]) and its outputs at column h * out_head of out (default
    n_out); with wider heads the other columns of out are left as they are.  32-bit sums."""
    _cuda(w)
    _need(x.is_cuda and out.is_cuda and (gate is None or gate.is_cuda), "kernels run on CUDA tensors only (there is no CPU path)")
    heads, n_out, n_in = w.shape
    T = x.shape[0]
    x_head = n_in if x_head is None else int(x_head)
    out_head = n_out if out_head is None else int(out_head)
    _need(x.dtype == w.dtype == out.dtype and w.is_contiguous(), "heads_linear: one dtype, dense weights")
    _need(x.stride(1) == 1 and out.stride(1) == 1 and x_head >= n_in and out_head >= n_out and tuple(x.shape) == (T, heads * x_head)
          and tuple(out.shape) == (T, heads * out_head), "heads_linear: shapes")
    per_head = gate is not None and gate.shape[1] == heads and n_out != 1
    _need(gate is None or (gate.dtype == torch.float32 and gate.stride(1) == 1 and tuple(gate.shape) in ((T, heads * n_out), (T, heads))),
          "heads_linear: gate float32 [T, heads * n_out] or [T, heads]")
    if x.dtype == torch.bfloat16 and T >= HEADS_LINEAR_LIBRARY_ROWS and n_in % 8 == 0 and n_out % 8 == 0 \
            and x.stride(0) % 8 == 0 and out.stride(0) % 8 == 0 and x_head % 8 == 0 and out_head % 8 == 0 \
            and (gate is None or out_head == n_out):
        # many rows: one batched library product over the heads (tensor cores, 32-bit sums), then the gate in place
        _gemm_lib_ready(x.device)
        _check(_lib.kernels().imparo_gemm_bf16_heads(_ptr(x), _ptr(w), _ptr(out), T, heads, n_out, n_in, x.stride(0), out.stride(0),
                                                     x_head, out_head, _stream()), "gemm_bf16_heads", "library")
        if gate is not None:
            _check(_lib.kernels().imparo_sigmoid_gate(_ptr(out), out.stride(0), _ptr(gate), gate.stride(0), _code(out), T,
                                                      heads * n_out, n_out if per_head else 1, _stream()), "sigmoid_gate")
        return
    _need(n_in * 32 <= 48 * 1024, "heads_linear: input size per head up to 1536")
    _check(_lib.kernels().imparo_heads_linear(_ptr(x), x.stride(0), _ptr(w), _ptr(gate), gate.stride(0) if gate is not None else 0,
                                              _ptr(out), out.stride(0), _code(x), T, heads, n_in, n_out, x_head, out_head,
                                              int(per_head), _stream()), "heads_linear")
