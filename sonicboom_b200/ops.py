"""Python face of the kernel library: each function checks its tensors, then calls one
`extern "C"` entry point on torch's current CUDA stream.

Nothing here computes with torch; a tensor that is not on a CUDA device, or a missing
library, is an error (there is no CPU path).  Shapes a kernel does not take are refused by
the kernel's own host-side checks, whose message is raised here.
"""
from __future__ import annotations

import ctypes

import torch

from . import abi as _abi
from .csrc import build as _build

F32, BF16 = 0, 1
EPI_NONE, EPI_BIAS, EPI_RESIDUAL, EPI_SWIGLU = 0, 1, 2, 3
SWIGLU_BLOCK = 8                 # rows of gate and up alternate in blocks of this many
SKINNY_MAX_ROWS = 64             # bfloat16 products of at most this many rows stream the weights


class KernelError(RuntimeError):
    pass


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        _lib = _abi.apply(_build.load(), _abi.CORE)
    return _lib


def _code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 and bfloat16 tensors, not {dtype}")


def _ptr(t):
    """The device address of a tensor as the typed entry points take it (an int; None is a null
    pointer).  A step makes a few thousand of these, so no ctypes object is made here."""
    if t is None:
        return None
    if not t.is_cuda:
        raise KernelError("kernels take CUDA tensors only; there is no CPU path")
    if not t.is_contiguous():
        raise KernelError("kernels take contiguous tensors")
    return t.data_ptr()


# torch.cuda.current_stream() resolves the device, builds a Stream object and costs several
# microseconds; a prompt step asks for the stream some four hundred times.  The raw handle of
# the current device's current stream is one call where torch has it.
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream():
    if _raw_stream is not None and _raw_device is not None:
        return _raw_stream(_raw_device())
    return torch.cuda.current_stream().cuda_stream


LAUNCHES = 0          # kernels launched through this module so far (a running count)


# Opt-in NVTX ranges around steps and schedule entries, in the manner of the reference's
# SONICBOOM_NVTX switch (core/src/model/gemma4_plan.cpp:50, 87-91): SB_TRACE=1 in the
# environment or `set_trace(True)`.  Off, `trace_range` hands out one shared no-op object.
import contextlib as _contextlib
import os as _os

TRACE = _os.environ.get("SB_TRACE", "0") not in ("", "0")
_NO_RANGE = _contextlib.nullcontext()


def set_trace(on: bool) -> None:
    global TRACE
    TRACE = bool(on)


class _Range:
    def __init__(self, name):
        self.name = name

    def __enter__(self):
        torch.cuda.nvtx.range_push(self.name)

    def __exit__(self, *exc):
        torch.cuda.nvtx.range_pop()


def trace_range(name: str):
    """A context manager that is an NVTX range when tracing is on, else nothing."""
    return _Range(name) if TRACE else _NO_RANGE


def _check(rc: int, what: str, launches: int = 1) -> None:
    global LAUNCHES
    if rc != 0:
        raise KernelError(f"{what}: {lib().sb_last_error().decode()}")
    LAUNCHES += launches


def _i32(t, what):
    if t.dtype != torch.int32:
        raise KernelError(f"{what} must be int32, got {t.dtype}")
    return _ptr(t)


def embed(tokens: torch.Tensor, table: torch.Tensor, out: torch.Tensor,
          scale: float = 1.0) -> torch.Tensor:
    """out[t] = table[tokens[t]] * scale as float32; an id outside the table gives a row of NaN."""
    n, width = tokens.numel(), table.shape[1]
    assert out.dtype == torch.float32 and out.shape == (n, width)
    _check(lib().sb_embed(_i32(tokens, "tokens"), n, _ptr(table), _code(table.dtype),
                          table.shape[0], width, ctypes.c_float(scale), _ptr(out), _stream()), "embed")
    return out


def add_bias(x: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """x[m, n] += bias[n] in place (x float32 [rows, width])."""
    assert x.dtype == torch.float32 and x.dim() == 2 and bias.numel() == x.shape[1]
    _check(lib().sb_add_bias(_ptr(x), _ptr(bias), _code(bias.dtype), x.shape[0], x.shape[1], _stream()),
           "add_bias")
    return x


def softcap(x: torch.Tensor, cap: float) -> torch.Tensor:
    """x = cap * tanh(x / cap) in place (float32)."""
    assert x.dtype == torch.float32 and x.is_contiguous()
    _check(lib().sb_softcap(_ptr(x), ctypes.c_size_t(x.numel()), ctypes.c_float(cap), _stream()),
           "softcap")
    return x


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
            rows: torch.Tensor | None = None) -> torch.Tensor:
    """out[r] = rmsnorm(x[rows[r]] or x[r]) * weight; x is the float32 residual stream."""
    assert x.dtype == torch.float32 and x.dim() == 2
    n = out.shape[0]
    width = x.shape[1]
    assert out.shape[1] == width and weight.numel() == width
    if rows is None:
        assert x.shape[0] == n
    _check(lib().sb_rmsnorm(_ptr(x), _i32(rows, "rows") if rows is not None else _ptr(None), n,
                            width, _ptr(weight), _code(weight.dtype), ctypes.c_float(eps),
                            _ptr(out), _code(out.dtype), _stream()), "rmsnorm")
    return out


def cast(x: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    if x.dtype == dtype:
        return x
    out = torch.empty_like(x, dtype=dtype)
    _check(lib().sb_cast(_ptr(x), _code(x.dtype), _ptr(out), _code(dtype),
                         ctypes.c_size_t(x.numel()), _stream()), "cast")
    return out


def linear(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int = EPI_NONE,
           bias: torch.Tensor | None = None, residual: torch.Tensor | None = None,
           kernel: str = "auto", norm: tuple | None = None,
           warm: torch.Tensor | None = None) -> torch.Tensor:
    """out = a @ w.T with a fused epilogue; a [M,K], w [N,K]; float32 accumulation.

    `norm` = (weight, eps, norm_out) also writes norm_out = rmsnorm(out, weight, eps) [M,N]
    (out must be float32): in the kernel that finishes the product where one does (the split-K
    decode form of the tcgen05 kernel), else with the norm kernel after it.
    `warm`: weights that a later kernel streams; the blocks of the tcgen05 kernel ask for them
    into L2 as they end (other kernels ignore it).  A hint: it changes no result.  It pays only
    for a consumer that cannot request its own weights early (see `requests_weights_late`).

    bfloat16 operands run on tensor cores: `kernel` "tc5" (TMA + tcgen05), "skinny" (weights
    streamed into mma.sync fragments, at most SKINNY_MAX_ROWS rows), "tiled" (mma.sync tiles),
    or "auto", which picks between the first two (see `_pick_kernel`).  float32 operands, inner
    sizes that are not multiples of 8, and `kernel="plain"` run the plain FFMA kernel.  A
    bfloat16 activation with a float32 weight is cast to float32 first.  The split-K decode
    form keeps one workspace per device, so products on one device must be ordered in a stream.
    """
    M, K = a.shape
    N = w.shape[0]
    assert w.shape[1] == K, f"linear: a is [{M},{K}], w is {tuple(w.shape)}"
    n_out = N // 2 if epilogue == EPI_SWIGLU else N
    assert tuple(out.shape) == (M, n_out), f"linear: out is {tuple(out.shape)}, want {(M, n_out)}"
    if a.dtype != w.dtype:
        a = cast(a, torch.float32)
        if w.dtype != torch.float32:
            raise KernelError("linear: a float32 activation needs float32 weights")
    args = (_ptr(a), _code(a.dtype), _ptr(w), _code(w.dtype), M, N, K, epilogue, _ptr(bias),
            _code(bias.dtype) if bias is not None else 0, _ptr(residual), _ptr(out),
            _code(out.dtype), _stream())
    if residual is not None:
        assert residual.dtype == torch.float32 and tuple(residual.shape) == (M, N)
    if bias is not None:
        assert bias.numel() == N
    fast = a.dtype == torch.bfloat16 and kernel != "plain" and K % 8 == 0
    l = lib()
    if norm is not None:
        norm_w, norm_eps, norm_out = norm
        assert out.dtype == torch.float32 and epilogue != EPI_SWIGLU
        assert norm_w.numel() == N and tuple(norm_out.shape) == (M, N)
        fuses = fast and kernel in ("auto", "tc5") and bool(l.sb_gemm_tc5_fuses_norm(
            M, N, K, _sm_count(a.device), epilogue, _code(out.dtype), 0))
        if fuses and (kernel == "tc5" or FORCE_DECODE_KERNEL != "skinny"):
            kernel = "tc5"
        else:
            linear(a, w, out, epilogue, bias, residual, kernel, warm=warm)
            rmsnorm(out, norm_w, norm_eps, norm_out)
            return out
    if kernel == "auto" and fast:
        kernel = _pick_kernel(M, N, K, a.device)
    if fast and kernel in ("tc5", "tc5_normal"):
        form = 1 if kernel == "tc5_normal" else 0
        ws = _tc5_workspace(M, N, K, a.device) if form == 0 else None
        extras = None
        if norm is not None or (warm is not None and WARM):
            extras = LinearExtras()
            if norm is not None:
                extras.norm_weight, extras.norm_weight_dtype = norm_w.data_ptr(), _code(norm_w.dtype)
                extras.norm_eps, extras.norm_out = norm_eps, norm_out.data_ptr()
                extras.norm_out_dtype = _code(norm_out.dtype)
            if warm is not None and WARM:
                extras.warm, extras.warm_bytes = warm.data_ptr(), warm.numel() * warm.element_size()
        _check(l.sb_gemm_tc5_ex(*args[:-1], _ptr(ws), ctypes.c_size_t(ws.numel() if ws is not None else 0),
                                _sm_count(a.device), form,
                                ctypes.byref(extras) if extras is not None else None, _stream()),
               "linear (tcgen05 kernel)",
               launches=2 if ws is not None else 1)        # a split product adds its reduce kernel
    elif fast and kernel == "skinny":
        _check(l.sb_gemm_skinny(*args), "linear (weight-streaming kernel)")
    elif fast and kernel == "tiled":
        _check(l.sb_gemm_tiled(*args), "linear (tiled kernel)")
    elif kernel in ("plain", "auto") or not fast:
        _check(l.sb_gemm_plain(*args), "linear (plain kernel)")
    else:
        raise KernelError(f"linear: unknown kernel {kernel!r}")
    return out


class RopeStore(ctypes.Structure):
    """SbRopeStore of the kernel library: the rotation + cache write that finishes a q|k|v product."""
    _fields_ = [("n_q_heads", ctypes.c_int), ("n_kv_heads", ctypes.c_int), ("hd", ctypes.c_int),
                ("rot", ctypes.c_int), ("inv_freq", ctypes.c_void_p), ("row_seq", ctypes.c_void_p),
                ("row_pos", ctypes.c_void_p), ("page_off", ctypes.c_void_p), ("page_ids", ctypes.c_void_p),
                ("page_size", ctypes.c_int), ("cache", ctypes.c_void_p), ("q_out", ctypes.c_void_p)]


class LinearExtras(ctypes.Structure):
    """SbLinearExtras of the kernel library: what may accompany a product."""
    _fields_ = [("norm_weight", ctypes.c_void_p), ("norm_weight_dtype", ctypes.c_int),
                ("norm_eps", ctypes.c_float), ("norm_out", ctypes.c_void_p),
                ("norm_out_dtype", ctypes.c_int), ("warm", ctypes.c_void_p),
                ("warm_bytes", ctypes.c_size_t), ("rope", ctypes.POINTER(RopeStore))]


def qkv_rope_store(h: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None, n_q_heads: int,
                   n_kv_heads: int, head_dim: int, rotary_dim: int, inv_freq: torch.Tensor, row_seq,
                   row_pos, page_off, page_ids, page_size: int, cache: torch.Tensor | None,
                   q_out: torch.Tensor) -> torch.Tensor:
    """The fused [q | k | v] projection of the rows `h` (+ bias), the rotation of q and k, q into
    `q_out` [rows, heads, hd] and k, v into the cache pages (`cache=None`: the weight holds the
    query rows only).  Where the split-K decode form of the tcgen05 product runs (9 to 64 rows of
    bfloat16), its reduce kernel does the rotation and the cache write too and the float32 row
    is never written; else the product and `rope_store` run one after the other."""
    M, K = h.shape
    N = w.shape[0]
    has_kv = cache is not None
    l = lib()
    fused = (h.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and q_out.dtype == torch.bfloat16
             and (not has_kv or cache.dtype == torch.bfloat16) and K % 8 == 0
             and (bias is None or bias.numel() == N)
             and _pick_kernel(M, N, K, h.device) == "tc5"
             and bool(l.sb_gemm_tc5_fuses_rope(M, N, K, _sm_count(h.device), n_q_heads, n_kv_heads, head_dim,
                                              rotary_dim, 1 if has_kv else 0)))
    if not fused:
        qkv = torch.empty((M, N), dtype=torch.float32, device=h.device)
        linear(h, w, qkv, EPI_BIAS if bias is not None else EPI_NONE, bias=bias)
        return rope_store(qkv, n_q_heads, n_kv_heads, head_dim, rotary_dim, inv_freq, row_seq, row_pos,
                          page_off, page_ids, page_size, cache, q_out)
    assert inv_freq.dtype == torch.float32 and inv_freq.numel() >= rotary_dim // 2
    rope = RopeStore(n_q_heads, n_kv_heads, head_dim, rotary_dim, inv_freq.data_ptr(),
                     _i32(row_seq, "row_seq"), _i32(row_pos, "row_pos"),
                     _i32(page_off, "page_off") if has_kv else None,
                     _i32(page_ids, "page_ids") if has_kv else None, page_size,
                     cache.data_ptr() if has_kv else None, _ptr(q_out))
    extras = LinearExtras()
    extras.rope = ctypes.pointer(rope)
    ws = _tc5_workspace(M, N, K, h.device)
    _check(l.sb_gemm_tc5_ex(_ptr(h), BF16, _ptr(w), BF16, M, N, K, EPI_BIAS if bias is not None else EPI_NONE,
                            _ptr(bias), _code(bias.dtype) if bias is not None else 0, _ptr(None), _ptr(None), F32,
                            _ptr(ws), ctypes.c_size_t(ws.numel()), _sm_count(h.device), 0,
                            ctypes.byref(extras), _stream()),
           "q|k|v product with rotation (tcgen05 kernel)", launches=2)
    return q_out


def _warm_args(warm):
    """(pointer, bytes) of an L2 hint as the kernels take it."""
    if warm is None or not WARM:
        return _ptr(None), ctypes.c_size_t(0)
    return _ptr(warm), ctypes.c_size_t(warm.numel() * warm.element_size())


WARM = _os.environ.get("SB_WARM", "1") != "0"       # L2 hints on (SB_WARM=0: off, for measurements)
# "skinny" or "tc5": overrides the choice below (for measurements; SB_DECODE_KERNEL in the environment)
FORCE_DECODE_KERNEL = _os.environ.get("SB_DECODE_KERNEL") or None


def _pick_kernel(M: int, N: int, K: int, device) -> str:
    """Which bfloat16 product kernel "auto" means.  The tcgen05 kernel, except for small
    matrices at up to 8 rows: there the kernel that streams W into mma.sync fragments has lower
    fixed costs (measured on B200 at the 7B layer sizes, alone inside CUDA graphs: 9 us against
    12 us for the 4608 x 3584 product at 8 rows, while at 64 rows the tcgen05 kernel takes 12 us
    and the streaming kernel 19 us; inside the decode step, where the tcgen05 kernel requests its
    weights while the kernel before it ends, the streaming kernel wins by 0.5 % of the step at
    8 rows and loses by 1.3 % at 16)."""
    if M > 8:
        return "tc5"
    if FORCE_DECODE_KERNEL:
        return FORCE_DECODE_KERNEL
    tiles = (N + 127) // 128
    if tiles >= _sm_count(device) or K >= 8192:
        return "tc5"
    return "skinny"


def requests_weights_late(M: int, N: int, K: int, device) -> bool:
    """Whether the bfloat16 product kernel that "auto" picks for these sizes starts only when
    the kernel before it has ended (it is launched without programmatic dependent launch), so
    that its weights are worth an L2 hint from an earlier kernel."""
    kernel = _pick_kernel(M, N, K, device)
    cls = PDL_TC5 if kernel == "tc5" else PDL_SKINNY
    return not (int(lib().sb_pdl_enabled()) & cls)


_sm_counts: dict = {}
_tc5_buffers: dict = {}          # device -> list of workspaces (never freed:
                                 # captured graphs may hold their addresses)


def _sm_count(device) -> int:
    n = _sm_counts.get(device)
    if n is None:
        key = torch.device(device).index or 0
        n = _sm_counts[device] = torch.cuda.get_device_properties(key).multi_processor_count
    return n


def _tc5_workspace(M: int, N: int, K: int, device):
    """Workspace of a tcgen05 product that splits K (the decode form, and the many-rows form when
    it has few row tiles): the partial sums.  One buffer per device serves every call on the
    stream; it only grows."""
    l = lib()
    need = int(l.sb_gemm_tc5_scratch_bytes(M, N, K, _sm_count(device)))
    if need == 0:
        return None
    key = torch.device(device).index or 0
    bufs = _tc5_buffers.setdefault(key, [])
    if not bufs or bufs[-1].numel() < need:
        bufs.append(torch.empty(max(need, 16 << 20), dtype=torch.uint8, device=device))
    return bufs[-1]


PDL_TC5, PDL_SKINNY, PDL_ATTENTION, PDL_ELEMENTWISE, PDL_REDUCE, PDL_OTHER, PDL_ALL = 1, 2, 4, 8, 16, 32, 63


def set_pdl(level) -> None:
    """Which kernels are launched with programmatic dependent launch: a mask of the PDL_* bits
    (0 none, PDL_ALL every kernel; the default is every class but PDL_SKINNY).  The
    environment variable SB_PDL sets it at start."""
    level = int(level)
    lib().sb_set_pdl(level)
    for l in _attn_libs.values():
        if l is not None:
            l.sb_set_pdl(level)


def tc5_status() -> int:
    """0 unless a tcgen05 kernel gave up on a bounded wait since the last call (synchronizes)."""
    return int(lib().sb_tc5_status())


def tc5_tile_width(M: int, N: int) -> int:
    """The tile width the tcgen05 product of M rows and N features runs with in its many-rows
    form (0: that form does not run): for tests that want every width covered."""
    sms = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    return int(lib().sb_gemm_tc5_tile_width(int(M), int(N), sms))


def force_tc5_tile_width(width: int) -> None:
    """256, 240, 224, 208 or 192: every many-rows tcgen05 product uses that tile width (for
    measurements and tests); 0: chosen by the sizes again."""
    lib().sb_gemm_tc5_force_width(int(width))


def set_tc5_pairs(mode: int) -> None:
    """Whether the tcgen05 product of more than 128 rows runs on pairs of SMs (a cluster of two
    blocks on one 256-row tile): 1 yes, 0 no (one block per 128-row tile), -1 by SB_TC5_PAIR
    (default yes).  The result is the same to the bit either way."""
    lib().sb_gemm_tc5_pairs(int(mode))


def rope_store(qkv: torch.Tensor, n_q_heads: int, n_kv_heads: int, head_dim: int, rotary_dim: int,
               inv_freq: torch.Tensor, row_seq, row_pos, page_off, page_ids, page_size: int,
               cache: torch.Tensor | None, q_out: torch.Tensor) -> torch.Tensor:
    """Rotates q and k, writes q to q_out [rows, heads, hd] and k, v into the cache pages.
    With cache=None the input row holds queries only (a layer that reads another's cache)."""
    n = qkv.shape[0]
    has_kv = cache is not None
    assert qkv.dtype == torch.float32
    assert qkv.shape[1] == (n_q_heads + (2 * n_kv_heads if has_kv else 0)) * head_dim
    assert inv_freq.dtype == torch.float32 and inv_freq.numel() >= rotary_dim // 2
    _check(lib().sb_rope_store(
        _ptr(qkv), n, n_q_heads, n_kv_heads, head_dim, rotary_dim, _ptr(inv_freq),
        _i32(row_seq, "row_seq"), _i32(row_pos, "row_pos"),
        _i32(page_off, "page_off") if has_kv else _ptr(None),
        _i32(page_ids, "page_ids") if has_kv else _ptr(None), page_size,
        _ptr(cache), _code(cache.dtype) if has_kv else _code(q_out.dtype), _ptr(q_out),
        _code(q_out.dtype), 1 if has_kv else 0, _stream()), "rope_store")
    return q_out


_attn_libs: dict = {}
_attn_counter_bufs: dict = {}    # device -> zeroed int32 buffers (kernels leave them zero; never freed)


def _attn_counters(n: int, device) -> torch.Tensor:
    """Arrival counters of the split attention's merge: zero between launches."""
    key = torch.device(device).index or 0
    bufs = _attn_counter_bufs.setdefault(key, [])
    if not bufs or bufs[-1].numel() < n:
        bufs.append(torch.zeros(max(n, 1 << 16), dtype=torch.int32, device=device))
    return bufs[-1]



def attention_lib(head_dim: int):
    """The tensor-core attention library of one head size, or None when the head size is
    outside what those kernels are written for (multiples of 16 up to 256)."""
    if head_dim not in _attn_libs:
        if head_dim in _build.HEAD_DIMS:
            al = _abi.apply(_build.load_attention(head_dim), _abi.ATTENTION)
            # SB_ATTN=mma|tma in the environment: one kernel family for every step (for measurements)
            al.sb_attention_force_mma({"mma": 1, "tma": 2}.get(_os.environ.get("SB_ATTN", ""), 0))
            _attn_libs[head_dim] = al
        else:
            _attn_libs[head_dim] = None
    return _attn_libs[head_dim]


def attention(q: torch.Tensor, out: torch.Tensor, plan, group_index: int, cache: torch.Tensor,
              n_q_heads: int, n_kv_heads: int, head_dim: int, window: int, scale: float,
              kernel: str = "auto", warm: torch.Tensor | None = None) -> torch.Tensor:
    """Causal grouped-query attention of the step's rows over one cache entry's pages.

    bfloat16 runs the tensor-core kernels (built for the head size at first use); float32, a
    head size those kernels do not take, or `kernel="plain"` run the plain kernel.  `"mma"` keeps
    to the mma.sync kernels where the tensor-memory prefill kernel or the persistent TMA decode
    kernel would run (head sizes 64, 128); `"tma"` runs that decode kernel whatever the number of
    key splits (by itself it runs from about a wave of splits on).
    `warm`: a tensor the kernel after this one will stream (weights); the decode kernel asks for
    it into L2 while it merges its partial results.  A hint: it changes no result."""
    n = q.shape[0]
    g = plan.groups[group_index]
    al = attention_lib(head_dim) if (q.dtype == torch.bfloat16 and cache.dtype == torch.bfloat16
                                     and kernel != "plain") else None
    if al is not None:
        need = int(al.sb_attention_scratch_bytes(n, n_q_heads, n_kv_heads, plan.max_new, plan.max_len))
        scratch = plan.scratch(need, q.device)
        counters = _attn_counters(plan.n_seqs * n_kv_heads, q.device)
        if kernel in ("mma", "tma"):
            al.sb_attention_force_mma(1 if kernel == "mma" else 2)
        rc = al.sb_attention(
            _ptr(q), _ptr(out), n, plan.n_seqs, plan.max_new, _i32(plan.seq_row0, "seq_row0"),
            _i32(plan.seq_pos0, "seq_pos0"), _i32(g.page_off, "page_off"),
            _i32(g.page_ids, "page_ids"), g.page_size, _ptr(cache), n_q_heads, n_kv_heads,
            head_dim, window, ctypes.c_float(scale), _ptr(scratch),
            ctypes.c_size_t(scratch.numel() if scratch is not None else 0),
            _ptr(counters), counters.numel(), plan.max_len, cache.shape[0], _sm_count(q.device),
            *_warm_args(warm), _stream())
        if kernel in ("mma", "tma"):
            al.sb_attention_force_mma({"mma": 1, "tma": 2}.get(_os.environ.get("SB_ATTN", ""), 0))
        if rc != 0:
            raise KernelError(f"attention: {al.sb_last_error().decode()}")
        global LAUNCHES
        LAUNCHES += int(al.sb_attention_last_launches())
    else:
        _check(lib().sb_attention_plain(
            _ptr(q), _ptr(out), _code(q.dtype), n, _i32(plan.row_seq, "row_seq"),
            _i32(plan.row_pos, "row_pos"), _i32(g.page_off, "page_off"),
            _i32(g.page_ids, "page_ids"), g.page_size, _ptr(cache), _code(cache.dtype),
            n_q_heads, n_kv_heads, head_dim, window, ctypes.c_float(scale), _stream()),
            "attention (plain kernel)")
    return out


def attention_status(head_dim: int) -> int:
    """0 when no tensor-memory attention kernel of this head size has given up on a wait since the
    last call (else the code of that wait); -1 when the head size has no such kernel."""
    al = attention_lib(head_dim)
    return int(al.sb_attention_status()) if al is not None else -1


def sample_params_size() -> int:
    return lib().sb_sample_params_size()


def sample(logits: torch.Tensor, params: torch.Tensor, history: torch.Tensor | None,
           out_tokens: torch.Tensor, fed_pos: torch.Tensor | None = None) -> torch.Tensor:
    """One token per logits row; `params` is a uint8 tensor of packed per-row records.  With
    `fed_pos` (int32 per row) the draw's position is fed_pos + 1 instead of the record's.
    A row whose logits are not finite may get -1: `check_tokens` turns that into an error."""
    n, vocab = logits.shape
    assert logits.dtype == torch.float32 and params.dtype == torch.uint8
    assert params.numel() == n * sample_params_size()
    stride = history.shape[1] if history is not None else 0
    _check(lib().sb_sample(_ptr(logits), n, vocab, _ptr(params),
                           _i32(history, "history") if history is not None else _ptr(None),
                           stride, _i32(fed_pos, "fed_pos") if fed_pos is not None else _ptr(None),
                           _i32(out_tokens, "out_tokens"), _stream()), "sample")
    return out_tokens


def check_tokens(ids: list, live: list | None = None) -> list:
    """Sampled ids as read on the host: raises where the sampler chose no token (rows whose
    `live` entry is false are not looked at)."""
    bad = [i for i, t in enumerate(ids) if t < 0 and (live is None or live[i])]
    if bad:
        raise KernelError(f"the sampler chose no token for row {bad[0]}: its logits are not finite")
    return ids


def check_status() -> None:
    """Raises KernelError if a kernel of any loaded library gave up on one of its bounded waits
    since the last look (its output is then incomplete).  Reading synchronizes with the device,
    so this is called where the host waits anyway."""
    if _lib is None:
        return
    code = tc5_status()
    if code:
        raise KernelError(f"a tcgen05 product kernel gave up on a bounded wait (code {code}): "
                          "results since the last check are incomplete")
    for hd, l in _attn_libs.items():
        if l is not None:
            code = int(l.sb_attention_status())
            if code > 0:
                raise KernelError(f"the tensor-memory attention kernel of head size {hd} gave up "
                                  f"on a bounded wait (code {code}): results since the last check "
                                  "are incomplete")


def add_i32(x: torch.Tensor, delta: int) -> torch.Tensor:
    """x += delta on the device (int32)."""
    _check(lib().sb_add_i32(_i32(x, "x"), x.numel(), int(delta), _stream()), "add_i32")
    return x


def advance_rows(pos: torch.Tensor, last: torch.Tensor) -> torch.Tensor:
    """pos[i] = min(pos[i] + 1, last[i]) on the device (int32): the positions of a captured
    decode batch move on, each row at most to the last position it holds pages for."""
    assert pos.numel() == last.numel()
    _check(lib().sb_advance_rows(_i32(pos, "pos"), _i32(last, "last"), pos.numel(), _stream()),
           "advance_rows")
    return pos


def random_normal(out: torch.Tensor, key0: int, key1: int, mean: float, std: float) -> torch.Tensor:
    """Fills `out` (float32 or bfloat16, contiguous) with mean + std * z, z standard normal drawn
    from the counter-based generator keyed by (key0, key1) and the element index."""
    _check(lib().sb_random_normal(_ptr(out), _code(out.dtype), ctypes.c_size_t(out.numel()),
                                  ctypes.c_uint32(key0 & 0xffffffff), ctypes.c_uint32(key1 & 0xffffffff),
                                  ctypes.c_float(mean), ctypes.c_float(std), _stream()),
           "random_normal")
    return out
