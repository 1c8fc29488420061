"""Python face of the CUDA launchers: each function checks its tensors, passes raw device
pointers and the current stream to an ``extern "C"`` launcher, and raises on any error.

There is no CPU path: a tensor that is not on a CUDA device is an error, and so is a
library that cannot be built or loaded.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_ulonglong, c_void_p
from typing import Optional

import torch

from .build import load_library

F32, BF16 = 0, 1
PAGE = 64
_CODES = {torch.float32: F32, torch.bfloat16: BF16}
_ERRORS = {2001: "a size or dtype this kernel does not take", 2002: "inconsistent arguments",
           2003: "the tensor-map encoder of the CUDA driver is not available",
           2004: "the CUDA driver refused a tensor map"}


class KernelError(RuntimeError):
    pass


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _CODES[dtype]
    except KeyError:
        raise KernelError(f"kernels take float32 or bfloat16, not {dtype}") from None


launches = 0      # kernels launched by this module since import (benchmarks read the difference)


def _check(code: int, what: str, n_kernels: int = 1) -> None:
    global launches
    launches += n_kernels
    if code != 0:
        why = _ERRORS.get(code, f"CUDA error {code}")
        raise KernelError(f"{what}: {why}")


def _ptr(t: Optional[torch.Tensor], what: str = "tensor") -> Optional[int]:
    if t is None:
        return None
    if not t.is_cuda:
        raise KernelError(f"{what} must live on a CUDA device (there is no CPU path)")
    if not t.is_contiguous():
        raise KernelError(f"{what} must be contiguous")
    return t.data_ptr()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The current CUDA stream's handle (called once per launch: the short way where torch has it)."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _i32(t: Optional[torch.Tensor], what: str) -> Optional[int]:
    if t is not None and t.dtype != torch.int32:
        raise KernelError(f"{what} must be int32, got {t.dtype}")
    return _ptr(t, what)


def _f32(t: Optional[torch.Tensor], what: str) -> Optional[int]:
    if t is not None and t.dtype != torch.float32:
        raise KernelError(f"{what} must be float32, got {t.dtype}")
    return _ptr(t, what)


def _f64(t: Optional[torch.Tensor], what: str) -> Optional[int]:
    if t is not None and t.dtype != torch.float64:
        raise KernelError(f"{what} must be float64, got {t.dtype}")
    return _ptr(t, what)


_configured: set[str] = set()


def _lib(name: str) -> ctypes.CDLL:
    lib = load_library(name)
    if name not in _configured:
        _SIGNATURES[name](lib)
        _configured.add(name)
    return lib


def _sig_ops(lib: ctypes.CDLL) -> None:
    lib.mf_embed.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_float,
                             c_void_p, c_void_p]
    lib.mf_rmsnorm.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float,
                               c_void_p]
    lib.mf_rope_kvstore.argtypes = ([c_void_p, c_int, c_void_p] + [c_void_p] * 10 + [c_int] * 9 +
                                    [c_void_p, c_void_p])
    lib.mf_add_rmsnorm.argtypes = [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
                                   c_int, c_int, c_float, c_void_p]
    lib.mf_swiglu.argtypes = [c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p]
    lib.mf_gather_rows.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p]
    lib.mf_cast.argtypes = [c_void_p, c_int, c_void_p, c_int, c_longlong, c_void_p]


def _sig_gemm_simt(lib: ctypes.CDLL) -> None:
    lib.mf_gemm_simt.argtypes = [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int,
                                 c_int, c_int, c_int, c_longlong, c_longlong, c_longlong, c_int,
                                 c_void_p]


def _sig_attention(lib: ctypes.CDLL) -> None:
    lib.mf_attention_packed.argtypes = [c_void_p] * 7 + [c_int] * 5 + [c_float, c_int, c_void_p]
    lib.mf_attention_paged.argtypes = ([c_void_p] * 6 + [c_int, c_int, c_void_p, c_void_p] +
                                       [c_int] * 7 + [c_float, c_int, c_int, c_longlong, c_void_p,
                                                      c_int, c_void_p])


def _sig_sampling(lib: ctypes.CDLL) -> None:
    lib.mf_sample.argtypes = [c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p, c_void_p,
                              c_void_p, c_float, c_int, c_float, c_float, c_float, c_float,
                              c_ulonglong, c_int, c_void_p]
    lib.mf_sampler_state_ints.argtypes = []


def _sig_gemm_tc(lib: ctypes.CDLL) -> None:
    lib.mf_gemm_tc.argtypes = [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p,
                               c_longlong, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
                               c_void_p, c_void_p]
    lib.mf_splitk_reduce.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_longlong, c_int, c_int,
                                     c_int, c_int, c_void_p]
    lib.mf_gemm_tc_workspace_floats.argtypes = [c_int, c_int, c_int, c_int]
    lib.mf_gemm_tc_workspace_floats.restype = c_longlong
    lib.mf_gemm_tc_plan.argtypes = [c_int, c_int, c_int, c_int, c_void_p, c_void_p]
    lib.mf_gemm_pair_plan.argtypes = [c_int, c_int, c_int, c_void_p, c_void_p]
    lib.mf_gemm_pair_dual_mode.argtypes = [c_int]
    lib.mf_gemm_pair_dual_mode.restype = None
    lib.mf_gemm_pair_group_m.argtypes = [c_int]
    lib.mf_gemm_pair_group_m.restype = None
    lib.mf_gemm_tc_fused.argtypes = [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p,
                                     c_longlong, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
                                     c_void_p, c_int, c_int, c_float, c_void_p, c_longlong, c_void_p,
                                     c_void_p, c_void_p, c_void_p]
    lib.mf_gemm_tc_prep_parts.argtypes = [c_int, c_int, c_int]
    lib.mf_wait_probe.argtypes = [c_void_p, ctypes.c_uint, c_ulonglong, c_void_p, c_void_p]


def _sig_attention_prefill(lib: ctypes.CDLL) -> None:
    lib.mf_attention_prefill_mma.argtypes = [c_void_p] * 5 + [c_int] * 6 + [c_float, c_void_p]


def _sig_attention_prefill_tc(lib: ctypes.CDLL) -> None:
    lib.mf_attention_prefill_tc.argtypes = [c_void_p] * 5 + [c_int] * 7 + [c_float, c_void_p, c_void_p]
    lib.mf_attention_prefill_tc_paged.argtypes = ([c_void_p] * 6 + [c_int, c_int, c_void_p] + [c_int] * 7 +
                                                  [c_float, c_longlong, c_void_p, c_void_p])


_SIGNATURES = {"attention_prefill_tc": _sig_attention_prefill_tc,
               "attention_prefill": _sig_attention_prefill, "gemm_tc": _sig_gemm_tc, "ops": _sig_ops, "gemm_simt": _sig_gemm_simt, "attention": _sig_attention,
               "sampling": _sig_sampling}


# ---------------------------------------------------------------------------------------
# row-wise ops
# ---------------------------------------------------------------------------------------
def embed(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, status: torch.Tensor,
          scale: float = 1.0) -> None:
    """out[t] = table[ids[t]] * scale in float32; an id outside the table sets status bit 1."""
    n, width = out.shape
    vocab = table.shape[0]
    if table.shape[1] != width or ids.numel() != n:
        raise KernelError("embed: shapes do not fit")
    _check(_lib("ops").mf_embed(_ptr(table, "table"), dtype_code(table.dtype), _i32(ids, "ids"),
                                _f32(out, "out"), n, width, vocab, float(scale),
                                _i32(status, "status"), _stream()), "embed")


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
            rows: Optional[torch.Tensor] = None) -> None:
    """out[r] = rmsnorm(x[rows[r]] or x[r]) * weight.  ``weight`` and ``rows`` are read while
    the kernel before this one may still run: weights, or inputs of the step."""
    n, width = out.shape
    if x.shape[1] != width or weight.numel() != width:
        raise KernelError("rmsnorm: shapes do not fit")
    if rows is None and x.shape[0] != n:
        raise KernelError("rmsnorm: row counts do not fit")
    _check(_lib("ops").mf_rmsnorm(_f32(x, "x"), _f32(weight, "weight"), _i32(rows, "rows"),
                                  _ptr(out, "out"), dtype_code(out.dtype), n, width, float(eps),
                                  _stream()), "rmsnorm")


def add_rmsnorm(h: torch.Tensor, partial: Optional[torch.Tensor], n_partials: int,
                bias: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                out: torch.Tensor) -> None:
    """h += bias + sum of the K splits in ``partial`` [n_partials, rows, width]; out = rmsnorm(h)."""
    n, width = out.shape
    if h.shape != (n, width) or weight.numel() != width:
        raise KernelError("add_rmsnorm: shapes do not fit")
    if n_partials > 0 and (partial is None or partial.numel() < n_partials * n * width):
        raise KernelError("add_rmsnorm: the partial sums are too small")
    _check(_lib("ops").mf_add_rmsnorm(_f32(h, "h"), _f32(partial, "partial"), int(n_partials),
                                      _f32(bias, "bias"), _f32(weight, "weight"), _ptr(out, "out"),
                                      dtype_code(out.dtype), n, width, float(eps), _stream()),
           "add_rmsnorm")


def rope_kvstore(qkv: torch.Tensor, positions: torch.Tensor, token_row: torch.Tensor,
                 seq_end: torch.Tensor, inv_freq: Optional[torch.Tensor], q_out: torch.Tensor,
                 k_out: Optional[torch.Tensor], v_out: Optional[torch.Tensor],
                 k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor],
                 page_table: Optional[torch.Tensor], table_stride: int, ring: int,
                 n_heads: int, n_kv: int, head_dim: int, rotary_dim: int, style: int,
                 status: torch.Tensor, n_partials: int = 0,
                 bias: Optional[torch.Tensor] = None) -> None:
    """``n_partials`` > 0: ``qkv`` is [n_partials, tokens, width], the K splits a deferred
    projection left; they are added here in split order, with ``bias``.

    The kernel reads ``positions``, ``token_row``, ``seq_end``, ``page_table``, ``inv_freq`` and
    ``bias`` while the kernel before it may still run (it only waits for that kernel before it
    touches ``qkv``).  They must therefore be final before the step's first kernel starts, as
    the engine's step inputs are (one copy to the device in front of the step), or be written
    by an ordinary launch, which this kernel waits for in full."""
    if n_partials > 0:
        if qkv.dim() != 3 or qkv.shape[0] != n_partials:
            raise KernelError("rope_kvstore: partial sums must be [splits, tokens, width]")
        n, width = qkv.shape[1], qkv.shape[2]
    else:
        n, width = qkv.shape
    if width != (n_heads + 2 * n_kv) * head_dim:
        raise KernelError("rope_kvstore: qkv has the wrong width")
    if bias is not None and bias.numel() != width:
        raise KernelError("rope_kvstore: bias has the wrong length")
    dt = q_out.dtype
    for t in (k_out, v_out, k_cache, v_cache):
        if t is not None and t.dtype != dt:
            raise KernelError("rope_kvstore: q, k, v and the cache must share one dtype")
    if (k_cache is None) != (v_cache is None) or (k_cache is not None and page_table is None):
        raise KernelError("rope_kvstore: the cache needs keys, values and a page table")
    _check(_lib("ops").mf_rope_kvstore(
        _f32(qkv, "qkv"), int(n_partials), _f32(bias, "bias"), _i32(positions, "positions"),
        _i32(token_row, "token_row"),
        _i32(seq_end, "seq_end"), _f64(inv_freq, "inv_freq"), _ptr(q_out, "q_out"),
        _ptr(k_out, "k_out"), _ptr(v_out, "v_out"), _ptr(k_cache, "k_cache"),
        _ptr(v_cache, "v_cache"), _i32(page_table, "page_table"), int(table_stride), int(ring),
        n, n_heads, n_kv, head_dim, rotary_dim, style, dtype_code(dt), _i32(status, "status"),
        _stream()), "rope_kvstore")


def swiglu(gate_up: torch.Tensor, out: torch.Tensor, interleaved: bool = False) -> None:
    """out = silu(gate) * up; ``interleaved``: the columns of ``gate_up`` alternate gate, up
    instead of all gates first."""
    n, nf = out.shape
    if gate_up.shape != (n, 2 * nf):
        raise KernelError("swiglu: shapes do not fit")
    _check(_lib("ops").mf_swiglu(_ptr(gate_up, "gate_up"), dtype_code(gate_up.dtype),
                                 _ptr(out, "out"), dtype_code(out.dtype), n, nf,
                                 1 if interleaved else 0, _stream()),
           "swiglu")


def gather_rows(x: torch.Tensor, rows: torch.Tensor, out: torch.Tensor) -> None:
    n, width = out.shape
    if x.shape[1] != width or rows.numel() != n:
        raise KernelError("gather_rows: shapes do not fit")
    _check(_lib("ops").mf_gather_rows(_f32(x, "x"), _i32(rows, "rows"), _f32(out, "out"), n, width,
                                      _stream()), "gather_rows")


def cast(src: torch.Tensor, out: torch.Tensor) -> None:
    if src.numel() != out.numel():
        raise KernelError("cast: sizes differ")
    _check(_lib("ops").mf_cast(_ptr(src, "src"), dtype_code(src.dtype), _ptr(out, "out"),
                               dtype_code(out.dtype), src.numel(), _stream()), "cast")


# ---------------------------------------------------------------------------------------
# matrix product on the FP32 pipe
# ---------------------------------------------------------------------------------------
def gemm_simt(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor,
              accumulate: bool = False) -> None:
    """out[M,N] (+)= a[M,K] @ w[N,K]^T + bias.  Rows may be strided (last dim contiguous)."""
    m, k = a.shape
    n = w.shape[0]
    if w.shape[1] != k or out.shape != (m, n):
        raise KernelError(f"gemm: shapes do not fit: a {tuple(a.shape)}, w {tuple(w.shape)}, "
                          f"out {tuple(out.shape)}")
    for t, what in ((a, "a"), (w, "w"), (out, "out")):
        if not t.is_cuda:
            raise KernelError(f"gemm: {what} must live on a CUDA device (there is no CPU path)")
        if t.stride(1) != 1:
            raise KernelError(f"gemm: {what} must be contiguous along its last dimension")
    if bias is not None and bias.numel() != n:
        raise KernelError("gemm: bias has the wrong length")
    _check(_lib("gemm_simt").mf_gemm_simt(
        a.data_ptr(), dtype_code(a.dtype), w.data_ptr(), dtype_code(w.dtype), _f32(bias, "bias"),
        out.data_ptr(), dtype_code(out.dtype), m, n, k, a.stride(0), w.stride(0), out.stride(0),
        1 if accumulate else 0, _stream()), "gemm_simt")


# ---------------------------------------------------------------------------------------
# matrix product on the tensor cores (bfloat16 x bfloat16, float32 accumulation)
# ---------------------------------------------------------------------------------------
EPI_STORE, EPI_ACCUM, EPI_SWIGLU = 0, 1, 2


def gemm_tc_supported(x: torch.Tensor, w: torch.Tensor) -> bool:
    """The tensor-core kernel takes bfloat16 operands whose rows start on 16-byte
    boundaries (TMA); anything else goes to the FP32-pipe kernel."""
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.dim() == 2
            and w.dim() == 2 and x.shape[1] % 8 == 0 and x.stride(1) == 1 and w.stride(1) == 1
            and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0
            and w.data_ptr() % 16 == 0)


_PLANS: dict = {}


def gemm_tc_plan(m: int, n: int, k: int, epi: int = EPI_STORE) -> tuple[int, int]:
    """(token tile, K splits) the kernel uses for these sizes (a function of the sizes only:
    asked once per shape)."""
    return _gemm_tc_shape(m, n, k, epi)[:2]


def gemm_pair_plan(m: int, n: int, k: int) -> tuple[int, bool]:
    """(token tile, two token tiles a pair at once) of the CTA-pair kernel, which runs products
    of 256 tokens and more."""
    nt, dual = ctypes.c_int(0), ctypes.c_int(0)
    _lib("gemm_tc").mf_gemm_pair_plan(m, n, k, ctypes.addressof(nt), ctypes.addressof(dual))
    return nt.value, bool(dual.value)


def gemm_pair_dual_mode(mode: int) -> None:
    """0: a pair never takes two token tiles at once; 1: where the kernel's cost model says so
    (the default); 2: always.  The result's bits are the same in every mode."""
    _lib("gemm_tc").mf_gemm_pair_dual_mode(int(mode))


def gemm_pair_group_m(group_m: int) -> None:
    """The CTA-pair kernel walks the token tiles in groups of this many (0: chosen from the sizes,
    the default).  The order of the tiles changes no bits."""
    _lib("gemm_tc").mf_gemm_pair_group_m(int(group_m))


def _gemm_tc_shape(m: int, n: int, k: int, epi: int) -> tuple[int, int, int]:
    """(token tile, K splits, workspace floats) of a product of these sizes."""
    key = (m, n, k, epi)
    got = _PLANS.get(key)
    if got is None:
        lib = _lib("gemm_tc")
        nt, sp = ctypes.c_int(0), ctypes.c_int(0)
        lib.mf_gemm_tc_plan(m, n, k, epi, ctypes.addressof(nt), ctypes.addressof(sp))
        got = (nt.value, sp.value, int(lib.mf_gemm_tc_workspace_floats(m, n, k, epi)))
        _PLANS[key] = got
    return got


def gemm_tc(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor,
            epi: int, status: torch.Tensor) -> None:
    """out (+)= x @ w^T + bias on tcgen05.  EPI_SWIGLU: w's rows alternate gate, up and out is
    [M, N/2] bfloat16 = silu(gate) * up."""
    m, k = x.shape
    n = w.shape[0]
    if w.shape[1] != k:
        raise KernelError(f"gemm: shapes do not fit: x {tuple(x.shape)}, w {tuple(w.shape)}")
    want_cols = n // 2 if epi == EPI_SWIGLU else n
    if out.shape != (m, want_cols) or out.stride(1) != 1:
        raise KernelError(f"gemm: out has shape {tuple(out.shape)}, expected {(m, want_cols)}")
    if not gemm_tc_supported(x, w):
        raise KernelError("gemm_tc: operands must be bfloat16 with 16-byte aligned rows")
    if bias is not None and bias.numel() != n:
        raise KernelError("gemm: bias has the wrong length")
    lib = _lib("gemm_tc")
    need = _gemm_tc_shape(m, n, k, epi)[2]
    ws = torch.empty(need, dtype=torch.float32, device=x.device) if need else None
    _check(lib.mf_gemm_tc(x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), _f32(bias, "bias"),
                          out.data_ptr(), out.stride(0), dtype_code(out.dtype), m, n, k, epi,
                          _ptr(ws, "workspace"), None, _i32(status, "status"), _stream()),
           "gemm_tc", 2 if need else 1)


class RowScale:
    """A norm whose 1/rms is still to be applied to the rows of an activation: the rows hold
    x' = h * g (g: the norm's weight), ``ssq`` [parts, rows] the sums of h^2 per group of
    columns, as the product before left them.  The product that reads x' multiplies row t's
    results by ``rsqrt(ssq[:, t].sum() / width + eps)``."""

    __slots__ = ("ssq", "width", "eps")

    def __init__(self, ssq: torch.Tensor, width: int, eps: float):
        self.ssq, self.width, self.eps = ssq, int(width), float(eps)


_PREP_PARTS: dict = {}


def gemm_tc_prep_parts(m: int, n: int, k: int) -> int:
    """Column groups whose sums of squares a residual-completing product of these sizes writes
    (the first dimension of its ``ssq``), or 0 if no kernel folds the next norm in at these
    sizes."""
    key = (m, n, k)
    got = _PREP_PARTS.get(key)
    if got is None:
        got = int(_lib("gemm_tc").mf_gemm_tc_prep_parts(m, n, k))
        _PREP_PARTS[key] = got
    return got


def gemm_tc_fused(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor,
                  epi: int, status: torch.Tensor, row_scale: Optional[RowScale] = None,
                  prep_x: Optional[torch.Tensor] = None, prep_weight: Optional[torch.Tensor] = None,
                  prep_ssq: Optional[torch.Tensor] = None, defer: bool = False) -> Optional[torch.Tensor]:
    """``gemm_tc`` with a norm folded in on either side.  ``row_scale``: ``x`` holds x' = h * g
    of a norm and row t's results are multiplied by its 1/rms.  ``prep_x`` [M, N] bfloat16,
    ``prep_weight`` [N] float32 and ``prep_ssq`` [gemm_tc_prep_parts(M, N, K), M] float32
    (EPI_ACCUM only): ``out`` is complete when the call returns and the three hold what the
    norm that reads ``out`` next needs.  ``defer``: if the product is split along K, returns the
    float32 partial sums [splits, M, N] (``out`` untouched, may be None) instead of adding them."""
    m, k = x.shape
    n = w.shape[0]
    if w.shape[1] != k:
        raise KernelError(f"gemm: shapes do not fit: x {tuple(x.shape)}, w {tuple(w.shape)}")
    if not gemm_tc_supported(x, w):
        raise KernelError("gemm_tc: operands must be bfloat16 with 16-byte aligned rows")
    want_cols = n // 2 if epi == EPI_SWIGLU else n
    if out is not None and (out.shape != (m, want_cols) or out.stride(1) != 1):
        raise KernelError(f"gemm: out has shape {tuple(out.shape)}, expected {(m, want_cols)}")
    if bias is not None and bias.numel() != n:
        raise KernelError("gemm: bias has the wrong length")
    if row_scale is not None and (row_scale.ssq.dim() != 2 or row_scale.ssq.shape[1] != m):
        raise KernelError("gemm: the sums of squares must be [parts, rows]")
    if prep_x is not None:
        parts = gemm_tc_prep_parts(m, n, k)
        if parts == 0:
            raise KernelError("gemm: no kernel folds the next norm in at these sizes")
        if (prep_x.shape != (m, n) or prep_x.dtype != torch.bfloat16 or prep_x.stride(1) != 1
                or prep_weight is None or prep_weight.numel() != n or prep_ssq is None
                or prep_ssq.shape != (parts, m)):
            raise KernelError("gemm: the next norm's tensors have the wrong shapes")
    lib = _lib("gemm_tc")
    need = _gemm_tc_shape(m, n, k, epi)[2]
    ws = None
    if need and prep_x is None:
        ws = torch.empty(need, dtype=torch.float32, device=x.device)
    splits = ctypes.c_int(0)
    if defer:
        if ws is None:
            return None
        target, ldo, code = ws, n, F32
    else:
        target, ldo, code = out, out.stride(0), dtype_code(out.dtype)
    _check(lib.mf_gemm_tc_fused(
        x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), _f32(bias, "bias") if not defer else None,
        target.data_ptr(), ldo, code, m, n, k, epi, _ptr(ws, "workspace"),
        ctypes.addressof(splits) if defer else None,
        _f32(row_scale.ssq, "ssq") if row_scale is not None else None,
        row_scale.ssq.shape[0] if row_scale is not None else 0,
        row_scale.width if row_scale is not None else 0,
        row_scale.eps if row_scale is not None else 0.0,
        _ptr(prep_x, "prep_x"), prep_x.stride(0) if prep_x is not None else 0,
        _f32(prep_weight, "prep_weight"), _f32(prep_ssq, "prep_ssq"), _i32(status, "status"),
        _stream()), "gemm_tc", 2 if (need and prep_x is None and not defer) else 1)
    if defer:
        if splits.value < 1:
            raise KernelError("gemm_tc: a split product reported no splits")
        return ws[:splits.value * m * n].view(splits.value, m, n)
    return None


def gemm_tc_partial_sums(x: torch.Tensor, w: torch.Tensor,
                         status: torch.Tensor) -> Optional[torch.Tensor]:
    """If the kernel would split x @ w^T along K, runs only the splits and returns their
    float32 partial sums [splits, M, N] for the caller's next kernel to add; returns None
    (and runs nothing) if the product is not split."""
    m, k = x.shape
    n = w.shape[0]
    if not gemm_tc_supported(x, w) or w.shape[1] != k:
        return None
    need = _gemm_tc_shape(m, n, k, EPI_STORE)[2]
    if need == 0:
        return None
    lib = _lib("gemm_tc")
    ws = torch.empty(need, dtype=torch.float32, device=x.device)
    splits = ctypes.c_int(0)
    _check(lib.mf_gemm_tc(x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), None,
                          ws.data_ptr(), n, F32, m, n, k, EPI_STORE, ws.data_ptr(),
                          ctypes.addressof(splits), _i32(status, "status"), _stream()),
           "gemm_tc")
    if splits.value < 1:
        raise KernelError("gemm_tc: a split product reported no splits")
    return ws[:splits.value * m * n].view(splits.value, m, n)


def wait_probe(status: torch.Tensor, max_tries: int, max_wait_ns: int,
               waited_ns: Optional[torch.Tensor] = None) -> None:
    """Runs the product kernels' bounded barrier wait on a barrier that nothing arrives at,
    with the given limits (never above the kernels' own).  The wait runs out, bit 4 of
    ``status`` is set and the kernel returns; ``waited_ns`` (int64 [1]) receives how long the
    wait lasted.  Nothing faults and nothing is left in flight."""
    if waited_ns is not None and (waited_ns.dtype != torch.int64 or not waited_ns.is_cuda):
        raise KernelError("wait_probe: waited_ns must be an int64 tensor on the device")
    _check(_lib("gemm_tc").mf_wait_probe(_i32(status, "status"), int(max_tries), int(max_wait_ns),
                                         None if waited_ns is None else waited_ns.data_ptr(),
                                         _stream()), "wait_probe")


def splitk_reduce(partial: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor,
                  accumulate: bool) -> None:
    """out (+)= bias + the sum of ``partial`` [splits, M, N] over its first dimension."""
    splits, m, n = partial.shape
    if out.shape != (m, n) or out.stride(1) != 1:
        raise KernelError("splitk_reduce: out has the wrong shape")
    _check(_lib("gemm_tc").mf_splitk_reduce(_f32(partial, "partial"), splits, _f32(bias, "bias"),
                                            out.data_ptr(), out.stride(0), dtype_code(out.dtype),
                                            m, n, 1 if accumulate else 0, _stream()),
           "splitk_reduce")


# ---------------------------------------------------------------------------------------
# attention
# ---------------------------------------------------------------------------------------
def attention_packed(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, row_seq: torch.Tensor,
                     row_pos: torch.Tensor, cu_seqlens: torch.Tensor, out: torch.Tensor,
                     n_heads: int, n_kv: int, head_dim: int, window: int, scale: float) -> None:
    rows = q.shape[0]
    if q.dtype != k.dtype or q.dtype != v.dtype or q.dtype != out.dtype:
        raise KernelError("attention: q, k, v and out must share one dtype")
    _check(_lib("attention").mf_attention_packed(
        _ptr(q, "q"), _ptr(k, "k"), _ptr(v, "v"), _i32(row_seq, "row_seq"), _i32(row_pos, "row_pos"),
        _i32(cu_seqlens, "cu_seqlens"), _ptr(out, "out"), rows, n_heads, n_kv, head_dim,
        int(window), float(scale), dtype_code(q.dtype), _stream()), "attention_packed")


def attention_prefill_supported(q: torch.Tensor, n_heads: int, n_kv: int, head_dim: int) -> bool:
    """The tensor-core kernel for whole prompts takes bfloat16 and head sizes 64 and 128."""
    return q.dtype == torch.bfloat16 and head_dim in (64, 128) and n_heads % n_kv == 0


def attention_prefill(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_seqlens: torch.Tensor,
                      out: torch.Tensor, n_seqs: int, max_len: int, n_heads: int, n_kv: int,
                      head_dim: int, window: int, scale: float) -> None:
    """Causal attention of whole sequences (positions 0..len-1) packed one after another, on
    tensor cores.  ``max_len`` is the longest sequence (it sizes the grid)."""
    for t in (q, k, v, out):
        if t.dtype != torch.bfloat16:
            raise KernelError("attention_prefill takes bfloat16")
    _check(_lib("attention_prefill").mf_attention_prefill_mma(
        _ptr(q, "q"), _ptr(k, "k"), _ptr(v, "v"), _i32(cu_seqlens, "cu_seqlens"), _ptr(out, "out"),
        int(n_seqs), int(max_len), n_heads, n_kv, head_dim, int(window), float(scale), _stream()),
        "attention_prefill")


def attention_prefill_tc(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_seqlens: torch.Tensor,
                         out: torch.Tensor, n_seqs: int, max_len: int, n_heads: int, n_kv: int,
                         head_dim: int, window: int, scale: float, status: torch.Tensor) -> None:
    """The same attention of whole sequences on tcgen05 (S and O in tensor memory)."""
    for t in (q, k, v, out):
        if t.dtype != torch.bfloat16:
            raise KernelError("attention_prefill_tc takes bfloat16")
    _check(_lib("attention_prefill_tc").mf_attention_prefill_tc(
        _ptr(q, "q"), _ptr(k, "k"), _ptr(v, "v"), _i32(cu_seqlens, "cu_seqlens"), _ptr(out, "out"),
        int(q.shape[0]), int(n_seqs), int(max_len), n_heads, n_kv, head_dim, int(window), float(scale),
        _i32(status, "status"), _stream()), "attention_prefill_tc")


def attention_prefill_tc_paged(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                               cu_seqlens: torch.Tensor, seq_end: torch.Tensor,
                               page_table: torch.Tensor, table_stride: int, ring: int,
                               out: torch.Tensor, n_seqs: int, max_len: int, n_heads: int, n_kv: int,
                               head_dim: int, window: int, scale: float,
                               status: torch.Tensor) -> None:
    """Attention of a step's packed tokens over the paged cache on tcgen05: sequence ``b``
    brings tokens ``cu_seqlens[b] .. cu_seqlens[b+1]-1`` at positions
    ``seq_end[b] - count .. seq_end[b] - 1``; the cache holds every position up to there, the
    step's own included.  ``max_len`` is the most tokens one sequence brings."""
    for t in (q, k_cache, v_cache, out):
        if t.dtype != torch.bfloat16:
            raise KernelError("attention_prefill_tc_paged takes bfloat16")
    _check(_lib("attention_prefill_tc").mf_attention_prefill_tc_paged(
        _ptr(q, "q"), _ptr(k_cache, "k_cache"), _ptr(v_cache, "v_cache"),
        _i32(cu_seqlens, "cu_seqlens"), _i32(seq_end, "seq_end"), _i32(page_table, "page_table"),
        int(table_stride), int(ring), _ptr(out, "out"), int(q.shape[0]), int(n_seqs), int(max_len),
        n_heads, n_kv, head_dim, int(window), float(scale), int(k_cache.shape[0]),
        _i32(status, "status"), _stream()), "attention_prefill_tc_paged")


def attention_paged(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                    row_seq: torch.Tensor, row_pos: torch.Tensor, page_table: torch.Tensor,
                    table_stride: int, ring: int, out: torch.Tensor,
                    partial: Optional[torch.Tensor], n_heads: int, n_kv: int, head_dim: int,
                    window: int, chunk: int, n_chunks: int, scale: float,
                    force_generic: bool = False, status: Optional[torch.Tensor] = None,
                    old_keys_final: bool = False) -> None:
    """Attention of ``rows`` queries over the paged cache.  ``partial`` (float32,
    rows*n_heads*n_chunks*(head_dim+2)) is scratch for the key chunks; with it, bfloat16 and
    head size 64 or 128 run on the tensor-core kernels, everything else on the generic one.
    With ``status`` (the device status word) the tensor-core kernel is the one that streams the
    keys through a TMA ring, whose bounded waits report there.  ``old_keys_final``: each row is the only new
    token of its sequence in this step (the keys below its position were cached before the step
    began), which lets that kernel fetch them while the kernel before it still runs."""
    rows = q.shape[0]
    if q.dtype != k_cache.dtype or q.dtype != v_cache.dtype or q.dtype != out.dtype:
        raise KernelError("attention: q, the cache and out must share one dtype")
    need = rows * n_heads * n_chunks * (head_dim + 2)
    if partial is not None and partial.numel() < need:
        raise KernelError("attention: the scratch for key chunks is too small")
    if n_chunks > 1 and partial is None:
        raise KernelError("attention: several key chunks need scratch to merge them")
    _check(_lib("attention").mf_attention_paged(
        _ptr(q, "q"), _ptr(k_cache, "k_cache"), _ptr(v_cache, "v_cache"), _i32(row_seq, "row_seq"),
        _i32(row_pos, "row_pos"), _i32(page_table, "page_table"), int(table_stride), int(ring),
        _ptr(out, "out"), _f32(partial, "partial"), rows, n_heads, n_kv, head_dim, int(window),
        int(chunk), int(n_chunks), float(scale), dtype_code(q.dtype), 1 if force_generic else 0,
        int(k_cache.shape[0]), _i32(status, "status"), 1 if old_keys_final else 0,
        _stream()), "attention_paged", 2 if n_chunks > 1 else 1)


# ---------------------------------------------------------------------------------------
# sampling
# ---------------------------------------------------------------------------------------
def sampler_state_ints() -> int:
    return int(_lib("sampling").mf_sampler_state_ints())


def sample(logits: torch.Tensor, out: torch.Tensor, *, temperature: float, top_k: int,
           top_p: float, repeat_penalty: float, frequency_penalty: float,
           presence_penalty: float, seed: int, slots: Optional[torch.Tensor] = None,
           state: Optional[torch.Tensor] = None, stream_ids: Optional[torch.Tensor] = None,
           update_state: bool = True) -> None:
    """Samples one token per row of ``logits`` (float32, changed in place) into ``out``."""
    rows, vocab = logits.shape
    if logits.stride(1) != 1:
        raise KernelError("sample: logits must be contiguous along the vocabulary")
    if not logits.is_cuda:
        raise KernelError("sample: logits must live on a CUDA device (there is no CPU path)")
    if logits.dtype != torch.float32:
        raise KernelError("sample: logits must be float32")
    _check(_lib("sampling").mf_sample(
        logits.data_ptr(), logits.stride(0), rows, vocab, _i32(slots, "slots"),
        _i32(state, "state"), _i32(stream_ids, "stream_ids"), _i32(out, "out"), float(temperature),
        int(top_k), float(top_p), float(repeat_penalty), float(frequency_penalty),
        float(presence_penalty), int(seed) & 0xFFFFFFFFFFFFFFFF, 1 if update_state else 0,
        _stream()), "sample")
