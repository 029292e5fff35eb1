"""Python faces of the CUDA kernels.

Every function takes CUDA tensors, checks what the kernel relies on (device,
dtype, contiguity, sizes) and launches on torch's current stream.  There is no
CPU path and no torch implementation behind these names: a tensor on the CPU,
or a kernel library that cannot be built, is an error.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Tuple, Optional

import torch

from . import build


class KernelError(RuntimeError):
    """A kernel refused its arguments or the launch failed."""


_CODES = {torch.float32: 0, torch.bfloat16: 1}

PAGE_ROWS = 64          # rows of one cache page


def code(dt: torch.dtype) -> int:
    try:
        return _CODES[dt]
    except KeyError:
        raise KernelError(f"kernels take float32 and bfloat16 tensors, not {dt}") from None


_RAW_STREAM = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_RAW_DEVICE = getattr(torch._C, "_cuda_getDevice", None)


def _stream() -> c_void_p:
    """The current stream's handle.  Every launch asks for it, so it is read through torch's raw accessors where
    this torch has them (a Stream object costs several microseconds to make)."""
    if _RAW_STREAM is not None and _RAW_DEVICE is not None:
        return c_void_p(_RAW_STREAM(_RAW_DEVICE()))
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t: Optional[torch.Tensor]) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


def _cuda(*ts: Optional[torch.Tensor]) -> None:
    for t in ts:
        if t is not None and not t.is_cuda:
            raise KernelError("this library computes on the GPU only: got a tensor on " + str(t.device))


_launches = 0


def launches() -> int:
    """How many kernel launches this process has made through this module (graph replays count their kernels)."""
    return _launches


def count_launches(n: int) -> None:
    global _launches
    _launches += n


def _check(lib, status: int, what: str, kernels: int = 1) -> None:
    global _launches
    if status == 0:
        _launches += kernels
        return
    if status < 0:
        raise KernelError(f"{what}: {lib.tb_error().decode()}")
    raise KernelError(f"{what}: CUDA error {status} at launch "
                      f"({torch.cuda.get_device_name() if torch.cuda.is_available() else 'no device'})")


def _rows_contig(t: torch.Tensor, what: str) -> None:
    if t.dim() != 2 or t.stride(1) != 1:
        raise KernelError(f"{what} must be 2-D with contiguous rows, got shape {tuple(t.shape)} strides {t.stride()}")


# ---------------------------------------------------------------------------
def embed(ids: torch.Tensor, table: torch.Tensor, scale: float, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[t] = float32(table[ids[t]]) * scale."""
    _cuda(ids, table, out)
    if ids.dtype != torch.int32 or ids.dim() != 1 or not ids.is_contiguous():
        raise KernelError("embed: ids must be a contiguous 1-D int32 tensor")
    if table.dim() != 2 or not table.is_contiguous():
        raise KernelError("embed: table must be contiguous [vocab, hidden]")
    V, H = table.shape
    if out is None:
        out = torch.empty((ids.numel(), H), dtype=torch.float32, device=ids.device)
    lib = build.load("embed")
    _check(lib, lib.tb_embed(_ptr(ids), _ptr(table), c_int(code(table.dtype)), _ptr(out), c_int(ids.numel()),
                             c_int(H), c_int(V), c_float(scale), _stream()), "embed")
    return out


def gather_rows(x: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
    """out[i] = x[rows[i]] for a float32 matrix."""
    _cuda(x, rows)
    if x.dtype != torch.float32 or x.dim() != 2 or not x.is_contiguous():
        raise KernelError("gather_rows: x must be contiguous float32 [rows, width]")
    if rows.dtype != torch.int32 or not rows.is_contiguous():
        raise KernelError("gather_rows: rows must be contiguous int32")
    out = torch.empty((rows.numel(), x.shape[1]), dtype=torch.float32, device=x.device)
    lib = build.load("embed")
    _check(lib, lib.tb_gather_rows(_ptr(x), _ptr(rows), _ptr(out), c_int(rows.numel()), c_int(x.shape[1]),
                                   c_int(x.shape[0]), _stream()), "gather_rows")
    return out


def random_normal(out: torch.Tensor, key, std: float) -> None:
    """Fill ``out`` (bfloat16 or float32) with the counter-based normal numbers of ``key`` = (k0, k1), times
    ``std``, rounded to bfloat16 (see random_init.cu; ``weights.random_init`` makes the key from seed and name)."""
    _cuda(out)
    if not out.is_contiguous():
        raise KernelError("random_normal: the tensor must be contiguous")
    lib = build.load("random_init")
    _check(lib, lib.tb_random_normal(_ptr(out), c_int(code(out.dtype)), c_longlong(out.numel()),
                                     ctypes.c_uint(key[0]), ctypes.c_uint(key[1]), c_float(std), _stream()),
           "random_normal")


# ---------------------------------------------------------------------------
def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float, offset: float, out_dtype: torch.dtype) -> torch.Tensor:
    """norm(x) * (offset + w), statistics in 32-bit."""
    _cuda(x, w)
    if x.dim() != 2 or not x.is_contiguous() or w.dim() != 1 or w.numel() != x.shape[1] or not w.is_contiguous():
        raise KernelError(f"rmsnorm: x {tuple(x.shape)} / w {tuple(w.shape)} do not fit")
    out = torch.empty(x.shape, dtype=out_dtype, device=x.device)
    lib = build.load("norm")
    _check(lib, lib.tb_rmsnorm(_ptr(x), c_int(code(x.dtype)), _ptr(w), c_int(code(w.dtype)), _ptr(out),
                               c_int(code(out_dtype)), c_int(x.shape[0]), c_int(x.shape[1]), c_float(eps),
                               c_float(offset), _stream()), "rmsnorm")
    return out


def add_rmsnorm(h: torch.Tensor, a: torch.Tensor, wa: torch.Tensor, eps_a: float, off_a: float,
                wb: Optional[torch.Tensor] = None, eps_b: float = 0.0, off_b: float = 0.0,
                out_dtype: Optional[torch.dtype] = None) -> Optional[torch.Tensor]:
    """h += norm_a(a) in place (h float32); with wb also returns norm_b(h).  ``a`` is [rows, width], or
    [splits, rows, width] partial sums (float32) that are added in split order on the way."""
    _cuda(h, a, wa, wb)
    if h.dtype != torch.float32 or h.dim() != 2 or not h.is_contiguous():
        raise KernelError("add_rmsnorm: the residual stream must be contiguous float32 [rows, width]")
    n_splits, split_stride = 1, 0
    if a.dim() == 3:
        if a.dtype != torch.float32:
            raise KernelError("add_rmsnorm: partial sums must be float32")
        n_splits, split_stride = a.shape[0], a.stride(0)
        if tuple(a.shape[1:]) != tuple(h.shape) or a.stride(1) != h.shape[1] or a.stride(2) != 1:
            raise KernelError(f"add_rmsnorm: partial sums {tuple(a.shape)} do not fit the stream {tuple(h.shape)}")
    elif a.shape != h.shape or not a.is_contiguous():
        raise KernelError(f"add_rmsnorm: branch {tuple(a.shape)} does not fit the stream {tuple(h.shape)}")
    if wa.numel() != h.shape[1] or (wb is not None and (wb.numel() != h.shape[1] or wb.dtype != wa.dtype)):
        raise KernelError("add_rmsnorm: norm weights do not fit (both must have the row width and one dtype)")
    out = None
    if wb is not None:
        out = torch.empty(h.shape, dtype=out_dtype, device=h.device)
    lib = build.load("norm")
    _check(lib, lib.tb_add_rmsnorm(_ptr(h), _ptr(a), c_int(code(a.dtype)), c_int(n_splits), c_longlong(split_stride),
                                   _ptr(wa), c_float(eps_a), c_float(off_a),
                                   _ptr(wb), c_float(eps_b), c_float(off_b), c_int(code(wa.dtype)),
                                   _ptr(out), c_int(code(out_dtype) if out is not None else 0),
                                   c_int(h.shape[0]), c_int(h.shape[1]), _stream()), "add_rmsnorm")
    return out


def residual_add(h: torch.Tensor, a: torch.Tensor) -> None:
    """h += a (a may be [splits, rows, width] partial sums: they are added one after the other)."""
    _cuda(h, a)
    if a.dim() == 3:
        a = sum_partials(a.contiguous())
    if h.dtype != torch.float32 or not h.is_contiguous() or not a.is_contiguous() or a.shape != h.shape:
        raise KernelError("residual_add: h must be contiguous float32 and a of the same shape")
    lib = build.load("norm")
    _check(lib, lib.tb_residual_add(_ptr(h), _ptr(a), c_int(code(a.dtype)), c_longlong(h.numel()), _stream()),
           "residual_add")


def fold_rmsnorm(h: torch.Tensor, a: torch.Tensor, w: torch.Tensor, eps: float, offset: float,
                 alpha: Optional[float], out_dtype: Optional[torch.dtype]) -> Optional[torch.Tensor]:
    """``alpha`` None: h += norm(a); a number: h <- norm(alpha * h + a) (the norm after the sum).  h float32, in
    place; ``a`` [rows, width] or float32 partial sums [splits, rows, width].  With ``out_dtype`` also returns the new
    h rounded to that dtype."""
    _cuda(h, a, w)
    if h.dtype != torch.float32 or h.dim() != 2 or not h.is_contiguous():
        raise KernelError("fold_rmsnorm: the residual stream must be contiguous float32 [rows, width]")
    n_splits, split_stride = 1, 0
    if a.dim() == 3:
        if a.dtype != torch.float32:
            raise KernelError("fold_rmsnorm: partial sums must be float32")
        n_splits, split_stride = a.shape[0], a.stride(0)
        if tuple(a.shape[1:]) != tuple(h.shape) or a.stride(1) != h.shape[1] or a.stride(2) != 1:
            raise KernelError(f"fold_rmsnorm: partial sums {tuple(a.shape)} do not fit the stream {tuple(h.shape)}")
    elif a.shape != h.shape or not a.is_contiguous():
        raise KernelError(f"fold_rmsnorm: branch {tuple(a.shape)} does not fit the stream {tuple(h.shape)}")
    if w.numel() != h.shape[1] or not w.is_contiguous():
        raise KernelError("fold_rmsnorm: the norm weight does not fit the row width")
    out = torch.empty(h.shape, dtype=out_dtype, device=h.device) if out_dtype is not None else None
    lib = build.load("norm")
    _check(lib, lib.tb_fold_rmsnorm(_ptr(h), c_int(0 if alpha is None else 1), c_float(alpha or 0.0), _ptr(a),
                                    c_int(code(a.dtype)), c_int(n_splits), c_longlong(split_stride), _ptr(w),
                                    c_int(code(w.dtype)), c_float(eps), c_float(offset), _ptr(out),
                                    c_int(code(out_dtype) if out is not None else 0), c_int(h.shape[0]),
                                    c_int(h.shape[1]), _stream()), "fold_rmsnorm")
    return out


def _branch(h: torch.Tensor, a: torch.Tensor, what: str):
    """(pointer, splits, split stride) of a float32 branch output [rows, width] or [splits, rows, width]."""
    if a.dtype != torch.float32:
        raise KernelError(f"{what}: branch outputs must be float32, got {a.dtype}")
    if a.dim() == 3:
        if tuple(a.shape[1:]) != tuple(h.shape) or a.stride(1) != h.shape[1] or a.stride(2) != 1:
            raise KernelError(f"{what}: partial sums {tuple(a.shape)} do not fit the stream {tuple(h.shape)}")
        return a, a.shape[0], a.stride(0)
    if a.shape != h.shape or not a.is_contiguous():
        raise KernelError(f"{what}: branch {tuple(a.shape)} does not fit the stream {tuple(h.shape)}")
    return a, 1, 0


def add_scaled_rmsnorm(h: torch.Tensor, branches, scale: float, w: Optional[torch.Tensor] = None, eps: float = 0.0,
                       offset: float = 0.0, out_dtype: Optional[torch.dtype] = None) -> Optional[torch.Tensor]:
    """``h += scale * (sum of the branches)`` in place (h float32; one or two float32 branch outputs, each [rows, width]
    or [splits, rows, width] partial sums); with ``w`` also returns ``norm(h) * (offset + w)`` in ``out_dtype``."""
    _cuda(h, w, *branches)
    if h.dtype != torch.float32 or h.dim() != 2 or not h.is_contiguous():
        raise KernelError("add_scaled_rmsnorm: the residual stream must be contiguous float32 [rows, width]")
    if not 1 <= len(branches) <= 2:
        raise KernelError(f"add_scaled_rmsnorm: one or two branches, got {len(branches)}")
    a, a_n, a_s = _branch(h, branches[0], "add_scaled_rmsnorm")
    b, b_n, b_s = _branch(h, branches[1], "add_scaled_rmsnorm") if len(branches) == 2 else (None, 0, 0)
    out = None
    if w is not None:
        if w.numel() != h.shape[1] or not w.is_contiguous():
            raise KernelError("add_scaled_rmsnorm: the norm weight does not fit the row width")
        out = torch.empty(h.shape, dtype=out_dtype, device=h.device)
    lib = build.load("norm")
    _check(lib, lib.tb_add_scaled_rmsnorm(_ptr(h), c_float(scale), _ptr(a), c_int(a_n), c_longlong(a_s), _ptr(b), c_int(b_n),
                                          c_longlong(b_s), _ptr(w), c_int(code(w.dtype) if w is not None else 0), c_float(eps),
                                          c_float(offset), _ptr(out), c_int(code(out_dtype) if out is not None else 0),
                                          c_int(h.shape[0]), c_int(h.shape[1]), _stream()), "add_scaled_rmsnorm")
    return out


def cast(x: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """A float32 tensor rounded to ``out_dtype``."""
    _cuda(x)
    if x.dtype != torch.float32 or not x.is_contiguous():
        raise KernelError("cast: wants a contiguous float32 tensor")
    out = torch.empty(x.shape, dtype=out_dtype, device=x.device)
    lib = build.load("norm")
    _check(lib, lib.tb_cast(_ptr(x), _ptr(out), c_int(code(out_dtype)), c_longlong(x.numel()), _stream()), "cast")
    return out


# ---------------------------------------------------------------------------
ACTIVATIONS = {"gelu_tanh": 0, "silu": 1, "clamped_swish": 2}
UNARY_ACTIVATIONS = {"relu2": 3}          # activations of a feed-forward without a gate branch: relu2(u) = relu(u)^2
ACTIVATIONS_WITH_LIMIT = ("clamped_swish",)


def gated_act(gu: torch.Tensor, activation: str, out_dtype: torch.dtype, limit: float = 0.0) -> torch.Tensor:
    """act(gu[:, :I]) * gu[:, I:]; for "clamped_swish" (which takes ``limit`` L):
    g' = min(g, L), u' = clamp(u, -L, L), g' sigmoid(1.702 g') (u' + 1)."""
    _cuda(gu)
    if gu.dim() != 2 or not gu.is_contiguous() or gu.shape[1] % 2:
        raise KernelError("gated_act: input must be contiguous [rows, 2*intermediate]")
    if activation not in ACTIVATIONS:
        raise KernelError(f"gated_act: unknown activation '{activation}' (known: {sorted(ACTIVATIONS)})")
    inter = gu.shape[1] // 2
    out = torch.empty((gu.shape[0], inter), dtype=out_dtype, device=gu.device)
    lib = build.load("activation")
    _check(lib, lib.tb_gated_act_limit(_ptr(gu), c_int(code(gu.dtype)), _ptr(out), c_int(code(out_dtype)),
                                       c_int(gu.shape[0]), c_int(inter), c_int(ACTIVATIONS[activation]),
                                       c_float(limit), _stream()), "gated_act")
    return out


def unary_act(part: torch.Tensor, activation: str, out_dtype: torch.dtype, col0: int = 0,
              cols: Optional[int] = None) -> torch.Tensor:
    """``act`` of columns ``col0 .. col0 + cols`` of a product given as float32 [rows, width] or partial sums
    [splits, rows, width] (added in split order); returns [rows, cols] in ``out_dtype``."""
    _cuda(part)
    if part.dim() == 2:
        part = part[None]
    if part.dtype != torch.float32 or part.dim() != 3 or part.stride(2) != 1:
        raise KernelError("unary_act: wants float32 [splits, rows, width] with contiguous rows")
    if activation not in UNARY_ACTIVATIONS:
        raise KernelError(f"unary_act: unknown activation '{activation}' (known: {sorted(UNARY_ACTIVATIONS)})")
    cols = part.shape[2] - col0 if cols is None else cols
    if col0 < 0 or cols < 1 or col0 + cols > part.shape[2]:
        raise KernelError(f"unary_act: columns {col0}..{col0 + cols} lie outside a width of {part.shape[2]}")
    out = torch.empty((part.shape[1], cols), dtype=out_dtype, device=part.device)
    lib = build.load("activation")
    _check(lib, lib.tb_unary_act(_ptr(part), c_int(part.shape[0]), c_longlong(part.stride(0)), c_longlong(part.stride(1)),
                                 c_int(col0), _ptr(out), c_int(code(out_dtype)), c_int(part.shape[1]), c_int(cols),
                                 c_int(UNARY_ACTIVATIONS[activation]), _stream()), "unary_act")
    return out


def token_gate(g: torch.Tensor, ids: torch.Tensor, table: torch.Tensor, col0: int,
               out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """out[t, j] = gelu_tanh(g[t, j]) * table[ids[t], col0 + j], computed in 32-bit, stored in ``out_dtype``
    (default: g's dtype).  ``g``: [tokens, dim], or [splits, tokens, dim] partial sums that are added on the way."""
    _cuda(g, ids, table)
    n_splits, split_stride = 1, 0
    if g.dim() == 3:
        n_splits, split_stride = g.shape[0], g.stride(0)
        if not g[0].is_contiguous():
            raise KernelError("token_gate: partial sums must be [splits, tokens, dim] with contiguous [tokens, dim]")
        g3, g = g, g[0]
    if g.dim() != 2 or not g.is_contiguous():
        raise KernelError("token_gate: g must be contiguous [tokens, dim]")
    if ids.dtype != torch.int32 or ids.numel() != g.shape[0] or not ids.is_contiguous():
        raise KernelError("token_gate: ids must be contiguous int32 [tokens]")
    if table.dim() != 2 or table.stride(1) != 1 or col0 < 0 or col0 + g.shape[1] > table.shape[1]:
        raise KernelError(f"token_gate: columns {col0}..{col0 + g.shape[1]} do not lie in a table of shape {tuple(table.shape)}")
    out = torch.empty(g.shape, dtype=out_dtype or g.dtype, device=g.device)
    lib = build.load("activation")
    _check(lib, lib.tb_token_gate(_ptr(g), c_int(code(g.dtype)), c_int(n_splits), c_longlong(split_stride), _ptr(ids), _ptr(table), c_int(code(table.dtype)),
                                  c_longlong(table.stride(0)), c_int(col0), c_int(table.shape[0]), _ptr(out),
                                  c_int(code(out.dtype)), c_int(g.shape[0]), c_int(g.shape[1]), _stream()), "token_gate")
    return out


def add_bias(x: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """x[r, :] += bias in place (x 2-D with contiguous rows, possibly a column slice of a wider matrix)."""
    _cuda(x, bias)
    _rows_contig(x, "add_bias: x")
    if bias.dim() != 1 or bias.numel() != x.shape[1] or not bias.is_contiguous():
        raise KernelError(f"add_bias: bias {tuple(bias.shape)} does not fit rows of width {x.shape[1]}")
    lib = build.load("activation")
    _check(lib, lib.tb_add_bias(_ptr(x), c_int(code(x.dtype)), c_longlong(x.stride(0)), _ptr(bias), c_int(code(bias.dtype)),
                                c_int(x.shape[0]), c_int(x.shape[1]), _stream()), "add_bias")
    return x


# ---------------------------------------------------------------------------
def gemm_simt(a: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype, softcap: float = 0.0,
              out: Optional[torch.Tensor] = None, out_scale: float = 1.0) -> torch.Tensor:
    """a[M,K] @ w[N,K]^T with 32-bit FMA (no tensor cores); the result times ``out_scale`` (after the cap)."""
    _cuda(a, w, out)
    _rows_contig(a, "gemm: a")
    _rows_contig(w, "gemm: w")
    if a.shape[1] != w.shape[1]:
        raise KernelError(f"gemm: a is {tuple(a.shape)}, w is {tuple(w.shape)}: inner sizes differ")
    M, K = a.shape
    N = w.shape[0]
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    else:
        _rows_contig(out, "gemm: out")
    lib = build.load("gemm_simt")
    _check(lib, lib.tb_gemm_simt_ex(_ptr(a), c_int(code(a.dtype)), _ptr(w), c_int(code(w.dtype)), _ptr(out),
                                    c_int(code(out.dtype)), c_int(M), c_int(N), c_int(K), c_longlong(a.stride(0)),
                                    c_longlong(w.stride(0)), c_longlong(out.stride(0)), c_float(softcap or 0.0),
                                    c_float(out_scale), _stream()), "gemm_simt")
    return out


# ---------------------------------------------------------------------------
class _RopeKvArgs(ctypes.Structure):
    _fields_ = [("qkv", c_void_p), ("row_stride", c_longlong),
                ("q_off", c_int), ("k_off", c_int), ("v_off", c_int),
                ("n_heads", c_int), ("n_kv_heads", c_int), ("head_dim", c_int), ("rotary_dim", c_int),
                ("inv_freq", c_void_p), ("positions", c_void_p), ("token_seq", c_void_p), ("len_after", c_void_p),
                ("k_pool", c_void_p), ("v_pool", c_void_p), ("page_table", c_void_p), ("pt_stride", c_int),
                ("page_rows", c_int), ("ring_rows", c_int),
                ("partial", c_void_p), ("n_splits", c_int), ("split_stride", c_longlong),
                ("partial_row_stride", c_longlong)]


def rope_kv(qkv: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int, rotary_dim: int,
            inv_freq: Optional[torch.Tensor], positions: torch.Tensor, token_seq: torch.Tensor,
            len_after: torch.Tensor, k_pool: Optional[torch.Tensor], v_pool: Optional[torch.Tensor],
            page_table: Optional[torch.Tensor], ring_rows: int, partial: Optional[torch.Tensor] = None) -> None:
    """Rotate q and k of ``qkv`` [T, (n_heads + 2 n_kv_heads) * head_dim] in place and store k, v
    in the cache line (``k_pool``/``v_pool`` [pages, n_kv_heads, PAGE_ROWS, head_dim]).  With ``partial``
    ([splits, T, width] float32 partial sums of the q/k/v product) the values are taken from their sum
    and ``qkv`` is only written."""
    _cuda(qkv, inv_freq, positions, token_seq, len_after, k_pool, v_pool, page_table, partial)
    if partial is not None and (partial.dtype != torch.float32 or partial.dim() != 3 or partial.shape[1:] != qkv.shape
                                or partial.stride(2) != 1):
        raise KernelError("rope_kv: partial sums must be float32 [splits, tokens, width] matching qkv")
    _rows_contig(qkv, "rope_kv: qkv")
    T = qkv.shape[0]
    if qkv.shape[1] != (n_heads + 2 * n_kv_heads) * head_dim:
        raise KernelError("rope_kv: qkv width does not fit the head counts")
    for name, t in (("positions", positions), ("token_seq", token_seq)):
        if t.dtype != torch.int32 or t.numel() != T or not t.is_contiguous():
            raise KernelError(f"rope_kv: {name} must be contiguous int32 [{T}]")
    if inv_freq is not None and (inv_freq.dtype != torch.float32 or inv_freq.numel() != rotary_dim // 2):
        raise KernelError("rope_kv: inv_freq must be float32 [rotary_dim/2]")
    if k_pool is not None:
        for p in (k_pool, v_pool):
            if p is None or p.dtype != qkv.dtype or not p.is_contiguous() or tuple(p.shape[1:]) != (n_kv_heads, PAGE_ROWS, head_dim):
                raise KernelError("rope_kv: cache pools must be contiguous [pages, n_kv_heads, PAGE_ROWS, head_dim] "
                                  "of the activations' dtype")
        if page_table is None or page_table.dtype != torch.int32 or page_table.dim() != 2 or page_table.stride(1) != 1:
            raise KernelError("rope_kv: page_table must be int32 [batch, pages]")
    a = _RopeKvArgs()
    a.qkv = qkv.data_ptr(); a.row_stride = qkv.stride(0)
    a.q_off = 0; a.k_off = n_heads * head_dim; a.v_off = (n_heads + n_kv_heads) * head_dim
    a.n_heads = n_heads; a.n_kv_heads = n_kv_heads; a.head_dim = head_dim; a.rotary_dim = rotary_dim
    a.inv_freq = inv_freq.data_ptr() if inv_freq is not None else None
    a.positions = positions.data_ptr(); a.token_seq = token_seq.data_ptr(); a.len_after = len_after.data_ptr()
    a.k_pool = k_pool.data_ptr() if k_pool is not None else None
    a.v_pool = v_pool.data_ptr() if v_pool is not None else None
    a.page_table = page_table.data_ptr() if page_table is not None else None
    a.pt_stride = page_table.stride(0) if page_table is not None else 0
    a.page_rows = PAGE_ROWS; a.ring_rows = ring_rows
    a.partial = partial.data_ptr() if partial is not None else None
    a.n_splits = partial.shape[0] if partial is not None else 0
    a.split_stride = partial.stride(0) if partial is not None else 0
    a.partial_row_stride = partial.stride(1) if partial is not None else 0
    lib = build.load("rope_kv")
    _check(lib, lib.tb_rope_kv(ctypes.byref(a), c_int(code(qkv.dtype)), c_int(T), _stream()), "rope_kv")


class _HeadNormKvArgs(ctypes.Structure):
    _fields_ = [("partial", c_void_p), ("n_splits", c_int), ("split_stride", c_longlong), ("partial_row_stride", c_longlong),
                ("out", c_void_p), ("out_row_stride", c_longlong),
                ("n_heads", c_int), ("n_kv_heads", c_int), ("head_dim", c_int),
                ("q_unit", c_int), ("k_unit", c_int), ("v_from_k", c_int),
                ("eps", c_float), ("temp_coef", c_float), ("temp_every", c_int),
                ("positions", c_void_p), ("token_seq", c_void_p), ("len_after", c_void_p),
                ("k_pool", c_void_p), ("v_pool", c_void_p), ("page_table", c_void_p), ("pt_stride", c_int),
                ("page_rows", c_int), ("ring_rows", c_int)]


def headnorm_kv(partial: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int, out_dtype: torch.dtype,
                q_unit: bool, k_unit: bool, v_from_k: bool, eps: float, temp_coef: float, temp_every: int,
                positions: torch.Tensor, token_seq: torch.Tensor, len_after: torch.Tensor,
                k_pool: Optional[torch.Tensor], v_pool: Optional[torch.Tensor], page_table: Optional[torch.Tensor],
                ring_rows: int) -> torch.Tensor:
    """From the q/k(/v) product's float32 partial sums [splits, T, width] to [T, (n_heads + 2 n_kv_heads) * head_dim]
    in ``out_dtype``: q and k heads divided by their root mean square (``q_unit``, ``k_unit``; eps inside the root),
    q times ``1 + temp_coef * ln(floor((pos + 1) / temp_every) + 1)`` (``temp_every`` 0: off), v the product's own
    v columns or, with ``v_from_k``, its k columns before the norm; k and v are also written to the cache line."""
    _cuda(partial, positions, token_seq, len_after, k_pool, v_pool, page_table)
    in_slots = n_heads + n_kv_heads * (1 if v_from_k else 2)
    if partial.dtype != torch.float32 or partial.dim() != 3 or partial.stride(2) != 1 or partial.shape[2] != in_slots * head_dim:
        raise KernelError(f"headnorm_kv: wants float32 partial sums [splits, tokens, {in_slots * head_dim}], "
                          f"got {tuple(partial.shape)} {partial.dtype}")
    T = partial.shape[1]
    for name, t in (("positions", positions), ("token_seq", token_seq)):
        if t.dtype != torch.int32 or t.numel() != T or not t.is_contiguous():
            raise KernelError(f"headnorm_kv: {name} must be contiguous int32 [{T}]")
    if k_pool is not None:
        for p in (k_pool, v_pool):
            if p is None or p.dtype != out_dtype or not p.is_contiguous() or tuple(p.shape[1:]) != (n_kv_heads, PAGE_ROWS, head_dim):
                raise KernelError("headnorm_kv: cache pools must be contiguous [pages, n_kv_heads, PAGE_ROWS, head_dim] "
                                  "of the output's dtype")
        if page_table is None or page_table.dtype != torch.int32 or page_table.dim() != 2 or page_table.stride(1) != 1:
            raise KernelError("headnorm_kv: page_table must be int32 [batch, pages]")
    out = torch.empty((T, (n_heads + 2 * n_kv_heads) * head_dim), dtype=out_dtype, device=partial.device)
    a = _HeadNormKvArgs()
    a.partial = partial.data_ptr(); a.n_splits = partial.shape[0]; a.split_stride = partial.stride(0)
    a.partial_row_stride = partial.stride(1)
    a.out = out.data_ptr(); a.out_row_stride = out.stride(0)
    a.n_heads = n_heads; a.n_kv_heads = n_kv_heads; a.head_dim = head_dim
    a.q_unit = int(bool(q_unit)); a.k_unit = int(bool(k_unit)); a.v_from_k = int(bool(v_from_k))
    a.eps = eps; a.temp_coef = temp_coef; a.temp_every = int(temp_every)
    a.positions = positions.data_ptr(); a.token_seq = token_seq.data_ptr(); a.len_after = len_after.data_ptr()
    a.k_pool = k_pool.data_ptr() if k_pool is not None else None
    a.v_pool = v_pool.data_ptr() if k_pool is not None else None
    a.page_table = page_table.data_ptr() if k_pool is not None else None
    a.pt_stride = page_table.stride(0) if k_pool is not None else 0
    a.page_rows = PAGE_ROWS; a.ring_rows = ring_rows
    lib = build.load("headnorm_kv")
    _check(lib, lib.tb_headnorm_kv(ctypes.byref(a), c_int(code(out_dtype)), c_int(T), _stream()), "headnorm_kv")
    return out


class _ProjNormKvArgs(ctypes.Structure):
    _fields_ = [("partial", c_void_p), ("n_splits", c_int), ("split_stride", c_longlong), ("partial_row_stride", c_longlong),
                ("out", c_void_p), ("out_row_stride", c_longlong), ("gate_out", c_void_p),
                ("n_heads", c_int), ("n_kv_heads", c_int), ("dim", c_int), ("vdim", c_int), ("D", c_int),
                ("q_norm_w", c_void_p), ("k_norm_w", c_void_p), ("eps", c_float), ("head_scale", c_void_p),
                ("rotary_dim", c_int), ("inv_freq", c_void_p),
                ("positions", c_void_p), ("token_seq", c_void_p), ("len_after", c_void_p),
                ("k_pool", c_void_p), ("v_pool", c_void_p), ("page_table", c_void_p), ("pt_stride", c_int),
                ("page_rows", c_int), ("ring_rows", c_int), ("bias", c_void_p)]


def projnorm_kv(partial: torch.Tensor, n_heads: int, n_kv_heads: int, dim: int, vdim: int, padded: int,
                out_dtype: torch.dtype, q_norm_w: Optional[torch.Tensor], k_norm_w: Optional[torch.Tensor], eps: float,
                head_scale: Optional[torch.Tensor], rotary_dim: int, inv_freq: Optional[torch.Tensor], has_gate: bool,
                positions: torch.Tensor, token_seq: torch.Tensor, len_after: torch.Tensor,
                k_pool: Optional[torch.Tensor], v_pool: Optional[torch.Tensor], page_table: Optional[torch.Tensor],
                ring_rows: int, bias: Optional[torch.Tensor] = None):
    """From the q/k/v(/gate) product's float32 partial sums [splits, T, H dim + G dim + G vdim (+ H)] to
    ([T, (H + 2 G) * padded] in ``out_dtype``, sigmoid of the gate columns float32 [T, H] or None): q and k divided by
    their root mean square over the whole projection times ``q_norm_w`` / ``k_norm_w`` (float32; None: no norm), q heads
    times ``head_scale[h]`` (float32 [H] or None), the first ``rotary_dim`` dims of every q and k head rotated at the
    token's position, every head padded with zeros to ``padded`` numbers; k and v are also written to the cache line
    (pools [pages, G, PAGE_ROWS, padded]).  ``bias``: float32, one number per column of the product (the width rounded
    up to a multiple of four), added to the summed row before anything else.  ``n_kv_heads`` 0: the product holds
    queries only."""
    _cuda(partial, q_norm_w, k_norm_w, head_scale, inv_freq, positions, token_seq, len_after, k_pool, v_pool, page_table, bias)
    H, G = n_heads, n_kv_heads
    in_width = H * dim + G * (dim + vdim) + (H if has_gate else 0)
    if partial.dtype != torch.float32 or partial.dim() != 3 or partial.stride(2) != 1 or partial.shape[2] < in_width:
        raise KernelError(f"projnorm_kv: wants float32 partial sums [splits, tokens, >= {in_width}], got {tuple(partial.shape)} {partial.dtype}")
    T = partial.shape[1]
    for name, t in (("positions", positions), ("token_seq", token_seq)):
        if t.dtype != torch.int32 or t.numel() != T or not t.is_contiguous():
            raise KernelError(f"projnorm_kv: {name} must be contiguous int32 [{T}]")
    for name, t, n in (("q_norm_w", q_norm_w, H * dim), ("k_norm_w", k_norm_w, G * dim), ("head_scale", head_scale, H),
                       ("inv_freq", inv_freq, rotary_dim // 2)):
        if t is not None and (t.dtype != torch.float32 or t.numel() != n or not t.is_contiguous()):
            raise KernelError(f"projnorm_kv: {name} must be contiguous float32 [{n}]")
    if rotary_dim and inv_freq is None:
        raise KernelError("projnorm_kv: a rotation needs its table")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() < (in_width + 3) // 4 * 4 or not bias.is_contiguous()):
        raise KernelError(f"projnorm_kv: the bias must be contiguous float32 [>= {(in_width + 3) // 4 * 4}]")
    if k_pool is not None:
        for p in (k_pool, v_pool):
            if p is None or p.dtype != out_dtype or not p.is_contiguous() or tuple(p.shape[1:]) != (G, PAGE_ROWS, padded):
                raise KernelError(f"projnorm_kv: cache pools must be contiguous [pages, {G}, PAGE_ROWS, {padded}] of the output's dtype")
        if page_table is None or page_table.dtype != torch.int32 or page_table.dim() != 2 or page_table.stride(1) != 1:
            raise KernelError("projnorm_kv: page_table must be int32 [batch, pages]")
    out = torch.empty((T, (H + 2 * G) * padded), dtype=out_dtype, device=partial.device)
    gate = torch.empty((T, H), dtype=torch.float32, device=partial.device) if has_gate else None
    a = _ProjNormKvArgs()
    a.partial = partial.data_ptr(); a.n_splits = partial.shape[0]; a.split_stride = partial.stride(0)
    a.partial_row_stride = partial.stride(1)
    a.out = out.data_ptr(); a.out_row_stride = out.stride(0); a.gate_out = gate.data_ptr() if gate is not None else None
    a.n_heads = H; a.n_kv_heads = G; a.dim = dim; a.vdim = vdim; a.D = padded
    a.q_norm_w = q_norm_w.data_ptr() if q_norm_w is not None else None
    a.k_norm_w = k_norm_w.data_ptr() if k_norm_w is not None else None
    a.eps = eps
    a.head_scale = head_scale.data_ptr() if head_scale is not None else None
    a.rotary_dim = rotary_dim; a.inv_freq = inv_freq.data_ptr() if (inv_freq is not None and rotary_dim) else None
    a.positions = positions.data_ptr(); a.token_seq = token_seq.data_ptr(); a.len_after = len_after.data_ptr()
    a.k_pool = k_pool.data_ptr() if k_pool is not None else None
    a.v_pool = v_pool.data_ptr() if k_pool is not None else None
    a.page_table = page_table.data_ptr() if k_pool is not None else None
    a.pt_stride = page_table.stride(0) if k_pool is not None else 0
    a.page_rows = PAGE_ROWS; a.ring_rows = ring_rows
    a.bias = bias.data_ptr() if bias is not None else None
    lib = build.load("projnorm_kv")
    _check(lib, lib.tb_projnorm_kv(ctypes.byref(a), c_int(code(out_dtype)), c_int(T), _stream()), "projnorm_kv")
    return out, gate


def head_gate(o: torch.Tensor, gate: torch.Tensor, n_heads: int) -> torch.Tensor:
    """Every head of an attention output ``o`` [T, n_heads * D] times its token's gate [T, n_heads] (float32), in place."""
    _cuda(o, gate)
    T = o.shape[0]
    if o.dim() != 2 or not o.is_contiguous() or o.shape[1] % n_heads or gate.dtype != torch.float32 \
            or tuple(gate.shape) != (T, n_heads) or not gate.is_contiguous():
        raise KernelError(f"head_gate: output {tuple(o.shape)} and gate {tuple(gate.shape)} do not fit {n_heads} heads")
    lib = build.load("projnorm_kv")
    _check(lib, lib.tb_head_gate(_ptr(o), c_int(code(o.dtype)), _ptr(gate), c_int(T), c_int(n_heads),
                                 c_int(o.shape[1] // n_heads), _stream()), "head_gate")
    return o


def head_difference(a: torch.Tensor, n_heads: int, D: int, vdim: int, lam: float, eps: float, out_scale: float) -> torch.Tensor:
    """An attention output whose heads come in pairs, ``a`` [T, n_heads * 2 * D] (per head: the first map's output,
    then the second's), folded to [T, n_heads * D]: ``o = a1 - lam * a2`` over the first ``vdim`` numbers of a head,
    divided by its root mean square (``eps`` inside the root), times ``out_scale``; zeros in the padding.  32-bit."""
    _cuda(a)
    T = a.shape[0]
    if a.dim() != 2 or not a.is_contiguous() or a.shape[1] != n_heads * 2 * D:
        raise KernelError(f"head_difference: {tuple(a.shape)} is not [T, {n_heads} * 2 * {D}] contiguous")
    out = torch.empty((T, n_heads * D), dtype=a.dtype, device=a.device)
    lib = build.load("projnorm_kv")
    _check(lib, lib.tb_head_difference(_ptr(a), _ptr(out), c_int(code(a.dtype)), c_int(T), c_int(n_heads), c_int(D), c_int(vdim),
                                       c_float(lam), c_float(eps), c_float(out_scale), _stream()), "head_difference")
    return out


class _Mamba2Args(ctypes.Structure):
    _fields_ = [("proj", c_void_p), ("proj_stride", c_longlong), ("dt", c_void_p), ("dt_stride", c_longlong),
                ("dt_splits", c_int), ("dt_split_stride", c_longlong),
                ("heads", c_int), ("P", c_int), ("N", c_int), ("groups", c_int), ("taps", c_int), ("norm_groups", c_int),
                ("conv_w", c_void_p), ("conv_b", c_void_p), ("dt_bias", c_void_p), ("A_log", c_void_p), ("D", c_void_p),
                ("norm_w", c_void_p), ("eps", c_float),
                ("state", c_void_p), ("state_stride", c_longlong),
                ("seq_start", c_void_p), ("token_seq", c_void_p), ("slot_ids", c_void_p),
                ("xbc", c_void_p), ("y", c_void_p), ("out", c_void_p), ("batch", c_int), ("n_tokens", c_int),
                ("chunk_state", c_void_p), ("chunk_decay", c_void_p), ("chunk_len", c_int), ("n_chunks", c_int)]


def mamba2_state_size(heads: int, P: int, N: int, groups: int, taps: int) -> int:
    """32-bit numbers of one sequence's state: S [heads, P, N], then the last taps-1 conv inputs [taps-1, channels]."""
    return heads * P * N + (taps - 1) * (heads * P + 2 * groups * N)


def mamba2(proj: torch.Tensor, dt_raw: torch.Tensor, heads: int, P: int, N: int, groups: int, taps: int, norm_groups: int,
           conv_w: torch.Tensor, conv_b: torch.Tensor, dt_bias: torch.Tensor, A_log: torch.Tensor, D: torch.Tensor,
           norm_w: torch.Tensor, eps: float, state: torch.Tensor, seq_start: torch.Tensor, token_seq: torch.Tensor,
           slot_ids: torch.Tensor, batch: int, one_token_each: bool, max_seq_len: int = 0) -> torch.Tensor:
    """Everything of the state-space mixer between its two products (see mamba2.cu): from the input product's rows
    ``proj`` [T, inner + channels] (compute dtype) and step sizes ``dt_raw`` [T, heads] (float32, before bias and
    softplus; or [splits, T, heads] partial sums) to the gated, normed [T, inner] that the output product reads, with the sequences' states (``state`` [slots, mamba2_state_size] float32, rows picked by ``slot_ids``) carried along.
    ``max_seq_len`` (the longest sequence of a step of whole prompts, 0 if unknown) lets few long prompts be cut into
    chunks that run side by side."""
    _cuda(proj, dt_raw, conv_w, conv_b, dt_bias, A_log, D, norm_w, state, seq_start, token_seq, slot_ids)
    inner, ch = heads * P, heads * P + 2 * groups * N
    _rows_contig(proj, "mamba2: proj")
    T = proj.shape[0]
    if proj.shape[1] != inner + ch:
        raise KernelError(f"mamba2: the input product has {proj.shape[1]} columns, the sizes ask for {inner + ch}")
    if dt_raw.dim() == 2:
        dt_raw = dt_raw[None]
    if dt_raw.dtype != torch.float32 or tuple(dt_raw.shape[1:]) != (T, heads) or dt_raw.stride(2) != 1:
        raise KernelError(f"mamba2: the step sizes must be float32 [splits, {T}, {heads}], got {tuple(dt_raw.shape)} {dt_raw.dtype}")
    wd = torch.float32          # the small tensors enter 32-bit arithmetic: the kernels take them in 32 bits
    for name, t, shape in (("conv", conv_w, (ch, taps)), ("conv bias", conv_b, (ch,)), ("dt_bias", dt_bias, (heads,)),
                           ("A_log", A_log, (heads,)), ("D", D, (heads,)), ("norm", norm_w, (inner,))):
        if tuple(t.shape) != shape or t.dtype != wd or not t.is_contiguous():
            raise KernelError(f"mamba2: {name} must be contiguous {shape} of dtype {wd}, got {tuple(t.shape)} {t.dtype}")
    if state.dtype != torch.float32 or state.dim() != 2 or state.stride(1) != 1 or \
            state.shape[1] != mamba2_state_size(heads, P, N, groups, taps):
        raise KernelError("mamba2: the state must be float32 [slots, mamba2_state_size]")
    dt = proj.dtype
    xbc = torch.empty((T, ch), dtype=dt, device=proj.device)
    y = torch.empty((T, inner), dtype=torch.float32, device=proj.device)
    out = torch.empty((T, inner), dtype=dt, device=proj.device)
    a = _Mamba2Args()
    a.proj = proj.data_ptr(); a.proj_stride = proj.stride(0)
    a.dt = dt_raw.data_ptr(); a.dt_stride = dt_raw.stride(1)
    a.dt_splits = dt_raw.shape[0]; a.dt_split_stride = dt_raw.stride(0)
    a.heads = heads; a.P = P; a.N = N; a.groups = groups; a.taps = taps; a.norm_groups = norm_groups
    a.conv_w = conv_w.data_ptr(); a.conv_b = conv_b.data_ptr(); a.dt_bias = dt_bias.data_ptr()
    a.A_log = A_log.data_ptr(); a.D = D.data_ptr(); a.norm_w = norm_w.data_ptr(); a.eps = eps
    a.state = state.data_ptr(); a.state_stride = state.stride(0)
    a.seq_start = seq_start.data_ptr(); a.token_seq = token_seq.data_ptr(); a.slot_ids = slot_ids.data_ptr()
    a.xbc = xbc.data_ptr(); a.y = y.data_ptr(); a.out = out.data_ptr(); a.batch = batch; a.n_tokens = T
    lib = build.load("mamba2")
    scan_launches = 1
    if not one_token_each and max_seq_len > 0:
        chunk_len = c_int(0)
        n_chunks = int(lib.tb_mamba2_plan(c_int(heads), c_int(P), c_int(batch), c_int(int(max_seq_len)), ctypes.byref(chunk_len)))
        if n_chunks > 1:
            chunk_state = torch.empty((batch, n_chunks, heads * P * N), dtype=torch.float32, device=proj.device)
            chunk_decay = torch.empty((batch, n_chunks, heads), dtype=torch.float32, device=proj.device)
            a.chunk_state = chunk_state.data_ptr(); a.chunk_decay = chunk_decay.data_ptr()
            a.chunk_len = chunk_len.value; a.n_chunks = n_chunks
            scan_launches = 2
    cd, cw = c_int(code(dt)), c_int(code(wd))
    _check(lib, lib.tb_mamba2_conv(ctypes.byref(a), cd, cw, c_int(int(bool(one_token_each))), _stream()), "mamba2_conv",
           1 if one_token_each or taps == 1 else 2)
    _check(lib, lib.tb_mamba2_scan(ctypes.byref(a), cd, cw, _stream()), "mamba2_scan", scan_launches)
    _check(lib, lib.tb_mamba2_gate_norm(ctypes.byref(a), cd, cw, _stream()), "mamba2_gate_norm")
    return out


# ---------------------------------------------------------------------------
def attn_prefill_simt(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, seq_start: torch.Tensor,
                      token_seq: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int,
                      scale: float, softcap: float, window: int) -> torch.Tensor:
    """Causal attention of packed sequences over their own tokens.  q [T, n_heads*hd] and
    k, v [T, n_kv_heads*hd] may be column slices of one wider matrix."""
    _cuda(q, k, v, seq_start, token_seq)
    for name, t in (("q", q), ("k", k), ("v", v)):
        _rows_contig(t, "attention: " + name)
    if k.stride(0) != v.stride(0) or k.dtype != q.dtype or v.dtype != q.dtype:
        raise KernelError("attention: k and v must share row stride and dtype with q")
    T = q.shape[0]
    out = torch.empty((T, n_heads * head_dim), dtype=q.dtype, device=q.device)
    lib = build.load("attention_simt")
    _check(lib, lib.tb_attn_prefill_simt(_ptr(q), _ptr(k), _ptr(v), c_longlong(q.stride(0)), c_longlong(k.stride(0)),
                                         _ptr(seq_start), _ptr(token_seq), _ptr(out), c_int(code(q.dtype)), c_int(T),
                                         c_int(n_heads), c_int(n_kv_heads), c_int(head_dim), c_float(scale),
                                         c_float(softcap or 0.0), c_int(window or 0), _stream()), "attn_prefill_simt")
    return out


class _DecodeArgs(ctypes.Structure):
    _fields_ = [("q", c_void_p), ("q_stride", c_longlong), ("k_pool", c_void_p), ("v_pool", c_void_p),
                ("page_table", c_void_p), ("pt_stride", c_int), ("len_after", c_void_p), ("out", c_void_p),
                ("partial", c_void_p),
                ("n_heads", c_int), ("n_kv_heads", c_int), ("hd", c_int), ("page_rows", c_int),
                ("ring_rows", c_int), ("window", c_int), ("n_splits", c_int),
                ("scale", c_float), ("cap", c_float), ("tickets", c_void_p),
                ("qkv_part", c_void_p), ("qkv_splits", c_int), ("qkv_split_stride", c_longlong),
                ("qkv_row_stride", c_longlong), ("inv_freq", c_void_p), ("rotary_dim", c_int)]


def attn_decode_simt(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, page_table: torch.Tensor,
                     len_after: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int, scale: float,
                     softcap: float, window: int, ring_rows: int, n_splits: int = 1,
                     scratch: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One query per sequence against the paged cache (the new token's k, v already stored)."""
    _cuda(q, k_pool, v_pool, page_table, len_after, scratch)
    _rows_contig(q, "attention: q")
    B = q.shape[0]
    if page_table.dtype != torch.int32 or page_table.dim() != 2 or page_table.stride(1) != 1 or page_table.shape[0] < B:
        raise KernelError("attention: page_table must be int32 [batch, pages]")
    if len_after.dtype != torch.int32 or len_after.numel() < B:
        raise KernelError("attention: len_after must be int32 [batch]")
    out = torch.empty((B, n_heads * head_dim), dtype=q.dtype, device=q.device)
    need = B * n_heads * n_splits * (head_dim + 2) if n_splits > 1 else 0
    if need and (scratch is None or scratch.dtype != torch.float32 or scratch.numel() < need):
        scratch = torch.empty(need, dtype=torch.float32, device=q.device)
    a = _DecodeArgs()
    a.q = q.data_ptr(); a.q_stride = q.stride(0)
    a.k_pool = k_pool.data_ptr(); a.v_pool = v_pool.data_ptr()
    a.page_table = page_table.data_ptr(); a.pt_stride = page_table.stride(0)
    a.len_after = len_after.data_ptr(); a.out = out.data_ptr()
    a.partial = scratch.data_ptr() if need else None
    a.n_heads = n_heads; a.n_kv_heads = n_kv_heads; a.hd = head_dim; a.page_rows = PAGE_ROWS
    a.ring_rows = ring_rows; a.window = window or 0; a.n_splits = n_splits
    a.scale = scale; a.cap = softcap or 0.0
    lib = build.load("attention_simt")
    _check(lib, lib.tb_attn_decode_simt(ctypes.byref(a), c_int(code(q.dtype)), c_int(B), _stream()), "attn_decode_simt")
    return out


# ---------------------------------------------------------------------------
def argmax(logits: torch.Tensor) -> torch.Tensor:
    """Greedy choice per row of float32 logits: int32 ids, the smallest index on a tie."""
    _cuda(logits)
    if logits.dtype != torch.float32:
        raise KernelError("argmax: logits must be float32")
    _rows_contig(logits, "argmax: logits")
    rows, V = logits.shape
    lib = build.load("sampling")
    lib.tb_argmax_scratch_bytes.restype = c_longlong
    nbytes = lib.tb_argmax_scratch_bytes(c_int(rows), c_int(V))
    scratch = torch.empty(max(int(nbytes), 8), dtype=torch.uint8, device=logits.device)
    out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    _check(lib, lib.tb_argmax(_ptr(logits), c_longlong(logits.stride(0)), c_int(rows), c_int(V), _ptr(out),
                              _ptr(scratch), _stream()), "argmax")
    return out


class _SampleArgs(ctypes.Structure):
    _fields_ = [("logits", c_void_p), ("row_stride", c_longlong), ("vocab", c_int),
                ("temperature", c_void_p), ("top_p", c_void_p), ("penalty", c_void_p), ("draw", c_void_p),
                ("recent", c_void_p), ("n_recent", c_int), ("out", c_void_p)]


WIDE_SAMPLING_FROM = 16384          # vocabularies from this size on are sampled by many CTAs per row


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_p: torch.Tensor, penalty: torch.Tensor,
           draw: torch.Tensor, recent: Optional[torch.Tensor], nucleus: bool = True) -> torch.Tensor:
    """Per row: repetition penalty over ``recent`` ids (changes ``logits`` in place), then argmax if
    the row's temperature is <= 0, else a nucleus draw with the row's ``draw`` in [0,1).  ``nucleus=False``:
    the caller knows that every row's top_p is >= 1 (saves the launches that search the threshold)."""
    _cuda(logits, temperature, top_p, penalty, draw, recent)
    if logits.dtype != torch.float32:
        raise KernelError("sample: logits must be float32")
    _rows_contig(logits, "sample: logits")
    rows, V = logits.shape
    for name, t in (("temperature", temperature), ("top_p", top_p), ("penalty", penalty), ("draw", draw)):
        if t.dtype != torch.float32 or t.numel() != rows or not t.is_contiguous():
            raise KernelError(f"sample: {name} must be contiguous float32 [{rows}]")
    if recent is not None and (recent.dtype != torch.int32 or recent.dim() != 2 or recent.shape[0] != rows
                               or not recent.is_contiguous()):
        raise KernelError("sample: recent must be contiguous int32 [rows, n]")
    out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    a = _SampleArgs()
    a.logits = logits.data_ptr(); a.row_stride = logits.stride(0); a.vocab = V
    a.temperature = temperature.data_ptr(); a.top_p = top_p.data_ptr(); a.penalty = penalty.data_ptr()
    a.draw = draw.data_ptr()
    a.recent = recent.data_ptr() if recent is not None else None
    a.n_recent = recent.shape[1] if recent is not None else 0
    a.out = out.data_ptr()
    lib = build.load("sampling")
    if V >= WIDE_SAMPLING_FROM:
        lib.tb_sample_wide_scratch_bytes.restype = c_longlong
        need = int(lib.tb_sample_wide_scratch_bytes(c_int(rows), c_int(V)))
        scratch = torch.empty(need, dtype=torch.uint8, device=logits.device)
        _check(lib, lib.tb_sample_wide(ctypes.byref(a), c_int(rows), _ptr(scratch), c_int(1 if nucleus else 0), _stream()),
               "sample", 10 if nucleus else 4)
        return out
    _check(lib, lib.tb_sample(ctypes.byref(a), c_int(rows), _stream()), "sample")
    return out


# ---------------------------------------------------------------------------
# Choice of kernel per call
# ---------------------------------------------------------------------------
_SMS = {}


def sm_count(device=None) -> int:
    idx = torch.cuda.current_device() if device is None else (torch.device(device).index or 0)
    if idx not in _SMS:
        _SMS[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    return _SMS[idx]


def gemm_tc_takes(a: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether the tensor-core GEMM takes these operands (bfloat16, K and row strides multiples
    of 8 elements, 16-byte aligned); otherwise the FMA kernel computes the product."""
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or a.dim() != 2 or w.dim() != 2:
        return False
    if a.stride(1) != 1 or w.stride(1) != 1 or a.shape[1] != w.shape[1]:
        return False
    K = a.shape[1]
    return (K % 8 == 0 and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


GEMM_TC_GATES = ("gelu_tanh", "silu", "clamped_swish")


def gemm_tc_gates(activation: str) -> bool:
    """Whether the tensor-core product's epilogue can apply this gated activation itself."""
    return activation in GEMM_TC_GATES


def gemm_tc(a: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype, softcap: float = 0.0,
            splits: Optional[int] = None, out: Optional[torch.Tensor] = None, partials: bool = False,
            gated_act: Optional[str] = None, act_limit: float = 0.0, out_scale: float = 1.0,
            unary_act: Optional[str] = None) -> torch.Tensor:
    """a[M,K] @ w[N,K]^T in bfloat16 on tcgen05 tensor cores with 32-bit accumulation.
    ``splits`` None: the library picks the K split (more than 1 only for few tokens and few weight rows).
    ``partials=True`` returns float32 [splits, M, N] whose sum over the first axis, taken in order, is the
    product: a consumer that reads the product once anyway adds them on the way and saves a pass.
    ``gated_act`` ("gelu_tanh" or "silu"): ``w`` holds gate and up rows interleaved in blocks of 16
    (see :func:`interleave_gate_up`); the result is bfloat16 [M, N/2] = act(gate) * up, taken on the
    32-bit accumulators in the epilogue ("clamped_swish" takes ``act_limit``).  ``out_scale``: the result times this
    number (not with a cap, a gate or partial sums).  ``unary_act`` ("relu2"): every output becomes act(output), taken
    on the 32-bit accumulators (no partial sums, no cap, no gate)."""
    _cuda(a, w, out)
    if unary_act is not None:
        if unary_act not in UNARY_ACTIVATIONS or partials or softcap or gated_act is not None or out_scale != 1.0 or not gemm_tc_takes(a, w):
            raise KernelError(f"gemm_tc: the unary epilogue knows {sorted(UNARY_ACTIVATIONS)} and takes no partials, cap, gate or scale")
        out = torch.empty((a.shape[0], w.shape[0]), dtype=out_dtype, device=a.device)
        lib = build.load("gemm_tc")
        _check(lib, lib.tb_gemm_tc_unary(_ptr(a), _ptr(w), _ptr(out), c_int(code(out_dtype)), c_int(a.shape[0]), c_int(w.shape[0]),
                                         c_int(a.shape[1]), c_longlong(a.stride(0)), c_longlong(w.stride(0)),
                                         c_longlong(out.stride(0)), c_int(1), _stream()), "gemm_tc")
        return out
    if not gemm_tc_takes(a, w):
        raise KernelError(f"gemm_tc does not take a {tuple(a.shape)}/{a.stride()} {a.dtype}, "
                          f"w {tuple(w.shape)}/{w.stride()} {w.dtype}")
    M, K = a.shape
    N = w.shape[0]
    lib = build.load("gemm_tc")
    if splits is None:
        splits = lib.tb_gemm_tc_splits(c_int(M), c_int(N), c_int(K), c_int(sm_count(a.device)))
    splits = int(lib.tb_gemm_tc_effective_splits(c_int(K), c_int(splits)))
    if gated_act is not None:
        if not gemm_tc_gates(gated_act):
            raise KernelError(f"gemm_tc: the epilogue does not know activation '{gated_act}' (known: {GEMM_TC_GATES})")
        if N % 32 or partials or softcap or out_scale != 1.0:
            raise KernelError("gemm_tc: the gated epilogue needs a multiple of 32 weight rows, no partials, no cap, no scale")
        out = torch.empty((M, N // 2), dtype=torch.bfloat16, device=a.device)
        _check(lib, lib.tb_gemm_tc_ex(_ptr(a), _ptr(w), _ptr(out), c_int(1), c_int(M), c_int(N), c_int(K),
                                      c_longlong(a.stride(0)), c_longlong(w.stride(0)), c_longlong(out.stride(0)),
                                      c_float(0.0), c_int(1), _ptr(None), c_int(1), c_int(ACTIVATIONS[gated_act]),
                                      c_float(act_limit), c_float(1.0), _stream()), "gemm_tc")
        return out
    if partials:
        if softcap or out_scale != 1.0:
            raise KernelError("gemm_tc: neither a soft cap nor a scale can be applied to partial sums")
        part = torch.empty((splits, M, N), dtype=torch.float32, device=a.device)
        if splits == 1:
            _check(lib, lib.tb_gemm_tc(_ptr(a), _ptr(w), _ptr(part), c_int(0), c_int(M), c_int(N), c_int(K),
                                       c_longlong(a.stride(0)), c_longlong(w.stride(0)), c_longlong(N),
                                       c_float(0.0), c_int(1), _ptr(None), c_int(1), c_int(-1), _stream()), "gemm_tc")
        else:
            _check(lib, lib.tb_gemm_tc(_ptr(a), _ptr(w), _ptr(None), c_int(0), c_int(M), c_int(N), c_int(K),
                                       c_longlong(a.stride(0)), c_longlong(w.stride(0)), c_longlong(N),
                                       c_float(0.0), c_int(splits), _ptr(part), c_int(0), c_int(-1), _stream()), "gemm_tc")
        return part
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    else:
        _rows_contig(out, "gemm: out")
    scratch = None
    if splits > 1:
        scratch = torch.empty(splits * M * N, dtype=torch.float32, device=a.device)
    _check(lib, lib.tb_gemm_tc_ex(_ptr(a), _ptr(w), _ptr(out), c_int(code(out.dtype)), c_int(M), c_int(N), c_int(K),
                                  c_longlong(a.stride(0)), c_longlong(w.stride(0)), c_longlong(out.stride(0)),
                                  c_float(softcap or 0.0), c_int(splits), _ptr(scratch), c_int(1), c_int(-1),
                                  c_float(0.0), c_float(out_scale), _stream()), "gemm_tc",
           2 if splits > 1 else 1)
    return out


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """[I, K] gate and up matrices -> [2I, K] with rows in blocks of 16: gate 0..15, up 0..15, gate 16..31, ...
    (the layout the gated epilogue of :func:`gemm_tc` expects; I must be a multiple of 16).  Run once, when
    the weights are bound."""
    I, K = gate.shape
    if up.shape != gate.shape or I % 16:
        raise KernelError("interleave_gate_up: gate and up must be [I, K] with I a multiple of 16")
    return torch.stack([gate.view(I // 16, 16, K), up.view(I // 16, 16, K)], dim=1).reshape(2 * I, K).contiguous()


def sum_partials(part: torch.Tensor) -> torch.Tensor:
    """[splits, rows, cols] float32 partial sums -> their sum, added in split order."""
    _cuda(part)
    if part.dtype != torch.float32 or part.dim() != 3 or not part.is_contiguous():
        raise KernelError("sum_partials: wants contiguous float32 [splits, rows, cols]")
    S, R, Cc = part.shape
    if S == 1:
        return part[0]
    out = torch.empty((R, Cc), dtype=torch.float32, device=part.device)
    lib = build.load("gemm_tc")
    _check(lib, lib.tb_sum_partials(_ptr(part), _ptr(out), c_int(R), c_int(Cc), c_int(S), _stream()), "sum_partials")
    return out


def kernel_errors() -> dict:
    """Error words of the kernels with bounded waits that this process has loaded: {} when no wait ever ran
    out.  Synchronises the device and clears the words."""
    out = {}
    loaded = build.loaded()
    if "gemm_tc" in loaded and gemm_tc_error():
        out["gemm_tc"] = "a bounded wait ran out"
    if "attention_decode" in loaded and attn_decode_error():
        out["attention_decode"] = "a bounded wait ran out"
    for name in loaded:
        if name.startswith("attention_prefill_tc@"):
            v = int(build.load(name).tb_attn_prefill_tc_error())
            if v:
                out[name] = f"error word {v}"
    return out


def gemm_tc_set_pair(mode: int) -> int:
    """Many-token products on pairs of SMs: 0 never, 1 whenever the shape allows, 2 where it pays (the default);
    returns the previous setting."""
    return int(build.load("gemm_tc").tb_gemm_tc_set_pair(c_int(int(mode))))


def gemm_tc_error() -> int:
    """Reads and clears the tensor-core GEMM's error word (synchronises): 0, or the role whose
    bounded wait ran out (1 loader, 2 MMA issuer, 3 epilogue; 4 to 6 the same roles of the kernel on pairs of SMs)."""
    return int(build.load("gemm_tc").tb_gemm_tc_error())


def attn_padded_head(dtype: torch.dtype, n: int) -> int:
    """The head size at which keys and values of up to ``n`` numbers a head are stored and attended to: in bfloat16 the
    next size that the tensor-core kernels of both prefill and decode take (64, 128, 256), beyond that the next multiple
    of 16; in float32 ``n`` itself (the generic kernel takes any size)."""
    if dtype != torch.bfloat16:
        return n
    for size in (64, 128, 256):
        if n <= size:
            return size
    return (n + 15) // 16 * 16


def attn_prefill_takes(dtype: torch.dtype, head_dim: int) -> bool:
    """Whether the tensor-core prefill kernel takes this shape (bfloat16, head_dim a multiple of 16 up to 256)."""
    return dtype == torch.bfloat16 and head_dim % 16 == 0 and 16 <= head_dim <= 256


def attn_prefill_lib(head_dim: int) -> str:
    return f"attention_prefill@TB_HD={head_dim}"


def attn_prefill_mma(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, seq_start: torch.Tensor, n_heads: int,
                     n_kv_heads: int, head_dim: int, scale: float, softcap: float, window: int,
                     max_seq_len: int) -> torch.Tensor:
    """Causal attention of packed sequences on tensor cores (see attention_prefill.cu); ``max_seq_len`` is the
    longest sequence of the batch (it sizes the grid)."""
    _cuda(q, k, v, seq_start)
    for name, t in (("q", q), ("k", k), ("v", v)):
        _rows_contig(t, "attention: " + name)
    if not attn_prefill_takes(q.dtype, head_dim) or k.dtype != q.dtype or v.dtype != q.dtype:
        raise KernelError(f"attn_prefill_mma does not take {q.dtype} with head_dim {head_dim}")
    if k.stride(0) != v.stride(0):
        raise KernelError("attention: k and v must share their row stride")
    if seq_start.dtype != torch.int32 or not seq_start.is_contiguous() or seq_start.numel() < 2:
        raise KernelError("attention: seq_start must be contiguous int32 [batch + 1]")
    T = q.shape[0]
    B = seq_start.numel() - 1
    out = torch.empty((T, n_heads * head_dim), dtype=q.dtype, device=q.device)
    lib = build.load(attn_prefill_lib(head_dim))
    _check(lib, lib.tb_attn_prefill_mma(_ptr(q), _ptr(k), _ptr(v), c_longlong(q.stride(0)), c_longlong(k.stride(0)),
                                        _ptr(seq_start), _ptr(out), c_int(B), c_int(max_seq_len), c_int(n_heads),
                                        c_int(n_kv_heads), c_int(head_dim), c_float(scale), c_float(softcap or 0.0),
                                        c_int(window or 0), _stream()), "attn_prefill_mma")
    return out


def attn_prefill_tc_takes(dtype: torch.dtype, head_dim: int) -> bool:
    """Whether the tcgen05 prefill kernel takes this shape (bfloat16, head_dim 64, 128 or 256)."""
    return dtype == torch.bfloat16 and head_dim in (64, 128, 256)


def attn_prefill_tc_lib(head_dim: int) -> str:
    return f"attention_prefill_tc@TB_HD={head_dim}"


def attn_prefill_tc(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, seq_start: torch.Tensor, seq_lens,
                    n_heads: int, n_kv_heads: int, head_dim: int, scale: float, softcap: float, window: int) -> torch.Tensor:
    """Causal attention of packed sequences on tcgen05 tensor cores (see attention_prefill_tc.cu).
    ``seq_lens``: the sequences' lengths on the host."""
    _cuda(q, k, v, seq_start)
    for name, t in (("q", q), ("k", k), ("v", v)):
        _rows_contig(t, "attention: " + name)
    if not attn_prefill_tc_takes(q.dtype, head_dim) or k.dtype != q.dtype or v.dtype != q.dtype:
        raise KernelError(f"attn_prefill_tc does not take {q.dtype} with head_dim {head_dim}")
    if k.stride(0) != v.stride(0):
        raise KernelError("attention: k and v must share their row stride")
    B = len(seq_lens)
    if seq_start.dtype != torch.int32 or not seq_start.is_contiguous() or seq_start.numel() != B + 1:
        raise KernelError("attention: seq_start must be contiguous int32 [batch + 1]")
    T = q.shape[0]
    out = torch.empty((T, n_heads * head_dim), dtype=q.dtype, device=q.device)
    lib = build.load(attn_prefill_tc_lib(head_dim))
    _check(lib, lib.tb_attn_prefill_tc(_ptr(q), _ptr(k), _ptr(v), c_longlong(q.stride(0)), c_longlong(k.stride(0)),
                                       _ptr(seq_start), _ptr(out), c_int(T), c_int(B), c_int(max(seq_lens)),
                                       c_int(n_heads), c_int(n_kv_heads), c_int(head_dim), c_float(scale),
                                       c_float(softcap or 0.0), c_int(window or 0), _stream()), "attn_prefill_tc", 2)
    return out


def attn_prefill_tc_error(head_dim: int) -> int:
    """Reads and clears the tcgen05 prefill attention's error word (synchronises); 0 = no wait ran out."""
    return int(build.load(attn_prefill_tc_lib(head_dim)).tb_attn_prefill_tc_error())


def attn_prefill(q, k, v, seq_start, token_seq, n_heads, n_kv_heads, head_dim, scale, softcap, window,
                 max_seq_len: int, seq_lens=None, memo: Optional[dict] = None) -> torch.Tensor:
    """Prefill attention, kernel chosen here: tcgen05 for head sizes 64/128/256, mma.sync for other multiples
    of 16, the generic kernel for the rest and for float32.  ``memo``: a per-step dict for what a kernel wants
    uploaded once per step and not once per layer (none does at present)."""
    if attn_prefill_tc_takes(q.dtype, head_dim) and seq_lens is not None:
        return attn_prefill_tc(q, k, v, seq_start, seq_lens, n_heads, n_kv_heads, head_dim, scale, softcap, window)
    if attn_prefill_takes(q.dtype, head_dim):
        return attn_prefill_mma(q, k, v, seq_start, n_heads, n_kv_heads, head_dim, scale, softcap, window, max_seq_len)
    return attn_prefill_simt(q, k, v, seq_start, token_seq, n_heads, n_kv_heads, head_dim, scale, softcap, window)


def attn_decode_takes(dtype: torch.dtype, n_heads: int, n_kv_heads: int, head_dim: int) -> bool:
    """Whether the bulk-copy decode kernel takes this shape (bfloat16, head_dim 32/64/128/256, up to 8
    query heads per kv head); other shapes run on the generic kernel."""
    if dtype != torch.bfloat16 or n_kv_heads <= 0 or n_heads % n_kv_heads:
        return False
    g = n_heads // n_kv_heads
    return (head_dim in (64, 128, 256) and 1 <= g <= 8) or (head_dim == 32 and g in (1, 2, 4, 8))


_TICKETS: dict = {}
_TICKET_SLOTS = 1 << 16


def _tickets(device: torch.device) -> torch.Tensor:
    """Zeroed counters with which the split pieces of a decode attention launch find out which of them
    finishes last; every launch leaves them at zero.  One array per device: launches that may overlap on
    the GPU (different streams with no order between them) must not both use split pieces."""
    t = _TICKETS.get(device.index)
    if t is None:
        if torch.cuda.is_current_stream_capturing():
            raise KernelError("attn_decode: the first launch on a device must not be inside a graph capture")
        t = _TICKETS[device.index] = torch.zeros(_TICKET_SLOTS, dtype=torch.int32, device=device)
    return t


def _decode_partials(part: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int, variant: str, rotate):
    """Checks the partial sums handed to a decode kernel that rotates by itself; returns them and a stand-in for q."""
    inv_freq, rotary_dim = rotate
    width = (n_heads + 2 * n_kv_heads) * head_dim
    if variant != "mma" or head_dim < 64:
        raise KernelError("attention: only the tensor-core decode kernel (head_dim >= 64) rotates by itself")
    if part.dtype != torch.float32 or part.dim() != 3 or part.shape[2] != width or part.stride(2) != 1:
        raise KernelError(f"attention: the q/k/v partial sums must be float32 [splits, batch, {width}]")
    if inv_freq is not None and (inv_freq.dtype != torch.float32 or inv_freq.numel() != rotary_dim // 2
                                 or rotary_dim % 2 or not 0 < rotary_dim <= head_dim):
        raise KernelError("attention: inv_freq must be float32 [rotary_dim/2], rotary_dim even and within head_dim")
    _cuda(inv_freq)
    return part, torch.empty((part.shape[1], 0), dtype=torch.bfloat16, device=part.device)


def _set_rotation(a, part, rotate) -> None:
    if part is None:
        a.qkv_part = None; a.qkv_splits = 0; a.qkv_split_stride = 0; a.qkv_row_stride = 0
        a.inv_freq = None; a.rotary_dim = 0
        return
    inv_freq, rotary_dim = rotate
    a.q = None; a.q_stride = 0
    a.qkv_part = part.data_ptr(); a.qkv_splits = part.shape[0]
    a.qkv_split_stride = part.stride(0); a.qkv_row_stride = part.stride(1)
    a.inv_freq = inv_freq.data_ptr() if inv_freq is not None else None
    a.rotary_dim = rotary_dim if inv_freq is not None else 0


def attn_decode_tma(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, page_table: torch.Tensor,
                    len_after: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int, scale: float,
                    softcap: float, window: int, ring_rows: int, n_splits: int = 1,
                    variant: str = "mma", rotate=None) -> torch.Tensor:
    """Decode attention with pages staged in shared memory by bulk copies (see attention_decode.cu).
    ``variant``: "mma" (tensor cores, the product path) or "lanes" (scalar, kept for comparison).
    ``rotate`` = (inv_freq or None, rotary_dim), "mma" only: ``q`` is then the float32 partial sums
    [splits, batch, (n_heads + 2 n_kv_heads) * head_dim] of the q/k/v product; the kernel adds them, rotates q and k
    at the new token's position, and writes k and v to the cache itself (no separate rotation kernel)."""
    _cuda(q, k_pool, v_pool, page_table, len_after)
    part = None
    if rotate is not None:
        part, q = _decode_partials(q, n_heads, n_kv_heads, head_dim, variant, rotate)
    _rows_contig(q, "attention: q")
    B = q.shape[0]
    if not attn_decode_takes(q.dtype, n_heads, n_kv_heads, head_dim):
        raise KernelError(f"attn_decode_tma does not take {q.dtype}, {n_heads}/{n_kv_heads} heads, head_dim {head_dim}")
    if page_table.dtype != torch.int32 or page_table.dim() != 2 or page_table.stride(1) != 1 or page_table.shape[0] < B:
        raise KernelError("attention: page_table must be int32 [batch, pages]")
    if len_after.dtype != torch.int32 or len_after.numel() < B:
        raise KernelError("attention: len_after must be int32 [batch]")
    if tuple(k_pool.shape[1:]) != (n_kv_heads, PAGE_ROWS, head_dim) or k_pool.shape != v_pool.shape \
            or not k_pool.is_contiguous() or not v_pool.is_contiguous() or k_pool.dtype != q.dtype:
        raise KernelError("attention: pools must be contiguous [pages, n_kv_heads, PAGE_ROWS, head_dim] of q's dtype")
    out = torch.empty((B, n_heads * head_dim), dtype=q.dtype, device=q.device)
    scratch = None
    if n_splits > 1:
        scratch = torch.empty(B * n_heads * n_splits * (head_dim + 2), dtype=torch.float32, device=q.device)
    a = _DecodeArgs()
    a.q = q.data_ptr(); a.q_stride = q.stride(0)
    a.k_pool = k_pool.data_ptr(); a.v_pool = v_pool.data_ptr()
    a.page_table = page_table.data_ptr(); a.pt_stride = page_table.stride(0)
    a.len_after = len_after.data_ptr(); a.out = out.data_ptr()
    a.partial = scratch.data_ptr() if scratch is not None else None
    a.n_heads = n_heads; a.n_kv_heads = n_kv_heads; a.hd = head_dim; a.page_rows = PAGE_ROWS
    a.ring_rows = ring_rows; a.window = window or 0; a.n_splits = n_splits
    a.scale = scale; a.cap = softcap or 0.0
    fused_fold = variant == "mma" and head_dim >= 64 and n_splits > 1 and B * n_kv_heads <= _TICKET_SLOTS
    a.tickets = _tickets(q.device).data_ptr() if fused_fold else None
    _set_rotation(a, part, rotate)
    lib = build.load("attention_decode")
    fn = lib.tb_attn_decode if variant == "mma" else lib.tb_attn_decode_lanes
    _check(lib, fn(ctypes.byref(a), c_int(code(q.dtype)), c_int(B), _stream()), "attn_decode",
           2 if (n_splits > 1 and not fused_fold) else 1)
    return out


def attn_decode_stream(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, page_table: torch.Tensor,
                       len_after: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int, scale: float,
                       softcap: float, window: int, ring_rows: int, n_ctas: Optional[int] = None,
                       rotate=None) -> torch.Tensor:
    """Decode attention on tensor cores with all pages of the launch dealt out evenly to ``n_ctas`` CTAs
    (default: one per SM), wherever the sequences end: the time of a launch follows the sum of the lengths,
    not the longest one (see attention_decode.cu).  ``rotate``: as in :func:`attn_decode_tma`."""
    _cuda(q, k_pool, v_pool, page_table, len_after)
    part = None
    if rotate is not None:
        part, q = _decode_partials(q, n_heads, n_kv_heads, head_dim, "mma", rotate)
    _rows_contig(q, "attention: q")
    B = q.shape[0]
    if not attn_decode_stream_takes(q.dtype, n_heads, n_kv_heads, head_dim, B):
        raise KernelError(f"attn_decode_stream does not take {q.dtype}, {n_heads}/{n_kv_heads} heads, "
                          f"head_dim {head_dim}, batch {B}")
    if page_table.dtype != torch.int32 or page_table.dim() != 2 or page_table.stride(1) != 1 or page_table.shape[0] < B:
        raise KernelError("attention: page_table must be int32 [batch, pages]")
    if len_after.dtype != torch.int32 or len_after.numel() < B:
        raise KernelError("attention: len_after must be int32 [batch]")
    if tuple(k_pool.shape[1:]) != (n_kv_heads, PAGE_ROWS, head_dim) or k_pool.shape != v_pool.shape \
            or not k_pool.is_contiguous() or not v_pool.is_contiguous() or k_pool.dtype != q.dtype:
        raise KernelError("attention: pools must be contiguous [pages, n_kv_heads, PAGE_ROWS, head_dim] of q's dtype")
    lib = build.load("attention_decode")
    if n_ctas is None:
        n_ctas = int(lib.tb_attn_decode_stream_ctas(c_int(sm_count(q.device)), c_int(head_dim)))
    lib.tb_attn_decode_stream_scratch_floats.restype = c_longlong
    need = int(lib.tb_attn_decode_stream_scratch_floats(c_int(n_ctas), c_int(n_heads), c_int(n_kv_heads), c_int(head_dim)))
    out = torch.empty((B, n_heads * head_dim), dtype=q.dtype, device=q.device)
    scratch = torch.empty(need, dtype=torch.float32, device=q.device)
    a = _DecodeArgs()
    a.q = q.data_ptr(); a.q_stride = q.stride(0)
    a.k_pool = k_pool.data_ptr(); a.v_pool = v_pool.data_ptr()
    a.page_table = page_table.data_ptr(); a.pt_stride = page_table.stride(0)
    a.len_after = len_after.data_ptr(); a.out = out.data_ptr()
    a.partial = scratch.data_ptr()
    a.n_heads = n_heads; a.n_kv_heads = n_kv_heads; a.hd = head_dim; a.page_rows = PAGE_ROWS
    a.ring_rows = ring_rows; a.window = window or 0; a.n_splits = 0
    a.scale = scale; a.cap = softcap or 0.0
    a.tickets = _tickets(q.device).data_ptr()
    _set_rotation(a, part, rotate)
    _check(lib, lib.tb_attn_decode_stream(ctypes.byref(a), c_int(code(q.dtype)), c_int(B), c_int(n_ctas), _stream()),
           "attn_decode_stream")
    return out


def attn_decode_rotates(dtype: torch.dtype, n_heads: int, n_kv_heads: int, head_dim: int) -> bool:
    """Whether :func:`attn_decode` can take the q/k/v partial sums and rotate by itself (``rotate=``)."""
    return attn_decode_takes(dtype, n_heads, n_kv_heads, head_dim) and head_dim >= 64


def attn_decode_stream_takes(dtype: torch.dtype, n_heads: int, n_kv_heads: int, head_dim: int, batch: int) -> bool:
    return (attn_decode_takes(dtype, n_heads, n_kv_heads, head_dim) and head_dim >= 64
            and batch <= 1024 and batch * n_kv_heads <= _TICKET_SLOTS)


def attn_decode_error() -> int:
    """Reads and clears the decode attention's error word (synchronises): 0, or 1 a bounded wait ran out, 2 the
    shared-memory block began less aligned than budgeted, 3 a CTA of the stream partition had more runs than its
    list holds.  After an error the ticket counters are zeroed again (a launch that gave up may have left them
    half counted)."""
    v = int(build.load("attention_decode").tb_attn_decode_error())
    if v:
        for t in _TICKETS.values():
            t.zero_()
    return v


def choose_decode_splits(batch: int, n_kv_heads: int, pages: int, sms: int) -> int:
    """In how many pieces decode attention cuts a sequence's pages.  A CTA serves one (sequence, kv head,
    piece); all CTAs of a launch are about equally long, so the launch takes ceil(CTAs / SMs) rounds.
    Among the piece counts that keep at least 4 pages per piece, take the one that wastes least of the
    last round (ties: fewer pieces)."""
    items = max(1, batch * n_kv_heads)
    best, best_eff = 1, 0.0
    for s in range(1, max(1, pages // 4) + 1):
        if s > 64:
            break
        ctas = items * s
        eff = ctas / (((ctas + sms - 1) // sms) * sms)
        # a piece pays its start-up and its share of the final fold: about four pages' worth (measured)
        per = (pages + s - 1) // s
        eff *= per / (per + 4.0)
        if eff > best_eff + 1e-9:
            best, best_eff = s, eff
    return best


_DECODE_PARTITION = None          # None: chosen per launch; "split" or "stream": forced (tests, comparisons)


def set_decode_partition(mode: Optional[str]) -> Optional[str]:
    """Forces decode attention's partition ("split", "stream") or gives the choice back (None); returns the
    previous setting.  Set it before an engine captures its decode graphs."""
    global _DECODE_PARTITION
    if mode not in (None, "split", "stream"):
        raise KernelError(f"decode partition {mode!r}: None, 'split' or 'stream'")
    was, _DECODE_PARTITION = _DECODE_PARTITION, mode
    return was


def decode_partition_is_stream(batch: int, n_kv_heads: int, pages: int, splits: int, uneven: int, sms: int) -> bool:
    """Whether decode attention deals its pages out as one stream (else every sequence is cut into ``splits``
    pieces).  A streaming launch costs about ten pages' time more (its CTAs walk several sequences: page prefix,
    a rotation and a fold per run), so it is taken when the pieces of the longest sequence are at least that much
    longer than an even share: ``uneven`` quarters of a piece's pages are saved at least.  And when cutting
    every sequence would take more than two rounds of CTAs: each round pays its start-up again."""
    per = (pages + splits - 1) // splits
    return uneven * per >= 4 * 10 or batch * n_kv_heads * splits > 2 * sms


def attn_decode_plan(batch: int, n_kv_heads: int, len_bucket: int, ring_rows: int, uneven: int, device) -> Tuple[bool, int]:
    """(whether the pages of a decode launch are dealt out as one stream, else in how many pieces every sequence
    is cut), from what a captured step may depend on."""
    rows = min(len_bucket, ring_rows) if ring_rows else len_bucket
    pages = max(1, (rows + PAGE_ROWS - 1) // PAGE_ROWS)
    sms = sm_count(device)
    splits = choose_decode_splits(batch, n_kv_heads, pages, sms)
    stream = decode_partition_is_stream(batch, n_kv_heads, pages, splits, int(uneven), sms)
    if _DECODE_PARTITION is not None:
        stream = _DECODE_PARTITION == "stream"
    return stream, splits


def attn_decode(q, k_pool, v_pool, page_table, len_after, n_heads, n_kv_heads, head_dim, scale, softcap, window,
                ring_rows, len_bucket: int, uneven: int = 0, rotate=None) -> torch.Tensor:
    """Decode attention, kernel and partition chosen here.  ``len_bucket``: an upper bound of the longest
    context of the batch (the engine passes a power of two so that the choice is stable across steps).
    ``uneven``: how much the batch's contexts differ in length (``engine.unevenness``, 0..3); if enough, the pages
    are dealt out to the CTAs as one stream, so that the launch's time follows the sum of the lengths and not
    the longest one."""
    B = q.shape[0] if rotate is None else q.shape[1]
    dt = q.dtype if rotate is None else torch.bfloat16
    stream, splits = attn_decode_plan(B, n_kv_heads, len_bucket, ring_rows, uneven, q.device)
    if stream and attn_decode_stream_takes(dt, n_heads, n_kv_heads, head_dim, B):
        return attn_decode_stream(q, k_pool, v_pool, page_table, len_after, n_heads, n_kv_heads, head_dim, scale,
                                  softcap, window, ring_rows, rotate=rotate)
    if attn_decode_takes(dt, n_heads, n_kv_heads, head_dim):
        variant = "lanes" if head_dim < 64 else "mma"     # a 64-byte row has no swizzled box for the tensor-core kernel
        return attn_decode_tma(q, k_pool, v_pool, page_table, len_after, n_heads, n_kv_heads, head_dim, scale,
                               softcap, window, ring_rows, splits, variant, rotate)
    if rotate is not None:
        raise KernelError("attention: this shape's decode kernel does not rotate by itself")
    return attn_decode_simt(q, k_pool, v_pool, page_table, len_after, n_heads, n_kv_heads, head_dim, scale,
                            softcap, window, ring_rows, splits)


# ---------------------------------------------------------------------------
# Layer norm, row-wise additions
# ---------------------------------------------------------------------------
def add_layernorm(h: torch.Tensor, a: Optional[torch.Tensor], w: torch.Tensor, b: torch.Tensor, eps: float,
                  out_dtype: torch.dtype) -> torch.Tensor:
    """``h += a`` in place (skipped if ``a`` is None), then returns the layer norm of ``h`` with weight and bias.
    ``h`` float32 [rows, width]; ``a`` [rows, width] or float32 partial sums [splits, rows, width]; ``w``, ``b``
    float32 [width]."""
    _cuda(h, a, w, b)
    if h.dtype != torch.float32 or h.dim() != 2 or not h.is_contiguous():
        raise KernelError("add_layernorm: the residual stream must be contiguous float32 [rows, width]")
    n_splits, split_stride, a_code = 1, 0, 0
    if a is not None:
        if a.dim() == 3:
            if a.dtype != torch.float32:
                raise KernelError("add_layernorm: partial sums must be float32")
            n_splits, split_stride = a.shape[0], a.stride(0)
            if tuple(a.shape[1:]) != tuple(h.shape) or a.stride(1) != h.shape[1] or a.stride(2) != 1:
                raise KernelError(f"add_layernorm: partial sums {tuple(a.shape)} do not fit the stream {tuple(h.shape)}")
        elif a.shape != h.shape or not a.is_contiguous():
            raise KernelError(f"add_layernorm: branch {tuple(a.shape)} does not fit the stream {tuple(h.shape)}")
        a_code = code(a.dtype)
    for name, t in (("weight", w), ("bias", b)):
        if t.dtype != torch.float32 or t.numel() != h.shape[1] or not t.is_contiguous():
            raise KernelError(f"add_layernorm: the {name} must be contiguous float32 [{h.shape[1]}]")
    out = torch.empty(h.shape, dtype=out_dtype, device=h.device)
    lib = build.load("layernorm")
    _check(lib, lib.tb_add_layernorm(_ptr(h), _ptr(a), c_int(a_code), c_int(n_splits), c_longlong(split_stride), _ptr(w),
                                     _ptr(b), c_float(eps), _ptr(out), c_int(code(out_dtype)), c_int(h.shape[0]),
                                     c_int(h.shape[1]), _stream()), "add_layernorm")
    return out


def add_rows(h: torch.Tensor, rows: Optional[torch.Tensor], vector: Optional[torch.Tensor]) -> None:
    """``h += rows + vector`` in place: ``rows`` float32 of h's shape, ``vector`` float32 [width]; either may be None."""
    _cuda(h, rows, vector)
    if h.dtype != torch.float32 or h.dim() != 2 or not h.is_contiguous():
        raise KernelError("add_rows: the residual stream must be contiguous float32 [rows, width]")
    if rows is not None and (rows.dtype != torch.float32 or rows.shape != h.shape or not rows.is_contiguous()):
        raise KernelError("add_rows: rows must be contiguous float32 of the stream's shape")
    if vector is not None and (vector.dtype != torch.float32 or vector.numel() != h.shape[1] or not vector.is_contiguous()):
        raise KernelError("add_rows: the vector must be contiguous float32 [width]")
    lib = build.load("layernorm")
    _check(lib, lib.tb_add_rows(_ptr(h), _ptr(rows), _ptr(vector), c_int(h.shape[0]), c_int(h.shape[1]), _stream()), "add_rows")


# ---------------------------------------------------------------------------
# Gated linear attention
# ---------------------------------------------------------------------------
class _GlaArgs(ctypes.Structure):
    _fields_ = [("proj", c_void_p), ("proj_stride", c_longlong),
                ("a1", c_void_p), ("a1_splits", c_int), ("a1_split_stride", c_longlong), ("rank", c_int),
                ("a2", c_void_p), ("a2_bias", c_void_p), ("inv_tau", c_float), ("q_scale", c_float),
                ("norm_w", c_void_p), ("eps", c_float), ("state", c_void_p), ("state_stride", c_longlong),
                ("seq_start", c_void_p), ("token_seq", c_void_p), ("slot_ids", c_void_p),
                ("decay", c_void_p), ("y", c_void_p), ("out", c_void_p),
                ("heads", c_int), ("D", c_int), ("V", c_int), ("batch", c_int), ("n_tokens", c_int),
                ("chunk_state", c_void_p), ("chunk_decay", c_void_p), ("chunk_len", c_int), ("n_chunks", c_int)]


def gla(proj: torch.Tensor, low: torch.Tensor, a2: torch.Tensor, a2_bias: torch.Tensor, tau: float, q_scale: float,
        norm_w: torch.Tensor, eps: float, heads: int, key_dim: int, value_dim: int, state: torch.Tensor,
        seq_start: torch.Tensor, token_seq: torch.Tensor, slot_ids: torch.Tensor, batch: int,
        max_seq_len: int = 0) -> torch.Tensor:
    """Gated linear attention between its products (see gla.cu).  ``max_seq_len`` (the longest sequence of a step of
    whole prompts, 0 if unknown or one token each) lets few long prompts be cut into chunks that run side by side.  ``proj`` [T, 2 H D + 2 H V]: q, k, v and the output
    gate's pre-activation, in the compute dtype; ``low`` float32 [splits, T, rank]: partial sums of the decay's first
    product; ``a2`` float32 [H D, rank], ``a2_bias`` float32 [H D], ``norm_w`` float32 [V]; ``state`` float32
    [slots, H D V], rows picked by ``slot_ids``, read and written.  Returns [T, H V] in the compute dtype."""
    _cuda(proj, low, a2, a2_bias, norm_w, state, seq_start, token_seq, slot_ids)
    _rows_contig(proj, "gla: proj")
    T = proj.shape[0]
    HD, HV = heads * key_dim, heads * value_dim
    if proj.shape[1] != 2 * HD + 2 * HV:
        raise KernelError(f"gla: the input product has {proj.shape[1]} columns, the sizes ask for {2 * HD + 2 * HV}")
    if low.dim() == 2:
        low = low[None]
    rank = low.shape[2]
    if low.dtype != torch.float32 or low.shape[1] != T or low.stride(2) != 1 or low.stride(1) != rank:
        raise KernelError(f"gla: the decay's first product must be float32 [splits, {T}, rank], got {tuple(low.shape)} {low.dtype}")
    for name, t, shape in (("a2", a2, (HD, rank)), ("a2 bias", a2_bias, (HD,)), ("norm", norm_w, (value_dim,))):
        if tuple(t.shape) != shape or t.dtype != torch.float32 or not t.is_contiguous():
            raise KernelError(f"gla: {name} must be contiguous float32 {shape}, got {tuple(t.shape)} {t.dtype}")
    if state.dtype != torch.float32 or state.dim() != 2 or state.stride(1) != 1 or state.shape[1] != HD * value_dim:
        raise KernelError(f"gla: the state must be float32 [slots, {HD * value_dim}]")
    dt = proj.dtype
    decay = torch.empty((T, HD), dtype=torch.float32, device=proj.device)
    y = torch.empty((T, HV), dtype=torch.float32, device=proj.device)
    out = torch.empty((T, HV), dtype=dt, device=proj.device)
    a = _GlaArgs()
    a.proj = proj.data_ptr(); a.proj_stride = proj.stride(0)
    a.a1 = low.data_ptr(); a.a1_splits = low.shape[0]; a.a1_split_stride = low.stride(0); a.rank = rank
    a.a2 = a2.data_ptr(); a.a2_bias = a2_bias.data_ptr(); a.inv_tau = 1.0 / tau; a.q_scale = q_scale
    a.norm_w = norm_w.data_ptr(); a.eps = eps; a.state = state.data_ptr(); a.state_stride = state.stride(0)
    a.seq_start = seq_start.data_ptr(); a.token_seq = token_seq.data_ptr(); a.slot_ids = slot_ids.data_ptr()
    a.decay = decay.data_ptr(); a.y = y.data_ptr(); a.out = out.data_ptr()
    a.heads = heads; a.D = key_dim; a.V = value_dim; a.batch = batch; a.n_tokens = T
    lib = build.load("gla")
    scan_launches = 1
    if max_seq_len > 0:
        chunk_len = c_int(0)
        n_chunks = int(lib.tb_gla_plan(c_int(heads), c_int(value_dim), c_int(batch), c_int(int(max_seq_len)),
                                       c_int(sm_count(proj.device)), ctypes.byref(chunk_len)))
        if n_chunks > 1 and batch * n_chunks <= 65535:
            chunk_state = torch.empty((batch, n_chunks, HD * value_dim), dtype=torch.float32, device=proj.device)
            chunk_decay = torch.empty((batch, n_chunks, HD), dtype=torch.float32, device=proj.device)
            a.chunk_state = chunk_state.data_ptr(); a.chunk_decay = chunk_decay.data_ptr()
            a.chunk_len = chunk_len.value; a.n_chunks = n_chunks
            scan_launches = 3
    _check(lib, lib.tb_gla_decay(ctypes.byref(a), _stream()), "gla_decay")
    _check(lib, lib.tb_gla_scan(ctypes.byref(a), c_int(code(dt)), _stream()), "gla_scan", scan_launches)
    _check(lib, lib.tb_gla_gate_norm(ctypes.byref(a), c_int(code(dt)), _stream()), "gla_gate_norm")
    return out


# ---------------------------------------------------------------------------
# Attention over cached latent rows
# ---------------------------------------------------------------------------
class _LatentRowsArgs(ctypes.Structure):
    _fields_ = [("dkv", c_void_p), ("splits", c_int), ("split_stride", c_longlong), ("norm_w", c_void_p), ("eps", c_float),
                ("inv_freq", c_void_p), ("rot_dims", c_int), ("C", c_int), ("R", c_int), ("n_tokens", c_int),
                ("positions", c_void_p), ("token_seq", c_void_p), ("page_table", c_void_p), ("pt_stride", c_int),
                ("page_rows", c_int), ("pool", c_void_p), ("rows", c_void_p),
                ("ring_rows", c_int), ("len_after", c_void_p), ("rot_scale", c_float), ("row_stride", c_longlong),
                ("Q", c_int), ("q_norm_w", c_void_p), ("cq_out", c_void_p), ("n_gate", c_int), ("gate_out", c_void_p)]


def latent_rows(part: torch.Tensor, norm_w: torch.Tensor, eps: float, inv_freq: Optional[torch.Tensor], rot_dims: int,
                C: int, R: int, positions: torch.Tensor, token_seq: torch.Tensor, pool: torch.Tensor,
                page_table: torch.Tensor, out_dtype: torch.dtype, ring_rows: int = 0,
                len_after: Optional[torch.Tensor] = None, rot_scale: float = 1.0,
                q_norm_w: Optional[torch.Tensor] = None, n_gate: int = 0):
    """From the down projection's partial sums ``part`` float32 [splits, T, C + R] to the cached rows: the first C
    columns RMS-normed times ``norm_w``, the last R rotated at the token's position; written to the paged ``pool``
    [pages, 1, PAGE_ROWS, C + R] and returned packed [T, C + R], both in ``out_dtype``.  ``ring_rows`` > 0: the cache
    line is a ring (row = position mod ring_rows; of a sequence with ``len_after`` tokens only the last ring_rows are
    written).  ``rot_scale``: the rotated columns come times this.  With ``q_norm_w`` (float32 [Q]) and/or ``n_gate`` the
    product carries more columns behind the C + R: Q numbers that are RMS-normed times ``q_norm_w`` (same eps) and
    ``n_gate`` numbers whose sigmoid is taken; the result is then (rows, normed [T, Q] in ``out_dtype`` or None,
    gates float32 [T, n_gate] or None)."""
    _cuda(part, norm_w, inv_freq, positions, token_seq, pool, page_table, len_after, q_norm_w)
    more = q_norm_w is not None or n_gate > 0
    Q = q_norm_w.numel() if q_norm_w is not None else 0
    if ring_rows and (len_after is None or ring_rows % PAGE_ROWS):
        raise KernelError("latent_rows: a ring needs the sequences' lengths and whole pages")
    if part.dim() == 2:
        part = part[None]
    T = part.shape[1]
    if part.dtype != torch.float32 or part.shape[2] < C + R + Q + n_gate or part.stride(2) != 1 \
            or (not more and (part.shape[2] != C + R or part.stride(1) != C + R)):
        raise KernelError(f"latent_rows: partial sums must be float32 [splits, T, {C + R + Q + n_gate}], got {tuple(part.shape)}")
    if q_norm_w is not None and (q_norm_w.dtype != torch.float32 or not q_norm_w.is_contiguous()):
        raise KernelError("latent_rows: the queries' norm weight must be contiguous float32")
    if norm_w.dtype != torch.float32 or norm_w.numel() != C or not norm_w.is_contiguous():
        raise KernelError(f"latent_rows: the norm weight must be contiguous float32 [{C}]")
    if rot_dims and (inv_freq is None or inv_freq.dtype != torch.float32 or inv_freq.numel() != rot_dims // 2):
        raise KernelError("latent_rows: inv_freq must be float32 [rot_dims / 2]")
    if pool.dtype != out_dtype or not pool.is_contiguous() or pool.shape[-1] != C + R or pool.shape[-2] != PAGE_ROWS \
            or (pool.dim() == 4 and pool.shape[1] != 1):
        raise KernelError(f"latent_rows: the pool must be contiguous {out_dtype} [pages, 1, {PAGE_ROWS}, {C + R}]")
    rows = torch.empty((T, C + R), dtype=out_dtype, device=part.device)
    a = _LatentRowsArgs()
    a.dkv = part.data_ptr(); a.splits = part.shape[0]; a.split_stride = part.stride(0)
    a.norm_w = norm_w.data_ptr(); a.eps = eps
    a.inv_freq = inv_freq.data_ptr() if rot_dims else None; a.rot_dims = rot_dims
    a.C = C; a.R = R; a.n_tokens = T
    a.positions = positions.data_ptr(); a.token_seq = token_seq.data_ptr()
    a.page_table = page_table.data_ptr(); a.pt_stride = page_table.stride(0); a.page_rows = PAGE_ROWS
    a.pool = pool.data_ptr(); a.rows = rows.data_ptr()
    a.ring_rows = ring_rows; a.len_after = len_after.data_ptr() if ring_rows else None; a.rot_scale = rot_scale
    a.row_stride = part.stride(1)
    cq = torch.empty((T, Q), dtype=out_dtype, device=part.device) if Q else None
    gates = torch.empty((T, n_gate), dtype=torch.float32, device=part.device) if n_gate else None
    a.Q = Q; a.q_norm_w = q_norm_w.data_ptr() if Q else None; a.cq_out = cq.data_ptr() if Q else None
    a.n_gate = n_gate; a.gate_out = gates.data_ptr() if n_gate else None
    lib = build.load("attention_latent")
    _check(lib, lib.tb_latent_rows(ctypes.byref(a), c_int(code(out_dtype)), _stream()), "latent_rows")
    return (rows, cq, gates) if more else rows


def head_linear(x: torch.Tensor, w: torch.Tensor, heads: int) -> torch.Tensor:
    """``y[t, h, :] = w[h] @ x[t, h, :]`` for ``x`` [T, heads * in] (rows may be a column slice) and ``w`` [heads, out, in]
    of x's dtype; returns [T, heads * out]."""
    _cuda(x, w)
    _rows_contig(x, "head_linear: x")
    if w.dim() != 3 or w.shape[0] != heads or not w.is_contiguous() or w.dtype != x.dtype or x.shape[1] != heads * w.shape[2]:
        raise KernelError(f"head_linear: x {tuple(x.shape)} {x.dtype} and w {tuple(w.shape)} {w.dtype} do not fit {heads} heads")
    T, out_dim, in_dim = x.shape[0], w.shape[1], w.shape[2]
    y = torch.empty((T, heads * out_dim), dtype=x.dtype, device=x.device)
    lib = build.load("attention_latent")
    _check(lib, lib.tb_head_linear(_ptr(x), c_longlong(x.stride(0)), _ptr(w), _ptr(y), c_longlong(y.stride(0)),
                                   c_int(code(x.dtype)), c_int(T), c_int(heads), c_int(in_dim), c_int(out_dim), _stream()),
           "head_linear")
    return y


class _LatentDecodeArgs(ctypes.Structure):
    _fields_ = [("q", c_void_p), ("q_stride", c_longlong), ("pool", c_void_p), ("page_table", c_void_p), ("pt_stride", c_int),
                ("page_rows", c_int), ("len_after", c_void_p), ("sink", c_void_p), ("out", c_void_p), ("out_stride", c_longlong),
                ("partial", c_void_p), ("heads", c_int), ("C", c_int), ("R", c_int), ("out_dim", c_int), ("n_splits", c_int),
                ("scale", c_float), ("window", c_int), ("ring_rows", c_int)]


def latent_decode(q: torch.Tensor, pool: torch.Tensor, page_table: torch.Tensor, len_after: torch.Tensor,
                  sink: Optional[torch.Tensor], heads: int, C: int, R: int, scale: float, len_bucket: int,
                  window: int = 0, ring_rows: int = 0) -> torch.Tensor:
    """One mapped query [heads * (C + R)] per sequence against its cached rows; returns [batch, heads * C] (the weighted
    sums of the rows' first C columns).  ``len_bucket``: an upper bound of the longest context, which the number of
    pieces a sequence is cut into depends on (and nothing else does, so that a captured step stays valid).
    ``window`` W > 0: only the last W rows are seen; ``ring_rows`` > 0: the line is a ring of that many rows."""
    _cuda(q, pool, page_table, len_after, sink)
    if ring_rows and (not 0 < window <= ring_rows or ring_rows % PAGE_ROWS):
        raise KernelError(f"latent_decode: a ring of {ring_rows} rows cannot hold a window of {window}")
    if window:
        len_bucket = min(len_bucket, window + 31)
    _rows_contig(q, "latent_decode: q")
    B = q.shape[0]
    if q.shape[1] != heads * (C + R) or pool.dtype != q.dtype:
        raise KernelError(f"latent_decode: q {tuple(q.shape)} does not fit {heads} heads of {C + R}")
    if sink is not None and (sink.dtype != torch.float32 or sink.numel() != heads or not sink.is_contiguous()):
        raise KernelError(f"latent_decode: the sink must be contiguous float32 [{heads}]")
    lib = build.load("attention_latent")
    mma = q.dtype == torch.bfloat16 and bool(lib.tb_latent_decode_mma_takes(c_int(C), c_int(R))) and q.stride(0) % 8 == 0 \
        and q.data_ptr() % 16 == 0
    # pieces: enough CTAs for about two per SM, none shorter than 128 keys (256 on the generic kernel)
    units = B * ((heads + 31) // 32 if heads > 16 else 1) if mma else B * heads          # the tensor-core kernel: up to 32 heads a CTA
    shortest = 128 if mma else 256
    pieces = max(1, min((len_bucket + shortest - 1) // shortest, max(1, (2 * sm_count(q.device)) // max(1, units))))
    out = torch.empty((B, heads * C), dtype=q.dtype, device=q.device)
    scratch = torch.empty(B * heads * pieces * (C + 2), dtype=torch.float32, device=q.device) if (pieces > 1 or mma) else None
    a = _LatentDecodeArgs()
    a.q = q.data_ptr(); a.q_stride = q.stride(0); a.pool = pool.data_ptr()
    a.page_table = page_table.data_ptr(); a.pt_stride = page_table.stride(0); a.page_rows = PAGE_ROWS
    a.len_after = len_after.data_ptr(); a.sink = sink.data_ptr() if sink is not None else None
    a.out = out.data_ptr(); a.out_stride = out.stride(0); a.partial = scratch.data_ptr() if scratch is not None else None
    a.heads = heads; a.C = C; a.R = R; a.out_dim = C; a.n_splits = pieces; a.scale = scale
    a.window = window or 0; a.ring_rows = ring_rows
    if mma:
        _check(lib, lib.tb_latent_decode_mma(ctypes.byref(a), c_int(B), _stream()), "latent_decode_mma", 2)
    else:
        _check(lib, lib.tb_latent_decode(ctypes.byref(a), c_int(code(q.dtype)), c_int(B), _stream()), "latent_decode",
               2 if pieces > 1 else 1)
    return out


def attn_prefill_sink(q, k, v, seq_start, token_seq, n_heads, head_dim, scale, sink, max_seq_len, seq_lens=None,
                      window: int = 0) -> torch.Tensor:
    """Causal prefill attention of packed sequences, one kv head per query head, whose softmax denominators also
    hold ``exp(sink[h])`` (``sink`` float32 [n_heads], or None).  bfloat16 runs on the tcgen05 kernel (head sizes 64, 128,
    256, with the sequences' lengths on the host in ``seq_lens``) or the mma.sync kernel (other multiples of 16),
    everything else on the generic kernel."""
    _cuda(q, k, v, seq_start, token_seq, sink)
    for name, t in (("q", q), ("k", k), ("v", v)):
        _rows_contig(t, "attention: " + name)
    if k.stride(0) != v.stride(0) or k.dtype != q.dtype or v.dtype != q.dtype:
        raise KernelError("attention: k and v must share row stride and dtype with q")
    if sink is not None and (sink.dtype != torch.float32 or sink.numel() != n_heads or not sink.is_contiguous()):
        raise KernelError(f"attention: the sink must be contiguous float32 [{n_heads}]")
    T = q.shape[0]
    out = torch.empty((T, n_heads * head_dim), dtype=q.dtype, device=q.device)
    aligned = all(t.data_ptr() % 16 == 0 and t.stride(0) % 8 == 0 for t in (q, k, v))
    if attn_prefill_tc_takes(q.dtype, head_dim) and aligned and seq_lens is not None:
        lib = build.load(attn_prefill_tc_lib(head_dim))
        B = len(seq_lens)
        _check(lib, lib.tb_attn_prefill_tc_ex(_ptr(q), _ptr(k), _ptr(v), c_longlong(q.stride(0)), c_longlong(k.stride(0)),
                                              _ptr(seq_start), _ptr(out), c_int(T), c_int(B), c_int(max(seq_lens)),
                                              c_int(n_heads), c_int(n_heads), c_int(head_dim), c_float(scale), c_float(0.0),
                                              c_int(window or 0), _ptr(sink), _stream()), "attn_prefill_tc", 2)
        return out
    if attn_prefill_takes(q.dtype, head_dim) and aligned:
        lib = build.load(attn_prefill_lib(head_dim))
        B = seq_start.numel() - 1
        _check(lib, lib.tb_attn_prefill_mma_ex(_ptr(q), _ptr(k), _ptr(v), c_longlong(q.stride(0)), c_longlong(k.stride(0)),
                                               _ptr(seq_start), _ptr(out), c_int(B), c_int(max_seq_len), c_int(n_heads),
                                               c_int(n_heads), c_int(head_dim), c_float(scale), c_float(0.0), c_int(window or 0),
                                               _ptr(sink), _stream()), "attn_prefill_mma")
        return out
    lib = build.load("attention_simt")
    _check(lib, lib.tb_attn_prefill_simt_ex(_ptr(q), _ptr(k), _ptr(v), c_longlong(q.stride(0)), c_longlong(k.stride(0)),
                                            _ptr(seq_start), _ptr(token_seq), _ptr(out), c_int(code(q.dtype)), c_int(T),
                                            c_int(n_heads), c_int(n_heads), c_int(head_dim), c_float(scale), c_float(0.0),
                                            c_int(window or 0), _ptr(sink), _stream()), "attn_prefill_simt")
    return out


# ---------------------------------------------------------------------------
# Attention whose heads' scores are mixed before the softmax
# ---------------------------------------------------------------------------
class _MixedAttnArgs(ctypes.Structure):
    _fields_ = [("q", c_void_p), ("q_stride", c_longlong), ("k", c_void_p), ("v", c_void_p), ("kv_stride", c_longlong),
                ("seq_start", c_void_p), ("token_seq", c_void_p), ("page_table", c_void_p), ("pt_stride", c_int),
                ("page_rows", c_int), ("ring_rows", c_int), ("len_after", c_void_p), ("out", c_void_p),
                ("out_stride", c_longlong), ("mix", c_void_p), ("partial", c_void_p), ("H", c_int), ("G", c_int), ("D", c_int),
                ("n_tokens", c_int), ("window", c_int), ("unit_sink", c_int), ("n_pieces", c_int), ("batch", c_int),
                ("max_seq_len", c_int), ("stages", c_int)]


def attn_mixed_padded_head(dtype: torch.dtype, n_heads: int, n: int) -> int:
    """The head size at which a mixer whose scores are mixed across heads stores keys and values of up to ``n`` numbers
    a head: in bfloat16 with up to 32 heads the next of 32, 64, 96, 128 (what the tensor-core form of its prefill
    kernel takes), else the next multiple of 8 (the generic kernels take any size; rows of whole 16-byte pieces)."""
    if dtype == torch.bfloat16 and n_heads <= 32 and n <= 128:
        return (n + 31) // 32 * 32
    return (n + 7) // 8 * 8


def _mixed_args(q, n_heads, n_kv_heads, head_dim, mix, window, unit_sink):
    _rows_contig(q, "attn_mixed: q")
    if q.shape[1] != n_heads * head_dim:
        raise KernelError(f"attn_mixed: q {tuple(q.shape)} does not hold {n_heads} heads of {head_dim}")
    if mix.dtype != torch.float32 or tuple(mix.shape) != (n_heads, n_heads) or not mix.is_contiguous():
        raise KernelError(f"attn_mixed: the mixing matrix must be contiguous float32 [{n_heads}, {n_heads}]")
    out = torch.empty((q.shape[0], n_heads * head_dim), dtype=q.dtype, device=q.device)
    a = _MixedAttnArgs()
    a.q = q.data_ptr(); a.q_stride = q.stride(0); a.out = out.data_ptr(); a.out_stride = out.stride(0)
    a.mix = mix.data_ptr(); a.H = n_heads; a.G = n_kv_heads; a.D = head_dim; a.n_tokens = q.shape[0]
    a.window = window or 0; a.unit_sink = int(bool(unit_sink)); a.n_pieces = 1; a.page_rows = PAGE_ROWS
    return a, out


def attn_mixed_prefill(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, seq_start: torch.Tensor, token_seq: torch.Tensor,
                       n_heads: int, n_kv_heads: int, head_dim: int, mix: torch.Tensor, window: int,
                       unit_sink: bool, max_seq_len: int = 0) -> torch.Tensor:
    """Causal attention of packed sequences whose scores are mixed across heads before the softmax:
    ``s_h = sum_g mix[h, g] (q_g . k)`` (``mix`` float32 [H, H]; the caller folds the scale in).  ``window`` W > 0: the
    last W positions are seen; -C: the positions of the query's own block of C, blocks counted from position 0; 0: all
    earlier ones.  ``unit_sink``: the softmax denominator also holds exp(0).  ``max_seq_len``: the longest sequence
    of the step; with it the tensor-core form runs where it takes the shapes (it sizes that form's grid)."""
    _cuda(q, k, v, seq_start, token_seq, mix)
    for name, t in (("k", k), ("v", v)):
        _rows_contig(t, "attn_mixed: " + name)
    if k.stride(0) != v.stride(0) or k.dtype != q.dtype or v.dtype != q.dtype or k.shape[1] != n_kv_heads * head_dim:
        raise KernelError("attn_mixed: k and v must share row stride and dtype with q and hold the kv heads")
    a, out = _mixed_args(q, n_heads, n_kv_heads, head_dim, mix, window, unit_sink)
    a.k = k.data_ptr(); a.v = v.data_ptr(); a.kv_stride = k.stride(0)
    a.seq_start = seq_start.data_ptr(); a.token_seq = token_seq.data_ptr()
    a.batch = seq_start.numel() - 1; a.max_seq_len = int(max_seq_len)
    lib = build.load("attention_mixed")
    pieces, scratch = 1, None
    if max_seq_len and lib.tb_attn_mixed_prefill_mma_takes(c_int(code(q.dtype)), c_int(n_heads), c_int(n_kv_heads), c_int(head_dim)):
        # the tensor-core form takes 16 queries of all heads a CTA: a short step's tiles are fewer than the SMs, so the keys of a
        # tile are cut into pieces (CTAs of their own, folded afterwards) while that fills the GPU and a piece keeps 4 rounds
        ctas = (int(max_seq_len) + 15) // 16 * a.batch * ((n_heads + 15) // 16)
        reach = min(int(max_seq_len), abs(window)) if window else int(max_seq_len)
        pieces = max(1, min(4, (2 * sm_count(q.device)) // max(1, ctas), reach // 128))
        if pieces > 1:
            scratch = torch.empty(q.shape[0] * n_heads * pieces * (head_dim + 2), dtype=torch.float32, device=q.device)
            a.partial = scratch.data_ptr()
    a.n_pieces = pieces
    _check(lib, lib.tb_attn_mixed_prefill(ctypes.byref(a), c_int(code(q.dtype)), _stream()), "attn_mixed_prefill",
           2 if pieces > 1 else 1)
    return out


def attn_mixed_decode(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, page_table: torch.Tensor,
                      len_after: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int, mix: torch.Tensor, window: int,
                      unit_sink: bool, ring_rows: int, len_bucket: int) -> torch.Tensor:
    """One query per sequence against the paged cache, scores mixed across heads (see :func:`attn_mixed_prefill`).
    ``len_bucket``: an upper bound of the longest context, which the number of pieces depends on (and nothing else)."""
    _cuda(q, k_pool, v_pool, page_table, len_after, mix)
    for p in (k_pool, v_pool):
        if p.dtype != q.dtype or not p.is_contiguous() or tuple(p.shape[1:]) != (n_kv_heads, PAGE_ROWS, head_dim):
            raise KernelError("attn_mixed: cache pools must be contiguous [pages, n_kv_heads, PAGE_ROWS, head_dim] of q's dtype")
    a, out = _mixed_args(q, n_heads, n_kv_heads, head_dim, mix, window, unit_sink)
    B = q.shape[0]
    reach = min(len_bucket, abs(window)) if window else len_bucket
    pieces = max(1, min((reach + 255) // 256, max(1, (2 * sm_count(q.device)) // max(1, B))))
    scratch = torch.empty(B * n_heads * pieces * (head_dim + 2), dtype=torch.float32, device=q.device) if pieces > 1 else None
    a.k = k_pool.data_ptr(); a.v = v_pool.data_ptr(); a.page_table = page_table.data_ptr(); a.pt_stride = page_table.stride(0)
    a.ring_rows = ring_rows; a.len_after = len_after.data_ptr(); a.n_pieces = pieces
    a.partial = scratch.data_ptr() if scratch is not None else None
    lib = build.load("attention_mixed")
    _check(lib, lib.tb_attn_mixed_decode(ctypes.byref(a), c_int(code(q.dtype)), _stream()), "attn_mixed_decode",
           2 if pieces > 1 else 1)
    return out


# ---------------------------------------------------------------------------
# Experts behind a router
# ---------------------------------------------------------------------------
class _MoeRouteArgs(ctypes.Structure):
    _fields_ = [("logits", c_void_p), ("splits", c_int), ("split_stride", c_longlong), ("row_stride", c_longlong),
                ("correction", c_void_p), ("has_gate", c_int), ("idx", c_void_p), ("weight", c_void_p), ("gate", c_void_p),
                ("n_tokens", c_int), ("W", c_int), ("E", c_int), ("top", c_int), ("groups", c_int), ("keep", c_int),
                ("group_top", c_int), ("weight_eps", c_float), ("softmax", c_int), ("out_scale", c_float), ("bias", c_void_p)]


def moe_route(logits: torch.Tensor, experts: int, correction: Optional[torch.Tensor], has_gate: bool,
              top: int, groups: int, keep: int, group_top: int, weight_eps: float, score: str = "sigmoid",
              out_scale: float = 1.0, bias: Optional[torch.Tensor] = None):
    """Routing with groups (see moe.cu; ``score`` "sigmoid" or "softmax" over all experts; the weights come times
    ``out_scale``) from the router's logits: float32 [T, >= experts (+ 1)] or
    partial sums [splits, T, ...] of the router product (column ``experts`` is the shared expert's gate product if
    ``has_gate``).  ``bias``: float32 [experts] added to the logits themselves (``correction`` only steers the choice).
    Returns (chosen experts int32 [T, top], their weights float32 [T, top], the shared expert's gate
    float32 [T] or None)."""
    _cuda(logits, correction, bias)
    if logits.dim() == 2:
        logits = logits[None]
    E = experts
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() < E or not bias.is_contiguous()):
        raise KernelError(f"moe_route: the bias must be contiguous float32 [>= {E}]")
    T = logits.shape[1]
    if logits.dtype != torch.float32 or logits.stride(2) != 1 or logits.shape[2] < E + int(has_gate):
        raise KernelError(f"moe_route: logits must be float32 [splits, T, >= {E + int(has_gate)}], got {tuple(logits.shape)} {logits.dtype}")
    if correction is not None and (correction.dtype != torch.float32 or correction.numel() != E or not correction.is_contiguous()):
        raise KernelError(f"moe_route: the correction must be contiguous float32 [{E}]")
    idx = torch.empty((T, top), dtype=torch.int32, device=logits.device)
    weight = torch.empty((T, top), dtype=torch.float32, device=logits.device)
    gate = torch.empty((T,), dtype=torch.float32, device=logits.device) if has_gate else None
    a = _MoeRouteArgs()
    a.logits = logits.data_ptr(); a.splits = logits.shape[0]; a.split_stride = logits.stride(0); a.row_stride = logits.stride(1)
    a.correction = correction.data_ptr() if correction is not None else None
    a.has_gate = int(has_gate)
    a.idx = idx.data_ptr(); a.weight = weight.data_ptr(); a.gate = gate.data_ptr() if gate is not None else None
    a.n_tokens = T; a.W = 0; a.E = E; a.top = top; a.groups = groups; a.keep = keep; a.group_top = group_top
    a.weight_eps = weight_eps
    if score not in ("sigmoid", "softmax"):
        raise KernelError(f"moe_route: scores are 'sigmoid' or 'softmax', not '{score}'")
    a.softmax = int(score == "softmax"); a.out_scale = out_scale
    a.bias = bias.data_ptr() if bias is not None else None
    lib = build.load("moe")
    _check(lib, lib.tb_moe_route(ctypes.byref(a), _stream()), "moe_route")
    return idx, weight, gate


MOE_GROUPED_FROM = 128      # (token, expert) pairs from which the experts' products run grouped on the tensor cores
MOE_TCGEN05_FROM = 1024     # ... and from which the grouped products are the tcgen05 kernel's (tiles of 128 rows per expert)


class _MoePadArgs(ctypes.Structure):
    _fields_ = [("idx", c_void_p), ("pos", c_void_p), ("row_pair", c_void_p), ("tile_group", c_void_p),
                ("P", c_int), ("E", c_int), ("max_rows", c_int)]


def _moe_grouped_tc(x, gate_up_w, down_w, idx, weight, shared, gate, out, ungated=False):
    """The experts' products on the tcgen05 kernel: the pairs ordered by expert, each expert's stretch padded to whole
    tiles of 128 rows (see moe.cu and gemm_tc.cu's grouped mode).  Shapes depend on the sizes only.  ``ungated``:
    ``gate_up_w`` holds the up rows alone and the first product's epilogue is relu(u)^2."""
    T, W = x.shape
    E, ff2 = gate_up_w.shape[0], gate_up_w.shape[1]
    ff = ff2 if ungated else ff2 // 2
    top = idx.shape[1]
    P = T * top
    max_rows = ((P + 127) // 128 + min(E, P)) * 128
    ints = torch.empty(P + max_rows + max_rows // 128, dtype=torch.int32, device=x.device)
    pos, row_pair, tile_group = ints[:P], ints[P:P + max_rows], ints[P + max_rows:]
    lib = build.load("moe")
    g = _MoePadArgs()
    g.idx = idx.data_ptr(); g.pos = pos.data_ptr(); g.row_pair = row_pair.data_ptr(); g.tile_group = tile_group.data_ptr()
    g.P = P; g.E = E; g.max_rows = max_rows
    _check(lib, lib.tb_moe_group_padded(ctypes.byref(g), _stream()), "moe_group_padded")
    xs = torch.empty((max_rows, W), dtype=x.dtype, device=x.device)
    _check(lib, lib.tb_moe_gather_rows(_ptr(x), c_longlong(x.stride(0)), _ptr(row_pair), _ptr(xs), c_int(max_rows), c_int(W),
                                       c_int(top), _stream()), "moe_gather_rows")
    act = torch.empty((max_rows, ff), dtype=x.dtype, device=x.device)
    y = torch.empty((max_rows, W), dtype=torch.float32, device=x.device)
    gl = build.load("gemm_tc")
    if ungated:
        _check(gl, gl.tb_gemm_tc_grouped_unary(_ptr(xs), _ptr(gate_up_w), _ptr(act), c_int(code(x.dtype)), c_int(max_rows), c_int(ff),
                                               c_int(E), c_int(W), c_longlong(W), c_longlong(W), c_longlong(ff), _ptr(tile_group),
                                               c_int(1), _stream()), "gemm_tc_grouped")
    else:
        _check(gl, gl.tb_gemm_tc_grouped(_ptr(xs), _ptr(gate_up_w), _ptr(act), c_int(code(x.dtype)), c_int(max_rows), c_int(ff2),
                                         c_int(E), c_int(W), c_longlong(W), c_longlong(W), c_longlong(ff), _ptr(tile_group),
                                         c_int(ACTIVATIONS["silu"]), _stream()), "gemm_tc_grouped")
    _check(gl, gl.tb_gemm_tc_grouped(_ptr(act), _ptr(down_w), _ptr(y), c_int(code(torch.float32)), c_int(max_rows), c_int(W),
                                     c_int(E), c_int(ff), c_longlong(ff), c_longlong(ff), c_longlong(W), _ptr(tile_group),
                                     c_int(-1), _stream()), "gemm_tc_grouped")
    _check(lib, lib.tb_moe_combine_sorted(_ptr(y), _ptr(pos), _ptr(weight), _ptr(shared),
                                          c_int(shared.shape[0] if shared is not None else 0),
                                          c_longlong(shared.stride(0) if shared is not None else 0), _ptr(gate), _ptr(out),
                                          c_int(T), c_int(W), c_int(top), _stream()), "moe_combine_sorted")
    return out


class _MoeGroupArgs(ctypes.Structure):
    _fields_ = [("idx", c_void_p), ("perm", c_void_p), ("tile_expert", c_void_p), ("tile_row0", c_void_p),
                ("tile_rows", c_void_p), ("n_tiles", c_void_p), ("P", c_int), ("E", c_int), ("max_tiles", c_int)]


class _MoeGroupedArgs(ctypes.Structure):
    _fields_ = [("x", c_void_p), ("x_stride", c_longlong), ("gate_w", c_void_p), ("up_w", c_void_p), ("down_w", c_void_p),
                ("perm", c_void_p), ("tile_expert", c_void_p), ("tile_row0", c_void_p), ("tile_rows", c_void_p),
                ("n_tiles", c_void_p), ("weight", c_void_p), ("act", c_void_p), ("pair_out", c_void_p),
                ("W", c_int), ("ff", c_int), ("top", c_int)]


def _moe_grouped(x, gate_w, up_w, down_w, idx, weight, shared, gate, out):
    """The experts' products with the pairs grouped by expert (bfloat16, tensor cores; see moe.cu).  The grid holds the
    most tiles there can be, so nothing the host does depends on which experts were chosen."""
    T, W = x.shape
    E, ff = up_w.shape[0], up_w.shape[1]
    top = idx.shape[1]
    P = T * top
    max_tiles = (P + 127) // 128 + min(E, P)          # tiles of 128 pairs; every expert may end with one that is not full
    ints = torch.empty(P + 3 * max_tiles + 1, dtype=torch.int32, device=x.device)
    perm, te, tr0, trn, nt = (ints[:P], ints[P:P + max_tiles], ints[P + max_tiles:P + 2 * max_tiles],
                              ints[P + 2 * max_tiles:P + 3 * max_tiles], ints[P + 3 * max_tiles:])
    act = torch.empty((P, ff), dtype=x.dtype, device=x.device)
    pair_out = torch.empty((P, W), dtype=torch.float32, device=x.device)
    g = _MoeGroupArgs()
    g.idx = idx.data_ptr(); g.perm = perm.data_ptr(); g.tile_expert = te.data_ptr(); g.tile_row0 = tr0.data_ptr()
    g.tile_rows = trn.data_ptr(); g.n_tiles = nt.data_ptr(); g.P = P; g.E = E; g.max_tiles = max_tiles
    lib = build.load("moe")
    _check(lib, lib.tb_moe_group(ctypes.byref(g), _stream()), "moe_group")
    a = _MoeGroupedArgs()
    a.x = x.data_ptr(); a.x_stride = x.stride(0)
    a.gate_w = gate_w.data_ptr() if gate_w is not None else None; a.up_w = up_w.data_ptr(); a.down_w = down_w.data_ptr()
    a.perm = perm.data_ptr(); a.tile_expert = te.data_ptr(); a.tile_row0 = tr0.data_ptr(); a.tile_rows = trn.data_ptr()
    a.n_tiles = nt.data_ptr(); a.weight = weight.data_ptr(); a.act = act.data_ptr(); a.pair_out = pair_out.data_ptr()
    a.W = W; a.ff = ff; a.top = top
    _check(lib, lib.tb_moe_grouped(ctypes.byref(a), _ptr(shared), c_int(shared.shape[0] if shared is not None else 0),
                                   c_longlong(shared.stride(0) if shared is not None else 0), _ptr(gate), _ptr(out), c_int(T),
                                   c_int(max_tiles), _stream()), "moe_grouped", 3)
    return out


class _MoeExpertArgs(ctypes.Structure):
    _fields_ = [("x", c_void_p), ("x_stride", c_longlong), ("gate_w", c_void_p), ("up_w", c_void_p), ("down_w", c_void_p),
                ("idx", c_void_p), ("weight", c_void_p), ("act", c_void_p), ("shared", c_void_p), ("shared_splits", c_int),
                ("shared_split_stride", c_longlong), ("gate", c_void_p), ("out", c_void_p),
                ("n_tokens", c_int), ("W", c_int), ("ff", c_int), ("top", c_int), ("ungated", c_int)]


def moe_experts(x: torch.Tensor, gate_w: Optional[torch.Tensor], up_w: torch.Tensor, down_w: torch.Tensor, idx: torch.Tensor,
                weight: torch.Tensor, shared: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None,
                gate_up_w: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The weighted sum of every token's chosen experts ``down_e(silu(gate_e x) * up_e x)`` plus ``gate[t] * shared[t]``
    (``shared`` float32 partial sums [splits, T, W]); returns float32 [T, W].  Expert matrices: ``gate_w``, ``up_w``
    [E, ff, W] and ``down_w`` [E, W, ff] of x's dtype; ``gate_up_w`` [E, 2 ff, W]: every expert's gate and up rows
    interleaved (``interleave_gate_up``), which lets many tokens run on the tcgen05 product.  ``gate_w`` None: the
    experts have no gate matrix and are ``down_e(relu(up_e x)^2)``."""
    _cuda(x, gate_w, up_w, down_w, idx, weight, shared, gate, gate_up_w)
    _rows_contig(x, "moe: x")
    T, W = x.shape
    E, ff = up_w.shape[0], up_w.shape[1]
    top = idx.shape[1]
    ungated = gate_w is None
    for name, t, shape in (("gate", gate_w, (E, ff, W)), ("up", up_w, (E, ff, W)), ("down", down_w, (E, W, ff))):
        if t is None:
            continue
        if tuple(t.shape) != shape or t.dtype != x.dtype or not t.is_contiguous():
            raise KernelError(f"moe: the experts' {name} matrices must be contiguous {x.dtype} {shape}, got {tuple(t.shape)} {t.dtype}")
    if shared is not None:
        if shared.dim() == 2:
            shared = shared[None]
        if shared.dtype != torch.float32 or tuple(shared.shape[1:]) != (T, W) or shared.stride(2) != 1 or shared.stride(1) != W \
                or gate is None:
            raise KernelError("moe: the shared expert's output must be float32 [splits, T, W] and come with its gate")
    out = torch.empty((T, W), dtype=torch.float32, device=x.device)
    if x.dtype == torch.bfloat16 and T * top >= MOE_GROUPED_FROM and W % 8 == 0 and ff % 8 == 0 and x.stride(0) % 8 == 0 \
            and x.data_ptr() % 16 == 0:
        if ungated and T * top >= MOE_TCGEN05_FROM:
            return _moe_grouped_tc(x, up_w, down_w, idx, weight, shared, gate, out, ungated=True)
        if gate_up_w is not None and T * top >= MOE_TCGEN05_FROM and ff % 16 == 0:
            return _moe_grouped_tc(x, gate_up_w, down_w, idx, weight, shared, gate, out)
        return _moe_grouped(x, gate_w, up_w, down_w, idx, weight, shared, gate, out)
    act = torch.empty((T * top, ff), dtype=x.dtype, device=x.device)
    a = _MoeExpertArgs()
    a.x = x.data_ptr(); a.x_stride = x.stride(0)
    a.gate_w = gate_w.data_ptr() if gate_w is not None else None; a.up_w = up_w.data_ptr(); a.down_w = down_w.data_ptr()
    a.ungated = int(ungated)
    a.idx = idx.data_ptr(); a.weight = weight.data_ptr(); a.act = act.data_ptr()
    a.shared = shared.data_ptr() if shared is not None else None
    a.shared_splits = shared.shape[0] if shared is not None else 0
    a.shared_split_stride = shared.stride(0) if shared is not None else 0
    a.gate = gate.data_ptr() if gate is not None else None
    a.out = out.data_ptr(); a.n_tokens = T; a.W = W; a.ff = ff; a.top = top
    lib = build.load("moe")
    _check(lib, lib.tb_moe_gate_up(ctypes.byref(a), c_int(code(x.dtype)), _stream()), "moe_gate_up")
    _check(lib, lib.tb_moe_down(ctypes.byref(a), c_int(code(x.dtype)), _stream()), "moe_down")
    return out
