"""Python faces of csrc/headops.cu (norm, rotation and cache append of packed heads; pooled blocks; the difference of two
score maps) and csrc/streamops.cu (gated joins of the residual stream, the mean of normed branches, a scale)."""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional, Sequence

import torch

from ..csrc.build import load_module
from .ops import DT, KernelError, _check, _dt, _fn, _need_cuda, _ptr, _stream


class _HeadPrepParams(ctypes.Structure):
    _fields_ = [("proj", c_void_p), ("row_stride", c_int), ("n_q", c_int), ("n_k", c_int), ("d", c_int), ("kv_heads", c_int),
                ("dv", c_int), ("q_weight", c_void_p), ("k_weight", c_void_p), ("eps", c_float), ("rot", c_int), ("layout", c_int),
                ("cos_t", c_void_p), ("sin_t", c_void_p), ("table_rows", c_int), ("tok_pos", c_void_p), ("append", c_int),
                ("tok_seq", c_void_p), ("seq_start", c_void_p), ("seq_len_before", c_void_p), ("kpool", c_void_p),
                ("vpool", c_void_p), ("page_table", c_void_p), ("table_stride", c_int), ("ring", c_int), ("pinned", c_int),
                ("err", c_void_p)]


PAIR_LAYOUTS = {"halves": 0, "neighbours": 1}


def head_prep(proj: torch.Tensor, n_q: int, n_k: int, d: int, *, kv_heads: int = 0, dv: int = 0, q_weight=None, k_weight=None,
              eps: float = 0.0, tables=None, layout: str = "halves", tok_pos=None, append=None, err=None) -> None:
    """In place on packed projections [T, n_q d (+ n_k d + kv_heads dv)]: every query row and key row of d elements is
    RMS-normed over the row with q_weight / k_weight (float32 [d]; None: no norm) and its first `dims` elements are
    rotated by the token's position, tables = (cos, sin, dims) with float32 tables [rows, dims / 2]; layout "halves" pairs
    element i with i + dims / 2, "neighbours" 2i with 2i + 1.  Float32 arithmetic, one rounding.  With `append` the n_k
    key rows (kv_heads cache rows of n_k / kv_heads keys side by side) and the kv_heads value rows go to the token's place
    in the paged cache.  append = dict(tok_seq, seq_start, seq_len_before, kpool, vpool, page_table, ring, pinned)."""
    _need_cuda(proj, tok_pos, q_weight, k_weight)
    T = proj.shape[0]
    if tok_pos is None or tok_pos.numel() != T or err is None:
        raise KernelError("head_prep needs tok_pos (one position per packed token) and an error word")
    assert proj.stride(1) == 1
    for w in (q_weight, k_weight):
        assert w is None or (w.dtype == torch.float32 and w.numel() == d and w.is_contiguous())
    p = _HeadPrepParams()
    p.proj, p.row_stride, p.n_q, p.n_k, p.d, p.kv_heads, p.dv = proj.data_ptr(), proj.stride(0), n_q, n_k, d, kv_heads, dv
    p.q_weight, p.k_weight, p.eps = _ptr(q_weight), _ptr(k_weight), eps
    if tables is not None:
        cos, sin, dims = tables
        assert cos.dtype == sin.dtype == torch.float32 and cos.shape[1] == dims // 2 and cos.is_contiguous() and sin.is_contiguous()
        p.rot, p.layout, p.cos_t, p.sin_t, p.table_rows = dims, PAIR_LAYOUTS[layout], cos.data_ptr(), sin.data_ptr(), cos.shape[0]
    p.tok_pos, p.err = tok_pos.data_ptr(), err.data_ptr()
    if append is not None:
        a = append
        assert a["kpool"].dtype == proj.dtype and kv_heads > 0 and n_k % kv_heads == 0
        p.append = 1
        p.tok_seq, p.seq_start, p.seq_len_before = a["tok_seq"].data_ptr(), a["seq_start"].data_ptr(), a["seq_len_before"].data_ptr()
        p.kpool, p.vpool, p.page_table = a["kpool"].data_ptr(), a["vpool"].data_ptr(), a["page_table"].data_ptr()
        p.table_stride, p.ring, p.pinned = a["page_table"].shape[1], a["ring"], a.get("pinned", 0)
    f = _fn(load_module("headops.cu"), "llb_head_prep", [_HeadPrepParams, c_int, c_int, c_void_p])
    _check(f(p, _dt(proj), T, _stream()), "norm, rotation and cache append of heads")


class _PoolAppendParams(ctypes.Structure):
    _fields_ = [("k_new", c_void_p), ("v_new", c_void_p), ("row_stride", c_int), ("kv_heads", c_int), ("dk", c_int), ("dv", c_int),
                ("pool", c_int), ("kpool", c_void_p), ("vpool", c_void_p), ("page_table", c_void_p), ("table_stride", c_int),
                ("ring", c_int), ("pinned", c_int), ("pk", c_void_p), ("pv", c_void_p), ("ptable", c_void_p),
                ("ptable_stride", c_int), ("seq_start", c_void_p), ("seq_len_before", c_void_p)]


def pool_append(proj: torch.Tensor, key_col: int, kv_heads: int, dk: int, dv: int, pool: int, kv, blocks, seq_start, seq_len_before,
                n_seqs: int, max_new: int) -> None:
    """For every block of `pool` consecutive positions that this step completes, the mean of its keys and the mean of its
    values (float32 sums) go to row `block` of the cache view `blocks`.  The step's own keys (as the cache will hold them)
    and values stand in proj [T, ...] from column key_col on: kv_heads key rows of dk, then kv_heads value rows of dv;
    earlier positions are read from the token cache view `kv`."""
    _need_cuda(proj)
    assert proj.dtype == kv.k.dtype == blocks.k.dtype
    es = proj.element_size()
    p = _PoolAppendParams()
    p.k_new, p.v_new, p.row_stride = proj.data_ptr() + key_col * es, proj.data_ptr() + (key_col + kv_heads * dk) * es, proj.stride(0)
    p.kv_heads, p.dk, p.dv, p.pool = kv_heads, dk, dv, pool
    p.kpool, p.vpool, p.page_table = kv.k.data_ptr(), kv.v.data_ptr(), kv.page_table.data_ptr()
    p.table_stride, p.ring, p.pinned = kv.page_table.shape[1], kv.ring, kv.pinned
    p.pk, p.pv, p.ptable, p.ptable_stride = blocks.k.data_ptr(), blocks.v.data_ptr(), blocks.page_table.data_ptr(), blocks.page_table.shape[1]
    p.seq_start, p.seq_len_before = seq_start.data_ptr(), seq_len_before.data_ptr()
    f = _fn(load_module("headops.cu"), "llb_pool_append", [_PoolAppendParams, c_int, c_int, c_int, c_void_p])
    _check(f(p, _dt(proj), n_seqs, max_new, _stream()), "pooled blocks of keys and values")


def diff_combine(a: torch.Tensor, H: int, group: int, dv: int, lam: float, eps: float, mult: float, out_dtype: torch.dtype) -> torch.Tensor:
    """a [T, 2 H dv] float32: for every group of `group` query heads first their results under score map 1, then under
    map 2.  Returns [T, H dv]: (a1 - lam a2) divided by its root mean square over the head's dv elements, times mult."""
    _need_cuda(a)
    T = a.shape[0]
    assert a.dtype == torch.float32 and a.is_contiguous() and a.shape[1] == 2 * H * dv
    out = torch.empty((T, H * dv), dtype=out_dtype, device=a.device)
    f = _fn(load_module("headops.cu"), "llb_diff_combine", [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_float,
                                                            c_float, c_void_p])
    _check(f(_ptr(a), _ptr(out), DT[out_dtype], T, H, group, dv, lam, eps, mult, _stream()), "difference of two score maps")
    return out


class _StreamJoinParams(ctypes.Structure):
    _fields_ = [("x", c_void_p), ("delta", c_void_p), ("gate", c_void_p), ("ld_gate", c_int), ("rows_add", c_void_p),
                ("vec_add", c_void_p), ("weight", c_void_p), ("out", c_void_p), ("H", c_int), ("eps", c_float)]


def stream_join(x: torch.Tensor, delta: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None, *,
                rows_add: Optional[torch.Tensor] = None, vec_add: Optional[torch.Tensor] = None,
                weight: Optional[torch.Tensor] = None, eps: float = 0.0, out_dtype: Optional[torch.dtype] = None):
    """One pass over the rows of the float32 stream x [T, H]:  x += sigmoid(gate) * delta (gate: float32 logits [T, H],
    None: delta joins as it is) + rows_add (float32 [T, H]) + vec_add (float32 [H]), each optional; then, with `weight`
    (float32 [H]), returns x / sqrt(mean(x^2) + eps) * weight in out_dtype (else None)."""
    _need_cuda(x, delta, gate, rows_add, vec_add, weight)
    T, H = x.shape
    assert x.dtype == torch.float32 and x.is_contiguous()
    assert delta is None or (delta.shape == x.shape and delta.is_contiguous())
    assert gate is None or (delta is not None and gate.dtype == torch.float32 and gate.shape == x.shape and gate.stride(1) == 1)
    assert rows_add is None or (rows_add.dtype == torch.float32 and rows_add.shape == x.shape and rows_add.is_contiguous())
    for v in (vec_add, weight):
        assert v is None or (v.dtype == torch.float32 and v.numel() == H and v.is_contiguous())
    out = torch.empty((T, H), dtype=out_dtype or torch.float32, device=x.device) if weight is not None else None
    if out is None and delta is None and rows_add is None and vec_add is None:
        return None
    p = _StreamJoinParams()
    p.x, p.delta, p.gate, p.ld_gate = x.data_ptr(), _ptr(delta), _ptr(gate), gate.stride(0) if gate is not None else 0
    p.rows_add, p.vec_add, p.weight, p.out, p.H, p.eps = _ptr(rows_add), _ptr(vec_add), _ptr(weight), _ptr(out), H, eps
    f = _fn(load_module("streamops.cu"), "llb_stream_join", [_StreamJoinParams, c_int, c_int, c_int, c_void_p])
    _check(f(p, _dt(delta) if delta is not None else 0, DT[out.dtype] if out is not None else 0, T, _stream()),
           "gated join of the stream and norm")
    return out


class _BranchMeanParams(ctypes.Structure):
    _fields_ = [("x", c_void_p * 4), ("w", c_void_p * 4), ("n", c_int), ("out", c_void_p), ("H", c_int), ("eps", c_float),
                ("mult", c_float)]


def branch_mean(xs: Sequence[torch.Tensor], ws: Sequence[torch.Tensor], eps: float, mult: float) -> torch.Tensor:
    """float32 [T, H]: mult * sum_b x_b / sqrt(mean(x_b^2) + eps) * w_b over up to four branches (x_b float32 [T, H], w_b [H])."""
    _need_cuda(*xs, *ws)
    assert 1 <= len(xs) == len(ws) <= 4
    T, H = xs[0].shape
    p = _BranchMeanParams()
    for i, (x, w) in enumerate(zip(xs, ws)):
        assert x.dtype == torch.float32 and x.shape == (T, H) and x.is_contiguous() and w.numel() == H and w.is_contiguous()
        assert w.dtype == ws[0].dtype
        p.x[i], p.w[i] = x.data_ptr(), w.data_ptr()
    out = torch.empty((T, H), dtype=torch.float32, device=xs[0].device)
    p.n, p.out, p.H, p.eps, p.mult = len(xs), out.data_ptr(), H, eps, mult
    f = _fn(load_module("streamops.cu"), "llb_branch_mean", [_BranchMeanParams, c_int, c_int, c_void_p])
    _check(f(p, _dt(ws[0]), T, _stream()), "mean of normed branches")
    return out


def scale_(x: torch.Tensor, c: float) -> torch.Tensor:
    """x *= c in place (float32, contiguous)."""
    _need_cuda(x)
    assert x.dtype == torch.float32 and x.is_contiguous()
    f = _fn(load_module("streamops.cu"), "llb_scale_rows", [c_void_p, c_longlong, c_float, c_void_p])
    _check(f(_ptr(x), x.numel(), c, _stream()), "scale")
    return x
