from __future__ import annotations

import ctypes
import functools
from ctypes import c_double, c_float, c_int, c_longlong, c_ulonglong, c_void_p
from dataclasses import dataclass
from typing import Optional

import torch

from ..csrc.build import load_module, page_tokens
from .. import diagnostics
from ..diagnostics import timers

PAGE = page_tokens()           # tokens of a cache page (LLB_PAGE in csrc/common.cuh)
DT = {torch.float32: 0, torch.bfloat16: 1}


class KernelError(RuntimeError):
    pass


def _dt(t: torch.Tensor) -> int:
    try:
        return DT[t.dtype]
    except KeyError:
        raise KernelError(f"dtype {t.dtype} is not supported by the kernels (float32 or bfloat16)") from None


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _stream():
    # the raw handle of torch's current stream on the current device, without the Python layers in between
    return torch._C._cuda_getCurrentRawStream(torch._C._cuda_getDevice())


def _need_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise KernelError("the kernels of llaisys_b200 run on a CUDA device only; got a CPU tensor")


_basic = None


def _lib_basic():
    global _basic
    if _basic is None:
        _basic = load_module("basic.cu")
        _basic.llb_error_string.restype = ctypes.c_char_p
        _basic.llb_error_string.argtypes = [c_int]
    return _basic


_launches = 0

# LLAISYS_STAMPS=1: the kernels that can record cycle stamps (see csrc/common.cuh: the decode step's three short ones and
# the paired-SM product) are built with them; set_stamps() then switches them on for launches of a given grid size.  Off by default: the product's
# builds contain no stamp.
_STAMPS = {"LLB_STAMPS": 1} if __import__("os").environ.get("LLAISYS_STAMPS", "0") not in ("", "0") else {}
_stamp_libs = {}


def _stamped(source: str, defines: Optional[dict] = None):
    lib = load_module(source, {**(defines or {}), **_STAMPS} or None)
    if _STAMPS:
        _stamp_libs[source] = lib
    return lib


def set_stamps(source: str, buf: Optional[torch.Tensor], blocks: int = 0) -> None:
    """Cycle stamps of the kernels of `source` ("gemm_tc.cu", "gemm_tc2.cu", "attention_mma.cu", "mlp_tc.cu") into `buf` (int64
    [blocks, 16] on the device) for launches of exactly `blocks` blocks; None switches them off.  Needs
    LLAISYS_STAMPS=1 in the environment before the package is imported, and the module in use already."""
    lib = _stamp_libs.get(source)
    if lib is None:
        raise KernelError(f"no stamped build of {source} is loaded (LLAISYS_STAMPS=1, and run a step first)")
    lib.llb_set_stamps.argtypes = [c_void_p, ctypes.c_uint]
    lib.llb_set_stamps.restype = c_int
    rc = lib.llb_set_stamps(_ptr(buf), blocks)
    if rc:
        raise KernelError(f"llb_set_stamps: CUDA error {rc}")


def launch_count() -> int:
    """Kernels of this package launched so far by this process (a captured launch counts once,
    at capture; replays are counted by whoever replays)."""
    return _launches


def _check(rc: int, what: str, n: int = 1):
    global _launches
    _launches += n
    if timers.enabled:
        timers.mark(what)
    if rc <= -2000:
        raise KernelError(f"{what}: the kernel's shared-memory size was refused (CUDA error {-rc - 2000})")
    if rc <= -1000:
        raise KernelError(f"{what}: a tensor map could not be encoded (driver error {-rc - 1000})")
    if rc != 0:
        msg = _lib_basic().llb_error_string(rc)
        raise KernelError(f"{what}: CUDA error {rc} ({msg.decode() if msg else '?'})")


_configured = set()


def _fn(lib, name, argtypes):
    f = getattr(lib, name)
    if (id(lib), name) not in _configured:
        f.argtypes = argtypes
        f.restype = c_int
        _configured.add((id(lib), name))
    return f


# ------------------------------------------------------------------ row-wise kernels
def embedding(ids: torch.Tensor, table: torch.Tensor, err: torch.Tensor) -> torch.Tensor:
    """float32 [T, H] rows of `table` (float32 or bfloat16) for int32 `ids`; an id outside the
    table sets err[0] = 1 and yields a zero row."""
    _need_cuda(ids, table)
    T, (V, H) = ids.numel(), table.shape
    out = torch.empty((T, H), dtype=torch.float32, device=table.device)
    f = _fn(_lib_basic(), "llb_embedding", [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p])
    _check(f(_ptr(out), _ptr(table), _dt(table), _ptr(ids), T, H, V, _ptr(err), _stream()), "embedding")
    return out


def embedding_pair(ctx, table: torch.Tensor, scale: float, pair_table: Optional[torch.Tensor] = None, buckets: int = 0,
                   mul_prev: int = 0, mul_cur: int = 0, last: Optional[torch.Tensor] = None) -> torch.Tensor:
    """float32 [T, H]: table[id] * scale, plus (with pair_table [buckets + 1, H]) the row that the hash
    (previous id * mul_prev + id * mul_cur) mod buckets of a token and the one before it in its sequence names; a
    sequence's first token takes row `buckets`.  `last` (int32 [slots, 2]: token, position) carries every sequence's
    last token from step to step; the kernel reads and rewrites the rows of the step's sequences.  err 1: an id
    outside the table; err 3: `last` does not hold the token just before the step's first."""
    ids = ctx.tokens
    _need_cuda(ids, table, pair_table, last)
    T, (V, H) = ids.numel(), table.shape
    if pair_table is not None:
        assert pair_table.dtype == table.dtype and pair_table.shape == (buckets + 1, H) and last is not None
        assert last.dtype == torch.int32 and last.is_contiguous() and last.shape[1] == 2
    out = torch.empty((T, H), dtype=torch.float32, device=table.device)
    f = _fn(_lib_basic(), "llb_embedding_pair",
            [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
             c_int, c_float, c_longlong, c_longlong, c_longlong, c_void_p, c_void_p])
    _check(f(_ptr(out), _ptr(table), _ptr(pair_table), _dt(table), _ptr(ids), _ptr(ctx.tok_pos), _ptr(ctx.tok_seq),
             _ptr(ctx.seq_start), _ptr(ctx.seq_slot), _ptr(last), T, H, V, scale, buckets, mul_prev, mul_cur, _ptr(ctx.err),
             _stream()), "embedding (scaled, with pair rows)")
    return out


def rmsnorm_multi(x: torch.Tensor, weights, eps: float, out_dtype: torch.dtype):
    """One root mean square per row of the float32 stream x [T, H], one output per weight (one or two):
    out_i = x / sqrt(mean(x^2) + eps) * w_i."""
    _need_cuda(x, *weights)
    assert x.dtype == torch.float32 and x.is_contiguous() and 1 <= len(weights) <= 2
    assert all(w.dtype == weights[0].dtype and w.is_contiguous() for w in weights)
    T, H = x.shape
    outs = [torch.empty((T, H), dtype=out_dtype, device=x.device) for _ in weights]
    f = _fn(_lib_basic(), "llb_rmsnorm_multi", [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int,
                                                c_float, c_void_p])
    _check(f(_ptr(x), _ptr(weights[0]), _ptr(weights[1]) if len(weights) > 1 else None, _dt(weights[0]), _ptr(outs[0]),
             _ptr(outs[1]) if len(outs) > 1 else None, DT[out_dtype], T, H, eps, _stream()), "rmsnorm (shared root mean square)")
    return outs


def relu_squared_(x: torch.Tensor) -> torch.Tensor:
    """x <- max(x, 0)^2 in place (contiguous)."""
    _need_cuda(x)
    assert x.is_contiguous()
    f = _fn(_lib_basic(), "llb_relu_squared", [c_void_p, c_int, c_longlong, c_void_p])
    _check(f(_ptr(x), _dt(x), x.numel(), _stream()), "relu squared")
    return x


ROW_ACTS = {None: 0, "relu_squared": 1, "gelu": 2, "gelu_tanh": 3}


def act_rows_(x: torch.Tensor, act: Optional[str], logit: Optional[torch.Tensor] = None, scale: float = 1.0) -> torch.Tensor:
    """In place on x [T, cols] (row stride free): x[t] <- act(x[t]) * scale * sigmoid(logit[t]) (scale alone without
    `logit`, a float32 [T] view with any stride); act None, "relu_squared", "gelu" (erf form) or "gelu_tanh"."""
    _need_cuda(x, logit)
    assert x.dim() == 2 and x.stride(1) == 1
    if logit is not None:
        assert logit.dtype == torch.float32 and logit.dim() == 1 and logit.numel() == x.shape[0]
    f = _fn(_lib_basic(), "llb_act_rows", [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int, c_float, c_void_p])
    _check(f(_ptr(x), _dt(x), x.shape[0], x.stride(0), x.shape[1], ROW_ACTS[act], _ptr(logit),
             logit.stride(0) if logit is not None else 0, float(scale), _stream()), f"activation of rows ({act})")
    return x


class _StreamUpdateParams(ctypes.Structure):
    _fields_ = [("cur", c_void_p), ("delta", c_void_p), ("n_part", c_int), ("part_stride", c_longlong), ("delta_scale", c_float),
                ("write_back", c_int), ("mix", c_void_p), ("n", c_int), ("x0", c_void_p), ("planes", c_void_p),
                ("plane_stride", c_longlong), ("dst", c_void_p), ("weight", c_void_p), ("out", c_void_p), ("rows", c_void_p),
                ("H", c_int), ("eps", c_float)]


def stream_update(cur: torch.Tensor, delta: Optional[torch.Tensor] = None, delta_scale: float = 1.0, *, mix: Optional[torch.Tensor] = None,
                  x0: Optional[torch.Tensor] = None, planes: Optional[torch.Tensor] = None, dst: Optional[torch.Tensor] = None,
                  weight: Optional[torch.Tensor] = None, eps: float = 0.0, out_dtype: Optional[torch.dtype] = None,
                  rows: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """One pass over the rows of the float32 stream `cur` [T, H]:

        v = cur + delta_scale * delta            (delta [T, H] or [parts, T, H]; written back to cur unless `rows`)
        y = sum_j mix[j] X_j                     (with mix, float32 [n]: X_0 = x0, X_1 .. X_{n-2} the planes [n - 2, T, H],
                                                  X_{n-1} = v; without mix y = v)
        dst = y                                  (with dst, float32)
        returns y / sqrt(mean(y^2) + eps) * weight in out_dtype (with weight), else None

    With rows (int32) only those rows are worked on, nothing is written back, and dst / the result have len(rows) rows."""
    _need_cuda(cur, delta, mix, x0, planes, dst, weight, rows)
    assert cur.dtype == torch.float32 and cur.is_contiguous() and cur.dim() == 2
    T, H = cur.shape
    R = T if rows is None else rows.numel()
    p = _StreamUpdateParams()
    p.cur, p.H, p.eps, p.delta_scale = cur.data_ptr(), H, float(eps), float(delta_scale)
    if delta is not None:
        assert delta.shape[-2:] == cur.shape and delta.is_contiguous()
        p.delta, p.n_part, p.part_stride = delta.data_ptr(), (delta.shape[0] if delta.dim() == 3 else 1), (delta.stride(0) if delta.dim() == 3 else 0)
        p.write_back = int(rows is None)
    if mix is not None:
        n = mix.numel()
        assert mix.dtype == torch.float32 and mix.is_contiguous() and n >= 1
        p.mix, p.n = mix.data_ptr(), n
        if n > 1:
            assert x0 is not None and x0.dtype == torch.float32 and x0.is_contiguous() and x0.shape == cur.shape
            p.x0 = x0.data_ptr()
        if n > 2:
            assert planes is not None and planes.dtype == torch.float32 and planes.shape[0] >= n - 2 and planes.shape[1:] == cur.shape
            assert planes.stride(1) == H and planes.stride(2) == 1
            p.planes, p.plane_stride = planes.data_ptr(), planes.stride(0)
    if dst is not None:
        assert dst.dtype == torch.float32 and dst.is_contiguous() and dst.shape == (R, H)
        p.dst = dst.data_ptr()
    out = None
    if weight is not None:
        assert weight.numel() == H and weight.is_contiguous()
        out = torch.empty((R, H), dtype=out_dtype or torch.float32, device=cur.device)
        p.weight, p.out = weight.data_ptr(), out.data_ptr()
    p.rows = _ptr(rows)
    f = _fn(_lib_basic(), "llb_stream_update", [_StreamUpdateParams, c_int, c_int, c_int, c_int, c_void_p])
    _check(f(p, _dt(delta) if delta is not None else 0, _dt(weight) if weight is not None else 0,
             DT[out.dtype] if out is not None else 0, R, _stream()), "stream update (scaled add, depth average, norm)")
    return out


def rope_lead_append(proj: torch.Tensor, nh: int, nkvh: int, dk: int, dv: int, rot: int, *, cos=None, sin=None, tok_pos=None,
                     append=None, err=None):
    """In place on packed projections [T, nh dk (+ nkvh dk + nkvh dv)]: rotate the first `rot` dimensions of the query
    heads and of the nkvh key heads (pairs (j, j + rot/2), tables [rows, rot/2]) and, with `append`, write keys and
    values to the paged cache.  nkvh 0: the rows hold queries only.
    append = dict(tok_seq, seq_start, seq_len_before, kpool, vpool, page_table, ring, pinned)."""
    _need_cuda(proj, tok_pos)
    T = proj.shape[0]
    assert proj.stride(1) == 1
    if tok_pos is None or tok_pos.numel() != T or err is None:
        raise KernelError("rope_lead_append needs tok_pos (one position per packed token) and an error word")
    if cos is None:
        rot = 0
    a = append or {}
    pt = a.get("page_table")
    f = _fn(_lib_basic(), "llb_rope_lead_append",
            [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int,
             c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p])
    _check(f(_ptr(proj), _dt(proj), T, proj.stride(0), nh, nkvh, dk, dv, rot, _ptr(cos), _ptr(sin),
             cos.shape[0] if cos is not None else 0, _ptr(tok_pos), int(append is not None), _ptr(a.get("tok_seq")),
             _ptr(a.get("seq_start")), _ptr(a.get("seq_len_before")), _ptr(a.get("kpool")), _ptr(a.get("vpool")), _ptr(pt),
             pt.shape[1] if pt is not None else 0, a.get("ring", 1), a.get("pinned", 0), _ptr(err), _stream()),
           "rotation of leading dimensions / cache append")


def gather_i32(dst: torch.Tensor, src: torch.Tensor, idx: torch.Tensor):
    """dst[i] = src[idx[i]] (int32, on the device)."""
    _need_cuda(dst, src, idx)
    assert dst.dtype == src.dtype == idx.dtype == torch.int32 and dst.numel() == idx.numel()
    f = _fn(_lib_basic(), "llb_gather_i32", [c_void_p, c_void_p, c_void_p, c_int, c_void_p])
    _check(f(_ptr(dst), _ptr(src), _ptr(idx), idx.numel(), _stream()), "gather_i32")


def scatter_i32(dst: torch.Tensor, idx: torch.Tensor, src: torch.Tensor):
    """dst[idx[i]] = src[i] (int32, on the device; idx without repeats)."""
    _need_cuda(dst, src, idx)
    assert dst.dtype == src.dtype == idx.dtype == torch.int32 and src.numel() == idx.numel()
    f = _fn(_lib_basic(), "llb_scatter_i32", [c_void_p, c_void_p, c_void_p, c_int, c_void_p])
    _check(f(_ptr(dst), _ptr(idx), _ptr(src), idx.numel(), _stream()), "scatter_i32")


def add_rmsnorm(residual: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                out_dtype: torch.dtype, rows: Optional[torch.Tensor] = None, want_out: bool = True):
    """residual (float32 [T, H]) += delta, then out = residual * weight / sqrt(mean(residual^2) + eps).

    delta is [T, H] or [parts, T, H] (partial sums, added in order).  With `rows` (int32) only those
    rows are normalised, into an [len(rows), H] output, and the residual is left as it was."""
    _need_cuda(residual, delta, weight, rows)
    T, H = residual.shape
    n_part, stride = 1, 0
    if delta is not None:
        if delta.dim() == 3:
            n_part, stride = delta.shape[0], delta.stride(0)
        assert delta.shape[-2:] == residual.shape and delta.is_contiguous()
    R = T if rows is None else rows.numel()
    out = torch.empty((R, H), dtype=out_dtype, device=residual.device) if want_out else None
    f = _fn(_lib_basic(), "llb_add_rmsnorm", [c_void_p, c_void_p, c_int, c_int, c_longlong, c_void_p, c_int,
                                              c_void_p, c_int, c_void_p, c_int, c_int, c_float, c_int, c_void_p])
    _check(f(_ptr(residual), _ptr(delta), _dt(delta) if delta is not None else 0, n_part, stride,
             _ptr(weight), _dt(weight), _ptr(out), DT[out_dtype], _ptr(rows), R, H, eps,
             0 if rows is not None else 1, _stream()), "add_rmsnorm")
    return out


def residual_add(residual: torch.Tensor, delta: torch.Tensor):
    _need_cuda(residual, delta)
    n_part, stride = (delta.shape[0], delta.stride(0)) if delta.dim() == 3 else (1, 0)
    f = _fn(_lib_basic(), "llb_residual_add", [c_void_p, c_void_p, c_int, c_int, c_longlong, c_longlong, c_void_p])
    _check(f(_ptr(residual), _ptr(delta), _dt(delta), n_part, stride, residual.numel(), _stream()), "residual_add")


def swiglu(gate_up: torch.Tensor) -> torch.Tensor:
    """[T, 2I] (gate columns first) -> [T, I]: up * gate / (1 + exp(-gate))."""
    _need_cuda(gate_up)
    T, I2 = gate_up.shape
    out = torch.empty((T, I2 // 2), dtype=gate_up.dtype, device=gate_up.device)
    f = _fn(_lib_basic(), "llb_swiglu", [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(out), _ptr(gate_up), _dt(gate_up), T, I2 // 2, _stream()), "swiglu")
    return out


GLU_ACTS = {"silu": 0, "relu": 1, "gelu_tanh": 2, "swish_clamped": 3}


def glu(gate_up: torch.Tensor, act: str, out_dtype: Optional[torch.dtype] = None, limit: float = 0.0, alpha: float = 1.0) -> torch.Tensor:
    """[T, 2I] (gate columns first) -> [T, I]: act(gate) * up with act "silu", "relu" or "gelu_tanh", in float32 with
    one rounding at the output.  "swish_clamped": g = min(gate, limit), u = clamp(up, -limit, limit),
    out = g sigmoid(alpha g) (u + 1)."""
    _need_cuda(gate_up)
    assert gate_up.is_contiguous()
    T, I2 = gate_up.shape
    out = torch.empty((T, I2 // 2), dtype=out_dtype or gate_up.dtype, device=gate_up.device)
    f = _fn(_lib_basic(), "llb_glu", [c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_float, c_float, c_void_p])
    _check(f(_ptr(out), _dt(out), _ptr(gate_up), _dt(gate_up), T, I2 // 2, GLU_ACTS[act], float(limit), float(alpha), _stream()),
           f"gated activation ({act})")
    return out


def scaled_norm_add(residual: torch.Tensor, delta: Optional[torch.Tensor], w_post: Optional[torch.Tensor], mult: float,
                    w_next: Optional[torch.Tensor], eps: float, offset: float, out_dtype: Optional[torch.dtype] = None):
    """residual (float32 [T, H]) += mult * delta / sqrt(mean(delta^2) + eps) * (w_post + offset); with w_next also returns
    residual / sqrt(mean(residual^2) + eps) * (w_next + offset) of the new rows, from the same pass.  Without delta
    only the second half (a plain norm of the stream)."""
    _need_cuda(residual, delta, w_post, w_next)
    assert residual.dtype == torch.float32 and residual.is_contiguous()
    T, H = residual.shape
    if delta is not None:
        assert delta.shape == residual.shape and delta.is_contiguous() and w_post is not None
    w = w_post if w_post is not None else w_next
    assert w is not None and (w_next is None or w_post is None or w_next.dtype == w_post.dtype)
    out = torch.empty((T, H), dtype=out_dtype, device=residual.device) if w_next is not None else None
    f = _fn(_lib_basic(), "llb_scaled_norm_add", [c_void_p, c_void_p, c_int, c_void_p, c_float, c_void_p, c_int, c_void_p, c_int,
                                                  c_int, c_int, c_float, c_float, c_void_p])
    _check(f(_ptr(residual), _ptr(delta), _dt(delta) if delta is not None else 0, _ptr(w_post), mult, _ptr(w_next), _dt(w),
             _ptr(out), DT[out_dtype] if out is not None else 0, T, H, eps, offset, _stream()), "normed output into the stream")
    return out


def dense_binary(out: torch.Tensor, a: torch.Tensor, b: torch.Tensor, op: str):
    """out = a + b (op "add") or out = b * a / (1 + exp(-a)) (op "swiglu": a the gate, b the up
    projection) on contiguous tensors of one dtype and one shape."""
    _need_cuda(out, a, b)
    assert out.dtype == a.dtype == b.dtype and out.shape == a.shape == b.shape
    assert out.is_contiguous() and a.is_contiguous() and b.is_contiguous()
    f = _fn(_lib_basic(), "llb_dense_binary", [c_void_p, c_void_p, c_void_p, c_int, c_longlong, c_int, c_void_p])
    _check(f(_ptr(out), _ptr(a), _ptr(b), _dt(out), out.numel(), {"add": 0, "swiglu": 1}[op], _stream()), op)


def rope_append(qkv: torch.Tensor, nh: int, nkvh: int, dh: int, *, cos=None, sin=None, tok_pos=None,
                append=None, err=None):
    """In place on the packed projections [T, (nh + 2 nkvh) dh]: rotate the query and key heads
    (when cos/sin tables are given) and/or write keys and values to the paged cache.

    append = dict(tok_seq, seq_start, seq_len_before, kpool, vpool, page_table, ring)."""
    _need_cuda(qkv, tok_pos)
    T = qkv.shape[0]
    assert qkv.stride(1) == 1
    if tok_pos is None or tok_pos.numel() != T or err is None:
        raise KernelError("rope_append needs tok_pos (one position per packed token) and an error word")
    do_rope, do_app = cos is not None, append is not None
    a = append or {}
    pt = a.get("page_table")
    f = _fn(_lib_basic(), "llb_rope_append",
            [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p,
             c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p])
    _check(f(_ptr(qkv), _dt(qkv), T, qkv.stride(0), nh, nkvh, dh, int(do_rope), _ptr(cos), _ptr(sin),
             cos.shape[0] if do_rope else 0, _ptr(tok_pos), int(do_app), _ptr(a.get("tok_seq")),
             _ptr(a.get("seq_start")), _ptr(a.get("seq_len_before")), _ptr(a.get("kpool")), _ptr(a.get("vpool")),
             _ptr(pt), pt.shape[1] if do_app else 0, a.get("ring", 1), _ptr(err), _stream()), "rope_append")


def fill_normal(out: torch.Tensor, key: int, mean: float, std: float, first: int = 0):
    """out (contiguous, float32 or bfloat16) <- mean + std * z(key, first + i): the counter-based
    normal numbers of csrc/random_init.cu, whose host twin is weights/rng.py."""
    _need_cuda(out)
    assert out.is_contiguous()
    f = _fn(load_module("random_init.cu"), "llb_fill_normal",
            [c_void_p, c_int, c_longlong, c_longlong, c_ulonglong, c_double, c_double, c_void_p])
    with torch.cuda.device(out.device):
        _check(f(_ptr(out), _dt(out), out.numel(), first, key & 0xFFFFFFFFFFFFFFFF, mean, std, _stream()), "fill_normal")


# ------------------------------------------------------------------ matrix products
_TC_SCRATCH_ELEMS = 16 * 1024 * 1024        # float32 partial tiles of split-K launches (64 MB)
_TC_COUNTERS = 1 << 16
_tc_res = {}
TC_ENABLED = True                            # tests switch the tensor-core path off to compare


def _tc_resources(device):
    """Per device: the scratch of split-K partial tiles, the tile counters (zero between
    launches) and the error word of the tensor-core kernels.  Allocated once, so launches inside
    a CUDA graph capture allocate nothing."""
    device = _dev_key(device)
    r = _tc_res.get(device)
    if r is None:
        if diagnostics.CANARY:
            scratch, raw_s = diagnostics.guarded((_TC_SCRATCH_ELEMS,), torch.float32, device, fill_zero=False)
            counters, raw_c = diagnostics.guarded((_TC_COUNTERS,), torch.int32, device)
            _tc_guards[device] = [("tensor-core scratch", raw_s), ("tensor-core tile counters", raw_c)]
        else:
            scratch = torch.empty(_TC_SCRATCH_ELEMS, dtype=torch.float32, device=device)
            counters = torch.zeros(_TC_COUNTERS, dtype=torch.int32, device=device)
        r = (scratch, counters, torch.zeros(1, dtype=torch.int32, device=device))
        _tc_res[device] = r
    return r


_tc_guards = {}


def check_guards(device) -> None:
    """Raises KernelError if the guard words around the tensor-core scratch or counters of `device` were
    overwritten (they exist only under LLAISYS_CANARY=1)."""
    broken = [what for what, raw in _tc_guards.get(_dev_key(device), []) if not diagnostics.guards_intact(raw)]
    if broken:
        raise KernelError("guard words overwritten around: " + ", ".join(broken))


def _dev_key(device) -> torch.device:
    device = torch.device(device)
    if device.type == "cuda" and device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    return device


def tc_error(device, clear: bool = True) -> int:
    """Error word of the tensor-core kernels on `device` (0: none; 101-104, 111-114, 121-122, 131-136, 141, 151-153: a bounded
    wait ran out).  Reading it waits for the device; a code that was found is cleared, so that it is
    reported once."""
    r = _tc_res.get(_dev_key(device))
    if not r:
        return 0
    code = int(r[2].item())
    if code and clear:
        r[2].zero_()
    return code


_sm_counts = {}


def _sm_count(device) -> int:
    n = _sm_counts.get(device)
    if n is None:
        n = _sm_counts[device] = torch.cuda.get_device_properties(device).multi_processor_count
    return n


_TC_STAGES = {False: {16: 5, 32: 4, 64: 4, 128: 6, 256: 4}, True: {16: 3, 32: 3, 64: 4, 128: 4, 256: 3}}


@functools.lru_cache(maxsize=4096)
def tc_plan(T: int, rows_out: int, K: int, sms: int, dual: bool = False):
    """(tokens per tile, K splits) of a tensor-core launch.

    The tile is the smallest that holds the tokens.  When the weight has fewer row blocks than
    the device can run CTAs (decode), K is split 2, 4, 8 or 16 ways over a thread-block cluster that
    reduces through shared memory.  The split minimises a cost fitted to measurements on a B200
    (microseconds): k-blocks per CTA times 0.0155 per KB of a pipeline stage, plus, when split,
    1.2 + 0.0015 * tile tokens * accumulators * splits for the cluster reduction; the CTAs must
    all be resident at once (two per SM while a CTA's shared memory stays under 113 KB; with one
    per SM, clusters of eight fill a GPC unevenly, so fewer CTAs are allowed)."""
    bn = 16 if T <= 16 else 32 if T <= 32 else 64 if T <= 64 else 128 if T <= 128 else 256
    tiles = -(-rows_out // 128) * -(-T // bn)
    kblocks = -(-K // 64)
    accs = 2 if dual else 1
    stage_kb = accs * 16 + bn / 8
    recv_kb = bn / 2 if bn <= 32 and not dual else 0          # the push reduction's receive buffer
    two_per_sm = stage_kb * _TC_STAGES[dual][bn] + recv_kb <= 112
    capacity = (sms * 2 * 280) // 296 if two_per_sm else (sms * 112) // 148
    best, best_cost = 1, kblocks * stage_kb * 0.0155
    if bn <= 128:
        # sixteen (a cluster of non-portable size) for 64-token tiles and for up to four tokens: measured in the
        # whole step, +2.7 % at batch 64, +1.5 % at batch 1 and 2, +4 % at batch 4, nothing at batch 6, but -1 % at
        # batch 8 and 32, although the product alone is faster there too
        for s in (2, 4, 8, 16):
            if s > kblocks // 2 or tiles * s > capacity or (s == 16 and bn != 64 and T > 4):
                break
            if (s - 1) * -(-kblocks // s) >= kblocks:      # a CTA of the cluster would be left without a k-block
                continue
            cost = -(-kblocks // s) * stage_kb * 0.0155 + 1.2 + 0.0015 * bn * accs * s
            if cost < best_cost:
                best, best_cost = s, cost
    return bn, best


def _tc_ok(x, weight, bias) -> bool:
    return (TC_ENABLED and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.shape[1] % 8 == 0
            and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0)


def _pair_ok(out, rows_out) -> bool:
    return out.dtype == torch.bfloat16 and rows_out % 8 == 0 and out.stride(0) % 8 == 0 and out.data_ptr() % 16 == 0


def _gemm_tc_pair(x, weight, bias, out, dual_offset=0):
    """The product on pairs of SMs (csrc/gemm_tc2.cu): persistent, for many tokens, bfloat16 output."""
    M, K = x.shape
    N = weight.shape[0]
    err = _tc_resources(x.device)[2]
    f = _fn(_stamped("gemm_tc2.cu"), "llb_gemm_tc2",
            [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p])
    _check(f(_ptr(x), _ptr(weight), _ptr(bias), _dt(bias) if bias is not None else 0, _ptr(out), M, N, K,
             x.stride(0), out.stride(0), dual_offset, _sm_count(x.device) // 2, _ptr(err), _stream()),
           "linear (tensor cores, paired SMs)")


def _gemm_tc(x, weight, bias, out, dual_offset=0, plan=None):
    M, K = x.shape
    N = weight.shape[0]
    if plan is None and M > 256 and _pair_ok(out, dual_offset or N):
        plan = ("pair",)
    if plan is not None and plan[0] == "pair":
        return _gemm_tc_pair(x, weight, bias, out, dual_offset)
    scratch, counters, err = _tc_resources(x.device)
    # gate/up for 17 to 64 tokens: a block per 64 outputs (gate and up rows side by side in one accumulator), twice as
    # many blocks as with a tile of 128 gate rows, which without a K split leaves half of the SMs idle at these sizes
    side_by_side = plan is not None and plan[0] == "gateup"
    if plan is None and dual_offset and 16 < M <= 64:
        side_by_side = True
    if side_by_side and dual_offset and bias is None and _pair_ok(out, dual_offset):
        bn = plan[1] if plan is not None else (32 if M <= 32 else 64)
        f = _fn(_stamped("gemm_tc.cu"), "llb_gemm_tc_gateup",
                [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p])
        _check(f(_ptr(x), _ptr(weight), _ptr(out), M, dual_offset, K, x.stride(0), out.stride(0), bn, _ptr(err), _stream()),
               "gate/up (tensor cores, rows side by side)")
        return
    if side_by_side:
        plan = None
    plan = plan or tc_plan(M, dual_offset or N, K, _sm_count(x.device), bool(dual_offset))
    bn, splits = plan[0], plan[1]
    cluster = plan[2] if len(plan) > 2 else 1            # (bn, splits, 0) forces the reduction through scratch
    f = _fn(_stamped("gemm_tc.cu"), "llb_gemm_tc",
            [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
             c_int, c_int, c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_void_p])
    _check(f(_ptr(x), _ptr(weight), _ptr(bias), _dt(bias) if bias is not None else 0, _ptr(out), _dt(out),
             M, N, K, x.stride(0), out.stride(0), bn, splits, cluster, dual_offset, _ptr(scratch), scratch.numel(),
             _ptr(counters), counters.numel(), _ptr(err), _stream()), "linear (tensor cores)")


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
           out_dtype: Optional[torch.dtype] = None, plan=None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x [M, K] (row stride free) times weight [N, K] transposed, plus bias [N]; float32 accumulation.  `out`: an
    [M, N] tensor or view (row stride free) that receives the result instead of a new tensor.

    bfloat16 operands with K a multiple of 8 run on the tensor cores (csrc/gemm_tc.cu); everything
    else (float32, a 32-bit weight under 16-bit activations, odd K) on the CUDA cores (csrc/gemm_simt.cu)."""
    _need_cuda(x, weight, bias)
    M, K = x.shape
    N, K2 = weight.shape
    if K != K2:
        raise KernelError(f"linear: x has {K} columns but the weight has {K2}")
    assert x.stride(1) == 1 and weight.is_contiguous()
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype or x.dtype, device=x.device)
    else:
        assert out.shape == (M, N) and out.stride(1) == 1 and out.is_cuda
    if M == 0:
        return out
    if _tc_ok(x, weight, bias) and (out.is_contiguous() or (out.data_ptr() % 16 == 0 and out.stride(0) % 8 == 0 and N % 8 == 0)):
        _gemm_tc(x, weight, bias, out, plan=plan)
        return out
    lib = load_module("gemm_simt.cu")
    f = _fn(lib, "llb_gemm_simt", [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int,
                                   c_int, c_int, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(x), _dt(x), _ptr(weight), _dt(weight), _ptr(bias), _dt(bias) if bias is not None else 0,
             _ptr(out), _dt(out), M, N, K, x.stride(0), out.stride(0), _stream()), "linear")
    return out


def linear_into_ok(x: torch.Tensor, weight: torch.Tensor, bias, stream: torch.Tensor) -> bool:
    """True when linear_into() takes these operands: bfloat16 on the tensor cores, a float32 stream with 16-byte
    aligned rows."""
    return (_tc_ok(x, weight, bias) and x.shape[0] > 0 and stream.dtype == torch.float32 and stream.stride(1) == 1
            and stream.stride(0) % 4 == 0 and stream.data_ptr() % 16 == 0 and stream.shape == (x.shape[0], weight.shape[0]))


def into_plan(T: int, N: int, K: int, sms: int):
    """(tokens per tile, K ranges) of linear_into() for up to 256 tokens: the smallest tile that holds the tokens, and as
    many K ranges as keep every block at two k-blocks or more and all blocks resident at once (two per SM while a
    block's ring stays under half of an SM's shared memory)."""
    bn = 16 if T <= 16 else 32 if T <= 32 else 64 if T <= 64 else 128 if T <= 128 else 256
    tiles = -(-N // 128) * -(-T // bn)
    kblocks = -(-K // 64)
    room = 2 * sms if bn <= 64 else sms
    return bn, max(1, min(kblocks // 2, room // tiles))


def linear_into(x: torch.Tensor, weight: torch.Tensor, bias, stream: torch.Tensor, ksplit: int = 0) -> None:
    """stream [T, N] (float32) += x weight^T + bias in place: a projection that ends in the residual add.  Up to 256
    tokens: csrc/gemm_tc.cu (INTO), the K range divided over blocks that each add their partial tile by a TMA
    reduction; more: the paired-SM kernel (csrc/gemm_tc2.cu, INTO).  ksplit: K ranges per tile (0: chosen)."""
    _need_cuda(x, weight, bias, stream)
    T, K = x.shape
    N = weight.shape[0]
    err = _tc_resources(x.device)[2]
    if T <= 256:
        bn, splits = into_plan(T, N, K, _sm_count(x.device))
        f = _fn(_stamped("gemm_tc.cu"), "llb_gemm_tc_into",
                [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p])
        _check(f(_ptr(x), _ptr(weight), _ptr(bias), _dt(bias) if bias is not None else 0, _ptr(stream), T, N, K, x.stride(0),
                 stream.stride(0), bn, ksplit or splits, _ptr(err), _stream()), "linear into the residual stream (tensor cores)")
        return
    f = _fn(_stamped("gemm_tc2.cu"), "llb_gemm_tc2_into",
            [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p])
    _check(f(_ptr(x), _ptr(weight), _ptr(bias), _dt(bias) if bias is not None else 0, _ptr(stream), T, N, K, x.stride(0),
             stream.stride(0), ksplit, _sm_count(x.device) // 2, _ptr(err), _stream()), "linear into the residual stream (tensor cores, paired SMs)")


def linear_swiglu(x: torch.Tensor, gate_up: torch.Tensor, plan=None) -> torch.Tensor:
    """up(x) * silu(gate(x)) for the fused [2I, K] matrix (gate rows first): [M, I].  On the
    tensor cores the two products share one kernel and the [M, 2I] intermediate is never written."""
    _need_cuda(x, gate_up)
    I = gate_up.shape[0] // 2
    if _tc_ok(x, gate_up, None) and x.shape[0] > 0:
        out = torch.empty((x.shape[0], I), dtype=x.dtype, device=x.device)
        _gemm_tc(x, gate_up, None, out, dual_offset=I, plan=plan)
        return out
    return swiglu(linear(x, gate_up))


FUSED_MLP = __import__("os").environ.get("LLAISYS_FUSED_MLP", "1") != "0"     # tests switch the one-launch feed-forward off to compare
_MLP_STAGES = int(__import__("os").environ.get("LLAISYS_MLP_STAGES", "0"))     # depth of its TMA ring (0: the kernel's choice)
# LLAISYS_MLP_WAIT_LIMIT: a build of that kernel whose bounded waits give up after this many tries (for trying out changes)
_MLP_DEFINES = ({"LLB_WAIT_LIMIT": int(__import__("os").environ["LLAISYS_MLP_WAIT_LIMIT"])}
                if __import__("os").environ.get("LLAISYS_MLP_WAIT_LIMIT") else None)


def mlp_fused_ok(x: torch.Tensor, gate_up: torch.Tensor, down: torch.Tensor, residual: torch.Tensor) -> bool:
    """True when the whole SwiGLU feed-forward of these tokens can run as one launch (csrc/mlp_tc.cu):
    bfloat16 operands, at most 32 tokens, widths that are multiples of 8 and an output width whose
    accumulators fit tensor memory."""
    if not (FUSED_MLP and TC_ENABLED and x.is_cuda and x.dtype == gate_up.dtype == down.dtype == torch.bfloat16
            and residual.dtype == torch.float32 and residual.is_contiguous() and x.stride(1) == 1 and x.stride(0) % 8 == 0
            and not ((x.data_ptr() | gate_up.data_ptr() | down.data_ptr()) & 15)):
        return False
    T, H = x.shape
    I = down.shape[1]
    if gate_up.shape != (2 * I, H) or down.shape != (H, I) or residual.shape != (T, H):
        return False
    f = _stamped("mlp_tc.cu", _MLP_DEFINES).llb_mlp_fused_ok
    f.argtypes, f.restype = [c_int, c_int, c_int], c_int
    return bool(f(T, H, I))


def mlp_fused(x: torch.Tensor, gate_up: torch.Tensor, down: torch.Tensor, residual: torch.Tensor, stages: int = 0) -> None:
    """residual [T, H] (float32) += down(up(x) * silu(gate(x))) in one launch; gate_up is [2I, H] with the gate rows
    first, down [H, I].  See mlp_fused_ok() for what it takes."""
    _need_cuda(x, gate_up, down, residual)
    T, H = x.shape
    I = down.shape[1]
    err = _tc_resources(x.device)[2]
    stages = stages or _MLP_STAGES
    f = _fn(_stamped("mlp_tc.cu", _MLP_DEFINES), "llb_mlp_fused",
            [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p])
    _check(f(_ptr(x), x.stride(0), _ptr(gate_up), _ptr(down), _ptr(residual), T, H, I, _sm_count(x.device), stages,
             _ptr(err), _stream()), "feed-forward (one launch, tensor cores)")


# ------------------------------------------------------------------ attention
class _AttnParams(ctypes.Structure):
    _fields_ = [("q", c_void_p), ("k_new", c_void_p), ("v_new", c_void_p), ("row_stride", c_int),
                ("out", c_void_p), ("kpool", c_void_p), ("vpool", c_void_p), ("page_table", c_void_p),
                ("table_stride", c_int), ("ring", c_int), ("seq_start", c_void_p),
                ("seq_len_before", c_void_p), ("nh", c_int), ("nkvh", c_int), ("window", c_int),
                ("scale", c_float), ("all_from_cache", c_int), ("n_splits", c_int), ("part_o", c_void_p), ("part_ml", c_void_p),
                ("keep_first", c_int), ("pinned", c_int), ("sink", c_int),
                ("sink_logits", c_void_p), ("v_in_k", c_int), ("kv_row_stride", c_int),
                ("dist_r1", c_void_p), ("dist_r2", c_void_p), ("q_temp_coef", c_float), ("q_temp_every", c_int),
                ("chunk", c_int), ("maps", c_int), ("out_f32", c_int), ("pool", c_int), ("pool_k", c_void_p), ("pool_v", c_void_p),
                ("pool_table", c_void_p), ("pool_table_stride", c_int)]


class _MmaAttnParams(ctypes.Structure):
    _fields_ = [("q", c_void_p), ("k_new", c_void_p), ("v_new", c_void_p), ("row_stride", c_int),
                ("out", c_void_p), ("kpool", c_void_p), ("vpool", c_void_p), ("page_table", c_void_p),
                ("table_stride", c_int), ("ring", c_int), ("seq_start", c_void_p),
                ("seq_len_before", c_void_p), ("nh", c_int), ("nkvh", c_int), ("window", c_int),
                ("scale", c_float), ("all_from_cache", c_int), ("n_splits", c_int), ("part_o", c_void_p),
                ("part_ml", c_void_p), ("rope_cos", c_void_p), ("rope_sin", c_void_p), ("rope_rows", c_int),
                ("append_new", c_int), ("cluster", c_int), ("err", c_void_p),
                ("keep_first", c_int), ("pinned", c_int), ("sink", c_int), ("sink_logits", c_void_p),
                ("dist_r1", c_void_p), ("dist_r2", c_void_p), ("q_temp_coef", c_float), ("q_temp_every", c_int),
                ("chunk", c_int), ("maps", c_int), ("out_f32", c_int), ("v_split", c_int), ("pool", c_int), ("pool_k", c_void_p),
                ("pool_v", c_void_p), ("pool_table", c_void_p), ("pool_table_stride", c_int)]


MMA_ATTENTION = True                         # tests switch the tensor-core attention off to compare


def _mma_ok(qkv, dh) -> bool:
    return MMA_ATTENTION and qkv.dtype == torch.bfloat16 and dh % 16 == 0 and dh <= 128 and qkv.stride(0) % 8 == 0


_decode16 = {}


def prefill_ext_ok(qkv: torch.Tensor, dh: int, dv: int) -> bool:
    """True when the mma.sync prefill kernel takes chunks, several score maps and pooled blocks for these operands."""
    return _mma_ok(qkv, dh) and dv in (dh, 2 * dh)


def decode_clusters16(dtype: torch.dtype, dh: int) -> int:
    """Clusters of sixteen blocks of the decode attention kernel that the device holds at once
    (0 where that kernel or that cluster size does not apply)."""
    if not (MMA_ATTENTION and dtype == torch.bfloat16 and dh % 16 == 0 and dh <= 128):
        return 0
    if dh not in _decode16:
        f = _mma_lib(dh).llb_attn_mma_decode_max_clusters
        f.argtypes, f.restype = [c_int], c_int
        _decode16[dh] = int(f(16))
    return _decode16[dh]


def decode_fusion_ok(dtype: torch.dtype, dh: int) -> bool:
    """True when decode attention can itself rotate the query and the new key and append the
    new key and value to the cache (the tensor-core kernel), so that no kernel has to do it before."""
    return MMA_ATTENTION and dtype == torch.bfloat16 and dh % 16 == 0 and dh <= 128


class _TcAttnParams(ctypes.Structure):
    _fields_ = [("out", c_void_p), ("page_table", c_void_p), ("table_stride", c_int), ("seq_start", c_void_p),
                ("seq_len_before", c_void_p), ("nh", c_int), ("nkvh", c_int), ("window", c_int), ("scale", c_float),
                ("err", c_void_p), ("n_split", c_int), ("keep_first", c_int), ("sink", c_int)]


TC_ATTENTION = True                          # tests switch the tcgen05 prefill attention off to compare


def prefill_tc_ok(dtype: torch.dtype, dh: int) -> bool:
    """True when prefill attention can run on tcgen05 (csrc/attention_tc.cu): bfloat16, head size 64
    or 128.  That kernel reads every key, those of the step included, from the cache."""
    return TC_ATTENTION and dtype == torch.bfloat16 and dh in (64, 128)


def require_head_dim(dh: int, even: bool = True) -> None:
    """Raises unless some attention kernel of this package takes heads of `dh` elements: the CUDA-core
    kernel (both precisions) takes any size up to 256 (even, where whole heads are rotated in halves); the
    tensor-core kernels take multiples of 16 up to 128 (mma.sync) and 64 or 128 (tcgen05) and are chosen
    where they apply."""
    if dh <= 0 or (even and dh % 2) or dh > 256:
        raise KernelError(f"attention: head size {dh} is not supported ({'even, ' if even else ''}at most 256)")


def _mma_lib(dh: int):
    lib = _stamped("attention_mma.cu", {"LLB_HEAD_DIM": dh})
    return lib


def _attn_lib(dh: int, dv: Optional[int] = None):
    require_head_dim(dh, even=False)
    if dv is None or dv == dh:
        return load_module("attention_simt.cu", {"LLB_HEAD_DIM": dh})
    require_head_dim(dv, even=False)
    return load_module("attention_simt.cu", {"LLB_HEAD_DIM": dh, "LLB_VALUE_DIM": dv})


@dataclass(frozen=True)
class AttnExtras:
    """What the plain causal (windowed) softmax attention does not have: values of a width of their own, first keys
    that stay visible behind a window (`keep_first`, held in `pinned` pages ahead of the cache ring), and a
    value-less sink term in the softmax's denominator: of score 0 (`sink`), or of a learned score per query head
    (`sink_logits`, float32 [heads]); a penalty on distance, `dist_bias` = (r1, r2), float32 [heads] each: the score of
    query position i and key position j loses r1[h] ln(1 + r2[h] (i - j)); a query temperature, `q_temp` = (coef, every):
    the query at position p is multiplied by 1 + coef ln(floor((p + 1) / every) + 1).  The last two run on the mma.sync
    kernels (bfloat16, keys and values of one width that is a multiple of 16 up to 128) and on the CUDA-core kernel (every
    other case, both precisions), not on the tcgen05 prefill kernel.

    Four more, on the CUDA-core kernel (both precisions, prompts and single tokens) and, for prompts in bfloat16 with keys
    of a multiple of 16 up to 128 elements and values as wide or twice as wide, on the mma.sync prefill kernel: `chunk` (the query at position p sees no key before floor(p / chunk) * chunk);
    `maps` (that many key heads share one value head: `nkvh` counts key heads, query head h uses key head h / (nh / nkvh)
    and value head (h / (nh / nkvh)) / maps, and a cache key row holds the maps' keys side by side); `out_f32` (the result
    is float32 whatever the operands are); `pool` = (P, blocks): beside the keys of a window W, one key and value per block
    of P positions that lies wholly before the window (block b is seen from position p when b P + P - 1 <= p - W), read
    at row b of the cache view `blocks`; tokens and blocks share one softmax."""
    value_dim: Optional[int] = None
    keep_first: int = 0
    pinned: int = 0
    sink: bool = False
    sink_logits: Optional[torch.Tensor] = None
    dist_bias: Optional[tuple] = None
    q_temp: Optional[tuple] = None
    chunk: int = 0
    maps: int = 1
    out_f32: bool = False
    pool: Optional[tuple] = None

    def plain(self, dh: int) -> bool:
        return (self.value_dim in (None, dh) and not self.keep_first and not self.pinned and not self.sink
                and self.sink_logits is None and not self.positional() and not self.cuda_core_only())

    def cuda_core_only(self) -> bool:
        """True with an option that only the CUDA-core kernel (and the mma.sync prefill kernel) has."""
        return bool(self.chunk) or self.maps > 1 or self.out_f32 or self.pool is not None

    def positional(self) -> bool:
        """True with an option that makes a score depend on the positions themselves."""
        return self.dist_bias is not None or self.q_temp is not None


def _attn_params(qkv, out, nh, nkvh, dh, kpool, vpool, page_table, ring, seq_start, seq_len_before,
                 window, scale, cls=None, extras: Optional[AttnExtras] = None):
    es = qkv.element_size()
    p = (cls or _AttnParams)()
    p.q = qkv.data_ptr()
    p.k_new = qkv.data_ptr() + nh * dh * es
    p.v_new = qkv.data_ptr() + (nh + nkvh) * dh * es
    if extras is not None:
        p.keep_first, p.pinned, p.sink = (extras.keep_first if window else 0), extras.pinned, int(extras.sink)
        if extras.sink_logits is not None:
            assert extras.sink_logits.dtype == torch.float32 and extras.sink_logits.numel() == nh
            p.sink_logits = extras.sink_logits.data_ptr()
        if extras.positional():
            if cls is not None and cls not in (_AttnParams, _MmaAttnParams):
                raise KernelError("attention: a distance penalty or a query temperature needs the CUDA-core or the mma.sync kernel")
            if extras.dist_bias is not None:
                r1, r2 = extras.dist_bias
                assert r1.dtype == r2.dtype == torch.float32 and r1.numel() == r2.numel() == nh and r1.is_cuda and r2.is_cuda
                p.dist_r1, p.dist_r2 = r1.data_ptr(), r2.data_ptr()
            if extras.q_temp is not None:
                p.q_temp_coef, p.q_temp_every = float(extras.q_temp[0]), int(extras.q_temp[1])
                if p.q_temp_every <= 0:
                    raise KernelError("attention: the query temperature's period must be positive")
        if extras.cuda_core_only():
            if cls is not None and cls not in (_AttnParams, _MmaAttnParams):
                raise KernelError("attention: chunks, several score maps, pooled blocks and float32 results need the CUDA-core or the mma.sync kernel")
            p.chunk, p.maps, p.out_f32 = int(extras.chunk), int(extras.maps), int(extras.out_f32)
            if extras.pool is not None:
                P, blocks = extras.pool
                if not window or P <= 0:
                    raise KernelError("attention: pooled blocks lie before a window; there is none")
                assert blocks.k.dtype == qkv.dtype and blocks.v is not None
                p.pool, p.pool_k, p.pool_v = int(P), blocks.k.data_ptr(), blocks.v.data_ptr()
                p.pool_table, p.pool_table_stride = blocks.page_table.data_ptr(), blocks.page_table.shape[1]
    p.row_stride = qkv.stride(0)
    p.out = out.data_ptr()
    p.kpool, p.vpool = kpool.data_ptr(), vpool.data_ptr()
    p.page_table, p.table_stride, p.ring = page_table.data_ptr(), page_table.shape[1], ring
    p.seq_start, p.seq_len_before = seq_start.data_ptr(), seq_len_before.data_ptr()
    p.nh, p.nkvh, p.window, p.scale = nh, nkvh, int(window or 0), scale
    p.all_from_cache, p.n_splits, p.part_o, p.part_ml = 0, 1, None, None
    return p


def attention_prefill(qkv, nh, nkvh, dh, kpool, vpool, page_table, ring, seq_start, seq_len_before,
                      n_seqs: int, max_new: int, window, scale, all_from_cache: bool = False,
                      tc_split: int = 0, extras: Optional[AttnExtras] = None) -> torch.Tensor:
    """Attention of the new tokens of each sequence over its cached keys (positions before the
    step) and the step's own keys, read from the packed projections `qkv` [T, (nh + 2 nkvh) dh]
    whose query and key heads are already rotated.  With all_from_cache the step's keys are
    read from the cache too (they were put there by an earlier call).  Returns [T, nh * dh].
    tc_split: CTAs per row block of the tcgen05 kernel (1, 2 or 4; 0: chosen by the number of row blocks)."""
    _need_cuda(qkv, kpool, vpool, page_table)
    assert qkv.dtype == kpool.dtype == vpool.dtype
    if extras is not None and not extras.plain(dh):
        return _attention_extras(False, qkv, nh, nkvh, dh, kpool, vpool, page_table, ring, seq_start, seq_len_before,
                                 n_seqs, max_new, window, scale, all_from_cache, 1, extras)
    out = torch.empty((qkv.shape[0], nh * dh), dtype=qkv.dtype, device=qkv.device)
    if all_from_cache and prefill_tc_ok(qkv.dtype, dh) and ring >= page_table.shape[1] and qkv.stride(0) % 8 == 0:
        _attention_prefill_tc(qkv, out, nh, nkvh, dh, kpool, vpool, page_table, seq_start, seq_len_before, n_seqs, max_new,
                              window, scale, tc_split)
        return out
    if _mma_ok(qkv, dh):
        p = _attn_params(qkv, out, nh, nkvh, dh, kpool, vpool, page_table, ring, seq_start, seq_len_before, window,
                         scale, _MmaAttnParams)
        p.all_from_cache = int(all_from_cache)
        f = _fn(_mma_lib(dh), "llb_attn_mma_prefill", [_MmaAttnParams, c_int, c_int, c_void_p])
        _check(f(p, n_seqs, max_new, _stream()), "attention_prefill (tensor cores)")
        return out
    p = _attn_params(qkv, out, nh, nkvh, dh, kpool, vpool, page_table, ring, seq_start, seq_len_before, window, scale)
    p.all_from_cache = int(all_from_cache)
    f = _fn(_attn_lib(dh), "llb_attn_prefill", [_AttnParams, c_int, c_int, c_int, c_void_p])
    _check(f(p, _dt(qkv), n_seqs, max_new, _stream()), "attention_prefill")
    return out


def _attention_prefill_tc(qkv, out, nh, nkvh, dh, kpool, vpool, page_table, seq_start, seq_len_before, n_seqs, max_new,
                          window, scale, tc_split=0, keep_first=0, sink=False):
    """The tcgen05 prefill kernel (csrc/attention_tc.cu): every key from a cache that keeps them all."""
    p = _TcAttnParams()
    p.out, p.page_table, p.table_stride = out.data_ptr(), page_table.data_ptr(), page_table.shape[1]
    p.seq_start, p.seq_len_before = seq_start.data_ptr(), seq_len_before.data_ptr()
    p.nh, p.nkvh, p.window, p.scale = nh, nkvh, int(window or 0), scale
    p.keep_first, p.sink = (int(keep_first) if window else 0), int(sink)
    p.err = _tc_resources(qkv.device)[2].data_ptr()
    # few row blocks (up to one and a half per SM): two CTAs share each block's key range, so that the longest
    # CTA gets shorter (measured at 12 heads: 30.5 vs 33.7 us at 2,048 tokens, 73 vs 64 us at 4,096; four CTAs
    # per block always lost to the cost of the merge)
    ctas = -(-max_new // 128) * nh * n_seqs
    p.n_split = tc_split if tc_split else (2 if ctas * 2 <= 3 * _sm_count(qkv.device) and dh >= 64 else 1)
    f = _fn(load_module("attention_tc.cu", {"LLB_HEAD_DIM": dh}), "llb_attn_tc_prefill",
            [c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, _TcAttnParams, c_int, c_int, c_void_p])
    _check(f(qkv.data_ptr(), qkv.shape[0], qkv.stride(0), kpool.data_ptr(), vpool.data_ptr(), kpool.shape[0],
             p, n_seqs, max_new, _stream()), "attention_prefill (tcgen05)")


def attention_decode(qkv, nh, nkvh, dh, kpool, vpool, page_table, ring, seq_start, seq_len_before,
                     n_seqs: int, window, scale, n_splits: int = 1, rope=None, append_new: bool = False,
                     extras: Optional[AttnExtras] = None) -> torch.Tensor:
    """Attention of one new token per sequence over the cache.

    By default the new token's (rotated) key and value are already in the cache.  Where
    decode_fusion_ok() holds, the kernel can do that work itself: rope = (cos, sin) tables makes it
    rotate the query heads (and the new key), append_new makes it take the new key and value from
    `qkv`, use them and write them to the cache."""
    _need_cuda(qkv, kpool, vpool, page_table)
    assert qkv.dtype == kpool.dtype == vpool.dtype
    if extras is not None and not extras.plain(dh):
        if rope is not None or append_new:
            raise KernelError("attention_decode: the fused rotation / append is not available with these options")
        return _attention_extras(True, qkv, nh, nkvh, dh, kpool, vpool, page_table, ring, seq_start, seq_len_before,
                                 n_seqs, 1, window, scale, True, n_splits, extras)
    out = torch.empty((qkv.shape[0], nh * dh), dtype=qkv.dtype, device=qkv.device)
    mma = _mma_ok(qkv, dh)
    p = _attn_params(qkv, out, nh, nkvh, dh, kpool, vpool, page_table, ring, seq_start, seq_len_before, window, scale,
                     _MmaAttnParams if mma else None)
    if (rope is not None or append_new) and not mma:
        raise KernelError("attention_decode: the fused rotation / append needs the tensor-core kernel (see decode_fusion_ok)")
    keep = None
    if mma:
        n_splits = min(n_splits, 64)
        if rope is not None:
            p.rope_cos, p.rope_sin, p.rope_rows = rope[0].data_ptr(), rope[1].data_ptr(), rope[0].shape[0]
        p.append_new = int(append_new)
        p.cluster = int(1 < n_splits <= 8 or n_splits == 16)      # few slices merge inside a cluster, through shared memory
        p.err = _tc_resources(qkv.device)[2].data_ptr()           # a bounded wait of that merge that runs out says so here
    p.n_splits = n_splits
    if n_splits > 1 and not (mma and p.cluster):
        part_o = torch.empty((n_seqs, nh, n_splits, dh), dtype=torch.float32, device=qkv.device)
        part_ml = torch.empty((n_seqs, nh, n_splits, 2), dtype=torch.float32, device=qkv.device)
        p.n_splits, p.part_o, p.part_ml = n_splits, part_o.data_ptr(), part_ml.data_ptr()
        keep = (part_o, part_ml)
    if mma:
        f = _fn(_mma_lib(dh), "llb_attn_mma_decode", [_MmaAttnParams, c_int, c_void_p])
        _check(f(p, n_seqs, _stream()), "attention_decode (tensor cores)", 2 if (n_splits > 1 and not p.cluster) else 1)
    else:
        f = _fn(_attn_lib(dh), "llb_attn_decode", [_AttnParams, c_int, c_int, c_void_p])
        _check(f(p, _dt(qkv), n_seqs, _stream()), "attention_decode", 2 if n_splits > 1 else 1)
    del keep
    return out


def _attention_extras(decode, qkv, nh, nkvh, dh, kpool, vpool, page_table, ring, seq_start, seq_len_before, n_seqs,
                      max_new, window, scale, all_from_cache, n_splits, extras: AttnExtras) -> torch.Tensor:
    """Attention with AttnExtras.  qkv holds nh query heads of dh, then (unless everything comes from the cache) nkvh key
    heads of dh and nkvh value heads of value_dim."""
    dv = extras.value_dim or dh
    out = torch.empty((qkv.shape[0], nh * dv), dtype=torch.float32 if extras.out_f32 else qkv.dtype, device=qkv.device)
    only_simt = extras.cuda_core_only()
    if (not only_simt and not decode and dv == dh and all_from_cache and prefill_tc_ok(qkv.dtype, dh) and not extras.pinned and scale > 0
            and extras.sink_logits is None and not extras.positional()
            and ring >= page_table.shape[1] and qkv.stride(0) % 8 == 0):
        # a cache that keeps every key, head size 64 or 128: the tcgen05 prefill kernel, as for the plain attention
        _attention_prefill_tc(qkv, out, nh, nkvh, dh, kpool, vpool, page_table, seq_start, seq_len_before, n_seqs, max_new,
                              window, scale, 0, extras.keep_first, extras.sink)
        return out
    if (only_simt and not decode and prefill_ext_ok(qkv, dh, dv) and not extras.keep_first and not extras.sink
            and extras.sink_logits is None and (extras.pool is None or not extras.positional())
            and not ((kpool.data_ptr() | vpool.data_ptr() | out.data_ptr()) & 15)):
        # prompts in bfloat16: the mma.sync prefill kernel with its extensions (a block owns one half of values twice as
        # wide as the keys, and repeats the scores for it)
        p = _attn_params(qkv, out, nh, nkvh, dh, kpool, vpool, page_table, ring, seq_start, seq_len_before, window, scale,
                         _MmaAttnParams, extras=extras)
        p.all_from_cache, p.v_split = int(all_from_cache), dv // dh
        f = _fn(_mma_lib(dh), "llb_attn_mma_prefill", [_MmaAttnParams, c_int, c_int, c_void_p])
        _check(f(p, n_seqs, max_new, _stream()), "attention_prefill (tensor cores)")
        return out
    if not only_simt and dv == dh and _mma_ok(qkv, dh):
        # keys and values of one width that the tensor-core kernel takes: the same kernels as the plain attention
        # (a distance penalty and a query temperature are applied to the score fragments in registers)
        p = _attn_params(qkv, out, nh, nkvh, dh, kpool, vpool, page_table, ring, seq_start, seq_len_before, window, scale,
                         _MmaAttnParams, extras=extras)
        p.all_from_cache = int(all_from_cache)
        if not decode:
            f = _fn(_mma_lib(dh), "llb_attn_mma_prefill", [_MmaAttnParams, c_int, c_int, c_void_p])
            _check(f(p, n_seqs, max_new, _stream()), "attention_prefill (tensor cores)")
            return out
        n_splits = min(n_splits, 64)
        p.cluster = int(1 < n_splits <= 8 or n_splits == 16)
        p.err = _tc_resources(qkv.device)[2].data_ptr()
        p.n_splits = n_splits
        keep = None
        if n_splits > 1 and not p.cluster:
            part_o = torch.empty((n_seqs, nh, n_splits, dh), dtype=torch.float32, device=qkv.device)
            part_ml = torch.empty((n_seqs, nh, n_splits, 2), dtype=torch.float32, device=qkv.device)
            p.part_o, p.part_ml = part_o.data_ptr(), part_ml.data_ptr()
            keep = (part_o, part_ml)
        f = _fn(_mma_lib(dh), "llb_attn_mma_decode", [_MmaAttnParams, c_int, c_void_p])
        _check(f(p, n_seqs, _stream()), "attention_decode (tensor cores)", 2 if (n_splits > 1 and not p.cluster) else 1)
        del keep
        return out
    p = _attn_params(qkv, out, nh, nkvh, dh, kpool, vpool, page_table, ring, seq_start, seq_len_before, window, scale,
                     extras=extras)
    p.v_new = qkv.data_ptr() + (nh + nkvh) * dh * qkv.element_size()
    p.all_from_cache = int(all_from_cache)
    lib = _attn_lib(dh, dv)
    if not decode:
        f = _fn(lib, "llb_attn_prefill", [_AttnParams, c_int, c_int, c_int, c_void_p])
        _check(f(p, _dt(qkv), n_seqs, max_new, _stream()), "attention_prefill")
        return out
    keep = None
    p.n_splits = n_splits
    if n_splits > 1:
        part_o = torch.empty((n_seqs, nh, n_splits, dv), dtype=torch.float32, device=qkv.device)
        part_ml = torch.empty((n_seqs, nh, n_splits, 2), dtype=torch.float32, device=qkv.device)
        p.part_o, p.part_ml = part_o.data_ptr(), part_ml.data_ptr()
        keep = (part_o, part_ml)
    f = _fn(lib, "llb_attn_decode", [_AttnParams, c_int, c_int, c_void_p])
    _check(f(p, _dt(qkv), n_seqs, _stream()), "attention_decode", 2 if n_splits > 1 else 1)
    del keep
    return out


# ------------------------------------------------------------------ routed experts
def _moe_lib():
    return load_module("moe.cu")


_moe_tile = None


def moe_tile_rows() -> int:
    global _moe_tile
    if _moe_tile is None:
        f = _moe_lib().llb_moe_tile_rows
        f.argtypes, f.restype = [], c_int
        _moe_tile = int(f())
    return _moe_tile


MOE_GATES = {"sigmoid": 0, "softmax_chosen": 1}


def moe_route(x: torch.Tensor, router: torch.Tensor, bias: Optional[torch.Tensor], top: int, route_scale: float,
              gate: str = "sigmoid", n_experts: Optional[int] = None, with_logits: bool = False, groups: Optional[tuple] = None,
              renorm: bool = False):
    """(int32 [T, top] experts, float32 [T, top] weights): the router's logits x router^T in float32 (a matrix product
    with float32 accumulation: on the tensor cores for bfloat16 operands, on the CUDA cores in float32).  gate "sigmoid":
    gates sigmoid(logits); the `top` largest of gate + bias are chosen (first maximum first); a weight is
    gate * route_scale.  gate "softmax_chosen": the `top` largest logits (+ bias) are chosen and the weights are the softmax
    over the chosen logits alone, times route_scale.  n_experts: the router's matrix has further rows after the experts'
    (other per-token logits that ride on the same product); with_logits also returns all logits [T, rows] (float32).
    groups = (count, keep): the experts form `count` equal groups of neighbours, a group's score is the sum of its two
    largest choice scores, and only experts of the `keep` best groups can be chosen.  renorm (gate "sigmoid"): the chosen
    gates are divided by their sum (+ 1e-20) before route_scale is applied."""
    _need_cuda(x, router, bias)
    T, H = x.shape
    rows = router.shape[0]
    E = rows if n_experts is None else int(n_experts)
    assert router.shape == (rows, H) and E <= rows and router.is_contiguous() and x.stride(1) == 1
    assert bias is None or (bias.dtype == torch.float32 and bias.numel() == E)
    plan = None
    if T > 256 and _tc_ok(x, router, None):
        # many tokens against a handful of rows: tiles of 64 tokens and the K range cut over a cluster, so that the
        # product runs on more than T / 256 blocks
        tiles, kblocks = -(-T // 64) * -(-rows // 128), -(-H // 64)
        splits = max([s for s in (1, 2, 4, 8) if s == 1 or (tiles * s <= 2 * _sm_count(x.device) and s <= kblocks // 2)])
        plan = (64, splits)
    z = linear(x, router, out_dtype=torch.float32, plan=plan)
    idx = torch.empty((T, top), dtype=torch.int32, device=x.device)
    wgt = torch.empty((T, top), dtype=torch.float32, device=x.device)
    n_groups, keep_groups = (int(groups[0]), int(groups[1])) if groups else (1, 1)
    if n_groups > 1 and (E % n_groups or not (1 <= keep_groups <= n_groups) or n_groups > 64):
        raise KernelError(f"router: {E} experts in {n_groups} groups of which {keep_groups} are kept cannot be (equal groups, at most 64)")
    f = _fn(_moe_lib(), "llb_moe_select", [c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_float, c_void_p, c_void_p, c_int,
                                           c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(z), z.stride(0), _ptr(bias), T, E, top, route_scale, _ptr(idx), _ptr(wgt), MOE_GATES[gate], n_groups, keep_groups,
             int(renorm), _stream()), "router's choice")
    return (idx, wgt, z) if with_logits else (idx, wgt)


class MoePlan:
    """(token, choice) pairs grouped by expert; see csrc/moe.cu."""
    __slots__ = ("slot_of", "pair_of", "tiles", "n_tiles", "max_tiles", "top", "n_pairs", "tile_rows")


def moe_plan(idx: torch.Tensor, n_experts: int, tile_rows: Optional[int] = None) -> MoePlan:
    """tile_rows: slots of a tile (default: what the CUDA-core product takes, 64)."""
    _need_cuda(idx)
    T, top = idx.shape
    N = T * top
    p = MoePlan()
    p.top, p.n_pairs, p.tile_rows = top, N, int(tile_rows or moe_tile_rows())
    p.max_tiles = N // p.tile_rows + min(n_experts, N)       # an expert that has pairs ends in one partial tile at most
    buf = torch.empty(2 * N + 3 * p.max_tiles + 1, dtype=torch.int32, device=idx.device)
    p.slot_of, p.pair_of = buf[:N], buf[N:2 * N]
    p.tiles, p.n_tiles = buf[2 * N:2 * N + 3 * p.max_tiles], buf[2 * N + 3 * p.max_tiles:]
    f = _fn(_moe_lib(), "llb_moe_plan", [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p])
    _check(f(_ptr(idx), N, n_experts, p.tile_rows, _ptr(p.slot_of), _ptr(p.pair_of), _ptr(p.tiles), p.max_tiles, _ptr(p.n_tiles),
             _stream()), "expert plan")
    return p


def moe_gemm(a: torch.Tensor, w: torch.Tensor, plan: MoePlan, gather: bool, act: Optional[str], out_dtype: torch.dtype) -> torch.Tensor:
    """out[slot] = act(a[row(slot)] w[expert(slot)]^T) for every slot of the plan; w is [E, N, K].  gather: `a` holds the
    tokens' rows [T, K] and a slot's row is its pair's token; else `a` is [slots, K].  act: None, "relu_squared" or "gelu"
    (the erf form)."""
    _need_cuda(a, w)
    E, N, K = w.shape
    assert w.is_contiguous() and a.stride(1) == 1 and a.shape[1] == K and plan.tile_rows <= moe_tile_rows()
    out = torch.empty((plan.n_pairs, N), dtype=out_dtype, device=a.device)
    f = _fn(_moe_lib(), "llb_moe_gemm", [c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_void_p, c_int, c_void_p, c_int, c_int,
                                         c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(a), _dt(a), a.stride(0), _ptr(plan.pair_of), plan.top, int(gather), _ptr(w), _dt(w), _ptr(out), DT[out_dtype],
             out.stride(0), _ptr(plan.tiles), plan.max_tiles, _ptr(plan.n_tiles), N, K, {None: 0, "relu_squared": 1, "gelu": 2}[act],
             _stream()), "experts' product")
    return out


def moe_tc_ok(x: torch.Tensor, up: torch.Tensor, down: torch.Tensor) -> bool:
    """True when the experts' products of these operands run on the tensor cores (csrc/moe_tc.cu): bfloat16, both
    reduction lengths multiples of 8, 16-byte aligned bases."""
    return (TC_ENABLED and x.is_cuda and x.dtype == up.dtype == down.dtype == torch.bfloat16 and up.shape[2] % 8 == 0
            and down.shape[2] % 8 == 0 and not ((up.data_ptr() | down.data_ptr()) & 15))


def moe_tc_tile_rows(n_pairs: int, n_experts: int) -> int:
    """Slots of a tile of the tensor-core product: 16, 64 or 128 by the pairs an expert gets on average (a function of
    the step's shape alone)."""
    avg = n_pairs / max(1, n_experts)
    return 16 if avg <= 16 else 64 if avg <= 96 else 128


def moe_gather_rows(x: torch.Tensor, plan: MoePlan) -> torch.Tensor:
    """[slots, H]: row slot is the row of x [T, H] of the slot's token."""
    _need_cuda(x)
    assert x.stride(1) == 1
    out = torch.empty((plan.n_pairs, x.shape[1]), dtype=x.dtype, device=x.device)
    f = _fn(_moe_lib(), "llb_moe_gather_rows", [c_void_p, c_int, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p])
    _check(f(_ptr(x), _dt(x), x.stride(0), _ptr(plan.pair_of), plan.top, _ptr(out), plan.n_pairs, x.shape[1], _stream()),
           "experts' rows in slot order")
    return out


def moe_gemm_tc(a: torch.Tensor, w: torch.Tensor, plan: MoePlan, epilogue: str, out: Optional[torch.Tensor] = None,
                wgt: Optional[torch.Tensor] = None, out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """The experts' product on tcgen05 over activations in slot order a [slots, K] (bfloat16), w [E, N, K].
    epilogue "store" / "relu_squared" / "gelu" (erf form): returns [slots, N] in out_dtype; "weighted_add": `out` is the float32 stream
    [T, N] and row token(slot) gets wgt[pair(slot)] * product added (float32 atomics)."""
    _need_cuda(a, w, out, wgt)
    E, N, K = w.shape
    assert w.is_contiguous() and a.stride(1) == 1 and a.shape == (plan.n_pairs, K) and a.dtype == w.dtype == torch.bfloat16
    assert plan.max_tiles and plan.tile_rows in (16, 64, 128)
    code = {"store": 0, "relu_squared": 1, "weighted_add": 2, "gelu": 3}[epilogue]
    if code == 2:
        assert out is not None and out.dtype == torch.float32 and out.stride(1) == 1 and out.shape[1] == N and wgt is not None
    else:
        out = torch.empty((plan.n_pairs, N), dtype=out_dtype, device=a.device)
    err = _tc_resources(a.device)[2]
    f = _fn(load_module("moe_tc.cu"), "llb_moe_gemm_tc",
            [c_void_p, c_int, c_longlong, c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_int, c_void_p, c_int, c_void_p, c_int,
             c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p])
    _check(f(_ptr(a), a.stride(0), plan.n_pairs, _ptr(w), E, N, K, _ptr(out), _dt(out), out.stride(0), _ptr(plan.tiles),
             plan.max_tiles, _ptr(plan.n_tiles), plan.tile_rows, code, _ptr(plan.pair_of), _ptr(wgt), plan.top, _ptr(err), _stream()),
           "experts' product (tensor cores)")
    return out


def moe_combine(stream: torch.Tensor, y: torch.Tensor, plan: MoePlan, wgt: torch.Tensor) -> None:
    """stream[t] += sum_k wgt[t, k] * y[slot_of[t, k]] (float32 stream, k in order)."""
    _need_cuda(stream, y, wgt)
    T, H = stream.shape
    assert stream.dtype == torch.float32 and stream.is_contiguous() and y.shape[1] == H and y.stride(1) == 1
    f = _fn(_moe_lib(), "llb_moe_combine", [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(stream), _ptr(y), _dt(y), y.stride(0), _ptr(plan.slot_of), _ptr(wgt), T, plan.top, H, _stream()),
           "experts' weighted sum")


# ------------------------------------------------------------------ choice of the next token
_argmax_counters = {}          # device -> int32 [4096], zero between launches (the split arg-max's per-row counters)


def argmax(logits: torch.Tensor) -> torch.Tensor:
    """int32 index of the first maximum of every row of float32 logits [R, V]."""
    _need_cuda(logits)
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    R, V = logits.shape
    out = torch.empty((R,), dtype=torch.int32, device=logits.device)
    # few rows of a wide vocabulary: several blocks share a row, so that the device's SMs all read
    parts = min(64, (2 * _sm_count(logits.device)) // max(R, 1), V // 2048)
    if parts >= 2 and R <= 4096:
        counters = _argmax_counters.get(logits.device)
        if counters is None:
            counters = _argmax_counters[logits.device] = torch.zeros(4096, dtype=torch.int32, device=logits.device)
        part = torch.empty((R * parts, 2), dtype=torch.int32, device=logits.device)
        f = _fn(load_module("sampling.cu"), "llb_argmax_split",
                [c_void_p, c_longlong, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p])
        _check(f(_ptr(logits), logits.stride(0), R, V, parts, _ptr(part), _ptr(counters), _ptr(out), _stream()), "argmax")
        return out
    f = _fn(load_module("sampling.cu"), "llb_argmax", [c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p])
    _check(f(_ptr(logits), logits.stride(0), R, V, _ptr(out), _stream()), "argmax")
    return out


def sample(logits: torch.Tensor, temperature: float, top_k: int, top_p: float, seed: int,
           keys: Optional[torch.Tensor] = None, steps: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One token per row of float32 logits [R, V]; see csrc/sampling.cu for the rule.  keys and
    steps (int32 [R]) are the request number and the number of tokens the request has drawn."""
    _need_cuda(logits, keys, steps)
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    R, V = logits.shape
    out = torch.empty((R,), dtype=torch.int32, device=logits.device)
    f = _fn(load_module("sampling.cu"), "llb_sample",
            [c_void_p, c_longlong, c_int, c_int, c_void_p, c_float, c_int, c_float, c_ulonglong,
             c_void_p, c_void_p, c_void_p])
    _check(f(_ptr(logits), logits.stride(0), R, V, _ptr(out), temperature, top_k, top_p,
             seed & 0xFFFFFFFFFFFFFFFF, _ptr(keys), _ptr(steps), _stream()), "sample")
    return out


def uniform(seed: int, key: int, step: int) -> float:
    """The uniform in [0, 1) that `sample` uses for (seed, key, step) (splitmix64 finaliser)."""
    mask, G = 0xFFFFFFFFFFFFFFFF, 0x9E3779B97F4A7C15

    def mix(z):
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & mask
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & mask
        return z ^ (z >> 31)

    z = mix((mix((seed + G * (key + 1)) & mask) + G * (step + 1)) & mask)
    return (z >> 11) / 9007199254740992.0
