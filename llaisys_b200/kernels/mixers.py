"""Python faces of the kernels of the recurrent and the latent mixers (csrc/gla.cu, csrc/latent.cu, and the CUDA-core
attention kernel of csrc/attention_simt.cu run over a cache of latent rows)."""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_void_p
from typing import Optional

import torch

from ..csrc.build import load_module
from .ops import DT, KernelError, _AttnParams, _attn_lib, _check, _dt, _fn, _need_cuda, _ptr, _sm_count, _stream


class _GlaParams(ctypes.Structure):
    _fields_ = [("q", c_void_p), ("k", c_void_p), ("v", c_void_p), ("row_stride", c_int), ("z", c_void_p), ("z_stride", c_int),
                ("state", c_void_p), ("seq_start", c_void_p), ("seq_slot", c_void_p), ("out", c_void_p), ("H", c_int),
                ("dk", c_int), ("dv", c_int), ("q_scale", c_float), ("inv_tau", c_float), ("z_is_decay", c_int),
                ("head_decay", c_void_p), ("act", c_int)]


GLA_MAX_KEY_DIM = 256


def gla_scan(proj: torch.Tensor, H: int, dk: int, dv: int, z: Optional[torch.Tensor], state: torch.Tensor, seq_start: torch.Tensor,
             seq_slot: torch.Tensor, n_seqs: int, q_scale: float, decay_root: float, head_decay: Optional[torch.Tensor] = None,
             act: Optional[str] = None) -> torch.Tensor:
    """The gated-linear-attention recurrence over the new tokens of every sequence: proj [T, >= 2 H dk + H dv] holds the
    heads' queries, then keys, then values; z [T, H dk] (float32) the decay logits; state [slots, H dk dv] (float32) is
    read at row seq_slot[b] and left holding the state after the step.  Returns o [T, H dv] in float32.  For more than
    64 tokens the decays are formed by a pass of their own over z (in place), once per token and channel.
    head_decay (float32 [H]) instead of z: one constant decay per head, S <- decay_h S + k v^T.  act "silu": q, k and v
    pass through silu (in float32) on their way into the recurrence."""
    _need_cuda(proj, z, state, head_decay)
    assert (z is None) != (head_decay is None)
    assert z is None or (z.dtype == torch.float32 and z.stride(1) == 1)
    assert head_decay is None or (head_decay.dtype == torch.float32 and head_decay.numel() == H and head_decay.is_contiguous())
    assert state.dtype == torch.float32 and state.is_contiguous()
    assert proj.stride(1) == 1 and state.shape[1] == H * dk * dv
    if dk > GLA_MAX_KEY_DIM:
        raise KernelError(f"gated linear attention: {dk} key channels a head; the kernel takes up to {GLA_MAX_KEY_DIM}")
    T = proj.shape[0]
    out = torch.empty((T, H * dv), dtype=torch.float32, device=proj.device)
    p = _GlaParams()
    es = proj.element_size()
    p.q, p.k, p.v = proj.data_ptr(), proj.data_ptr() + H * dk * es, proj.data_ptr() + 2 * H * dk * es
    p.row_stride, p.z, p.z_stride = proj.stride(0), _ptr(z), z.stride(0) if z is not None else 0
    p.head_decay, p.act = _ptr(head_decay), {None: 0, "silu": 1}[act]
    p.state, p.seq_start, p.seq_slot, p.out = state.data_ptr(), seq_start.data_ptr(), seq_slot.data_ptr(), out.data_ptr()
    p.H, p.dk, p.dv, p.q_scale, p.inv_tau = H, dk, dv, q_scale, 1.0 / decay_root
    if z is not None and T > 64 and z.is_contiguous():
        g = _fn(load_module("gla.cu"), "llb_gla_decay", [c_void_p, ctypes.c_longlong, c_float, c_void_p])
        _check(g(_ptr(z), z.numel(), 1.0 / decay_root, _stream()), "gated linear attention (decays)")
        p.z_is_decay = 1
    f = _fn(load_module("gla.cu"), "llb_gla_scan", [_GlaParams, c_int, c_int, c_int, c_void_p])
    _check(f(p, _dt(proj), n_seqs, _sm_count(proj.device), _stream()), "gated linear attention (recurrence)")
    return out


SCAN_CHUNK = 64               # tokens of a chunk of a long step of the constant-decay recurrence
SCAN_CHUNKED_FROM = 256       # steps whose longest sequence brings at least this many tokens run chunk by chunk


def scan_chunks(n_new, device, chunk: int = SCAN_CHUNK):
    """The chunks of a step whose sequences bring n_new[b] tokens: int32 device tensors chunk_start [NC + 1] (first packed
    token of every chunk), chunk_len [NC], seq_chunk0 [B + 1] (first chunk of every sequence), chunk_row [NC] (0 .. NC - 1)."""
    starts, lens, seq0, at = [], [], [0], 0
    for n in n_new:
        for c0 in range(0, n, chunk):
            starts.append(at + c0)
            lens.append(min(chunk, n - c0))
        at += n
        seq0.append(len(starts))
    starts.append(at)
    flat = torch.tensor(starts + lens + seq0 + list(range(len(lens))), dtype=torch.int32).to(device)
    nc, b = len(lens), len(n_new)
    return flat[:nc + 1], flat[nc + 1:2 * nc + 1], flat[2 * nc + 1:2 * nc + 2 + b], flat[2 * nc + 2 + b:]


def gla_scan_chunked(proj: torch.Tensor, H: int, dk: int, dv: int, state: torch.Tensor, seq_slot: torch.Tensor, n_seqs: int,
                     head_decay: torch.Tensor, chunks, act: Optional[str] = None) -> torch.Tensor:
    """The constant-decay recurrence (gla_scan with head_decay) of a long step, its chunks side by side: the recurrence over
    every chunk from a zero state, one pass that turns the chunks' local states into the states they start with (and
    leaves the sequences' states as the step ends them), and the recurrence over every chunk again.  chunks: scan_chunks()
    of the step.  Returns o [T, H dv] in float32; differs from the token-by-token walk by float32 rounding only."""
    chunk_start, chunk_len, seq_chunk0, chunk_row = chunks
    nc = chunk_len.numel()
    n_state = H * dk * dv
    tmp = torch.zeros((nc, n_state), dtype=torch.float32, device=proj.device)
    gla_scan(proj, H, dk, dv, None, tmp, chunk_start, chunk_row, nc, 1.0, 1.0, head_decay=head_decay, act=act)
    f = _fn(load_module("gla.cu"), "llb_gla_chunk_prefix", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                                           c_int, c_void_p])
    _check(f(_ptr(tmp), _ptr(state), _ptr(seq_chunk0), _ptr(chunk_len), _ptr(seq_slot), _ptr(head_decay), dk * dv, n_state, n_seqs,
             _stream()), "constant-decay recurrence (chunks' starting states)")
    return gla_scan(proj, H, dk, dv, None, tmp, chunk_start, chunk_row, nc, 1.0, 1.0, head_decay=head_decay, act=act)


def gla_out(o: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor, H: int, dv: int, eps: float,
            out_dtype: torch.dtype, gate_act: str = "silu") -> torch.Tensor:
    """[T, H dv]: every head's o (float32) RMS-normed over its dv channels with `weight` [dv], times silu(gate) (gate a
    [T, H dv] view with any row stride, in the output's dtype)."""
    _need_cuda(o, gate, weight)
    T = o.shape[0]
    assert o.dtype == torch.float32 and o.is_contiguous() and gate.dtype == out_dtype and gate.stride(1) == 1
    out = torch.empty((T, H * dv), dtype=out_dtype, device=o.device)
    f = _fn(load_module("gla.cu"), "llb_gla_out", [c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int,
                                                  c_int, c_float, c_int, c_void_p])
    _check(f(_ptr(o), _ptr(gate), gate.stride(0), _ptr(weight), _dt(weight), _ptr(out), DT[out_dtype], T, H, dv, eps,
             {"silu": 0, "sigmoid": 1}[gate_act], _stream()),
           "gated linear attention (head norm and gate)")
    return out


class _MinGruParams(ctypes.Structure):
    _fields_ = [("proj", c_void_p), ("ld", c_int), ("a_off", c_int), ("u_off", c_int), ("g_off", c_int), ("width", c_int),
                ("state", c_void_p), ("seq_start", c_void_p), ("seq_slot", c_void_p), ("out", c_void_p), ("chunk_a", c_void_p),
                ("chunk_b", c_void_p), ("chunk", c_int), ("n_chunks", c_int)]


MINGRU_CHUNK = 64            # tokens of a chunk of a long step (256 beyond 4,096 tokens a sequence)


def mingru(proj: torch.Tensor, width: int, state: torch.Tensor, seq_start: torch.Tensor, seq_slot: torch.Tensor, n_seqs: int,
           max_new: int, out_dtype: torch.dtype, offsets=None) -> torch.Tensor:
    """The minGRU recurrence over the new tokens of every sequence: proj [T, >= 3 width] holds the gate logits, the
    candidate inputs and the output gate (`offsets` = their first columns, default 0, width, 2 width), biases included;
    state [slots, width] (float32) is read at row seq_slot[b] and left holding the state after the step.  Returns
    y [T, width] = state_t * silu(output gate) in out_dtype.  Steps of more than one chunk of tokens a sequence are cut
    into chunks that run side by side (three launches instead of one)."""
    _need_cuda(proj, state)
    assert proj.stride(1) == 1 and state.dtype == torch.float32 and state.is_contiguous() and state.shape[1] == width
    T = proj.shape[0]
    a_off, u_off, g_off = offsets or (0, width, 2 * width)
    out = torch.empty((T, width), dtype=out_dtype, device=proj.device)
    p = _MinGruParams()
    p.proj, p.ld, p.a_off, p.u_off, p.g_off, p.width = proj.data_ptr(), proj.stride(0), a_off, u_off, g_off, width
    p.state, p.seq_start, p.seq_slot, p.out = state.data_ptr(), seq_start.data_ptr(), seq_slot.data_ptr(), out.data_ptr()
    p.chunk = MINGRU_CHUNK if max_new <= 4096 else 256
    p.n_chunks = -(-max_new // p.chunk)
    scratch, launches = None, 1
    if p.n_chunks > 1:
        scratch = torch.empty((2, n_seqs, p.n_chunks, width), dtype=torch.float32, device=proj.device)
        p.chunk_a, p.chunk_b = scratch[0].data_ptr(), scratch[1].data_ptr()
        launches = 3
    f = _fn(load_module("mingru.cu"), "llb_mingru", [_MinGruParams, c_int, c_int, c_int, c_void_p])
    _check(f(p, _dt(proj), DT[out_dtype], n_seqs, _stream()), "minGRU recurrence", launches)
    del scratch
    return out


class _LatentPrepParams(ctypes.Structure):
    _fields_ = [("proj", c_void_p), ("row_stride", c_int), ("q_off", c_int), ("q_rank", c_int), ("kv_off", c_int),
                ("kv_rank", c_int), ("kr_off", c_int), ("rope_dim", c_int), ("rot", c_int), ("wq", c_void_p), ("wkv", c_void_p),
                ("eps", c_float), ("cos_t", c_void_p), ("sin_t", c_void_p), ("table_rows", c_int), ("tok_pos", c_void_p),
                ("q_out", c_void_p), ("kv_out", c_void_p), ("append", c_int), ("tok_seq", c_void_p), ("seq_start", c_void_p),
                ("seq_len_before", c_void_p), ("pool", c_void_p), ("page_table", c_void_p), ("table_stride", c_int),
                ("ring", c_int), ("pinned", c_int), ("err", c_void_p), ("halves", c_int)]


def latent_prep(proj: torch.Tensor, q_rank: int, kv_rank: int, rope_dim: int, wq: Optional[torch.Tensor], wkv: Optional[torch.Tensor],
                eps: float, tables, tok_pos: torch.Tensor, err: torch.Tensor, append: Optional[dict] = None, halves: bool = False,
                kv_off: Optional[int] = None):
    """From the fused down projections proj [T, q_rank (+ kv_rank + rope_dim) ...]: the RMS-normed query latent
    [T, q_rank] and, when the layer projects its own (wkv given), the rows [normed latent | rotated shared key part]
    [T, kv_rank + rope_dim]; tables = (cos, sin, rotated dims) or None.  append = dict(tok_seq, seq_start,
    seq_len_before, pool, page_table, ring, pinned) also writes those rows into the paged cache.  halves: the rotated
    pairs are (i, i + dims / 2) instead of (2i, 2i + 1).  q_rank 0 (wq None): the layer has no query latent; kv_off then
    says where the key/value latent's columns start (default: after the query latent)."""
    _need_cuda(proj, wq, wkv, tok_pos)
    T = proj.shape[0]
    assert proj.stride(1) == 1 and tok_pos.numel() == T
    own = wkv is not None
    assert (q_rank > 0) == (wq is not None) and (own or q_rank > 0)
    q_out = torch.empty((T, q_rank), dtype=proj.dtype, device=proj.device) if q_rank > 0 else None
    kv_out = torch.empty((T, kv_rank + rope_dim), dtype=proj.dtype, device=proj.device) if own else None
    p = _LatentPrepParams()
    p.proj, p.row_stride, p.q_off, p.q_rank = proj.data_ptr(), proj.stride(0), 0, q_rank
    off = q_rank if kv_off is None else int(kv_off)
    p.kv_off, p.kv_rank, p.kr_off, p.rope_dim = off, kv_rank if own else 0, off + kv_rank, rope_dim
    p.wq, p.wkv, p.eps, p.halves = _ptr(wq), _ptr(wkv), eps, int(halves)
    if own and wq is not None and wkv.dtype != wq.dtype:
        raise KernelError("latent_prep: the two norm weights must have one dtype")
    if tables is not None and own:
        cos, sin, rot = tables
        p.cos_t, p.sin_t, p.table_rows, p.rot = cos.data_ptr(), sin.data_ptr(), cos.shape[0], rot
    p.tok_pos, p.q_out, p.kv_out, p.err = tok_pos.data_ptr(), _ptr(q_out), _ptr(kv_out), err.data_ptr()
    if append is not None and own:
        a = append
        p.append, p.tok_seq, p.seq_start, p.seq_len_before = 1, a["tok_seq"].data_ptr(), a["seq_start"].data_ptr(), a["seq_len_before"].data_ptr()
        p.pool, p.page_table, p.table_stride = a["pool"].data_ptr(), a["page_table"].data_ptr(), a["page_table"].shape[1]
        p.ring, p.pinned = a["ring"], a.get("pinned", 0)
    f = _fn(load_module("latent.cu"), "llb_latent_prep", [_LatentPrepParams, c_int, c_int, c_int, c_void_p])
    _check(f(p, _dt(proj), _dt(wq if wq is not None else wkv), T, _stream()), "latent attention (norms, key rotation, cache rows)")
    return q_out, kv_out


def latent_append(rows: torch.Tensor, tok_pos: torch.Tensor, append: dict) -> None:
    """rows [T, width] into the tokens' rows of the paged cache (a pool of one key head of `width` elements)."""
    _need_cuda(rows, tok_pos)
    assert rows.is_contiguous()
    a = append
    f = _fn(load_module("latent.cu"), "llb_latent_append", [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                                            c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(rows), _dt(rows), rows.shape[0], rows.shape[1], _ptr(tok_pos), _ptr(a["tok_seq"]), _ptr(a["seq_start"]),
             _ptr(a["seq_len_before"]), _ptr(a["pool"]), _ptr(a["page_table"]), a["page_table"].shape[1], a["ring"],
             a.get("pinned", 0), _stream()), "latent attention (cache append)")


class _HeadMatmulParams(ctypes.Structure):
    _fields_ = [("x", c_void_p), ("x_stride", c_int), ("x_head", c_int), ("m", c_void_p), ("y", c_void_p), ("y_stride", c_int),
                ("y_head", c_int), ("T", c_int), ("H", c_int), ("n_in", c_int), ("n_out", c_int), ("tail", c_int), ("rot", c_int),
                ("cos_t", c_void_p), ("sin_t", c_void_p), ("table_rows", c_int), ("tok_pos", c_void_p), ("gate", c_void_p),
                ("gate_stride", c_int), ("err", c_void_p), ("halves", c_int), ("gate_elems", c_int)]


def head_matmul(x: torch.Tensor, m: torch.Tensor, *, tail: int = 0, tables=None, tok_pos=None, gate: Optional[torch.Tensor] = None,
                err: Optional[torch.Tensor] = None, halves: bool = False, gate_elems: bool = False) -> torch.Tensor:
    """y[t, h, :n_out] = x[t, h, :n_in] m[h] for x [T, H (n_in + tail)] and m [H, n_in, n_out], float32 accumulation; the
    `tail` elements after a head's inputs follow its outputs in y [T, H (n_out + tail)], the first `rot` of them rotated in
    pairs (2i, 2i+1) by tables = (cos, sin, rot) at the tokens' positions; with gate ([T, >= H] view) every head's
    outputs are multiplied by sigmoid(gate[t, h]), or, with gate_elems, output element i of head h by
    sigmoid(gate[t, h n_out + i]) (gate a [T, >= H n_out] view).  halves: the rotated pairs are (i, i + rot / 2)."""
    _need_cuda(x, m, gate, tok_pos)
    T = x.shape[0]
    H, n_in, n_out = m.shape
    assert x.stride(1) == 1 and m.is_contiguous() and m.dtype == x.dtype and x.shape[1] == H * (n_in + tail)
    y = torch.empty((T, H * (n_out + tail)), dtype=x.dtype, device=x.device)
    p = _HeadMatmulParams()
    p.x, p.x_stride, p.x_head, p.m = x.data_ptr(), x.stride(0), n_in + tail, m.data_ptr()
    p.y, p.y_stride, p.y_head = y.data_ptr(), y.stride(0), n_out + tail
    p.T, p.H, p.n_in, p.n_out, p.tail = T, H, n_in, n_out, tail
    p.halves, p.gate_elems = int(halves), int(gate_elems)
    if tail and tables is not None:
        cos, sin, rot = tables
        if tok_pos is None or err is None:
            raise KernelError("head_matmul: a rotated tail needs the tokens' positions and an error word")
        p.cos_t, p.sin_t, p.table_rows, p.rot, p.tok_pos, p.err = cos.data_ptr(), sin.data_ptr(), cos.shape[0], rot, tok_pos.data_ptr(), err.data_ptr()
    if gate is not None:
        assert gate.dtype == x.dtype and gate.stride(1) == 1
        p.gate, p.gate_stride = gate.data_ptr(), gate.stride(0)
    f = _fn(load_module("latent.cu"), "llb_head_matmul", [_HeadMatmulParams, c_int, c_void_p])
    _check(f(p, _dt(x), _stream()), "per-head matrix product")
    return y


def rope_pairs_(x: torch.Tensor, H: int, head: int, off: int, tables, tok_pos: torch.Tensor, err: torch.Tensor,
                halves: bool = False) -> None:
    """In place on x [T, >= H head] (row stride free): of every head's elements from `off` on, the pairs (2i, 2i+1)
    (with halves: (i, i + rot / 2)), i < rot / 2, are rotated by tables = (cos, sin, rot) at the tokens' positions."""
    _need_cuda(x, tok_pos)
    if tables is None:
        return
    cos, sin, rot = tables
    assert x.stride(1) == 1 and off + rot <= head
    f = _fn(load_module("latent.cu"), "llb_rope_pairs", [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
                                                         c_int, c_void_p, c_void_p, c_int, c_void_p])
    _check(f(_ptr(x), _dt(x), x.shape[0], x.stride(0), H, head, off, rot, _ptr(cos), _ptr(sin), cos.shape[0], _ptr(tok_pos), _ptr(err),
             int(halves), _stream()), "rotation of pairs")


def head_gate_(x: torch.Tensor, gate: torch.Tensor, H: int) -> torch.Tensor:
    """In place on x [T, H width] (contiguous): head h of token t times sigmoid(gate[t, h]) (gate a [T, >= H] view)."""
    _need_cuda(x, gate)
    assert x.is_contiguous() and gate.dtype == x.dtype and gate.stride(1) == 1 and x.shape[1] % H == 0
    f = _fn(load_module("latent.cu"), "llb_head_gate", [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(x), _ptr(gate), gate.stride(0), _dt(x), x.shape[0], H, x.shape[1] // H, _stream()), "per-head output gate")
    return x


LATENT_MAX_ROW = 640          # the widest cache row (latent + rotated part) the attention kernel's key tile holds


def require_latent_row(width: int, value_width: int) -> None:
    if not (0 < value_width <= width <= LATENT_MAX_ROW):
        raise KernelError(f"latent attention: cache rows of {width} elements ({value_width} of them the latent) are not supported "
                          f"(at most {LATENT_MAX_ROW})")


def latent_attention(decode: bool, q: torch.Tensor, nh: int, width: int, value_width: int, kv_new: Optional[torch.Tensor],
                     pool: torch.Tensor, page_table: torch.Tensor, ring: int, pinned: int, seq_start: torch.Tensor,
                     seq_len_before: torch.Tensor, n_seqs: int, max_new: int, window: Optional[int], scale: float,
                     sink_logits: Optional[torch.Tensor], n_splits: int = 1) -> torch.Tensor:
    """Softmax attention of nh query heads q [T, nh width] over one shared row per position: the key is the whole row
    [width], the value its first `value_width` elements.  Rows of positions before the step come from the paged pool,
    the step's own from kv_new [T, width] (None: from the pool too, where an earlier call has put them).  Causal, with
    an optional window and a learned sink score per head (float32 [nh]) in the softmax's denominator.
    Returns [T, nh value_width]."""
    _need_cuda(q, kv_new, pool, page_table, sink_logits)
    require_latent_row(width, value_width)
    assert q.dtype == pool.dtype and q.stride(1) == 1 and (kv_new is None or (kv_new.dtype == q.dtype and kv_new.is_contiguous()))
    assert sink_logits is None or (sink_logits.dtype == torch.float32 and sink_logits.numel() == nh)
    out = torch.empty((q.shape[0], nh * value_width), dtype=q.dtype, device=q.device)
    p = _AttnParams()
    p.q, p.row_stride, p.out = q.data_ptr(), q.stride(0), out.data_ptr()
    if kv_new is not None:
        p.k_new, p.kv_row_stride = kv_new.data_ptr(), kv_new.stride(0)
    p.kpool, p.page_table, p.table_stride, p.ring, p.pinned = pool.data_ptr(), page_table.data_ptr(), page_table.shape[1], ring, pinned
    p.seq_start, p.seq_len_before = seq_start.data_ptr(), seq_len_before.data_ptr()
    p.nh, p.nkvh, p.window, p.scale = nh, 1, int(window or 0), scale
    p.all_from_cache = int(kv_new is None)
    p.sink_logits, p.v_in_k, p.n_splits = _ptr(sink_logits), 1, 1
    lib = _attn_lib(width, value_width) if width <= 256 else load_module("attention_simt.cu", {"LLB_HEAD_DIM": width, "LLB_VALUE_DIM": value_width})
    if not decode:
        f = _fn(lib, "llb_attn_prefill", [_AttnParams, c_int, c_int, c_int, c_void_p])
        _check(f(p, _dt(q), n_seqs, max_new, _stream()), "latent attention (prefill)")
        return out
    keep = None
    p.n_splits = n_splits
    if n_splits > 1:
        part_o = torch.empty((n_seqs, nh, n_splits, value_width), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((n_seqs, nh, n_splits, 2), dtype=torch.float32, device=q.device)
        p.part_o, p.part_ml = part_o.data_ptr(), part_ml.data_ptr()
        keep = (part_o, part_ml)
    f = _fn(lib, "llb_attn_decode", [_AttnParams, c_int, c_int, c_void_p])
    _check(f(p, _dt(q), n_seqs, _stream()), "latent attention (decode)", 2 if n_splits > 1 else 1)
    del keep
    return out
