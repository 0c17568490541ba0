from __future__ import annotations

import torch

from .. import kernels
from .attention import decode_splits
from .base import KVNeed, Mixer, TensorDecl, build_part, register_part


@register_part("mixer", "windowed_sink_attention")
class WindowedSinkAttention(Mixer):
    """Causal grouped-query attention over the paged cache with six options the plain one does not have:

      * keys and queries of `key_dim` elements, values (and the heads' outputs) of `value_dim`;
      * a window that keeps a sequence's first keys: the query at position i sees key j <= i when i - j < window or
        j < keep_first (the kept keys stay at their true positions);
      * a sink: the softmax's denominator has one more term e^0 that carries no value, so the weights are
        e^{s_j} / (1 + sum e^{s_j}) and may sum to less than one;
      * a penalty on distance (`distance_bias`): the score of query position i and key position j loses
        r1[h] ln(1 + r2[h] (i - j)), with two numbers per query head (tensors `r1`, `r2`, [num_heads]);
      * a query temperature (`q_temp` = {coef, every}): the query at position p is multiplied by
        1 + coef ln(floor((p + 1) / every) + 1), i.e. queries sharpen as the sequence grows, in steps of `every`;
      * a layer without key and value projections (`own_kv` false) that reads the rotated keys and the values another
        layer stored in the cache (the run order's `cache_of`), with queries, window and everything else its own.

    Query heads h of a group of num_heads / num_kv_heads share key/value head h / group.  Scores are (q . k) * scale.
    The position encoding is a part of category "position" that hands out leading_tables() (rotation of a head's
    first dimensions).  Projections have no bias; q (and k, v when the layer has them) are one matrix.

    Cache: `cache_window` says what the layer's cache keeps: None (every key: needed when other layers read it, and
    then this layer's window is only a mask) or the window, kept in a ring of pages behind ceil(keep_first / page)
    pinned ones.  With a ring, a step of several tokens attends over the cache (earlier positions) and the step's own
    projections and appends afterwards, so that the ring is never overwritten by keys the step's queries still need;
    otherwise (and in decode) keys and values are appended first and attention reads the cache alone.

    params: hidden_size, num_heads, num_kv_heads, key_dim, value_dim, scale, window, keep_first, sink, own_kv,
    cache_window, position (PartSpec or None: no rotation), distance_bias, q_temp, names (local tensor names of q, k, v, o,
    r1, r2; default those).
    """

    def __init__(self, spec, env):
        super().__init__(spec, env)
        p = spec.params
        self.hidden, self.nh, self.nkvh = int(p["hidden_size"]), int(p["num_heads"]), int(p["num_kv_heads"])
        self.dk, self.dv = int(p["key_dim"]), int(p["value_dim"])
        if self.nkvh <= 0 or self.nh % self.nkvh:
            raise ValueError(f"{self.nh} query heads cannot share {self.nkvh} key/value heads")
        kernels.require_head_dim(self.dk, even=False)      # (the rotated part of a head is even; the head need not be)
        kernels.require_head_dim(self.dv, even=False)
        self.scale = float(p["scale"])
        self.window = int(p["window"]) if p.get("window") is not None else None
        if self.window is not None and self.window <= 0:
            raise ValueError(f"a window holds at least one key, got {self.window}")
        self.keep_first = max(0, int(p.get("keep_first", 0))) if self.window is not None else 0
        self.sink = bool(p.get("sink", False))
        self.own_kv = bool(p.get("own_kv", True))
        self.cache_window = p.get("cache_window")
        if self.cache_window is not None and (self.window is None or self.cache_window < self.window):
            raise ValueError("the cache must keep at least the keys the window shows")
        self.position = build_part("position", p["position"], env) if p.get("position") else None
        if self.position is not None and not hasattr(self.position, "leading_tables"):
            raise ValueError("this mixer takes a position encoding that rotates a head's leading dimensions")
        self.rot = self.position.dims if self.position is not None else 0
        self.names = dict({"q": "q", "k": "k", "v": "v", "o": "o", "r1": "r1", "r2": "r2"}, **(p.get("names") or {}))
        self.distance_bias = bool(p.get("distance_bias", False))
        self.q_temp = None
        if p.get("q_temp"):
            self.q_temp = (float(p["q_temp"]["coef"]), int(p["q_temp"]["every"]))
            if self.q_temp[1] <= 0:
                raise ValueError(f"the query temperature's period must be positive, got {self.q_temp[1]}")
        self.w_in = self.w_o = self.r1 = self.r2 = None

    capturable = True

    def prepare(self, max_positions):
        if self.position is not None:
            self.position.prepare(max_positions)

    def kv_need(self):
        return KVNeed(self.nkvh, self.dk, self.dv, self.cache_window, self.keep_first if self.cache_window is not None else 0)

    def tensors(self):
        n = self.names
        t = {n["q"]: TensorDecl((self.nh * self.dk, self.hidden)), n["o"]: TensorDecl((self.hidden, self.nh * self.dv))}
        if self.own_kv:
            t[n["k"]] = TensorDecl((self.nkvh * self.dk, self.hidden))
            t[n["v"]] = TensorDecl((self.nkvh * self.dv, self.hidden))
        if self.distance_bias:
            t[n["r1"]] = TensorDecl((self.nh,), init="one_plus_normal", use="vector")
            t[n["r2"]] = TensorDecl((self.nh,), init="one_plus_normal", use="vector")
        return t

    def load(self, tensors):
        n = self.names
        ts = [tensors[n["q"]]] + ([tensors[n["k"]], tensors[n["v"]]] if self.own_kv else [])
        dt = ts[0].dtype
        for t in ts[1:]:
            dt = torch.promote_types(dt, t.dtype)
        self.w_in = torch.cat([t.to(dt) for t in ts], dim=0).contiguous()
        self.w_o = tensors[n["o"]].contiguous()
        if self.distance_bias:
            self.r1, self.r2 = tensors[n["r1"]].float().contiguous(), tensors[n["r2"]].float().contiguous()

    def forward(self, x, ctx, call):
        return kernels.linear(self._attend(x, ctx, call), self.w_o)

    def forward_into(self, x, ctx, call, residual):
        if not (x.dtype == torch.bfloat16 and self.w_o.dtype == torch.bfloat16
                and kernels.linear_into_ok(x.new_empty((x.shape[0], self.nh * self.dv)), self.w_o, None, residual)):
            return False
        kernels.linear_into(self._attend(x, ctx, call), self.w_o, None, residual)
        return True

    def _splits(self, ctx) -> int:
        """Slices of the key range in decode: as the plain attention chooses them, but no more than the tiles a window
        (and the kept first keys) can span."""
        from ..cache.kv import pinned_pages, ring_pages
        splits = decode_splits(ctx, self.nkvh)
        if self.window is not None:
            splits = min(splits, ring_pages(self.window) + pinned_pages(self.window, self.keep_first))
        return max(1, splits)

    def _attend(self, x, ctx, call):
        """Projections, rotation, cache append and attention: [T, nh * value_dim], before the output projection."""
        kv = ctx.kv(call)
        if kv.writable != self.own_kv:
            raise ValueError("a layer with key/value projections keeps its own cache; one without reads another layer's")
        proj = kernels.linear(x, self.w_in)
        nkv_here = self.nkvh if self.own_kv else 0
        tables = self.position.leading_tables(ctx.max_position + 1) if self.position is not None else None
        cos, sin = tables if tables is not None else (None, None)
        append = None
        if kv.writable:
            append = dict(tok_seq=ctx.tok_seq, seq_start=ctx.seq_start, seq_len_before=ctx.seq_len_before, kpool=kv.k,
                          vpool=kv.v, page_table=kv.page_table, ring=kv.ring, pinned=kv.pinned)
        extras = kernels.AttnExtras(value_dim=self.dv, keep_first=self.keep_first, pinned=kv.pinned, sink=self.sink,
                                    dist_bias=(self.r1, self.r2) if self.distance_bias else None, q_temp=self.q_temp)
        common = (proj, self.nh, self.nkvh, self.dk, kv.k, kv.v, kv.page_table, kv.ring, ctx.seq_start, ctx.seq_len_before,
                  ctx.n_seqs)
        ring_cache = kv.writable and self.cache_window is not None
        if ctx.is_decode or not ring_cache:
            kernels.rope_lead_append(proj, self.nh, nkv_here, self.dk, self.dv, self.rot, cos=cos, sin=sin,
                                     tok_pos=ctx.tok_pos, append=append, err=ctx.err)
            if ctx.is_decode:
                return kernels.attention_decode(*common, self.window, self.scale, n_splits=self._splits(ctx), extras=extras)
            return kernels.attention_prefill(*common, ctx.max_new, self.window, self.scale, all_from_cache=True, extras=extras)
        kernels.rope_lead_append(proj, self.nh, nkv_here, self.dk, self.dv, self.rot, cos=cos, sin=sin,
                                 tok_pos=ctx.tok_pos, err=ctx.err)
        out = kernels.attention_prefill(*common, ctx.max_new, self.window, self.scale, all_from_cache=False, extras=extras)
        kernels.rope_lead_append(proj, self.nh, nkv_here, self.dk, self.dv, 0, tok_pos=ctx.tok_pos, append=append, err=ctx.err)
        return out
