from __future__ import annotations

import math

import torch

from .. import kernels
from .attention import decode_splits
from .base import KVNeed, Mixer, TensorDecl, build_part, register_part


def _fuse(ts):
    dt = ts[0].dtype
    for t in ts[1:]:
        dt = torch.promote_types(dt, t.dtype)
    return torch.cat([t.to(dt) for t in ts], dim=0).contiguous()


class _NormedHeads(Mixer):
    """What the two mixers below share: grouped-query attention over the paged cache whose query and key rows are RMS-normed
    over their elements (one weight for all query rows, one for all key rows; `qk_norm` false: no norm) and then rotated
    by a position part that hands out pair_tables() (layout "halves" or "neighbours"), both in one kernel and in
    float32 (kernels.head_prep), which also stores keys and values.  Projections have no bias; q, k and v are one matrix.
    The cache is a ring: a step of several tokens attends over the cache (earlier positions) and the step's own
    projections and appends afterwards; a step of single tokens appends first and attends over the cache alone."""
    capturable = True

    def _common(self, p):
        self.hidden, self.nh, self.nkvh = int(p["hidden_size"]), int(p["num_heads"]), int(p["num_kv_heads"])
        self.dk, self.dv = int(p["key_dim"]), int(p["value_dim"])
        if self.nkvh <= 0 or self.nh % self.nkvh:
            raise ValueError(f"{self.nh} query heads cannot share {self.nkvh} key/value heads")
        kernels.require_head_dim(self.dk, even=False)
        kernels.require_head_dim(self.dv, even=False)
        self.scale, self.eps = float(p["scale"]), float(p.get("eps", 0.0))
        self.qk_norm = bool(p.get("qk_norm", True))
        self.position = build_part("position", p["position"], self.env) if p.get("position") else None
        if self.position is not None and not hasattr(self.position, "pair_tables"):
            raise ValueError("this mixer takes a position encoding that hands out pair tables")
        self.names = dict({"q": "q", "k": "k", "v": "v", "o": "o", "q_norm": "q.norm", "k_norm": "k.norm"}, **(p.get("names") or {}))
        self.w_in = self.w_o = self.q_norm = self.k_norm = None

    def prepare(self, max_positions):
        if self.position is not None:
            self.position.prepare(max_positions)

    def _tensors(self, maps: int):
        n = self.names
        t = {n["q"]: TensorDecl((self.nh * maps * self.dk, self.hidden)), n["k"]: TensorDecl((self.nkvh * maps * self.dk, self.hidden)),
             n["v"]: TensorDecl((self.nkvh * self.dv, self.hidden)), n["o"]: TensorDecl((self.hidden, self.nh * self.dv))}
        if self.qk_norm:
            t[n["q_norm"]] = TensorDecl((self.dk,), init="one_plus_normal", use="vector")
            t[n["k_norm"]] = TensorDecl((self.dk,), init="one_plus_normal", use="vector")
        return t

    def _load_norms(self, tensors):
        if self.qk_norm:
            self.q_norm = tensors[self.names["q_norm"]].float().contiguous()
            self.k_norm = tensors[self.names["k_norm"]].float().contiguous()

    def _prep(self, proj, ctx, maps: int, append=None, rotate: bool = True):
        tables = self.position.pair_tables(ctx.max_position + 1) if (rotate and self.position is not None) else None
        kernels.head_prep(proj, self.nh * maps, self.nkvh * maps, self.dk, kv_heads=self.nkvh, dv=self.dv,
                          q_weight=self.q_norm if rotate else None, k_weight=self.k_norm if rotate else None, eps=self.eps,
                          tables=tables, layout=self.position.pair_layout if self.position is not None else "halves",
                          tok_pos=ctx.tok_pos, append=append, err=ctx.err)

    def _decode(self, ctx, common, maps: int, window, extras, splits: int):
        """Attention of single tokens over the caches alone (their rows are appended already).  bfloat16 operands that the
        mma.sync prefill kernel takes run there as a step of one token per sequence: a block per query head walks the
        whole visible range on the tensor cores, which at windows of thousands of keys is several times faster than the
        CUDA-core kernel with its key range cut into slices and a merge behind it."""
        if kernels.prefill_ext_ok(common[0], self.dk, self.dv):
            return kernels.attention_prefill(*common, 1, window, self.scale, all_from_cache=True, extras=extras)
        return kernels.attention_decode(*common, window, self.scale, n_splits=splits, extras=extras)

    @staticmethod
    def _append_args(ctx, kv):
        return dict(tok_seq=ctx.tok_seq, seq_start=ctx.seq_start, seq_len_before=ctx.seq_len_before, kpool=kv.k, vpool=kv.v,
                    page_table=kv.page_table, ring=kv.ring, pinned=kv.pinned)


@register_part("mixer", "differential_attention")
class DifferentialAttention(_NormedHeads):
    """Attention with two score maps per head over one set of values.  Every query head and every key/value head carries
    two query (key) rows of `key_dim` elements, [map 1, map 2]; each map is a softmax attention of its own (scores
    (q . k) * scale) over the head's values, giving a1 and a2, and the head's result is

        o = a1 - lambda * a2,   lambda = exp(sum(lq1 * lk1)) - exp(sum(lq2 * lk2)) + diff     (one number for the layer)
        out = o / sqrt(mean(o^2) + eps) * (1 - diff)                                          (over the head's value_dim)

    followed by the output projection.  Masks: `chunk` C (the query at position p sees the keys j <= p with
    floor(j / C) = floor(p / C); chunks count from the sequence's first position) and/or `window`; neither: causal.

    On the device the two maps are 2 H query heads against 2 G key heads that share G value heads (`maps` of the
    attention kernel); the rows of the query matrix are reordered when they are loaded so that the query heads of one
    key head are neighbours.  The two results leave the attention kernel in float32, as the difference cancels.

    params: hidden_size, num_heads, num_kv_heads, key_dim, value_dim, scale, diff, eps, chunk, window, qk_norm, position,
    names (q, k, v, o, q_norm, k_norm, lq1, lk1, lq2, lk2)."""

    def __init__(self, spec, env):
        super().__init__(spec, env)
        p = spec.params
        self._common(p)
        self.diff = float(p["diff"])
        self.chunk = int(p["chunk"]) if p.get("chunk") else 0
        self.window = int(p["window"]) if p.get("window") else None
        if self.chunk < 0 or (self.window is not None and self.window <= 0):
            raise ValueError("a chunk or a window holds at least one key")
        self.names = dict({"lq1": "lq1", "lk1": "lk1", "lq2": "lq2", "lk2": "lk2"}, **self.names)
        self.lam = None

    def _kept(self):
        """How far back the cache has to reach: the chunk, the window, or (None) everything."""
        spans = [s for s in (self.chunk or None, self.window) if s]
        return min(spans) if spans else None

    def kv_need(self):
        return KVNeed(self.nkvh, 2 * self.dk, self.dv, self._kept())

    def tensors(self):
        t = self._tensors(2)
        for k in ("lq1", "lk1", "lq2", "lk2"):
            t[self.names[k]] = TensorDecl((self.dk,), use="vector")
        return t

    def load(self, tensors):
        n = self.names
        r = self.nh // self.nkvh
        wq = tensors[n["q"]]
        # rows [head][map][element] -> [key/value head][map][head of the group][element]
        wq = wq.reshape(self.nkvh, r, 2, self.dk, self.hidden).permute(0, 2, 1, 3, 4).reshape(self.nh * 2 * self.dk, self.hidden)
        self.w_in = _fuse([wq, tensors[n["k"]], tensors[n["v"]]])
        self.w_o = tensors[n["o"]].contiguous()
        self._load_norms(tensors)
        l = [tensors[n[k]].float().cpu() for k in ("lq1", "lk1", "lq2", "lk2")]
        self.lam = float(torch.exp((l[0] * l[1]).sum()) - torch.exp((l[2] * l[3]).sum()) + torch.tensor(self.diff, dtype=torch.float32))

    def forward(self, x, ctx, call):
        kv = ctx.kv(call)
        proj = kernels.linear(x, self.w_in)
        extras = kernels.AttnExtras(value_dim=self.dv, pinned=kv.pinned, chunk=self.chunk, maps=2, out_f32=True)
        common = (proj, 2 * self.nh, 2 * self.nkvh, self.dk, kv.k, kv.v, kv.page_table, kv.ring, ctx.seq_start, ctx.seq_len_before,
                  ctx.n_seqs)
        if ctx.is_decode:
            self._prep(proj, ctx, 2, append=self._append_args(ctx, kv))
            splits = decode_splits(ctx, 2 * self.nkvh)
            if self._kept() is not None:
                splits = max(1, min(splits, -(-self._kept() // kernels.ops.PAGE) + 1))
            a = self._decode(ctx, common, 2, self.window, extras, splits)
        else:
            self._prep(proj, ctx, 2)
            a = kernels.attention_prefill(*common, ctx.max_new, self.window, self.scale, all_from_cache=False, extras=extras)
            self._prep(proj, ctx, 2, append=self._append_args(ctx, kv), rotate=False)
        y = kernels.diff_combine(a, self.nh, self.nh // self.nkvh, self.dv, self.lam, self.eps, 1.0 - self.diff, x.dtype)
        return kernels.linear(y, self.w_o, out_dtype=torch.float32)


@register_part("mixer", "pooled_window_attention")
class PooledWindowAttention(_NormedHeads):
    """Sliding-window attention that still sees what has left the window, in blocks: the query at position p sees the
    keys j with 0 <= p - j < window and, beside them, one key and one value for every block of `pool` consecutive
    positions that lies wholly before the window (block b = positions b P .. b P + P - 1, seen when b P + P - 1 <= p - window).
    A block's key is the mean of its P keys as the cache holds them (normed and rotated), its value the mean of its P
    values; tokens and blocks share one softmax.  Positions that have left the window while their block is incomplete or
    not yet wholly outside are not seen.

    The mixer is two users of the cache: a ring of token rows that reaches back max(window, pool) positions, and a group
    of block rows (one per P tokens, all kept) that kernels.pool_append fills as blocks complete, before the step's
    attention runs.

    Without a pool (0 or absent) the mixer is a plain sliding window with normed and rotated heads and one user of the cache.

    params: hidden_size, num_heads, num_kv_heads, key_dim, value_dim, scale, window, pool, eps, qk_norm, position, names."""

    def __init__(self, spec, env):
        super().__init__(spec, env)
        p = spec.params
        self._common(p)
        self.window, self.pool = int(p["window"]), int(p.get("pool") or 0)          # pool 0: no blocks, a plain window
        if self.window <= 0 or self.pool < 0:
            raise ValueError(f"window {self.window} must be positive and pool {self.pool} not negative")

    def kv_need(self):
        return KVNeed(self.nkvh, self.dk, self.dv, max(self.window, self.pool))

    def cache_users(self):
        if not self.pool:
            return [(self.kv_need(), 0)]
        return [(self.kv_need(), 0), (KVNeed(self.nkvh, self.dk, self.dv, None, every=self.pool), 0)]

    def tensors(self):
        return self._tensors(1)

    def load(self, tensors):
        n = self.names
        self.w_in = _fuse([tensors[n["q"]], tensors[n["k"]], tensors[n["v"]]])
        self.w_o = tensors[n["o"]].contiguous()
        self._load_norms(tensors)

    def forward(self, x, ctx, call):
        kv, blocks = ctx.kv(call), (ctx.kv(call + 1) if self.pool else None)
        proj = kernels.linear(x, self.w_in)
        # single tokens: norm, rotation and append in one launch (the ring still holds the block's earlier positions);
        # longer steps append after the attention, so that the ring is not overwritten under the step's own queries
        self._prep(proj, ctx, 1, append=self._append_args(ctx, kv) if ctx.is_decode else None)
        if self.pool:
            kernels.pool_append(proj, self.nh * self.dk, self.nkvh, self.dk, self.dv, self.pool, kv, blocks, ctx.seq_start,
                                ctx.seq_len_before, ctx.n_seqs, ctx.max_new)
        extras = kernels.AttnExtras(value_dim=self.dv, pinned=kv.pinned, pool=(self.pool, blocks) if self.pool else None)
        common = (proj, self.nh, self.nkvh, self.dk, kv.k, kv.v, kv.page_table, kv.ring, ctx.seq_start, ctx.seq_len_before,
                  ctx.n_seqs)
        if ctx.is_decode:
            pages = -(-self.window // kernels.ops.PAGE) + 1 + (blocks.page_table.shape[1] if blocks is not None else 0)
            splits = max(1, min(decode_splits(ctx, self.nkvh), pages))
            a = self._decode(ctx, common, 1, self.window, extras, splits)
        else:
            a = kernels.attention_prefill(*common, ctx.max_new, self.window, self.scale, all_from_cache=False, extras=extras)
            self._prep(proj, ctx, 1, append=self._append_args(ctx, kv), rotate=False)
        return kernels.linear(a, self.w_o, out_dtype=torch.float32)


@register_part("mixer", "lightning_attention")
class LightningAttention(Mixer):
    """Linear attention with one constant decay per head: q = silu(Wq h), k = silu(Wk h) (heads x key_dim), v = silu(Wv h)
    (heads x value_dim); per head S <- decay_h S + k v^T, o = S^T q, with S [key_dim, value_dim] in float32 in the cache's
    fixed-size state of the sequence (zero at its start).  The heads' results, side by side, are RMS-normed together with
    one weight over all of them, multiplied by sigmoid(Wg h) and projected.  q, k and v leave their product in float32;
    the recurrence is the kernel of the gated linear attention with the decay taken from a table per head.  A step in which
    some sequence brings 256 tokens or more runs in chunks of 64 tokens side by side (kernels.gla_scan_chunked): with a
    constant decay a chunk's effect on the state is a^n S + (what the chunk reaches from zero).

    params: hidden_size, num_heads, key_dim, value_dim, decay (one number per head), eps, names (q, k, v, g, o, norm)."""
    capturable = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        p = spec.params
        self.hidden, self.nh, self.dk, self.dv = int(p["hidden_size"]), int(p["num_heads"]), int(p["key_dim"]), int(p["value_dim"])
        self.eps = float(p["eps"])
        decay = [float(d) for d in p["decay"]]
        if len(decay) != self.nh or any(not (0.0 <= d <= 1.0) or math.isnan(d) for d in decay):
            raise ValueError(f"one decay in [0, 1] per head ({self.nh}), got {decay}")
        if self.dk > kernels.mixers.GLA_MAX_KEY_DIM:
            raise kernels.KernelError(f"lightning attention: {self.dk} key channels a head; the kernel takes up to "
                                      f"{kernels.mixers.GLA_MAX_KEY_DIM}")
        self.decay = torch.tensor(decay, dtype=torch.float32, device=env.device)
        self.names = dict({"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "norm": "norm"}, **(p.get("names") or {}))
        self.w_in = self.w_gate = self.w_norm = self.w_o = None

    def state_size(self):
        return self.nh * self.dk * self.dv

    def tensors(self):
        n, D, K, V = self.names, self.hidden, self.nh * self.dk, self.nh * self.dv
        return {n["q"]: TensorDecl((K, D)), n["k"]: TensorDecl((K, D)), n["v"]: TensorDecl((V, D)), n["g"]: TensorDecl((V, D)),
                n["o"]: TensorDecl((D, V)), n["norm"]: TensorDecl((V,), init="one_plus_normal", use="vector")}

    def load(self, tensors):
        n = self.names
        self.w_in = _fuse([tensors[n["q"]], tensors[n["k"]], tensors[n["v"]]])
        self.w_gate = tensors[n["g"]].contiguous()
        self.w_norm = tensors[n["norm"]].contiguous()
        self.w_o = tensors[n["o"]].contiguous()

    def forward(self, x, ctx, call):
        qkv = kernels.linear(x, self.w_in, out_dtype=torch.float32)
        gate = kernels.linear(x, self.w_gate)
        n_new = getattr(ctx, "n_new", None)
        if n_new and max(n_new) >= kernels.mixers.SCAN_CHUNKED_FROM:
            chunks = getattr(ctx, "_scan_chunks", None)          # one plan per step, shared by the step's layers
            if chunks is None:
                chunks = kernels.scan_chunks(n_new, x.device)
                try:
                    ctx._scan_chunks = chunks
                except AttributeError:
                    pass
            o = kernels.gla_scan_chunked(qkv, self.nh, self.dk, self.dv, ctx.state(call), ctx.seq_slot, ctx.n_seqs, self.decay,
                                         chunks, act="silu")
        else:
            o = kernels.gla_scan(qkv, self.nh, self.dk, self.dv, None, ctx.state(call), ctx.seq_start, ctx.seq_slot, ctx.n_seqs,
                                 1.0, 1.0, head_decay=self.decay, act="silu")
        y = kernels.gla_out(o, gate, self.w_norm, 1, self.nh * self.dv, self.eps, x.dtype, gate_act="sigmoid")
        return kernels.linear(y, self.w_o, out_dtype=torch.float32)


@register_part("mixer", "parallel_mixers")
class ParallelMixers(Mixer):
    """Several mixers side by side that read the same input; the result is the mean of their outputs, each first
    RMS-normed over the model width with a weight of its own.  The branches are mixers of any kind, built from their
    own specs (their tensors lie under their own prefixes); their users of the cache follow one another.

    params: hidden_size, eps, branches: [{part: PartSpec of category "mixer", out: the local name of the branch's norm
    weight}]."""

    def __init__(self, spec, env):
        super().__init__(spec, env)
        p = spec.params
        self.hidden, self.eps = int(p["hidden_size"]), float(p["eps"])
        self.branches = [build_part("mixer", b["part"], env) for b in p["branches"]]
        self.out_names = [str(b["out"]) for b in p["branches"]]
        if not (1 <= len(self.branches) <= 4):
            raise ValueError(f"one to four branches, got {len(self.branches)}")
        self.out_w = []

    @property
    def capturable(self):
        return all(b.capturable for b in self.branches)

    def children(self):
        return list(self.branches)

    def prepare(self, max_positions):
        for b in self.branches:
            b.prepare(max_positions)

    def cache_users(self):
        return [u for b in self.branches for u in b.cache_users()]

    def tensors(self):
        return {n: TensorDecl((self.hidden,), init="one_plus_normal", use="vector") for n in self.out_names}

    def load(self, tensors):
        self.out_w = [tensors[n].float().contiguous() for n in self.out_names]

    def forward(self, x, ctx, call):
        outs = []
        for b in self.branches:
            y = b.forward(x, ctx, call)
            outs.append(y if y.dtype == torch.float32 else y.float())
            call += len(b.cache_users())
        return kernels.branch_mean(outs, self.out_w, self.eps, 1.0 / len(outs))
