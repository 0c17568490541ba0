from __future__ import annotations

import torch

from .. import kernels
from .base import KVNeed, Mixer, TensorDecl, build_part, register_part


@register_part("mixer", "latent_attention")
class LatentAttention(Mixer):
    """Causal softmax attention whose queries, keys and values pass through low-rank latents; a token leaves one row
    [c (kv_rank) | rotated shared key part (rope_dim)] in the cache for all heads together.

        cq = rms_norm(Wdq h; w)                  q[h] = Wuq[h] cq = [q_n (nope_dim) | q_r (rope_dim)], q_r rotated
        [c' | k_r] = Wdkv h                      c = rms_norm(c'; w), k_r rotated (one for all heads)
        k_n[h] = Wuk[h] c,  v[h] = Wuv[h] c
        score(i, j) = (q_n[h]_i . k_n[h]_j + q_r[h]_i . k_r_j) * scale      for j <= i (and i - j < window)
        weights = softmax over the visible j, with one more term e^(sink[h]) in the denominator that carries no value
        out = Wo concat_h(sigmoid(Wg h)_h * sum_j weight_j v[h]_j)

    The up projections of keys and values never run over the cache: q_n . (Wuk[h] c) = (Wuk[h]^T q_n) . c and
    sum_j w_j Wuv[h] c_j = Wuv[h] sum_j w_j c_j, so the heads' queries are carried into the latent space (a per-head
    product), attention runs over the cached rows as one key/value head shared by all query heads (key: the whole row,
    value: its first kv_rank elements), and the latent result is carried into each head's value space.  Scores,
    softmax and all norms are float32.

    A step of whole prompts (no sequence of the step has history) in bfloat16, with heads whose query/key and value sizes
    are equal and fit the tensor-core attention kernel, goes the other way round: the heads' keys and values of the
    step's tokens are made from the step's rows by one matrix product (Wuk, an identity block that copies the rotated
    part into every head, and Wuv stacked), and the framework's tensor-core attention runs over them as ordinary heads,
    with the learned sink as its extra term; nothing is read from the cache, which is still appended to as always.

    Variants.  `q_rank` None: the queries pass through no latent, q = Wq h (tensor `q`).  `gate` "elements": the output
    gate has a value per element of the concatenated heads (Wg is [heads * value_dim, hidden]) instead of one per head
    ("head", what `head_gate` true means).  The position encoding's `pair_layout` says which dimensions of the rotated
    part pair up: neighbours (2i, 2i+1) or halves (i, i + dims/2).

    `own_kv` false: the layer has no Wdkv and reads the rows another layer cached (the run order's `cache_of`), with
    its own up projections, queries, window and everything else.

    Cache: one key head of kv_rank + rope_dim elements, no value pool.  `cache_window` None keeps every row (needed
    when other layers read the cache; the window is then a mask only), otherwise a ring of pages for the window: a step
    of several tokens then attends over the cache and the step's own rows and appends afterwards; single tokens, and
    caches that keep every row, append first.

    params: hidden_size, num_heads, nope_dim, rope_dim, value_dim, q_rank, kv_rank, scale, window, eps, sink, head_gate,
    gate, own_kv, cache_window, position (PartSpec of a position encoding with pair_tables()), names.
    """
    capturable = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        p = spec.params
        self.hidden, self.nh = int(p["hidden_size"]), int(p["num_heads"])
        self.dn, self.dr, self.dv = int(p["nope_dim"]), int(p["rope_dim"]), int(p["value_dim"])
        self.q_rank, self.kv_rank = (int(p["q_rank"]) if p.get("q_rank") else 0), int(p["kv_rank"])
        self.scale, self.eps = float(p["scale"]), float(p["eps"])
        self.window = int(p["window"]) if p.get("window") is not None else None
        if self.window is not None and self.window <= 0:
            raise ValueError(f"a window holds at least one key, got {self.window}")
        self.sink = bool(p.get("sink", False))
        self.gate = p.get("gate") or ("head" if p.get("head_gate", False) else None)
        if self.gate not in (None, "head", "elements"):
            raise ValueError(f"the output gate is per 'head' or per 'elements', got {self.gate!r}")
        self.head_gate = self.gate is not None
        self.own_kv = bool(p.get("own_kv", True))
        self.cache_window = p.get("cache_window")
        if self.cache_window is not None and (self.window is None or self.cache_window < self.window):
            raise ValueError("the cache must keep at least the keys the window shows")
        self.row = self.kv_rank + self.dr
        kernels.require_latent_row(self.row, self.kv_rank)
        self.position = build_part("position", p["position"], env) if p.get("position") else None
        if self.position is not None and not hasattr(self.position, "pair_tables"):
            raise ValueError("this mixer takes a position encoding that hands out pair_tables()")
        self.halves = getattr(self.position, "pair_layout", "neighbours") == "halves"
        self.names = dict({"q": "q", "dq": "dq", "dq_norm": "dq.norm", "uq": "uq", "dkv": "dkv", "dkv_norm": "dkv.norm", "uk": "uk",
                           "uv": "uv", "sink": "sink", "g": "g", "o": "o"}, **(p.get("names") or {}))
        self.w_in = self.w_uq = self.w_uk = self.w_uv_t = self.w_o = self.w_qn = self.w_kvn = self.sink_logits = None
        self.w_kv_heads = None

    def prepare(self, max_positions):
        if self.position is not None:
            self.position.prepare(max_positions)

    def kv_need(self):
        return KVNeed(1, self.row, 0, self.cache_window)

    def tensors(self):
        n, D, H = self.names, self.hidden, self.nh
        t = {n["uk"]: TensorDecl((H * self.dn, self.kv_rank)),
             n["uv"]: TensorDecl((H * self.dv, self.kv_rank)), n["o"]: TensorDecl((D, H * self.dv))}
        if self.q_rank:
            t[n["dq"]] = TensorDecl((self.q_rank, D))
            t[n["dq_norm"]] = TensorDecl((self.q_rank,), init="one_plus_normal", use="vector")
            t[n["uq"]] = TensorDecl((H * (self.dn + self.dr), self.q_rank))
        else:
            t[n["q"]] = TensorDecl((H * (self.dn + self.dr), D))
        if self.own_kv:
            t[n["dkv"]] = TensorDecl((self.row, D))
            t[n["dkv_norm"]] = TensorDecl((self.kv_rank,), init="one_plus_normal", use="vector")
        if self.sink:
            t[n["sink"]] = TensorDecl((H,), use="vector")
        if self.head_gate:
            t[n["g"]] = TensorDecl((H if self.gate == "head" else H * self.dv, D))
        return t

    def load(self, tensors):
        n, H = self.names, self.nh
        ts = [tensors[n["dq"] if self.q_rank else n["q"]]] + ([tensors[n["dkv"]]] if self.own_kv else []) + ([tensors[n["g"]]] if self.head_gate else [])
        dt = ts[0].dtype
        for t in ts[1:]:
            dt = torch.promote_types(dt, t.dtype)
        rows = sum(t.shape[0] for t in ts)
        if rows % 8:                                   # whole 16-byte pieces of output rows: the faster products want them
            ts.append(torch.zeros((8 - rows % 8, self.hidden), dtype=dt, device=ts[0].device))
        self.w_in = torch.cat([t.to(dt) for t in ts], dim=0).contiguous()       # [query latent or queries | kv latent, key part | gates]
        self.q_cols = self.q_rank if self.q_rank else H * (self.dn + self.dr)
        self.gate_off = self.q_cols + (self.row if self.own_kv else 0)
        self.w_uq = tensors[n["uq"]].contiguous() if self.q_rank else None
        self.w_uk = tensors[n["uk"]].reshape(H, self.dn, self.kv_rank).contiguous()                 # [h, nope, latent]
        self.w_uv_t = tensors[n["uv"]].reshape(H, self.dv, self.kv_rank).transpose(1, 2).contiguous()   # [h, latent, value]
        self.w_o = tensors[n["o"]].contiguous()
        self.w_qn = tensors[n["dq_norm"]].float().contiguous() if self.q_rank else None
        self.w_kvn = tensors[n["dkv_norm"]].float().contiguous() if self.own_kv else None
        self.sink_logits = tensors[n["sink"]].float().contiguous() if self.sink else None
        dk = self.dn + self.dr
        if self.w_o.dtype == torch.bfloat16 and dk == self.dv and dk % 16 == 0 and dk <= 128 and self.row % 8 == 0:
            # rows [c | k_r] -> every head's [Wuk[h] c | k_r], then every head's Wuv[h] c
            w = torch.zeros((H * dk + H * self.dv, self.row), dtype=self.w_o.dtype, device=self.w_o.device)
            keys = w[:H * dk].view(H, dk, self.row)
            keys[:, :self.dn, :self.kv_rank] = tensors[n["uk"]].reshape(H, self.dn, self.kv_rank)
            keys[:, self.dn:, self.kv_rank:] = torch.eye(self.dr, dtype=w.dtype, device=w.device)
            w[H * dk:, :self.kv_rank] = tensors[n["uv"]]
            self.w_kv_heads = w

    def _splits(self, ctx) -> int:
        """Slices of the key range in decode: all query heads of a sequence share one block per slice, so enough slices to
        fill the device, at most one per page that the window (or the widest page table of the step) can span: a function
        of the step's shape alone, so a captured step stays valid as sequences grow."""
        from ..cache.kv import ring_pages
        pages = max(ctx.widths) if ctx.widths else 1
        if self.window is not None:
            pages = min(pages, ring_pages(self.window))
        return max(1, min((2 * ctx.sm_count) // max(1, ctx.n_seqs), pages, 64))

    def forward(self, x, ctx, call):
        kv = ctx.kv(call)
        if kv.writable != self.own_kv:
            raise ValueError("a layer with its own latent projection keeps its own cache; one without reads another layer's")
        proj = kernels.linear(x, self.w_in)
        tables = self.position.pair_tables(ctx.max_position + 1) if self.position is not None else None
        append = None
        if kv.writable:
            append = dict(tok_seq=ctx.tok_seq, seq_start=ctx.seq_start, seq_len_before=ctx.seq_len_before, pool=kv.k,
                          page_table=kv.page_table, ring=kv.ring, pinned=kv.pinned)
        ring_cache = kv.writable and self.cache_window is not None
        after = ring_cache and not ctx.is_decode          # a ring is appended to after a step of several tokens
        cq, rows = None, None
        if self.q_rank or kv.writable:
            cq, rows = kernels.latent_prep(proj, self.q_rank, self.kv_rank, self.dr, self.w_qn, self.w_kvn, self.eps, tables,
                                           ctx.tok_pos, ctx.err, append=None if after else append, halves=self.halves,
                                           kv_off=self.q_cols)
        # the step's rows by the pool they go to, for the layers of this step that read this layer's cache
        shared = ctx.__dict__.setdefault("step_rows", {})
        if kv.writable:
            shared[kv.k.data_ptr()] = rows
        step_rows = shared.get(kv.k.data_ptr())
        if (self.w_kv_heads is not None and kernels.ops.MMA_ATTENTION and not ctx.is_decode and step_rows is not None
                and step_rows.shape[0] == x.shape[0] and not any(ctx.lens_before)):
            heads = self._whole_prompts(cq, proj, step_rows, tables, kv, ctx)
            if after:
                kernels.latent_append(rows, ctx.tok_pos, append)
            if self.gate == "head":
                kernels.head_gate_(heads, proj[:, self.gate_off:], self.nh)
            elif self.gate == "elements":
                kernels.head_gate_(heads, proj[:, self.gate_off:], self.nh * self.dv)
            return kernels.linear(heads, self.w_o, out_dtype=_delta_dtype(heads))
        q = kernels.linear(cq, self.w_uq) if self.q_rank else proj[:, :self.q_cols]
        q_lat = kernels.head_matmul(q, self.w_uk, tail=self.dr, tables=tables, tok_pos=ctx.tok_pos, err=ctx.err, halves=self.halves)
        o_lat = kernels.latent_attention(ctx.is_decode, q_lat, self.nh, self.row, self.kv_rank, rows if after else None, kv.k,
                                         kv.page_table, kv.ring, kv.pinned, ctx.seq_start, ctx.seq_len_before, ctx.n_seqs,
                                         ctx.max_new, self.window, self.scale, self.sink_logits,
                                         n_splits=self._splits(ctx) if ctx.is_decode else 1)
        if after:
            kernels.latent_append(rows, ctx.tok_pos, append)
        heads = kernels.head_matmul(o_lat, self.w_uv_t, gate=proj[:, self.gate_off:] if self.head_gate else None,
                                    gate_elems=self.gate == "elements")
        return kernels.linear(heads, self.w_o, out_dtype=_delta_dtype(heads))

    def _whole_prompts(self, cq, proj, rows, tables, kv, ctx):
        """Attention of a step without history on the tensor cores: [T, heads * value_dim], before gate and output."""
        H, dk = self.nh, self.dn + self.dr
        packed = torch.empty((rows.shape[0], 3 * H * dk), dtype=rows.dtype, device=rows.device)     # queries | keys | values, by head
        if self.q_rank:
            kernels.linear(cq, self.w_uq, out=packed[:, :H * dk])
        else:
            packed[:, :H * dk].copy_(proj[:, :self.q_cols])
        kernels.rope_pairs_(packed, H, dk, self.dn, tables, ctx.tok_pos, ctx.err, halves=self.halves)
        kernels.linear(rows, self.w_kv_heads, out=packed[:, H * dk:])
        extras = kernels.AttnExtras(sink_logits=self.sink_logits) if self.sink else None
        return kernels.attention_prefill(packed, H, H, dk, kv.k, kv.k, kv.page_table, kv.ring, ctx.seq_start, ctx.seq_len_before,
                                         ctx.n_seqs, ctx.max_new, self.window, self.scale, all_from_cache=False, extras=extras)


def _delta_dtype(x):
    """What a part's last product hands on to the norm of its output (see parts/mlp.py: delta_dtype)."""
    from .mlp import delta_dtype
    return delta_dtype(x)
