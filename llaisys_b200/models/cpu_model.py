"""A decoder on the CPU, put together from the plain float32 operators of `cpu_ops`: one sequence,
a contiguous cache per attention call, the prompt in one step and then one token per step,
greedy choice of the next token.

This is what xsmccc/llaisys' own model is (src/models/qwen2/qwen2.cpp:53-87: operators on the
CPU, float32, one sequence), and it serves here as the second implementation that the command
line's --test compares the engine's tokens with (test/test_infer.py:193-195 compares with a
second implementation too), and as the model behind --device cpu.  It reads the same `ModelSpec`
and the same tensors by name as the engine does, shares no code with the engine's parts or
kernels, and knows the built-in part kinds only (those of both built-in architectures).
"""
from __future__ import annotations

from typing import Dict, List, Sequence

import numpy as np

from .. import cpu_ops
from ..config.spec import ModelSpec, PartSpec

_KNOWN = {"embedding": {"token_embedding", "scaled_pair_embedding"}, "norm": {"rms_norm"},
          "mixer": {"gqa_attention", "windowed_sink_attention", "gated_linear_attention", "latent_attention", "min_gru",
                    "differential_attention", "pooled_window_attention", "lightning_attention", "parallel_mixers"},
          "ffn": {"swiglu_mlp", "routed_experts", "gated_mlp"},
          "block": {"pre_norm_residual", "parallel_residual", "sandwich_residual", "depth_averaged_residual", "gated_residual"},
          "head": {"lm_head"}, "reentry": {"embedding_and_offset"},
          "position": {"rope_half_split", "rope_leading", "rope_interleaved"}}


class CpuModel:
    def __init__(self, spec: ModelSpec, tensors: Dict[str, np.ndarray]):
        """tensors: name -> float32 array, the names being those of the weights file."""
        self.spec, self.w = spec, tensors
        for kind, cat in [(spec.embedding.kind, "embedding"), (spec.final_norm.kind, "norm"), (spec.head.kind, "head")]:
            self._known(cat, kind)
        for layer in spec.layers:
            self._known("block", layer.block)
            for sub in layer.sublayers:
                self._known(sub.category, sub.part.kind)
                if sub.norm is not None:
                    self._known("norm", sub.norm.kind)
                for part in [sub.part] + [b["part"] for b in sub.part.params.get("branches", [])]:
                    self._known("mixer" if part is not sub.part else sub.category, part.kind)
                    pos = part.params.get("position")
                    if pos is not None:
                        self._known("position", pos.kind)
        if spec.reentry is not None:
            self._known("reentry", spec.reentry.kind)
        self.reset()

    @staticmethod
    def _known(category: str, kind: str):
        if kind not in _KNOWN[category]:
            raise NotImplementedError(f"the CPU model knows the built-in parts only, not the {category} {kind!r}")

    @classmethod
    def from_folder(cls, folder) -> "CpuModel":
        from ..config.registry import load_config
        from ..weights.loader import FolderSource
        src = FolderSource(folder)
        return cls(load_config(folder).to_spec(), {n: src.get(n).float().numpy() for n in src.entries()})

    def reset(self) -> None:
        self.length = 0
        self.last_token = None                                       # the token before the next step's first (pair embedding)
        self.cache: List[dict] = [{} for _ in self.spec.order]       # per entry of the run order: mixer index -> (k, v)

    # ---- parts
    def _norm(self, p: PartSpec, x):
        w = self.w[p.tensor_name(p.params.get("tensor", "weight"))]
        if p.params.get("offset"):
            w = w.astype(np.float32) + np.float32(p.params["offset"])       # stored as the distance from the offset
        return cpu_ops.rms_norm(x, w, p.params["eps"])

    def _gla(self, p: PartSpec, x, store: dict, key):
        a = p.params
        H, dk, dv = a["num_heads"], a["key_dim"], a["value_dim"]
        n = dict({"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "norm": "norm", "a1": "a1", "a2": "a2", "a2_bias": "a2.b"},
                 **(a.get("names") or {}))
        w = lambda k: self.w[p.tensor_name(n[k])]
        T = x.shape[0]
        q = cpu_ops.linear(x, w("q")).reshape(T, H, dk) * np.float32(a.get("query_scale", 1.0))
        k = cpu_ops.linear(x, w("k")).reshape(T, H, dk)
        v = cpu_ops.linear(x, w("v")).reshape(T, H, dv)
        z = cpu_ops.linear(cpu_ops.linear(x, w("a1")), w("a2"), w("a2_bias")).reshape(T, H, dk)
        if key not in store:
            store[key] = np.zeros((H, dk, dv), dtype=np.float32)
        o = cpu_ops.gated_linear_recurrence(q, k, v, z, store[key], a["decay_root"])
        o = cpu_ops.rms_norm(o, w("norm"), a["eps"]).reshape(T, H * dv)
        g = cpu_ops.linear(x, w("g"))
        return cpu_ops.linear(o * (g / (np.float32(1) + np.exp(-g))), w("o"))

    def _min_gru(self, p: PartSpec, x, store: dict, key):
        a = p.params
        n = dict({"z": "z", "z_bias": "z.b", "x": "x", "x_bias": "x.b", "g": "g", "o": "o"}, **(a.get("names") or {}))
        w = lambda k: self.w[p.tensor_name(n[k])]
        if key not in store:
            store[key] = np.zeros(a["width"], dtype=np.float32)
        S = cpu_ops.min_gru(cpu_ops.linear(x, w("z"), w("z_bias")), cpu_ops.linear(x, w("x"), w("x_bias")), store[key])
        g = cpu_ops.linear(x, w("g"))
        return cpu_ops.linear(S * (g * cpu_ops.sigmoid(g)), w("o"))

    def _latent(self, p: PartSpec, x, positions, store: dict, key, owner):
        """The heads' keys and values are made from the cached latents here (the engine carries the queries into the
        latent space instead)."""
        a = p.params
        H, dn, dr, dv, r = a["num_heads"], a["nope_dim"], a["rope_dim"], a["value_dim"], a["kv_rank"]
        n = dict({"q": "q", "dq": "dq", "dq_norm": "dq.norm", "uq": "uq", "dkv": "dkv", "dkv_norm": "dkv.norm", "uk": "uk", "uv": "uv",
                  "sink": "sink", "g": "g", "o": "o"}, **(a.get("names") or {}))
        w = lambda k: self.w[p.tensor_name(n[k])]
        if a.get("position") is None:
            rot = lambda t: t.astype(np.float32)
        elif a["position"].kind == "rope_leading":                # pairs (i, i + dims/2)
            pos = a["position"].params
            rot = lambda t: cpu_ops.rope_leading(t, positions, pos["dims"], pos["base"])
        else:
            pos = a["position"].params
            rot = lambda t: cpu_ops.rope_pairs(t, positions, pos["dims"], pos["base"], pos.get("yarn"))
        T = x.shape[0]
        if a.get("q_rank"):
            cq = cpu_ops.rms_norm(cpu_ops.linear(x, w("dq")), w("dq_norm"), a["eps"])
            q = cpu_ops.linear(cq, w("uq")).reshape(T, H, dn + dr)
        else:                                                     # no query latent
            q = cpu_ops.linear(x, w("q")).reshape(T, H, dn + dr)
        q = np.concatenate([q[:, :, :dn], rot(q[:, :, dn:])], axis=-1)
        if owner is None:
            d = cpu_ops.linear(x, w("dkv"))
            c, kr = cpu_ops.rms_norm(d[:, :r], w("dkv_norm"), a["eps"]), rot(d[:, None, r:])[:, 0]
            old = store.get(key)
            store[key] = (c, kr) if old is None else (np.concatenate([old[0], c]), np.concatenate([old[1], kr]))
            cs, krs = store[key]
        else:
            cs, krs = owner[key]
        L = cs.shape[0]
        k = np.concatenate([cpu_ops.linear(cs, w("uk")).reshape(L, H, dn), np.broadcast_to(krs[:, None, :], (L, H, dr))], axis=-1)
        v = cpu_ops.linear(cs, w("uv")).reshape(L, H, dv)
        o = cpu_ops.self_attention(q, k, v, a["scale"], a.get("window"), sink_logits=w("sink") if a.get("sink") else None)
        gate = a.get("gate") or ("head" if a.get("head_gate") else None)
        if gate is not None:
            g = cpu_ops.sigmoid(cpu_ops.linear(x, w("g")))
            o = o * (g[:, :, None] if gate == "head" else g.reshape(T, H, dv))
        return cpu_ops.linear(o.reshape(T, H * dv), w("o"))

    def _gated_mlp(self, p: PartSpec, x):
        n = dict({"gate": "gate_proj.weight", "up": "up_proj.weight", "down": "down_proj.weight"}, **(p.params.get("names") or {}))
        sfx = p.params.get("bias_suffix", ".b")
        b = (lambda k: self.w[p.tensor_name(n[k] + sfx)]) if p.params.get("bias") else (lambda k: None)
        g, u = cpu_ops.linear(x, self.w[p.tensor_name(n["gate"])], b("gate")), cpu_ops.linear(x, self.w[p.tensor_name(n["up"])], b("up"))
        return cpu_ops.linear(cpu_ops.glu(g, u, p.params.get("act", "silu")), self.w[p.tensor_name(n["down"])], b("down"))

    # ---- mixers with normed heads, blocks of keys, two score maps, a constant-decay recurrence
    def _normed_rows(self, p: PartSpec, x, positions, maps: int):
        """q [T, nh * maps, dk], k [T, nkvh * maps, dk] (normed over their elements, then rotated), v [T, nkvh, dv]."""
        a = p.params
        nh, nkvh, dk, dv = a["num_heads"], a["num_kv_heads"], a["key_dim"], a["value_dim"]
        n = dict({"q": "q", "k": "k", "v": "v", "o": "o", "q_norm": "q.norm", "k_norm": "k.norm"}, **(a.get("names") or {}))
        T = x.shape[0]
        q = cpu_ops.linear(x, self.w[p.tensor_name(n["q"])]).reshape(T, nh * maps, dk)
        k = cpu_ops.linear(x, self.w[p.tensor_name(n["k"])]).reshape(T, nkvh * maps, dk)
        v = cpu_ops.linear(x, self.w[p.tensor_name(n["v"])]).reshape(T, nkvh, dv)
        if a.get("qk_norm", True):
            q = cpu_ops.rms_norm(q, self.w[p.tensor_name(n["q_norm"])], a.get("eps", 0.0))
            k = cpu_ops.rms_norm(k, self.w[p.tensor_name(n["k_norm"])], a.get("eps", 0.0))
        pos = a.get("position")
        if pos is not None:
            pp = pos.params
            rot = lambda t: cpu_ops.rotate_pairs(t, positions, pp["dims"], pp["base"], pp.get("factor", 1.0), pos.kind == "rope_interleaved")
            q, k = rot(q), rot(k)
        return q, k, v, n

    @staticmethod
    def _kept(store, key, k, v):
        old = store.get(key)
        store[key] = (k, v) if old is None else (np.concatenate([old[0], k]), np.concatenate([old[1], v]))
        return store[key]

    def _differential(self, p: PartSpec, x, positions, store: dict, key):
        a = p.params
        nh, nkvh, dk, dv = a["num_heads"], a["num_kv_heads"], a["key_dim"], a["value_dim"]
        q, k, v, n = self._normed_rows(p, x, positions, 2)
        ks, vs = self._kept(store, key, k, v)
        T, L = x.shape[0], ks.shape[0]
        j, i = np.arange(L)[None, :], np.asarray(positions)[:, None]
        visible = j <= i
        if a.get("chunk"):
            visible &= (j // a["chunk"]) == (i // a["chunk"])
        if a.get("window"):
            visible &= i - j < a["window"]
        q, ks = q.reshape(T, nh, 2, dk), ks.reshape(L, nkvh, 2, dk)
        a1 = cpu_ops.masked_attention(q[:, :, 0], ks[:, :, 0], vs, a["scale"], visible)
        a2 = cpu_ops.masked_attention(q[:, :, 1], ks[:, :, 1], vs, a["scale"], visible)
        l = [self.w[p.tensor_name(dict({"lq1": "lq1", "lk1": "lk1", "lq2": "lq2", "lk2": "lk2"}, **(a.get("names") or {}))[t])].astype(np.float32)
             for t in ("lq1", "lk1", "lq2", "lk2")]
        lam = np.exp((l[0] * l[1]).sum()) - np.exp((l[2] * l[3]).sum()) + np.float32(a["diff"])
        o = a1 - np.float32(lam) * a2
        o = cpu_ops.rms_norm(o, np.ones(dv, dtype=np.float32), a.get("eps", 0.0)) * np.float32(1.0 - a["diff"])
        return cpu_ops.linear(o.reshape(T, nh * dv), self.w[p.tensor_name(n["o"])])

    def _pooled_window(self, p: PartSpec, x, positions, store: dict, key):
        a = p.params
        nh, dv, W, P = a["num_heads"], a["value_dim"], a["window"], a.get("pool") or 0
        q, k, v, n = self._normed_rows(p, x, positions, 1)
        ks, vs = self._kept(store, key, k, v)
        T, L = x.shape[0], ks.shape[0]
        P = P or L + 1                                             # no pool: no block is ever complete
        nb = L // P
        kb = ks[:nb * P].reshape(nb, P, *ks.shape[1:]).mean(axis=1, dtype=np.float32)
        vb = vs[:nb * P].reshape(nb, P, *vs.shape[1:]).mean(axis=1, dtype=np.float32)
        i = np.asarray(positions)[:, None]
        j, b = np.arange(L)[None, :], np.arange(nb)[None, :]
        visible = np.concatenate([(j <= i) & (i - j < W), b * P + P - 1 <= i - W], axis=1)
        o = cpu_ops.masked_attention(q, np.concatenate([ks, kb]), np.concatenate([vs, vb]), a["scale"], visible)
        return cpu_ops.linear(o.reshape(T, nh * dv), self.w[p.tensor_name(n["o"])])

    def _lightning(self, p: PartSpec, x, store: dict, key):
        a = p.params
        H, dk, dv = a["num_heads"], a["key_dim"], a["value_dim"]
        n = dict({"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "norm": "norm"}, **(a.get("names") or {}))
        w = lambda t: self.w[p.tensor_name(n[t])]
        T = x.shape[0]
        silu = lambda t: t * cpu_ops.sigmoid(t)
        q, k = silu(cpu_ops.linear(x, w("q"))).reshape(T, H, dk), silu(cpu_ops.linear(x, w("k"))).reshape(T, H, dk)
        v = silu(cpu_ops.linear(x, w("v"))).reshape(T, H, dv)
        if key not in store:
            store[key] = np.zeros((H, dk, dv), dtype=np.float32)
        o = cpu_ops.decayed_linear_recurrence(q, k, v, np.asarray(a["decay"], dtype=np.float32), store[key]).reshape(T, H * dv)
        o = cpu_ops.rms_norm(o, w("norm"), a["eps"]) * cpu_ops.sigmoid(cpu_ops.linear(x, w("g")))
        return cpu_ops.linear(o, w("o"))

    def _mixer_of(self, part: PartSpec, h, positions, store, key):
        if part.kind == "differential_attention":
            return self._differential(part, h, positions, store, key)
        if part.kind == "pooled_window_attention":
            return self._pooled_window(part, h, positions, store, key)
        if part.kind == "lightning_attention":
            return self._lightning(part, h, store, key)
        a = part.params                                            # parallel_mixers
        outs = [self._mixer_of(b["part"], h, positions, store, (key, i)) for i, b in enumerate(a["branches"])]
        ws = [self.w[part.tensor_name(b["out"])] for b in a["branches"]]
        return sum(cpu_ops.rms_norm(o, w, a["eps"]) for o, w in zip(outs, ws)) * np.float32(1.0 / len(outs))

    def _part(self, sub, h, positions, store, m, owner):
        """One part's output for normed input h."""
        kind = sub.part.kind
        if kind in ("differential_attention", "pooled_window_attention", "lightning_attention", "parallel_mixers"):
            return self._mixer_of(sub.part, h, positions, store, m)
        if kind == "gated_linear_attention":
            return self._gla(sub.part, h, store, m)
        if kind == "min_gru":
            return self._min_gru(sub.part, h, store, m)
        if kind == "latent_attention":
            return self._latent(sub.part, h, positions, store, m, owner)
        if kind == "windowed_sink_attention":
            return self._sink_attention(sub.part, h, positions, store, m, owner)
        if kind == "gqa_attention":
            return self._attention(sub.part, h, positions, store, m, owner)
        if kind == "routed_experts":
            return self._routed(sub.part, h)
        if kind == "gated_mlp":
            return self._gated_mlp(sub.part, h)
        return self._mlp(sub.part, h)

    def _embed(self, tokens):
        p = self.spec.embedding
        ids = np.asarray(tokens)
        if p.kind == "token_embedding":
            return cpu_ops.embedding(ids, self.w[p.tensor_name("weight")]).astype(np.float32)
        a = p.params
        x = cpu_ops.embedding(ids, self.w[p.tensor_name(a.get("tensor", "weight"))]).astype(np.float32) * np.float32(a.get("scale", 1.0))
        if a.get("pair"):
            pr = a["pair"]
            prev = np.concatenate([[self.last_token if self.last_token is not None else 0], ids[:-1]]).astype(np.int64)
            rows = (prev * int(pr["mul_prev"]) + ids.astype(np.int64) * int(pr["mul_cur"])) % int(pr["buckets"])
            if self.length == 0:
                rows[0] = int(pr["buckets"])
            x = cpu_ops.add(x, cpu_ops.embedding(rows, self.w[p.tensor_name(pr["tensor"])]))
        self.last_token = int(ids[-1])
        return x

    def _sink_attention(self, p: PartSpec, x, positions, store: dict, key, owner):
        a = p.params
        nh, nkvh, dk, dv = a["num_heads"], a["num_kv_heads"], a["key_dim"], a["value_dim"]
        n = dict({"q": "q", "k": "k", "v": "v", "o": "o", "r1": "r1", "r2": "r2"}, **(a.get("names") or {}))
        T = x.shape[0]
        pos = a.get("position")
        rot = (lambda t: cpu_ops.rope_leading(t, positions, pos.params["dims"], pos.params["base"])) if pos is not None else (lambda t: t)
        q = rot(cpu_ops.linear(x, self.w[p.tensor_name(n["q"])]).reshape(T, nh, dk))
        if a.get("q_temp"):
            q = q * cpu_ops.query_temperature(positions, a["q_temp"]["coef"], a["q_temp"]["every"])[:, None, None]
        bias = (self.w[p.tensor_name(n["r1"])], self.w[p.tensor_name(n["r2"])]) if a.get("distance_bias") else None
        if owner is None:
            k = rot(cpu_ops.linear(x, self.w[p.tensor_name(n["k"])]).reshape(T, nkvh, dk))
            v = cpu_ops.linear(x, self.w[p.tensor_name(n["v"])]).reshape(T, nkvh, dv)
            old = store.get(key)
            store[key] = (k, v) if old is None else (np.concatenate([old[0], k]), np.concatenate([old[1], v]))
            ks, vs = store[key]
        else:
            ks, vs = owner[key]
        o = cpu_ops.self_attention(q, ks, vs, a["scale"], a.get("window"), a.get("keep_first", 0), bool(a.get("sink")), dist_bias=bias)
        return cpu_ops.linear(o.reshape(T, nh * dv), self.w[p.tensor_name(n["o"])])

    def _routed(self, p: PartSpec, x):
        a = p.params
        n = {"router": "router", "bias": "correction", "expert_up": "e{e}.up", "expert_down": "e{e}.down",
             "shared_up": "shared.up", "shared_down": "shared.down", "shared_gate": "shared.sg", **(a.get("names") or {})}
        bias = self.w[p.tensor_name(n["bias"])] if a.get("use_bias", True) else None
        logits = cpu_ops.linear(x, self.w[p.tensor_name(n["router"])])
        if a.get("groups") or a.get("renorm"):
            g = a.get("groups")
            idx, wgt = cpu_ops.route_grouped(logits, a["top"], (g["count"], g["keep"]) if g else None, bool(a.get("renorm")),
                                             a.get("route_scale", 1.0))
        else:
            top_of = cpu_ops.route_top_softmax if a.get("gate") == "softmax_chosen" else cpu_ops.route_top
            idx, wgt = top_of(logits, bias, a["top"], a.get("route_scale", 1.0))
        act = cpu_ops.gelu if a.get("act") == "gelu" else cpu_ops.relu_squared
        gated = a.get("act") == "swish_clamped"
        out = np.zeros((x.shape[0], a["hidden_size"]), dtype=np.float32)
        for t in range(x.shape[0]):
            for e, wt in zip(idx[t], wgt[t]):
                up = self.w[p.tensor_name(n["expert_up"].format(e=int(e)))]
                down = self.w[p.tensor_name(n["expert_down"].format(e=int(e)))]
                if gated:
                    gate = self.w[p.tensor_name(n.get("expert_gate", "e{e}.gate").format(e=int(e)))]
                    y = cpu_ops.swish_clamped(cpu_ops.linear(x[t:t + 1], gate), cpu_ops.linear(x[t:t + 1], up), a["limit"], a.get("alpha", 1.0))
                else:
                    y = act(cpu_ops.linear(x[t:t + 1], up))
                out[t] += wt * cpu_ops.linear(y, down)[0]
        if a.get("shared_ff"):
            shared = cpu_ops.linear(act(cpu_ops.linear(x, self.w[p.tensor_name(n["shared_up"])])), self.w[p.tensor_name(n["shared_down"])])
            if a.get("shared_gate"):
                shared = shared * cpu_ops.sigmoid(cpu_ops.linear(x, self.w[p.tensor_name(n["shared_gate"])].reshape(1, -1)))
            out = cpu_ops.add(out, shared)
        return out

    def _attention(self, p: PartSpec, x, positions, store: dict, key, owner):
        a = p.params
        nh, nkvh, dh = a["num_heads"], a["num_kv_heads"], a["head_dim"]
        T = x.shape[0]
        bias = (lambda n: self.w[p.tensor_name(n)]) if a.get("qkv_bias") else (lambda n: None)
        q = cpu_ops.linear(x, self.w[p.tensor_name("q_proj.weight")], bias("q_proj.bias")).reshape(T, nh, dh)
        k = cpu_ops.linear(x, self.w[p.tensor_name("k_proj.weight")], bias("k_proj.bias")).reshape(T, nkvh, dh)
        v = cpu_ops.linear(x, self.w[p.tensor_name("v_proj.weight")], bias("v_proj.bias")).reshape(T, nkvh, dh)
        if a.get("position") is not None:
            theta = a["position"].params["theta"]
            q, k = cpu_ops.rope(q, positions, theta), cpu_ops.rope(k, positions, theta)
        if owner is None:
            old = store.get(key)
            store[key] = (k, v) if old is None else (np.concatenate([old[0], k]), np.concatenate([old[1], v]))
            ks, vs = store[key]
        else:
            ks, vs = owner[key]                       # an earlier entry's keys and values; nothing is appended
        o = cpu_ops.self_attention(q, ks, vs, a["scale"], a.get("window"))
        out_bias = self.w[p.tensor_name("o_proj.bias")] if a.get("out_bias") else None
        return cpu_ops.linear(o.reshape(T, nh * dh), self.w[p.tensor_name("o_proj.weight")], out_bias)

    def _mlp(self, p: PartSpec, x):
        g = cpu_ops.linear(x, self.w[p.tensor_name("gate_proj.weight")])
        u = cpu_ops.linear(x, self.w[p.tensor_name("up_proj.weight")])
        return cpu_ops.linear(cpu_ops.swiglu(g, u), self.w[p.tensor_name("down_proj.weight")])

    # ---- the model
    def step(self, tokens: Sequence[int]) -> np.ndarray:
        """Feeds the next tokens of the sequence; returns float32 logits [len(tokens), vocab]."""
        positions = np.arange(self.length, self.length + len(tokens))
        x = self._embed(tokens)
        first = x                                          # looped layers: the embedding's output joins again before later passes
        results = [x]                                      # depth-averaged layers: the embedding's output and every layer's result
        for c, call in enumerate(self.spec.order):
            if call.opens_pass is not None:
                re = self.spec.reentry
                offsets = self.w[re.tensor_name(re.params.get("tensor", "offset"))].astype(np.float32)
                if call.opens_pass > 0:
                    x = cpu_ops.add(x, first)
                x = cpu_ops.add(x, np.broadcast_to(offsets[call.opens_pass], x.shape))
            owner = self.cache[call.cache_of] if call.cache_of is not None else None
            m = 0
            layer = self.spec.layers[call.layer]
            parallel = layer.block == "parallel_residual"          # every sub-layer reads the stream as the layer found it
            x_in = x
            for sub in layer.sublayers:
                src = x_in if parallel else x
                h = self._norm(sub.norm, src) if sub.norm is not None else src
                y = self._part(sub, h, positions, self.cache[c], m, owner)
                if sub.category == "mixer":
                    m += 1
                if layer.block == "sandwich_residual":       # the part's output is normed and scaled on its way into the stream
                    y = self._norm(sub.post_norm, y) * np.float32(layer.params.get("mult", 1.0))
                elif layer.block == "depth_averaged_residual":
                    y = y * np.float32(layer.params.get("mult", 1.0))
                elif layer.block == "gated_residual":          # the part's output passes a gate computed from the same input
                    g = layer.params["gates"][layer.sublayers.index(sub)]
                    prefix = layer.params.get("prefix", "")
                    y = y * cpu_ops.sigmoid(cpu_ops.linear(h, self.w[f"{prefix}.{g}"], self.w[f"{prefix}.{g}.b"]))
                x = cpu_ops.add(y, x)
            if layer.block == "depth_averaged_residual":     # what goes on is a weighted sum of all results so far
                results.append(x)
                a = self.w[f"{layer.params['prefix']}.{layer.params.get('tensor', 'dwa')}"].astype(np.float32)
                x = sum(a[j] * r for j, r in enumerate(results))
        self.length += len(tokens)
        x = self._norm(self.spec.final_norm, x)
        head = self.spec.head
        name = head.params.get("tied_to") or head.tensor_name(head.params.get("tensor", "weight"))
        return cpu_ops.linear(x, self.w[name]) * np.float32(head.params.get("scale", 1.0))

    def generate(self, prompt: Sequence[int], max_new_tokens: int, stop_ids: Sequence[int] = ()) -> List[int]:
        """Greedy continuation: the new tokens (a stop token included)."""
        self.reset()
        logits = self.step(list(prompt))[-1]
        new: List[int] = []
        for _ in range(max_new_tokens):
            tok, _ = cpu_ops.argmax(logits)
            new.append(tok)
            if tok in stop_ids or len(new) == max_new_tokens:
                break
            logits = self.step([tok])[-1]
        return new
