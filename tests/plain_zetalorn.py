"""A plain, slow evaluation of the Zetalorn decoder in float64 numpy: one function per mechanism, whole sequences, no
cache, no code shared with the package.  `forward(config, tensors, tokens)` takes the parsed config.json, a dict of
arrays by tensor name and one sequence's token ids; it returns the logits at every position and the residual stream
after every layer run.

Notation: T tokens, stream width D, h a sub-layer's normed input, positions p = 0 .. T-1.
"""
from __future__ import annotations

import numpy as np


def rms(x, eps):
    return x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softmax_masked(scores, visible):
    """Rows of `scores` [.., T, N] turned into weights over the visible columns (visible: bool [T, N])."""
    s = np.where(visible, scores, -np.inf)
    s = s - s.max(axis=-1, keepdims=True)
    e = np.where(visible, np.exp(s), 0.0)
    return e / e.sum(axis=-1, keepdims=True)


def rotate(x, pos, dims, base, factor, layout):
    """x [T, n, d]: the first `dims` elements of every row turned by the angles pos * base^(-2i/dims) / factor.
    layout "neighbours": element 2i with 2i+1; "halves": element i with i + dims/2."""
    if not dims:
        return x
    half = dims // 2
    freq = base ** (-2.0 * np.arange(half) / dims) / factor
    ang = np.asarray(pos, dtype=np.float64)[:, None] * freq[None, :]                 # [T, half]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    out = x.copy()
    if layout == "neighbours":
        u, v = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = u * c - v * s
        out[..., 1:dims:2] = v * c + u * s
    else:
        u, v = x[..., :half], x[..., half:dims]
        out[..., :half] = u * c - v * s
        out[..., half:dims] = v * c + u * s
    return out


def chunk_mask(T, size):
    i, j = np.arange(T)[:, None], np.arange(T)[None, :]
    return (j <= i) & (i // size == j // size)


def window_mask(T, size):
    i, j = np.arange(T)[:, None], np.arange(T)[None, :]
    return (j <= i) & (i - j < size)


def pooled_mask(T, size, pool):
    """[T, T // pool]: query i sees block b when the block's last position has left the window."""
    i, b = np.arange(T)[:, None], np.arange(T // pool)[None, :]
    return b * pool + pool - 1 <= i - size


def differential_attention(h, w, m, eps, pos=None):
    """The mixer of an 'attention' layer.  w: the layer's mixer tensors by local name; m: its 'mixer' object."""
    T = h.shape[0]
    pos = np.arange(T) if pos is None else pos
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m.get("vdim", m["dim"])
    q = (h @ w["q"].T).reshape(T, H * 2, d)
    k = (h @ w["k"].T).reshape(T, G * 2, d)
    v = (h @ w["v"].T).reshape(T, G, dv)
    q = rms(q, eps) * w["q.norm"]
    k = rms(k, eps) * w["k.norm"]
    rot = m.get("rot") or {}
    factor = (rot.get("scaling") or {}).get("factor", 1.0)
    q = rotate(q, pos, rot.get("dims", 0), rot.get("base", 1.0), factor, "neighbours").reshape(T, H, 2, d)
    k = rotate(k, pos, rot.get("dims", 0), rot.get("base", 1.0), factor, "neighbours").reshape(T, G, 2, d)
    visible = chunk_mask(T, (m.get("mask") or {}).get("size") or T + 1)          # no mask: one chunk
    lam = np.exp((w["lq1"] * w["lk1"]).sum()) - np.exp((w["lq2"] * w["lk2"]).sum()) + m["diff"]
    out = np.zeros((T, H, dv))
    for hd in range(H):
        g = hd // (H // G)
        a = []
        for mp in range(2):
            s = (q[:, hd, mp] @ k[:, g, mp].T) * m["scale"]
            a.append(softmax_masked(s, visible) @ v[:, g])
        o = a[0] - lam * a[1]
        out[:, hd] = rms(o, eps) * (1.0 - m["diff"])
    return out.reshape(T, H * dv) @ w["o"].T


def pooled_window_attention(h, w, m, eps):
    """The left half of a 'parallel' mixer: a sliding window over tokens plus one mean key and value for every block
    of `pool` tokens that lies wholly before the window, in one softmax."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m.get("vdim", m["dim"])
    q = rms((h @ w["q"].T).reshape(T, H, d), eps) * w["q.norm"]
    k = rms((h @ w["k"].T).reshape(T, G, d), eps) * w["k.norm"]
    v = (h @ w["v"].T).reshape(T, G, dv)
    rot = m.get("rot") or {}
    factor = (rot.get("scaling") or {}).get("factor", 1.0)
    q = rotate(q, np.arange(T), rot.get("dims", 0), rot.get("base", 1.0), factor, "halves")
    k = rotate(k, np.arange(T), rot.get("dims", 0), rot.get("base", 1.0), factor, "halves")
    W, P = m["mask"]["size"], m["mask"].get("pool") or T + 1          # no pool: no block is ever complete
    nb = T // P
    kb = k[:nb * P].reshape(nb, P, G, d).mean(axis=1)
    vb = v[:nb * P].reshape(nb, P, G, dv).mean(axis=1)
    visible = np.concatenate([window_mask(T, W), pooled_mask(T, W, P)], axis=1)
    out = np.zeros((T, H, dv))
    for hd in range(H):
        g = hd // (H // G)
        keys = np.concatenate([k[:, g], kb[:, g]], axis=0)
        vals = np.concatenate([v[:, g], vb[:, g]], axis=0)
        out[:, hd] = softmax_masked((q[:, hd] @ keys.T) * m["scale"], visible) @ vals
    return out.reshape(T, H * dv) @ w["o"].T


def lightning_attention(h, w, m, eps):
    """The right half of a 'parallel' mixer: per head S <- decay S + k v^T, o = S^T q, token after token."""
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m.get("vdim", m["dim"])
    q = silu(h @ w["q"].T).reshape(T, H, d)
    k = silu(h @ w["k"].T).reshape(T, H, d)
    v = silu(h @ w["v"].T).reshape(T, H, dv)
    decay = np.broadcast_to(np.asarray(m["decay"], dtype=np.float64), (H,))
    S = np.zeros((H, d, dv))
    o = np.zeros((T, H, dv))
    for t in range(T):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = np.einsum("hkv,hk->hv", S, q[t])
    y = rms(o.reshape(T, H * dv), eps) * w["norm"]
    return (y * sigmoid(h @ w["g"].T)) @ w["o"].T


def parallel_mixer(h, w, m, eps):
    left = {k[len("left."):]: v for k, v in w.items() if k.startswith("left.") and k != "left.out"}
    right = {k[len("right."):]: v for k, v in w.items() if k.startswith("right.") and k != "right.out"}
    a = pooled_window_attention(h, left, m["left"], eps)
    b = lightning_attention(h, right, m["right"], eps)
    return 0.5 * (rms(a, eps) * w["left.out"] + rms(b, eps) * w["right.out"])


def route(h, w_router, r):
    """(chosen experts [T, top], their weights [T, top]) of the grouped sigmoid router."""
    s = sigmoid(h @ w_router.T)
    T, E = s.shape
    top, groups = r["top"], r.get("groups") or {"count": 1, "keep": 1}
    n, keep = groups["count"], groups["keep"]
    per = E // n
    by_group = s.reshape(T, n, per)
    gs = np.sort(by_group, axis=-1)[..., ::-1][..., :2].sum(axis=-1)                  # [T, n]
    kept = np.argsort(-gs, axis=-1, kind="stable")[:, :keep]
    allowed = np.zeros((T, n), dtype=bool)
    np.put_along_axis(allowed, kept, True, axis=1)
    masked = np.where(np.repeat(allowed, per, axis=1), s, -np.inf)
    idx = np.argsort(-masked, axis=-1, kind="stable")[:, :top]
    chosen = np.take_along_axis(s, idx, axis=1)
    return idx, chosen / (chosen.sum(axis=-1, keepdims=True) + 1e-20)


def expert(h, gate, up, down, limit):
    limit = np.inf if limit is None else limit
    g = np.minimum(h @ gate.T, limit)
    u = np.clip(h @ up.T, -limit, limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ down.T


def moe(h, w, mlp):
    idx, wgt = route(h, w["router"], mlp["router"])
    out = np.zeros((h.shape[0], w["e0.down"].shape[0]))
    for t in range(h.shape[0]):
        for e, c in zip(idx[t], wgt[t]):
            out[t] += c * expert(h[t:t + 1], w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"], mlp["expert"].get("limit"))[0]
    return out


def sub(tensors, prefix):
    return {k[len(prefix) + 1:]: v for k, v in tensors.items() if k.startswith(prefix + ".")}


def layer(x, i, cfg, tensors):
    eps = cfg["norm"]["eps"]
    L = cfg["layers"][i]
    w = sub(tensors, f"l{i}.mix")
    h = rms(x, eps) * tensors[f"l{i}.norm1"]
    y = differential_attention(h, w, L["mixer"], eps) if L["type"] == "attention" else parallel_mixer(h, w, L["mixer"], eps)
    x = x + sigmoid(h @ tensors[f"l{i}.rg1"].T + tensors[f"l{i}.rg1.b"]) * y
    if L.get("mlp") is not None:
        h = rms(x, eps) * tensors[f"l{i}.norm2"]
        x = x + sigmoid(h @ tensors[f"l{i}.rg2"].T + tensors[f"l{i}.rg2.b"]) * moe(h, sub(tensors, f"l{i}.mlp"), L["mlp"])
    return x


def run_order(cfg):
    """[(layer, pass number or None when the layer does not open a pass)] in the order the layers run."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    order = [(i, None) for i in range(loop["start"])]
    for t in range(loop["times"]):
        order += [(i, t if i == loop["start"] else None) for i in range(loop["start"], loop["stop"])]
    return order + [(i, None) for i in range(loop["stop"], n)]


def forward(cfg, tensors, tokens):
    tensors = {k: np.asarray(v, dtype=np.float64) for k, v in tensors.items()}
    x0 = tensors["embed"][np.asarray(tokens)]
    x, after = x0.copy(), []
    for i, t in run_order(cfg):
        if t is not None:
            if t > 0:
                x = x + x0
            x = x + tensors["loop.step"][t]
        x = layer(x, i, cfg, tensors)
        after.append(x.copy())
    h = rms(x, cfg["norm"]["eps"]) * tensors["final.norm"]
    return (h @ tensors["head"].T) * cfg.get("logit_scale", 1.0), np.stack(after)
