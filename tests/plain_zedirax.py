"""A plain, slow implementation of the Zedirax decoder in float64 numpy: one function per mechanism, whole
sequences, no cache, no state carried between calls, and no code shared with the package.

Notation: T tokens, stream width D, x [T, D] the residual stream, h the normed input of a mixer or feed-forward.
Weights come as a dict name -> array with the names of the weights file; matrices are [out, in].
"""
from __future__ import annotations

import math

import numpy as np


def rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    x = np.asarray(x, dtype=np.float64)
    return x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps)


def norm_plain(x, w, eps):
    return rms(x, eps) * np.asarray(w, dtype=np.float64)


def norm_offset(x, w, eps):
    """The layers' norm: the stored weight is the distance from one."""
    return rms(x, eps) * (1.0 + np.asarray(w, dtype=np.float64))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def gelu_erf(z):
    return 0.5 * z * (1.0 + np.vectorize(math.erf)(z / math.sqrt(2.0)))


def softmax_rows(s):
    e = np.exp(s - s.max(axis=-1, keepdims=True))
    return e / e.sum(axis=-1, keepdims=True)


# ---------------------------------------------------------------------------------------------- rotation
def rotate_halves(x, positions, dims, base):
    """Rotates the pairs (i, i + dims/2), i < dims/2, of the last axis of x [T, ..., n >= dims]; the rest passes."""
    half = dims // 2
    f = base ** (-2.0 * np.arange(half, dtype=np.float64) / dims)
    ang = np.asarray(positions, dtype=np.float64)[:, None] * f[None, :]
    shape = (len(positions),) + (1,) * (x.ndim - 2) + (half,)
    cos, sin = np.cos(ang).reshape(shape), np.sin(ang).reshape(shape)
    out = np.array(x, dtype=np.float64)
    u, v = out[..., :half].copy(), out[..., half:dims].copy()
    out[..., :half] = u * cos - v * sin
    out[..., half:dims] = v * cos + u * sin
    return out


# ---------------------------------------------------------------------------------------------- mixers
def mingru_candidate(u):
    """u + 1/2 where u >= 0, sigmoid(u) below: continuous, positive."""
    return np.where(u >= 0, u + 0.5, sigmoid(np.minimum(u, 0.0)))


def mingru_mixer(h, w, p, state=None):
    """The gated recurrence whose gates read the current token only.  Returns (output [T, D], final state [width])."""
    z = sigmoid(h @ w[p + ".z"].T + w[p + ".z.b"])
    c = mingru_candidate(h @ w[p + ".x"].T + w[p + ".x.b"])
    T, W = z.shape
    S = np.zeros(W) if state is None else np.array(state, dtype=np.float64)
    out = np.zeros((T, W))
    for t in range(T):
        S = (1.0 - z[t]) * S + z[t] * c[t]
        out[t] = S
    return (out * silu(h @ w[p + ".g"].T)) @ w[p + ".o"].T, S


def latent_attention_mixer(h, w, p, mix, eps, positions):
    """Attention whose keys and values come from one normed latent per token and one rotated key part for all heads."""
    H, dn, dr, dv, r = mix["heads"], mix["dim"], mix["rot_dim"], mix["vdim"], mix["kv_rank"]
    T = h.shape[0]
    rot = mix["rot"]
    q = (h @ w[p + ".q"].T).reshape(T, H, dn + dr)
    qr = rotate_halves(q[:, :, dn:], positions, rot["dims"], rot["base"])
    d = h @ w[p + ".dkv"].T
    c = norm_plain(d[:, :r], w[p + ".dkv.norm"], eps)
    kr = rotate_halves(d[:, r:], positions, rot["dims"], rot["base"])
    kn = (c @ w[p + ".uk"].T).reshape(T, H, dn)
    val = (c @ w[p + ".uv"].T).reshape(T, H, dv)
    s = (np.einsum("thd,shd->hts", q[:, :, :dn], kn) + np.einsum("thd,sd->hts", qr, kr)) * float(mix["scale"])
    i, j = np.asarray(positions)[:, None], np.asarray(positions)[None, :]
    s = np.where((j <= i)[None], s, -np.inf)
    o = np.einsum("hts,shv->thv", softmax_rows(s), val).reshape(T, H * dv)
    return (o * sigmoid(h @ w[p + ".g"].T)) @ w[p + ".o"].T


def query_temperature(positions, coef, every):
    """1 + coef ln(floor((p + 1) / every) + 1): one until position every - 1, then growing in steps."""
    p = np.asarray(positions, dtype=np.int64)
    return 1.0 + float(coef) * np.log(((p + 1) // int(every)) + 1.0)


def biased_attention_mixer(h, w, p, mix, positions):
    """Grouped-query attention without rotation: the query grows with its position, and a score loses
    r1 ln(1 + r2 distance) with two numbers per head."""
    H, G, dk, dv = mix["heads"], mix["kv_heads"], mix["dim"], mix["vdim"]
    T = h.shape[0]
    q = (h @ w[p + ".q"].T).reshape(T, H, dk)
    k = (h @ w[p + ".k"].T).reshape(T, G, dk)
    v = (h @ w[p + ".v"].T).reshape(T, G, dv)
    qt = mix.get("q_temp")
    if qt:
        q = q * query_temperature(positions, qt["coef"], qt["every"])[:, None, None]
    i, j = np.asarray(positions)[:, None], np.asarray(positions)[None, :]
    dist = np.maximum(i - j, 0).astype(np.float64)
    r1, r2 = np.asarray(w[p + ".r1"], dtype=np.float64), np.asarray(w[p + ".r2"], dtype=np.float64)
    o = np.zeros((T, H, dv))
    for hd in range(H):
        g = hd // (H // G)
        s = (q[:, hd] @ k[:, g].T) * float(mix["scale"]) - r1[hd] * np.log1p(r2[hd] * dist)
        s = np.where(j <= i, s, -np.inf)
        o[:, hd] = softmax_rows(s) @ v[:, g]
    return o.reshape(T, H * dv) @ w[p + ".o"].T


# ---------------------------------------------------------------------------------------------- feed-forwards
def dense_ff(h, w, p):
    return (gelu_tanh(h @ w[p + ".gate"].T + w[p + ".gate.b"]) * (h @ w[p + ".up"].T + w[p + ".up.b"])) @ w[p + ".down"].T \
        + w[p + ".down.b"]


def expert_ff(h, w, p):
    return gelu_erf(h @ w[p + ".up"].T) @ w[p + ".down"].T


def route(h, w, p, top):
    """(chosen experts [T, top], their weights [T, top]): the largest logits, softmax over the chosen ones only."""
    z = h @ w[p + ".router"].T
    idx = np.argsort(-z, axis=-1, kind="stable")[:, :top]
    return idx, softmax_rows(np.take_along_axis(z, idx, axis=-1))


def moe_ff(h, w, p, mlp):
    top = int(mlp["router"]["top"])
    idx, wgt = route(h, w, p, top)
    out = np.zeros((h.shape[0], w[p + ".e0.down"].shape[0]))
    for t in range(h.shape[0]):
        for k in range(top):
            out[t] += wgt[t, k] * expert_ff(h[t:t + 1], w, f"{p}.e{idx[t, k]}")[0]
    if mlp.get("shared") is not None:
        out = out + expert_ff(h, w, p + ".shared") * sigmoid(h @ w[p + ".shared.sg"].T)
    return out


# ---------------------------------------------------------------------------------------------- the model
def depth_average(xs, weights):
    """sum_j weights[j] xs[j] over the embedding output and every layer's result so far."""
    return sum(float(a) * x for a, x in zip(weights, xs))


def forward(cfg, w, tokens, collect=None):
    """Logits [T, vocab] of one whole sequence.  `collect`: a list that receives the stream after every layer."""
    w = {k: np.asarray(v, dtype=np.float64) for k, v in w.items()}
    eps, m = float(cfg["norm"]["eps"]), float(cfg.get("residual_mult", 1.0))
    positions = np.arange(len(tokens))
    x = w["embed"][np.asarray(tokens)]
    results = [x]
    for i, layer in enumerate(cfg["layers"]):
        p, mix = f"l{i}", layer["mixer"]
        h = norm_offset(x, w[p + ".norm1"], eps)
        if layer["type"] == "mingru":
            y, _ = mingru_mixer(h, w, p + ".mix")
        elif layer["type"] == "latent_attention":
            y = latent_attention_mixer(h, w, p + ".mix", mix, eps, positions)
        elif layer["type"] == "attention":
            y = biased_attention_mixer(h, w, p + ".mix", mix, positions)
        else:
            raise ValueError(layer["type"])
        x = x + m * y
        mlp = layer.get("mlp")
        if mlp is not None:
            h = norm_offset(x, w[p + ".norm2"], eps)
            x = x + m * (dense_ff(h, w, p + ".mlp") if mlp["kind"] == "dense" else moe_ff(h, w, p + ".mlp", mlp))
        results.append(x)
        x = depth_average(results, w[p + ".dwa"])
        if collect is not None:
            collect.append(x.copy())
    return norm_offset(x, w["final.norm"], eps) @ w["head"].T
