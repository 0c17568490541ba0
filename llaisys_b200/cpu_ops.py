"""The operators on the CPU: plain float32 numpy, one function per operator, written from the
formulas of xsmccc/llaisys' CPU operators (src/ops/*/cpu/*.cpp: inputs of any supported dtype are
computed in float32 and rounded once at the output, README.md:156).

This is the reference beside each CUDA operator, as that project keeps one (src/ops/linear/op.cpp:48-58
dispatches on the device): `llaisys_b200.ops.Ops` runs these when its operands live on the CPU, the
op tests compare the CUDA kernels with them, and the command line's --test and --device cpu
generate with a model put together from them.  It is not a fallback of the engine: the engine
runs on a CUDA device only.
"""
from __future__ import annotations

import numpy as np


def add(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """c = a + b (src/ops/add/cpu/add_cpu.cpp:8-16)."""
    return a.astype(np.float32) + b.astype(np.float32)


def argmax(vals: np.ndarray):
    """(index of the first maximum, the maximum): strict > scan from index 0
    (src/ops/argmax/cpu/argmax_cpu.cpp:14-27)."""
    v = vals.astype(np.float32).reshape(-1)
    i = int(np.argmax(v))
    return i, v[i]


def embedding(index: np.ndarray, weight: np.ndarray) -> np.ndarray:
    """out[t] = weight[index[t]] (src/ops/embedding/cpu/embedding_cpu.cpp:16-22)."""
    idx = np.asarray(index, dtype=np.int64)
    if idx.size and (idx.min() < 0 or idx.max() >= weight.shape[0]):
        raise IndexError(f"embedding: index outside the table of {weight.shape[0]} rows")
    return weight[idx]


def linear(x: np.ndarray, weight: np.ndarray, bias=None) -> np.ndarray:
    """y = x W^T + b with W [out, in], float32 accumulation (src/ops/linear/cpu/linear_cpu.cpp:21-40)."""
    y = x.astype(np.float32) @ weight.astype(np.float32).T
    if bias is not None:
        y = y + bias.astype(np.float32)
    return y


def rms_norm(x: np.ndarray, weight: np.ndarray, eps: float) -> np.ndarray:
    """y = (x * w) / sqrt(mean(x^2) + eps), eps inside the root (src/ops/rms_norm/cpu/rms_norm_cpu.cpp:15-34)."""
    x = x.astype(np.float32)
    ss = (x * x).sum(axis=-1, keepdims=True, dtype=np.float32)
    inv = np.float32(1.0) / np.sqrt(ss / np.float32(x.shape[-1]) + np.float32(eps))
    return (x * weight.astype(np.float32)) * inv


def rope(x: np.ndarray, pos_ids: np.ndarray, theta: float) -> np.ndarray:
    """Half-split rotation of x [seq, heads, d]: phi = p / theta^(2j/d) in double precision from theta
    held as a C float; (a, b) = (x[j], x[j + d/2]) -> (a cos - b sin, b cos + a sin)
    (src/ops/rope/cpu/rope_cpu.cpp:16-46)."""
    d = x.shape[-1]
    half = d // 2
    t = float(np.float32(theta))
    freq = 1.0 / np.power(t, 2.0 * np.arange(half, dtype=np.float64) / d)
    ang = np.asarray(pos_ids, dtype=np.float64)[:, None] * freq[None, :]
    cos, sin = np.cos(ang)[:, None, :].astype(np.float32), np.sin(ang)[:, None, :].astype(np.float32)
    x = x.astype(np.float32)
    a, b = x[..., :half], x[..., half:]
    return np.concatenate([a * cos - b * sin, b * cos + a * sin], axis=-1)


def rope_leading(x: np.ndarray, pos_ids: np.ndarray, dims: int, base: float) -> np.ndarray:
    """Rotation of the first `dims` dimensions of x [seq, heads, d] in pairs (i, i + dims/2) by the angle
    p * base^(-2i/dims); the other dimensions pass (not in xsmccc/llaisys)."""
    x = x.astype(np.float32)
    half = dims // 2
    if half == 0:
        return x
    freq = np.power(float(base), -2.0 * np.arange(half, dtype=np.float64) / dims)
    ang = np.asarray(pos_ids, dtype=np.float64)[:, None] * freq[None, :]
    cos, sin = np.cos(ang)[:, None, :].astype(np.float32), np.sin(ang)[:, None, :].astype(np.float32)
    a, b = x[..., :half], x[..., half:dims]
    return np.concatenate([a * cos - b * sin, b * cos + a * sin, x[..., dims:]], axis=-1)


def relu_squared(x: np.ndarray) -> np.ndarray:
    """max(x, 0)^2 (not in xsmccc/llaisys)."""
    r = np.maximum(x.astype(np.float32), np.float32(0))
    return r * r


def route_top(logits: np.ndarray, bias, top: int, scale: float):
    """(experts [T, top], weights [T, top]) of a router: gates 1 / (1 + e^-z); the `top` largest of gate + bias, the
    first maximum first; weights gate * scale, not renormalised (not in xsmccc/llaisys)."""
    gate = np.float32(1.0) / (np.float32(1.0) + np.exp(-logits.astype(np.float32)))
    choice = gate + (bias.astype(np.float32) if bias is not None else np.float32(0))
    idx = np.argsort(-choice, axis=-1, kind="stable")[:, :top]
    return idx, np.take_along_axis(gate, idx, axis=-1) * np.float32(scale)


def self_attention(q: np.ndarray, k: np.ndarray, v: np.ndarray, scale: float, window=None, keep_first: int = 0,
                   sink: bool = False, sink_logits=None, dist_bias=None) -> np.ndarray:
    """Causal grouped-query attention of q [qlen, nh, d] over k [kvlen, nkvh, d], v [kvlen, nkvh, dv], the queries being
    the last qlen of the kvlen positions: query i sees keys t <= kvlen - qlen + i; head h reads kv head
    h // (nh / nkvh); softmax with the maximum subtracted (src/ops/self_attention/cpu/self_attention_cpu.cpp:28-112).
    Not in that project: window (a query at position p sees only the keys p - window < t <= p), keep_first (the keys
    t < keep_first stay visible behind the window), sink (one more term e^0 in the denominator, without a value) and
    sink_logits [nh] (that term is e^sink_logits[h] instead), dist_bias = (r1 [nh], r2 [nh]) (the score of query position
    p and key position t loses r1[h] ln(1 + r2[h] (p - t)))."""
    qlen, nh, d = q.shape
    kvlen, nkvh, dv = v.shape
    group = nh // nkvh
    q, k, v = q.astype(np.float32), k.astype(np.float32), v.astype(np.float32)
    out = np.zeros((qlen, nh, dv), dtype=np.float32)
    t = np.arange(kvlen)
    cur = (kvlen - qlen + np.arange(qlen))[:, None]
    visible = t[None, :] <= cur
    if window is not None:
        visible &= (t[None, :] > cur - window) | (t[None, :] < keep_first)
    for h in range(nh):
        s = (q[:, h, :] @ k[:, h // group, :].T) * np.float32(scale)
        if dist_bias is not None:
            dist = np.maximum(cur - t[None, :], 0).astype(np.float32)
            s = s - np.float32(dist_bias[0][h]) * np.log1p(np.float32(dist_bias[1][h]) * dist)
        s = np.where(visible, s, -np.inf)
        m = s.max(axis=-1, keepdims=True)
        s0 = np.float32(sink_logits[h]) if sink_logits is not None else np.float32(0)
        if sink or sink_logits is not None:
            m = np.maximum(m, s0)
        e = np.where(visible, np.exp(s - m), 0.0).astype(np.float32)
        den = e.sum(axis=-1, keepdims=True) + (np.exp(s0 - m).astype(np.float32) if (sink or sink_logits is not None) else np.float32(0))
        out[:, h, :] = (e / den) @ v[:, h // group, :]
    return out


def swiglu(gate: np.ndarray, up: np.ndarray) -> np.ndarray:
    """out = up * gate / (1 + exp(-gate)) (src/ops/swiglu/cpu/swiglu_cpu.cpp:13-21)."""
    g, u = gate.astype(np.float32), up.astype(np.float32)
    return u * (g / (np.float32(1.0) + np.exp(-g)))


def rope_pairs(x: np.ndarray, pos_ids: np.ndarray, dims: int, base: float, yarn=None) -> np.ndarray:
    """Rotation of the neighbouring pairs (2i, 2i+1), i < dims/2, of the last axis of x [seq, heads, d] by the angle
    p * f_i; the other dimensions pass.  f_i = base^(-2i/dims), or with yarn = {factor, original, fast, slow} the
    rescaled frequencies and magnitude of parts/rope.py: yarn_frequencies (not in xsmccc/llaisys)."""
    import math
    x = x.astype(np.float32).copy()
    half = dims // 2
    if half == 0:
        return x
    i = np.arange(half, dtype=np.float64)
    f = np.power(float(base), -2.0 * i / dims)
    mag = 1.0
    if yarn:
        def turn_dim(turns):
            return dims * math.log(float(yarn["original"]) / (2.0 * math.pi * turns)) / (2.0 * math.log(float(base)))
        lo, hi = max(math.floor(turn_dim(float(yarn["fast"]))), 0), min(math.ceil(turn_dim(float(yarn["slow"]))), dims - 1)
        ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
        f = f / float(yarn["factor"]) * ramp + f * (1.0 - ramp)
        mag = 0.1 * math.log(float(yarn["factor"])) + 1.0
    ang = np.asarray(pos_ids, dtype=np.float64)[:, None] * f[None, :]
    cos, sin = (np.cos(ang) * mag)[:, None, :].astype(np.float32), (np.sin(ang) * mag)[:, None, :].astype(np.float32)
    u, v = x[..., 0:dims:2].copy(), x[..., 1:dims:2].copy()
    x[..., 0:dims:2] = u * cos - v * sin
    x[..., 1:dims:2] = v * cos + u * sin
    return x


def glu(gate: np.ndarray, up: np.ndarray, act: str) -> np.ndarray:
    """act(gate) * up with act "silu", "relu" or "gelu_tanh" (not in xsmccc/llaisys beyond swiglu)."""
    g, u = gate.astype(np.float32), up.astype(np.float32)
    if act == "relu":
        a = np.maximum(g, np.float32(0))
    elif act == "gelu_tanh":
        a = np.float32(0.5) * g * (np.float32(1) + np.tanh(np.float32(0.7978845608028654) * (g + np.float32(0.044715) * g * g * g)))
    else:
        a = g / (np.float32(1.0) + np.exp(-g))
    return a * u


def gated_linear_recurrence(q: np.ndarray, k: np.ndarray, v: np.ndarray, z: np.ndarray, state: np.ndarray, root: float):
    """o_t = S_t^T q_t with S_t = diag(sigmoid(z_t)^(1/root)) S_(t-1) + k_t v_t^T per head, float32: q, k, z
    [seq, heads, dk], v [seq, heads, dv], state [heads, dk, dv] (updated in place).  Returns o [seq, heads, dv]
    (not in xsmccc/llaisys)."""
    q, k, v = q.astype(np.float32), k.astype(np.float32), v.astype(np.float32)
    z = z.astype(np.float32)
    a = np.exp(-(np.maximum(-z, 0) + np.log1p(np.exp(-np.abs(z)))) / np.float32(root)).astype(np.float32)
    out = np.zeros(v.shape, dtype=np.float32)
    for t in range(q.shape[0]):
        state *= a[t][:, :, None]
        state += k[t][:, :, None] * v[t][:, None, :]
        out[t] = np.einsum("hkv,hk->hv", state, q[t])
    return out


def query_temperature(pos_ids: np.ndarray, coef: float, every: int) -> np.ndarray:
    """1 + coef ln(floor((p + 1) / every) + 1) per position (not in xsmccc/llaisys)."""
    p = np.asarray(pos_ids, dtype=np.int64)
    return (1.0 + float(coef) * np.log(((p + 1) // int(every)) + 1.0)).astype(np.float32)


def min_gru(a: np.ndarray, u: np.ndarray, state: np.ndarray) -> np.ndarray:
    """S_t = (1 - z_t) S_(t-1) + z_t c_t per channel, z = sigmoid(a), c = u + 1/2 where u >= 0 and sigmoid(u) below;
    a, u [seq, width], state [width] (updated in place).  Returns S [seq, width] (not in xsmccc/llaisys)."""
    a, u = a.astype(np.float32), u.astype(np.float32)
    z = np.float32(1) / (np.float32(1) + np.exp(-a))
    c = np.where(u >= 0, u + np.float32(0.5), np.float32(1) / (np.float32(1) + np.exp(-np.minimum(u, np.float32(0)))))
    out = np.zeros(a.shape, dtype=np.float32)
    for t in range(a.shape[0]):
        state += z[t] * (c[t] - state)
        out[t] = state
    return out


def gelu(x: np.ndarray) -> np.ndarray:
    """x Phi(x) with the error function (not in xsmccc/llaisys)."""
    import math
    x = x.astype(np.float32)
    return (np.float32(0.5) * x * (np.float32(1) + np.vectorize(math.erf, otypes=[np.float64])(x / math.sqrt(2.0)))).astype(np.float32)


def sigmoid(x: np.ndarray) -> np.ndarray:
    return np.float32(1) / (np.float32(1) + np.exp(-x.astype(np.float32)))


def route_top_softmax(logits: np.ndarray, bias, top: int, scale: float):
    """(experts [T, top], weights [T, top]): the `top` largest of logits + bias, the first maximum first; weights the
    softmax over the chosen logits alone, times scale (not in xsmccc/llaisys)."""
    z = logits.astype(np.float32)
    choice = z + (bias.astype(np.float32) if bias is not None else np.float32(0))
    idx = np.argsort(-choice, axis=-1, kind="stable")[:, :top]
    zc = np.take_along_axis(z, idx, axis=-1)
    e = np.exp(zc - zc.max(axis=-1, keepdims=True))
    return idx, (e / e.sum(axis=-1, keepdims=True)) * np.float32(scale)


def rotate_pairs(x: np.ndarray, pos_ids: np.ndarray, dims: int, base: float, factor: float = 1.0, neighbours: bool = False) -> np.ndarray:
    """Rotation of the first `dims` elements of the last axis of x [seq, rows, d] by the angles p * base^(-2i/dims) / factor,
    pairing element i with i + dims/2, or (neighbours) 2i with 2i + 1; angles in float64, the rest float32 (not in
    xsmccc/llaisys)."""
    x = x.astype(np.float32).copy()
    half = dims // 2
    if half == 0:
        return x
    f = np.power(float(base), -2.0 * np.arange(half, dtype=np.float64) / dims) / float(factor)
    ang = np.asarray(pos_ids, dtype=np.float64)[:, None] * f[None, :]
    cos, sin = np.cos(ang)[:, None, :].astype(np.float32), np.sin(ang)[:, None, :].astype(np.float32)
    a, b = (slice(0, dims, 2), slice(1, dims, 2)) if neighbours else (slice(0, half), slice(half, dims))
    u, v = x[..., a].copy(), x[..., b].copy()
    x[..., a] = u * cos - v * sin
    x[..., b] = v * cos + u * sin
    return x


def masked_attention(q: np.ndarray, k: np.ndarray, v: np.ndarray, scale: float, visible: np.ndarray) -> np.ndarray:
    """Softmax attention of q [qlen, nh, d] over k [n, nkvh, d], v [n, nkvh, dv] with a mask visible [qlen, n] given by the
    caller (windows, chunks, blocks of keys); head h reads kv head h // (nh / nkvh) (not in xsmccc/llaisys)."""
    qlen, nh, _ = q.shape
    nkvh, dv = v.shape[1], v.shape[2]
    group = nh // nkvh
    q, k, v = q.astype(np.float32), k.astype(np.float32), v.astype(np.float32)
    out = np.zeros((qlen, nh, dv), dtype=np.float32)
    for h in range(nh):
        s = np.where(visible, (q[:, h, :] @ k[:, h // group, :].T) * np.float32(scale), -np.inf)
        e = np.where(visible, np.exp(s - s.max(axis=-1, keepdims=True)), 0.0).astype(np.float32)
        out[:, h, :] = (e / e.sum(axis=-1, keepdims=True)) @ v[:, h // group, :]
    return out


def route_grouped(logits: np.ndarray, top: int, groups=None, renorm: bool = False, scale: float = 1.0):
    """(experts [T, top], weights [T, top]): gates 1 / (1 + e^-z); with groups = (count, keep) the experts form `count` equal
    groups of neighbours, a group's score is the sum of its two largest gates, and only experts of the `keep` best groups
    (first maximum first) can be chosen; the `top` largest gates among them; weights gate * scale, with renorm divided by
    the chosen gates' sum + 1e-20 (not in xsmccc/llaisys)."""
    gate = np.float32(1.0) / (np.float32(1.0) + np.exp(-logits.astype(np.float32)))
    T, E = gate.shape
    choice = gate.copy()
    if groups and groups[0] > 1:
        count, keep = groups
        by = gate.reshape(T, count, E // count)
        score = np.sort(by, axis=-1)[..., ::-1][..., :2].sum(axis=-1)
        kept = np.argsort(-score, axis=-1, kind="stable")[:, :keep]
        allowed = np.zeros((T, count), dtype=bool)
        np.put_along_axis(allowed, kept, True, axis=1)
        choice = np.where(np.repeat(allowed, E // count, axis=1), choice, -np.inf)
    idx = np.argsort(-choice, axis=-1, kind="stable")[:, :top]
    w = np.take_along_axis(gate, idx, axis=-1)
    if renorm:
        w = w / (w.sum(axis=-1, keepdims=True) + np.float32(1e-20))
    return idx, w * np.float32(scale)


def swish_clamped(gate: np.ndarray, up: np.ndarray, limit: float, alpha: float) -> np.ndarray:
    """g = min(gate, limit), u = clamp(up, -limit, limit): g sigmoid(alpha g) (u + 1) (not in xsmccc/llaisys)."""
    g = np.minimum(gate.astype(np.float32), np.float32(limit))
    u = np.clip(up.astype(np.float32), np.float32(-limit), np.float32(limit))
    return g * sigmoid(np.float32(alpha) * g) * (u + np.float32(1))


def decayed_linear_recurrence(q: np.ndarray, k: np.ndarray, v: np.ndarray, decay: np.ndarray, state: np.ndarray) -> np.ndarray:
    """Per head S <- decay_h S + k_t v_t^T, o_t = S^T q_t over q, k [T, H, dk], v [T, H, dv]; `state` [H, dk, dv] is
    updated in place (not in xsmccc/llaisys)."""
    T = q.shape[0]
    out = np.zeros((T,) + v.shape[1:], dtype=np.float32)
    a = decay.astype(np.float32)[:, None, None]
    for t in range(T):
        state *= a
        state += k[t][:, :, None].astype(np.float32) * v[t][:, None, :].astype(np.float32)
        out[t] = np.einsum("hkv,hk->hv", state, q[t].astype(np.float32))
    return out
