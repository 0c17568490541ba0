"""Shared by the Zedirax tests: small configurations that differ from one another in every size and option, model folders
with seeded weights shaped so that a fault shows, and the plain oracle's logits."""
from __future__ import annotations

import copy
import json
from pathlib import Path

import numpy as np
import torch

import plain_qwen2
import plain_zedirax as plain


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, shared_ff=None):
    d = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}
    if shared_ff:
        d["shared"] = {"ff": shared_ff}
    return d


def mingru(width, mlp=None):
    return {"type": "mingru", "mixer": {"width": width}, "mlp": mlp}


def latent(heads, dim, rot_dim, vdim, kv_rank, mlp=None, base=10000.0, scale=None):
    return {"type": "latent_attention", "mlp": mlp,
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
                      "scale": scale if scale is not None else (dim + rot_dim) ** -0.5, "rot": {"dims": rot_dim, "base": base}}}


def attention(heads, kv_heads, dim, vdim, q_temp=None, mlp=None, scale=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else dim ** -0.5}
    if q_temp:
        m["q_temp"] = {"coef": q_temp[0], "every": q_temp[1]}
    return {"type": "attention", "mixer": m, "mlp": mlp}


def config(vocab, width, layers, mult=None, eps=1e-5):
    c = {"architecture": "Zedirax", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if mult is not None:
        c["residual_mult"] = mult
    return c


# P: every kind of mixer and of feed-forward; the query temperature steps every 16 positions; keys and values of
#    different widths in both attentions; a recurrence narrower than the stream.
# Q: sizes that are no multiples of 8 (the CUDA-core products); attention first and a recurrence last; every head a
#    key/value head; one expert a token without a shared expert; no temperature; a temperature that steps at every
#    position; layers without a feed-forward; no residual constant in the configuration (it is 1).
# R: cache rows wider than 256 elements; a recurrence of 130 channels (two blocks of channels); one key/value head for
#    six query heads; every expert chosen; unrotated query/key part larger and smaller than the rotated one.
CONFIGS = {
    "P": config(211, 64, [
        mingru(40, dense(96)),
        latent(3, 16, 8, 24, 40, moe(6, 2, 40, 24), base=5000.0),
        attention(4, 2, 16, 24, q_temp=(0.4, 16), mlp=dense(80)),
        mingru(72, moe(5, 3, 24, 48)),
        attention(2, 1, 32, 16, q_temp=(1.5, 50), mlp=moe(4, 2, 16)),
        latent(2, 8, 16, 12, 24, dense(56), scale=0.3),
    ], mult=0.6),
    "Q": config(150, 44, [
        attention(3, 3, 18, 10, mlp=moe(4, 1, 20)),
        latent(5, 4, 2, 3, 7),
        mingru(33, dense(36)),
        attention(2, 2, 6, 14, q_temp=(0.25, 1)),
        mingru(44),
    ], eps=1e-6),
    "R": config(97, 48, [
        latent(2, 24, 8, 8, 264, moe(3, 3, 32, 16), base=300.0),
        mingru(130, dense(64)),
        attention(6, 1, 16, 16, q_temp=(0.7, 64), mlp=moe(2, 2, 16)),
        latent(6, 4, 12, 16, 20, dense(40)),
    ], mult=1.4),
}
DENSE_ROUTING = {"R"}          # every expert chosen: the choice cannot depend on rounding

GAIN = {torch.float32: 9.0, torch.bfloat16: 3.0}


def for_dtype(cfg: dict, dtype) -> dict:
    """Under bfloat16 every expert is chosen: which experts a token uses must not hang on 16-bit rounding of the stream
    (sparse routing in 16 bits is covered where both sides get the same input)."""
    if dtype != torch.bfloat16:
        return cfg

    def all_experts(c):
        for l in c["layers"]:
            if l["mlp"] and l["mlp"]["kind"] == "moe":
                l["mlp"]["router"]["top"] = l["mlp"]["router"]["experts"]
    return variant(cfg, all_experts)


def make_folder(tmp, cfg: dict, seed: int, gain: float, store="bfloat16") -> Path:
    """Seeded random weights, then: the matrices that make queries and keys scaled by `gain` (scores spread out, so a lost
    or misplaced key shows); the distance penalty's two numbers per head spread over positive ranges that differ between
    heads; the recurrence's gate biases spread so that channels forget at different speeds, its candidate inputs scaled so
    that both branches of the candidate occur; output gates scaled away from 1/2; router matrices scaled so that logits
    differ; the norms' stored weights spread over +-0.5 (an offset left out or applied twice shows); the depth weights
    spread, some negative, so that no earlier result drops out unnoticed."""
    from llaisys_b200.weights import SafetensorsFile, write_random_model, write_safetensors
    folder = write_random_model(Path(tmp), cfg, seed, store)
    f = SafetensorsFile(folder / "model.safetensors")
    rng = np.random.default_rng(seed + 1)
    out = {}
    for name in f.entries:
        t = f.get(name).clone()
        kind = cfg["layers"][int(name[1:name.index(".")])]["type"] if name[0] == "l" and name[1].isdigit() else None
        leaf = name.split(".mix.")[-1] if ".mix." in name else name.rsplit(".", 1)[-1]

        def uniform(lo, hi):
            return torch.from_numpy(rng.uniform(lo, hi, size=tuple(t.shape))).to(t.dtype)

        if ".mix." in name and kind == "attention" and leaf in ("q", "k"):
            t = (t.float() * gain).to(t.dtype)
        elif ".mix." in name and kind == "attention" and leaf == "r1":
            t = uniform(0.2, 1.5)
        elif ".mix." in name and kind == "attention" and leaf == "r2":
            t = uniform(0.05, 2.0)
        elif ".mix." in name and kind == "latent_attention" and leaf in ("q", "uk"):
            t = (t.float() * gain).to(t.dtype)
        elif ".mix." in name and kind == "latent_attention" and leaf == "dkv":
            rot = cfg["layers"][int(name[1:name.index(".")])]["mixer"]["rot_dim"]
            u = t.float()
            u[-rot:] *= gain * 2.0
            t = u.to(t.dtype)
        elif ".mix." in name and kind == "latent_attention" and leaf == "g":
            t = (t.float() * 10.0).to(t.dtype)
        elif ".mix." in name and kind == "mingru" and leaf == "z.b":
            t = uniform(-5.0, 2.0)
        elif ".mix." in name and kind == "mingru" and leaf in ("z", "x", "g"):
            t = (t.float() * 6.0).to(t.dtype)
        elif name.endswith(".router"):
            t = (t.float() * 25.0).to(t.dtype)
        elif name.endswith(".shared.sg"):
            t = (t.float() * 10.0).to(t.dtype)
        elif ".mlp." in name and not name.endswith(".b"):
            t = (t.float() * 4.0).to(t.dtype)
        elif name.endswith(".b") and ".mlp." in name:
            t = uniform(-0.5, 0.5)
        elif leaf.startswith("norm") and ".mix." not in name:
            t = uniform(-0.5, 0.5)
        elif name.endswith(".dwa"):
            n = t.numel()
            a = rng.uniform(-0.4, 1.0, size=n)
            a[-1] = rng.uniform(0.6, 1.0)
            t = torch.from_numpy(a / max(1.0, np.abs(a).sum() / 1.5)).to(t.dtype)
        out[name] = t
    write_safetensors(folder / "model.safetensors", out)
    return folder


class Oracle:
    """Plain logits of whole requests, computed once per request."""

    def __init__(self, folder):
        self.config = json.loads((Path(folder) / "config.json").read_text())
        self.weights = plain_qwen2.read_safetensors(Path(folder) / "model.safetensors")
        self._memo = {}

    def logits(self, tokens) -> np.ndarray:
        key = tuple(tokens)
        if key not in self._memo:
            self._memo[key] = plain.forward(self.config, self.weights, list(tokens))
        return self._memo[key]


def like_config(cfg: dict) -> dict:
    """What helpers.tolerance reads.  Its bfloat16 bound counts six roundings to 16 bits a layer; a layer of this design
    has about twice as many (normed input, projections, queries in the latent space, cached rows, weights' product, gated
    heads; normed input, two halves and their product, or expert activations), so a layer counts twice."""
    return {"num_hidden_layers": 2 * len(cfg["layers"])}


def random_requests(cfg: dict, lengths, seed: int):
    rng = np.random.default_rng(seed)
    return [rng.integers(0, cfg["vocab"], size=n).tolist() for n in lengths]


def variant(cfg: dict, edit) -> dict:
    c = copy.deepcopy(cfg)
    edit(c)
    return c


def compare(got, oracle, requests, dtype, cfg, what=""):
    """float32: every logits row within the absolute bound of helpers.tolerance.  bfloat16: no row beyond four bounds and
    at most one row in ten beyond one (a fault, a lost key or a stale state, moves whole ranges of positions by far more)."""
    import helpers
    like = like_config(cfg)
    if dtype == torch.float32:
        return helpers.compare(got, oracle, requests, dtype, like, what)
    ratios = []
    for r, toks in enumerate(requests):
        ref = oracle.logits(toks)
        tol = helpers.tolerance(dtype, like, ref)
        for p in range(len(toks)):
            assert (r, p) in got, f"{what}: no logits for request {r} position {p}"
            err = float(np.abs(got[(r, p)].astype(np.float64) - ref[p]).max())
            assert np.isfinite(err), f"{what}: non-finite logits at request {r} position {p}"
            ratios.append((err / tol, r, p))
    worst = max(ratios)
    over = sum(1 for x in ratios if x[0] > 1.0)
    assert worst[0] <= 4.0, f"{what}: request {worst[1]} position {worst[2]} is {worst[0]:.1f} bounds off"
    assert over <= max(1, len(ratios) // 10), f"{what}: {over} of {len(ratios)} rows are beyond the bound (worst {worst[0]:.1f} at {worst[1:]})"
    return worst[0], worst[1:]
