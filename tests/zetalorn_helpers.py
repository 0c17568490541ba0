"""Shared by the Zetalorn tests: small configurations that differ from one another in every size and option, model folders
with seeded weights shaped so that a fault shows, and the plain oracle's logits."""
from __future__ import annotations

import copy
import json
from pathlib import Path

import numpy as np
import torch

import plain_qwen2
import plain_zetalorn as plain


def moe(experts, top, ff, limit=1.5, groups=None):
    r = {"experts": experts, "top": top}
    if groups:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "router": r, "expert": {"ff": ff, "limit": limit}}


def rot(dims, base=10000.0, factor=None):
    r = {"dims": dims, "base": base}
    if factor is not None:
        r["scaling"] = {"factor": factor}
    return r


def attention(heads, kv_heads, dim, vdim, chunk, diff=0.3, rotation=None, mlp=None, scale=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else dim ** -0.5,
         "diff": diff, "mask": {"size": chunk}}
    if rotation:
        m["rot"] = rotation
    return {"type": "attention", "mixer": m, "mlp": mlp}


def parallel(left, right, mlp=None):
    """left = (heads, kv_heads, dim, vdim, window, pool, rotation); right = (heads, dim, vdim, decays)."""
    h, g, d, dv, window, pool, rotation = left
    l = {"heads": h, "kv_heads": g, "dim": d, "vdim": dv, "scale": d ** -0.5, "mask": {"size": window, "pool": pool}}
    if rotation:
        l["rot"] = rotation
    rh, rd, rdv, decay = right
    return {"type": "parallel", "mixer": {"left": l, "right": {"heads": rh, "dim": rd, "vdim": rdv, "decay": list(decay)}}, "mlp": mlp}


def config(vocab, width, layers, loop=None, logit_scale=None, eps=1e-5):
    c = {"architecture": "Zetalorn", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if loop:
        c["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    if logit_scale is not None:
        c["logit_scale"] = logit_scale
    return c


# P: both kinds of layer, a loop of two layers run three times, grouped routing, part of a head rotated in both layouts,
#    keys and values of different widths, a window that is no multiple of the pool, a chunk smaller than a page.
# Q: sizes that are no multiples of 8 (the CUDA-core products); every head a key/value head; a pool of one token and a
#    pool larger than the window; a window of one; no rotation in one layer, whole heads in another; layers without a
#    feed-forward; one expert a token without groups; no loop and no logit scale; a chunk of one page exactly.
# R: one key/value head for six query heads; a chunk larger than every prompt and a window larger than two pages; a loop
#    that covers every layer and runs once; every expert chosen; decays of 0 and 1.
CONFIGS = {
    "P": config(211, 64, [
        parallel((4, 2, 16, 24, 20, 8, rot(8, 5000.0)), (2, 8, 16, (0.6, 0.99)), moe(6, 2, 24, 1.0, groups=(3, 2))),
        attention(4, 2, 16, 24, 40, diff=0.25, rotation=rot(12, 20000.0, 2.0), mlp=moe(8, 3, 16, 1.5, groups=(4, 2))),
        parallel((2, 1, 32, 16, 70, 4, rot(32, 300.0, 4.0)), (3, 16, 8, (0.5, 0.9, 0.999)), moe(4, 2, 40, 0.7)),
        attention(2, 1, 24, 8, 65, diff=0.1, rotation=rot(24, 10000.0)),
    ], loop=(1, 3, 3), logit_scale=0.5),
    "Q": config(150, 44, [
        attention(3, 3, 18, 10, 64, diff=0.4, mlp=moe(4, 1, 20, 2.0)),
        parallel((3, 3, 6, 14, 9, 1, None), (1, 5, 7, (0.8,))),
        parallel((2, 2, 10, 6, 1, 3, rot(10, 1000.0)), (4, 3, 9, (0.3, 0.7, 0.95, 1.0)), moe(5, 2, 12, 0.5)),
        parallel((1, 1, 12, 12, 5, 16, rot(4, 50.0)), (2, 12, 4, (0.9, 0.2))),
    ], eps=1e-6),
    "R": config(97, 48, [
        parallel((6, 1, 16, 16, 150, 8, rot(16, 100000.0, 8.0)), (2, 24, 24, (0.0, 1.0)), moe(3, 3, 32, 1.2)),
        attention(6, 1, 16, 16, 5000, diff=0.5, rotation=rot(2, 7.0), mlp=moe(2, 2, 16, 3.0, groups=(2, 2))),
    ], loop=(0, 2, 1), logit_scale=2.0),
}

GAIN = {torch.float32: 4.0, torch.bfloat16: 2.0}


def variant(cfg: dict, edit) -> dict:
    c = copy.deepcopy(cfg)
    edit(c)
    return c


def for_dtype(cfg: dict, dtype) -> dict:
    """Under bfloat16 every expert is chosen: which experts a token uses must not hang on 16-bit rounding of the stream
    (sparse routing in 16 bits is covered where both sides get the same input)."""
    if dtype != torch.bfloat16:
        return cfg

    def all_experts(c):
        for l in c["layers"]:
            if l["mlp"]:
                r = l["mlp"]["router"]
                r["top"] = r["experts"]
                if r.get("groups"):
                    r["groups"]["keep"] = r["groups"]["count"]
    return variant(cfg, all_experts)


def make_folder(tmp, cfg: dict, seed: int, gain: float, store="bfloat16", edit=None) -> Path:
    """Seeded random weights, then: the weights of the query and key norms scaled by `gain` (scores spread out, so a lost
    or misplaced key shows); the layers' norm numbers, the branch norms and the gate biases spread (a norm left out or a
    gate stuck at 1/2 shows); gate matrices, router matrices and the recurrence's inputs scaled so that sigmoid and silu
    leave their linear range; expert matrices scaled so that the clamps are met; the four vectors behind lambda spread so
    that lambda differs from the configured constant; the passes' offsets scaled to the size of the stream; the head
    scaled so that logits are of size one.  `edit`
    (dict of tensors -> None) changes the result further."""
    from llaisys_b200.weights import SafetensorsFile, write_random_model, write_safetensors
    folder = write_random_model(Path(tmp), cfg, seed, store)
    f = SafetensorsFile(folder / "model.safetensors")
    rng = np.random.default_rng(seed + 1)
    out = {}
    for name in f.entries:
        t = f.get(name).clone()

        def uniform(lo, hi):
            return torch.from_numpy(np.asarray(rng.uniform(lo, hi, size=tuple(t.shape)))).to(t.dtype)

        def scaled(c):
            return (t.float() * c).to(t.dtype)

        leaf = name.rsplit(".", 1)[-1]
        if name.endswith(("q.norm", "k.norm")):
            t = (uniform(0.6, 1.4).float() * gain ** 0.5).to(t.dtype)
        elif leaf in ("norm1", "norm2") or name == "final.norm" or name.endswith((".left.out", ".right.out", ".right.norm")):
            t = uniform(0.5, 1.5)
        elif leaf in ("lq1", "lk1", "lq2", "lk2"):
            t = uniform(-0.4, 0.4)
        elif leaf in ("rg1", "rg2"):
            t = scaled(25.0)
        elif name.endswith((".rg1.b", ".rg2.b")):
            t = uniform(-1.5, 1.5)
        elif ".mix.right." in name and leaf in ("q", "k", "v", "g"):
            t = scaled(12.0)
        elif name.endswith(".router"):
            t = scaled(25.0)
        elif ".mlp." in name:
            t = scaled(8.0)
        elif name == "loop.step":
            t = scaled(1.5)
        elif name == "head":
            t = scaled(5.0)
        elif leaf in ("v", "o"):
            t = scaled(3.0)
        out[name] = t
    if edit:
        edit(out)
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
            self._memo[key] = plain.forward(self.config, self.weights, list(tokens))[0]
        return self._memo[key]


def like_config(cfg: dict) -> dict:
    """What helpers.tolerance reads.  Its bfloat16 bound counts six roundings to 16 bits a layer; a layer run of this
    design has about twice as many (normed input, projections, normed and rotated heads, cached rows, gated heads; normed
    input, gate and up rows, expert activations), so a run counts twice; looped layers count once per pass."""
    return {"num_hidden_layers": 2 * len(plain.run_order(cfg))}


def random_requests(cfg: dict, lengths, seed: int):
    rng = np.random.default_rng(seed)
    return [rng.integers(0, cfg["vocab"], size=n).tolist() for n in lengths]


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
