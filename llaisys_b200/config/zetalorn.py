"""Typed configuration of the Zetalorn decoder, read from its own config.json keys.

    architecture    "Zetalorn"
    vocab, width    vocabulary and stream width
    norm            {eps}
    logit_scale     what the logits are multiplied by (1 when absent)
    loop            {start, stop, times}: the layers start .. stop - 1 run `times` times in a row (absent: once)
    layers          list of {type: "attention" | "parallel", mixer: {...}, mlp: {...} or null}
      attention mixer   heads, kv_heads, dim (query/key size of one score map), vdim, scale, diff, mask: {size} (chunks),
                        rot: {dims, base, scaling: {factor}} (rotation of neighbouring pairs; scaling optional)
      parallel mixer    left: heads, kv_heads, dim, vdim, scale, mask: {size, pool} (window and pooled blocks; without
                              `pool` what has left the window is not seen),
                              rot: {dims, base, scaling} (rotation of halves)
                        right: heads, dim, vdim, decay (one number per head, or one for all)
                        (vdim absent: as wide as dim)
      mlp               {kind: "moe", router: {experts, top, groups: {count, keep}}, expert: {ff, limit}}   (groups and limit optional)

Tensor names: embed, loop.step, l<i>.norm1, l<i>.norm2 (one number each), l<i>.rg1, l<i>.rg1.b, l<i>.rg2, l<i>.rg2.b,
l<i>.mix.*, l<i>.mlp.*, final.norm, head.

A layer is `gated_residual`: x += sigmoid(Wg h + bg) * part(h), h = norm(x), for the mixer and then for the feed-forward;
every norm is an RMS norm with a single number as its weight.  Each pass over the looped layers is an entry of the run
order with a cache of its own; the entry that opens a pass adds the pass's offset (and, from the second pass on, the
embedding's output) to the stream.  The configuration names no longest sequence; MAX_POSITIONS is this library's bound.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .registry import register_architecture
from .spec import CallSpec, ConfigError, LayerSpec, ModelSpec, PartSpec, SubLayerSpec
from .vumezen import _dict, _float, _int

MAX_POSITIONS = 1 << 18
SWISH_ALPHA = 1.702           # the experts' activation is g * sigmoid(1.702 g): the design fixes the constant


@dataclass(frozen=True)
class ZetalornRotation:
    dims: int
    base: float
    factor: float


@dataclass(frozen=True)
class ZetalornAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    diff: float
    chunk: Optional[int]
    rot: Optional[ZetalornRotation]


@dataclass(frozen=True)
class ZetalornWindowed:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int
    pool: int
    rot: Optional[ZetalornRotation]


@dataclass(frozen=True)
class ZetalornLinear:
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]


@dataclass(frozen=True)
class ZetalornParallel:
    left: ZetalornWindowed
    right: ZetalornLinear


@dataclass(frozen=True)
class ZetalornMoE:
    experts: int
    top: int
    groups: Optional[Tuple[int, int]]
    ff: int
    limit: float


def _rotation(m: dict, where: str, dim: int) -> Optional[ZetalornRotation]:
    if m.get("rot") is None:
        return None
    rot = _dict(m, "rot", where)
    dims = _int(rot, "dims", f"{where}.rot", 0)
    if dims == 0:
        return None
    if dims % 2 or dims > dim:
        raise ConfigError(f"{where}: rot.dims={dims} must be even and at most dim={dim}")
    factor = 1.0
    if rot.get("scaling") is not None:
        factor = _float(_dict(rot, "scaling", f"{where}.rot"), "factor", f"{where}.rot.scaling")
    return ZetalornRotation(dims=dims, base=_float(rot, "base", f"{where}.rot"), factor=factor)


def _heads(m: dict, where: str):
    heads, kv_heads = _int(m, "heads", where), _int(m, "kv_heads", where)
    if heads % kv_heads:
        raise ConfigError(f"{where}: {heads} query heads cannot share {kv_heads} key/value heads")
    dim = _int(m, "dim", where)
    return heads, kv_heads, dim, (_int(m, "vdim", where) if m.get("vdim") is not None else dim), _float(m, "scale", where, positive=False)


def _mixer(kind, m: dict, where: str):
    if kind == "attention":
        heads, kv_heads, dim, vdim, scale = _heads(m, where)
        chunk = _int(_dict(m, "mask", where), "size", f"{where}.mask") if m.get("mask") is not None else None
        return ZetalornAttention(heads, kv_heads, dim, vdim, scale, diff=_float(m, "diff", where, positive=False), chunk=chunk,
                                 rot=_rotation(m, where, dim))
    if kind == "parallel":
        l, r = _dict(m, "left", where), _dict(m, "right", where)
        heads, kv_heads, dim, vdim, scale = _heads(l, f"{where}.left")
        mask = _dict(l, "mask", f"{where}.left")
        left = ZetalornWindowed(heads, kv_heads, dim, vdim, scale, window=_int(mask, "size", f"{where}.left.mask"),
                                pool=_int(mask, "pool", f"{where}.left.mask") if mask.get("pool") is not None else 0,
                                rot=_rotation(l, f"{where}.left", dim))
        rh = _int(r, "heads", f"{where}.right")
        decay = r.get("decay")
        if isinstance(decay, (int, float)) and not isinstance(decay, bool):
            decay = [decay] * rh                                   # one number for all heads
        if not isinstance(decay, list) or len(decay) != rh or any(isinstance(d, bool) or not isinstance(d, (int, float)) or not (0 <= d <= 1)
                                                                  for d in decay):
            raise ConfigError(f"{where}.right: 'decay' must list one number in [0, 1] for each of the {rh} heads, got {decay!r}")
        rd = _int(r, "dim", f"{where}.right")
        right = ZetalornLinear(rh, rd, _int(r, "vdim", f"{where}.right") if r.get("vdim") is not None else rd, tuple(float(d) for d in decay))
        return ZetalornParallel(left, right)
    raise ConfigError(f"{where}: the mixers of this architecture are 'attention' and 'parallel', got {kind!r}")


def _mlp(mlp, where: str):
    if mlp is None:
        return None
    if not isinstance(mlp, dict):
        raise ConfigError(f"{where} must be an object or null")
    if mlp.get("kind") != "moe":
        raise ConfigError(f"{where}: the feed-forward of this architecture is kind 'moe', got {mlp.get('kind')!r}")
    router, ex = _dict(mlp, "router", where), _dict(mlp, "expert", where)
    experts, top = _int(router, "experts", f"{where}.router"), _int(router, "top", f"{where}.router")
    if top > experts:
        raise ConfigError(f"{where}: a token cannot use {top} of {experts} experts")
    groups = None
    if router.get("groups") is not None:
        g = _dict(router, "groups", f"{where}.router")
        count, keep = _int(g, "count", f"{where}.router.groups"), _int(g, "keep", f"{where}.router.groups")
        if experts % count or keep > count or keep * (experts // count) < top:
            raise ConfigError(f"{where}: {experts} experts in {count} groups of which {keep} are kept cannot give {top} choices")
        groups = (count, keep)
    limit = _float(ex, "limit", f"{where}.expert") if ex.get("limit") is not None else float("inf")     # no limit: nothing is clamped
    return ZetalornMoE(experts, top, groups, ff=_int(ex, "ff", f"{where}.expert"), limit=limit)


@register_architecture("Zetalorn")
@dataclass(frozen=True)
class ZetalornConfig:
    vocab: int
    width: int
    eps: float
    logit_scale: float
    loop: Optional[Tuple[int, int, int]]      # (start, stop, times)
    mixers: Tuple[Any, ...]                   # ZetalornAttention or ZetalornParallel per layer
    ffs: Tuple[Any, ...]                      # ZetalornMoE or None per layer
    raw: Any = None

    @classmethod
    def from_dict(cls, d: dict) -> "ZetalornConfig":
        vocab, width = _int(d, "vocab", "config"), _int(d, "width", "config")
        eps = _float(_dict(d, "norm", "config"), "eps", "norm")
        scale = _float(d, "logit_scale", "config", positive=False) if "logit_scale" in d else 1.0
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config: 'layers' must be a non-empty list")
        mixers, ffs = [], []
        for i, layer in enumerate(layers):
            where = f"layers[{i}]"
            if not isinstance(layer, dict):
                raise ConfigError(f"{where} must be an object")
            mixers.append(_mixer(layer.get("type"), _dict(layer, "mixer", where), where))
            ffs.append(_mlp(layer.get("mlp"), f"{where}.mlp"))
        loop = None
        if d.get("loop") is not None:
            lp = _dict(d, "loop", "config")
            loop = (_int(lp, "start", "loop", 0), _int(lp, "stop", "loop"), _int(lp, "times", "loop"))
            if not (loop[0] < loop[1] <= len(layers)):
                raise ConfigError(f"loop: layers {loop[0]} .. {loop[1] - 1} do not lie among the {len(layers)} layers")
        return cls(vocab=vocab, width=width, eps=eps, logit_scale=scale, loop=loop, mixers=tuple(mixers), ffs=tuple(ffs),
                   raw=copy.deepcopy(d))

    def to_dict(self) -> Dict[str, Any]:
        return copy.deepcopy(self.raw)

    def order(self):
        """[(layer, the pass it opens or None)] in the order the layers run."""
        n = len(self.mixers)
        if self.loop is None:
            return [(i, None) for i in range(n)]
        start, stop, times = self.loop
        out = [(i, None) for i in range(start)]
        for t in range(times):
            out += [(i, t if i == start else None) for i in range(start, stop)]
        return out + [(i, None) for i in range(stop, n)]

    def _position(self, kind: str, width_key: str, dim: int, rot: Optional[ZetalornRotation]):
        if rot is None:
            return None
        return PartSpec(kind, {width_key: dim, "dims": rot.dims, "base": rot.base, "factor": rot.factor})

    def to_spec(self) -> ModelSpec:
        D = self.width
        norm = {"size": D, "eps": self.eps, "tensor": "", "scalar": True}
        layers = []
        for i, (m, ff) in enumerate(zip(self.mixers, self.ffs)):
            p = f"l{i}"
            if isinstance(m, ZetalornAttention):
                mixer = PartSpec("differential_attention", {
                    "hidden_size": D, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "key_dim": m.dim, "value_dim": m.vdim,
                    "scale": m.scale, "diff": m.diff, "eps": self.eps, "chunk": m.chunk, "window": None, "qk_norm": True,
                    "position": self._position("rope_interleaved", "width", m.dim, m.rot)}, prefix=f"{p}.mix")
            else:
                l, r = m.left, m.right
                left = PartSpec("pooled_window_attention", {
                    "hidden_size": D, "num_heads": l.heads, "num_kv_heads": l.kv_heads, "key_dim": l.dim, "value_dim": l.vdim,
                    "scale": l.scale, "window": l.window, "pool": l.pool, "eps": self.eps, "qk_norm": True,
                    "position": self._position("rope_leading", "head_dim", l.dim, l.rot)}, prefix=f"{p}.mix.left")
                right = PartSpec("lightning_attention", {
                    "hidden_size": D, "num_heads": r.heads, "key_dim": r.dim, "value_dim": r.vdim, "decay": list(r.decay),
                    "eps": self.eps}, prefix=f"{p}.mix.right")
                mixer = PartSpec("parallel_mixers", {"hidden_size": D, "eps": self.eps, "branches": [
                    {"part": left, "out": "left.out"}, {"part": right, "out": "right.out"}]}, prefix=f"{p}.mix")
            subs = [SubLayerSpec("mixer", mixer, PartSpec("rms_norm", norm, prefix=f"{p}.norm1"))]
            gates = ["rg1"]
            if ff is not None:
                ffn = PartSpec("routed_experts", {
                    "hidden_size": D, "experts": ff.experts, "top": ff.top, "expert_ff": ff.ff, "route_scale": 1.0, "gate": "sigmoid",
                    "act": "swish_clamped", "limit": ff.limit, "alpha": SWISH_ALPHA, "renorm": True,
                    "groups": {"count": ff.groups[0], "keep": ff.groups[1]} if ff.groups else None,
                    "shared_ff": None, "use_bias": False}, prefix=f"{p}.mlp")
                subs.append(SubLayerSpec("ffn", ffn, PartSpec("rms_norm", norm, prefix=f"{p}.norm2")))
                gates.append("rg2")
            layers.append(LayerSpec("gated_residual", tuple(subs), {"hidden_size": D, "prefix": p, "gates": gates}))
        reentry = None
        if self.loop is not None:
            reentry = PartSpec("embedding_and_offset", {"hidden_size": D, "passes": self.loop[2], "tensor": "step"}, prefix="loop")
        return ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab, hidden_size=D, max_positions=MAX_POSITIONS,
            embedding=PartSpec("scaled_pair_embedding", {"vocab_size": self.vocab, "hidden_size": D, "scale": 1.0,
                                                         "tensor": "embed", "pair": None}),
            layers=tuple(layers),
            order=tuple(CallSpec(layer=i, opens_pass=t) for i, t in self.order()),
            final_norm=PartSpec("rms_norm", norm, prefix="final.norm"),
            head=PartSpec("lm_head", {"vocab_size": self.vocab, "hidden_size": D, "tied_to": None, "tensor": "",
                                      "scale": self.logit_scale}, prefix="head"),
            stop_token_ids=(), reentry=reentry)
