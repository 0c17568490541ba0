"""Typed configuration of the Zedirax decoder, read from its own config.json keys.

    architecture    "Zedirax"
    vocab, width    vocabulary and stream width
    norm            {eps}
    residual_mult   what a sub-layer's output is multiplied by before it joins the stream (1 when absent)
    layers          list of {type: "mingru" | "latent_attention" | "attention", mixer: {...}, mlp: {...} or null}
      mingru mixer      width (channels of the recurrence)
      latent mixer      heads, dim (unrotated query/key part), rot_dim (rotated part; one key part shared by all heads),
                        vdim, kv_rank (latent size), scale, rot: {dims, base}
      attention mixer   heads, kv_heads, dim (query/key head size), vdim (value head size), scale,
                        q_temp: {coef, every} (optional)
      mlp               {kind: "dense", ff}  or  {kind: "moe", router: {experts, top}, expert: {ff}, shared: {ff} (optional)}

Tensor names: embed, l<i>.norm1, l<i>.norm2, l<i>.mix.*, l<i>.mlp.*, l<i>.dwa, final.norm, head.

A layer is `depth_averaged_residual`: x += m * part(norm(x)) for the mixer and then for the feed-forward, every norm an
RMS norm whose stored weight is the distance from one; what a layer hands on is a weighted sum of the embedding's output
and every layer's result so far (l<i>.dwa, i + 2 weights).  The configuration names no longest sequence;
MAX_POSITIONS is this library's own bound.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .registry import register_architecture
from .spec import CallSpec, ConfigError, LayerSpec, ModelSpec, PartSpec, SubLayerSpec
from .vumezen import _dict, _float, _int

MAX_POSITIONS = 1 << 18


@dataclass(frozen=True)
class ZediraxMinGRU:
    width: int


@dataclass(frozen=True)
class ZediraxLatent:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    rot_dims: int
    rot_base: float


@dataclass(frozen=True)
class ZediraxAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    q_temp: Optional[Tuple[float, int]]          # (coef, every)


@dataclass(frozen=True)
class ZediraxDense:
    ff: int


@dataclass(frozen=True)
class ZediraxMoE:
    experts: int
    top: int
    expert_ff: int
    shared_ff: Optional[int]


def _mixer(kind, m: dict, where: str):
    if kind == "mingru":
        return ZediraxMinGRU(width=_int(m, "width", where))
    if kind == "latent_attention":
        rot_dim = _int(m, "rot_dim", where, 0)
        rot_dims, rot_base = 0, 10000.0
        if rot_dim:
            rot = _dict(m, "rot", where)
            rot_dims, rot_base = _int(rot, "dims", f"{where}.rot", 0), _float(rot, "base", f"{where}.rot")
        mx = ZediraxLatent(heads=_int(m, "heads", where), dim=_int(m, "dim", where, 0), rot_dim=rot_dim, vdim=_int(m, "vdim", where),
                           kv_rank=_int(m, "kv_rank", where), scale=_float(m, "scale", where, positive=False),
                           rot_dims=rot_dims, rot_base=rot_base)
        if mx.rot_dims % 2 or mx.rot_dims > mx.rot_dim:
            raise ConfigError(f"{where}: rot.dims={mx.rot_dims} must be even and at most rot_dim={mx.rot_dim}")
        if mx.dim + mx.rot_dim == 0:
            raise ConfigError(f"{where}: a head needs query/key dimensions (dim + rot_dim > 0)")
        return mx
    if kind == "attention":
        q_temp = None
        if m.get("q_temp") is not None:
            qt = _dict(m, "q_temp", where)
            q_temp = (_float(qt, "coef", f"{where}.q_temp", positive=False), _int(qt, "every", f"{where}.q_temp"))
        mx = ZediraxAttention(heads=_int(m, "heads", where), kv_heads=_int(m, "kv_heads", where), dim=_int(m, "dim", where),
                              vdim=_int(m, "vdim", where), scale=_float(m, "scale", where, positive=False), q_temp=q_temp)
        if mx.heads % mx.kv_heads:
            raise ConfigError(f"{where}: {mx.heads} query heads cannot share {mx.kv_heads} key/value heads")
        return mx
    raise ConfigError(f"{where}: the mixers of this architecture are 'mingru', 'latent_attention' and 'attention', got {kind!r}")


def _mlp(mlp, where: str):
    if mlp is None:
        return None
    if not isinstance(mlp, dict):
        raise ConfigError(f"{where} must be an object or null")
    kind = mlp.get("kind")
    if kind == "dense":
        return ZediraxDense(ff=_int(mlp, "ff", where))
    if kind == "moe":
        router = _dict(mlp, "router", where)
        f = ZediraxMoE(experts=_int(router, "experts", f"{where}.router"), top=_int(router, "top", f"{where}.router"),
                       expert_ff=_int(_dict(mlp, "expert", where), "ff", f"{where}.expert"),
                       shared_ff=_int(_dict(mlp, "shared", where), "ff", f"{where}.shared") if mlp.get("shared") is not None else None)
        if f.top > f.experts:
            raise ConfigError(f"{where}: a token cannot use {f.top} of {f.experts} experts")
        return f
    raise ConfigError(f"{where}: the feed-forwards of this architecture are kind 'dense' and 'moe', got {kind!r}")


@register_architecture("Zedirax")
@dataclass(frozen=True)
class ZediraxConfig:
    vocab: int
    width: int
    eps: float
    residual_mult: float
    mixers: Tuple[Any, ...]                   # ZediraxMinGRU, ZediraxLatent or ZediraxAttention per layer
    ffs: Tuple[Any, ...]                      # ZediraxDense, ZediraxMoE or None per layer
    raw: Any = None

    @classmethod
    def from_dict(cls, d: dict) -> "ZediraxConfig":
        vocab, width = _int(d, "vocab", "config"), _int(d, "width", "config")
        eps = _float(_dict(d, "norm", "config"), "eps", "norm")
        mult = _float(d, "residual_mult", "config", positive=False) if "residual_mult" in d else 1.0
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
        return cls(vocab=vocab, width=width, eps=eps, residual_mult=mult, mixers=tuple(mixers), ffs=tuple(ffs),
                   raw=copy.deepcopy(d))

    def to_dict(self) -> Dict[str, Any]:
        return copy.deepcopy(self.raw)

    def to_spec(self) -> ModelSpec:
        D, L = self.width, len(self.mixers)
        norm = {"size": D, "eps": self.eps, "tensor": "", "offset": 1.0}
        layers = []
        for i, (m, ff) in enumerate(zip(self.mixers, self.ffs)):
            p = f"l{i}"
            if isinstance(m, ZediraxMinGRU):
                mixer = PartSpec("min_gru", {"hidden_size": D, "width": m.width}, prefix=f"{p}.mix")
            elif isinstance(m, ZediraxLatent):
                mixer = PartSpec("latent_attention", {
                    "hidden_size": D, "num_heads": m.heads, "nope_dim": m.dim, "rope_dim": m.rot_dim, "value_dim": m.vdim,
                    "q_rank": None, "kv_rank": m.kv_rank, "scale": m.scale, "window": None, "eps": self.eps, "sink": False,
                    "gate": "elements", "own_kv": True, "cache_window": None,
                    "position": PartSpec("rope_leading", {"head_dim": m.rot_dim, "dims": m.rot_dims, "base": m.rot_base})
                    if m.rot_dims else None,
                }, prefix=f"{p}.mix")
            else:
                mixer = PartSpec("windowed_sink_attention", {
                    "hidden_size": D, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "key_dim": m.dim, "value_dim": m.vdim,
                    "scale": m.scale, "window": None, "keep_first": 0, "sink": False, "own_kv": True, "cache_window": None,
                    "position": None, "distance_bias": True,
                    "q_temp": {"coef": m.q_temp[0], "every": m.q_temp[1]} if m.q_temp else None}, prefix=f"{p}.mix")
            subs = [SubLayerSpec("mixer", mixer, PartSpec("rms_norm", norm, prefix=f"{p}.norm1"))]
            if isinstance(ff, ZediraxDense):
                ffn = PartSpec("gated_mlp", {"hidden_size": D, "intermediate_size": ff.ff, "act": "gelu_tanh", "bias": True,
                                             "names": {"gate": "gate", "up": "up", "down": "down"}}, prefix=f"{p}.mlp")
            elif isinstance(ff, ZediraxMoE):
                ffn = PartSpec("routed_experts", {
                    "hidden_size": D, "experts": ff.experts, "top": ff.top, "expert_ff": ff.expert_ff, "route_scale": 1.0,
                    "gate": "softmax_chosen", "act": "gelu", "shared_ff": ff.shared_ff, "shared_gate": ff.shared_ff is not None,
                    "use_bias": False}, prefix=f"{p}.mlp")
            else:
                ffn = None
            if ffn is not None:
                subs.append(SubLayerSpec("ffn", ffn, PartSpec("rms_norm", norm, prefix=f"{p}.norm2")))
            layers.append(LayerSpec("depth_averaged_residual", tuple(subs),
                                    {"mult": self.residual_mult, "index": i, "layers": L, "prefix": p, "tensor": "dwa"}))
        return ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab, hidden_size=D, max_positions=MAX_POSITIONS,
            embedding=PartSpec("scaled_pair_embedding", {"vocab_size": self.vocab, "hidden_size": D, "scale": 1.0,
                                                         "tensor": "embed", "pair": None}),
            layers=tuple(layers),
            order=tuple(CallSpec(layer=i) for i in range(L)),
            final_norm=PartSpec("rms_norm", norm, prefix="final.norm"),
            head=PartSpec("lm_head", {"vocab_size": self.vocab, "hidden_size": D, "tied_to": None, "tensor": ""}, prefix="head"),
            stop_token_ids=())
