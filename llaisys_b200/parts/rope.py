from __future__ import annotations

import torch

from .. import kernels
from .base import PositionEncoding, register_part

# (head_dim, theta, device) -> (cos, sin): every layer of a model has a part of its own, and all
# of them rotate by the same angles, so they share one pair of tables.
_TABLES = {}


def _tables(head_dim: int, theta: float, device, rows: int):
    key = (head_dim, theta, str(device))
    have = _TABLES.get(key)
    if have is None or have[0].shape[0] < rows:
        half = head_dim // 2
        j = torch.arange(half, dtype=torch.float64)
        freq = 1.0 / torch.pow(torch.tensor(theta, dtype=torch.float64), 2.0 * j / head_dim)
        ang = torch.arange(rows, dtype=torch.float64)[:, None] * freq[None, :]
        have = (torch.cos(ang).to(torch.float32).to(device), torch.sin(ang).to(torch.float32).to(device))
        _TABLES[key] = have
    return have


@register_part("position", "rope_half_split")
class RotaryHalfSplit(PositionEncoding):
    """Rotary encoding over the pairs (j, j + d/2): phi = p / theta^(2j/d),
    (a, b) -> (a cos phi - b sin phi, b cos phi + a sin phi)
    (xsmccc/llaisys src/ops/rope/cpu/rope_cpu.cpp:16-46, which computes the angle in double
    precision from theta held as a C float).  The cos/sin table is built in float64 on the host
    and kept in float32.  prepare() sizes it once for the longest sequence the engine can hold;
    after that it never moves (a captured step has its address), and a position beyond it is an
    error.  A part that was never prepared grows its table on demand.  params: head_dim, theta."""
    capturable = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.head_dim = int(spec.params["head_dim"])
        self.theta = float(torch.tensor(float(spec.params["theta"]), dtype=torch.float32))
        if self.head_dim % 2:
            raise ValueError(f"rotary encoding needs an even head size, got {self.head_dim}")
        self._cos = self._sin = None
        self._prepared = False

    def table(self, positions: int):
        if self._cos is None or self._cos.shape[0] < positions:
            if self._prepared:
                raise ValueError(f"position {positions - 1} lies beyond the {self._cos.shape[0]} positions the "
                                 f"rotary table was prepared for")
            rows = max(positions, 2 * (self._cos.shape[0] if self._cos is not None else 0))
            self._cos, self._sin = _tables(self.head_dim, self.theta, self.env.device, rows)
        return self._cos, self._sin

    def prepare(self, max_positions):
        self._prepared = False
        self.table(max_positions)
        self._prepared = True

    def rotation_tables(self, positions: int):
        return self.table(positions)

    def apply(self, qkv, num_heads, num_kv_heads, ctx):
        cos, sin = self.table(ctx.max_position + 1)
        kernels.rope_append(qkv, num_heads, num_kv_heads, self.head_dim, cos=cos, sin=sin,
                            tok_pos=ctx.tok_pos, err=ctx.err)


def _leading_tables(dims: int, base: float, device, rows: int, factor: float = 1.0):
    key = ("leading", dims, base, str(device)) + ((factor,) if factor != 1.0 else ())
    have = _TABLES.get(key)
    if have is None or have[0].shape[0] < rows:
        half = dims // 2
        i = torch.arange(half, dtype=torch.float64)
        freq = torch.pow(torch.tensor(base, dtype=torch.float64), -2.0 * i / dims) / factor
        ang = torch.arange(rows, dtype=torch.float64)[:, None] * freq[None, :]
        have = (torch.cos(ang).to(torch.float32).to(device).contiguous(), torch.sin(ang).to(torch.float32).to(device).contiguous())
        _TABLES[key] = have
    return have


@register_part("position", "rope_leading")
class RotaryLeading(PositionEncoding):
    """Rotary encoding of the first `dims` dimensions of a head: dimension i pairs with i + dims/2 (i < dims/2) and the
    pair (a, b) at position p becomes (a cos phi - b sin phi, b cos phi + a sin phi), phi = p * base^(-2i/dims); the
    dimensions from `dims` on pass unchanged.  dims = head_dim is the half-split rotation of whole heads; dims = 0
    encodes nothing.  Tables [positions, dims/2] are built in float64 on the host and kept in float32, sized once by
    prepare().  Mixers that rotate in their own kernels take the tables through pair_tables(); `pair_layout` tells them
    which dimensions pair up.  params: head_dim, dims, base, factor (default 1: every frequency is divided by it, the
    linear stretching of positions)."""
    capturable = True
    pair_layout = "halves"

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.head_dim, self.dims, self.base = int(spec.params["head_dim"]), int(spec.params["dims"]), float(spec.params["base"])
        self.factor = float(spec.params.get("factor", 1.0))
        if self.factor <= 0:
            raise ValueError(f"the frequencies' divisor must be positive, got {self.factor}")
        if self.dims % 2 or not (0 <= self.dims <= self.head_dim):
            raise ValueError(f"rotated dimensions must be even and at most the head size {self.head_dim}, got {self.dims}")
        self._tables = None
        self._prepared = False

    def leading_tables(self, positions: int):
        """(cos, sin), each float32 [rows >= positions, dims / 2]; None when nothing is rotated."""
        if self.dims == 0:
            return None
        if self._tables is None or self._tables[0].shape[0] < positions:
            if self._prepared:
                raise ValueError(f"position {positions - 1} lies beyond the {self._tables[0].shape[0]} positions the "
                                 f"rotary table was prepared for")
            rows = max(positions, 2 * (self._tables[0].shape[0] if self._tables is not None else 0))
            self._tables = _leading_tables(self.dims, self.base, self.env.device, rows, self.factor)
        return self._tables

    def prepare(self, max_positions):
        self._prepared = False
        self.leading_tables(max_positions)
        self._prepared = True

    def rotation_tables(self, positions: int):
        return self.leading_tables(positions) if self.dims == self.head_dim else None

    def pair_tables(self, positions: int):
        """(cos, sin, dims), the tables float32 [rows >= positions, dims / 2]; None when nothing is rotated."""
        t = self.leading_tables(positions)
        return None if t is None else (t[0], t[1], self.dims)

    def apply(self, qkv, num_heads, num_kv_heads, ctx):
        t = self.leading_tables(ctx.max_position + 1)
        if t is not None:
            kernels.rope_lead_append(qkv, num_heads, num_kv_heads, self.head_dim, self.head_dim, self.dims, cos=t[0], sin=t[1],
                                     tok_pos=ctx.tok_pos, err=ctx.err)


def yarn_frequencies(dims: int, base: float, yarn):
    """float64 frequencies [dims / 2] of a rotation with the wavelength-dependent rescaling known as YaRN, and the factor
    both cos and sin are multiplied by.  yarn = {factor, original, fast, slow}: with d(r) = dims ln(original / (2 pi r)) /
    (2 ln base) the dimension whose wavelength makes r turns over `original` positions, lo = max(floor(d(fast)), 0),
    hi = min(ceil(d(slow)), dims - 1) and ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), the frequency is
    f_i / factor * ramp_i + f_i (1 - ramp_i) (slow dimensions are stretched, fast ones kept) and the magnitude
    0.1 ln(factor) + 1.  None: plain frequencies base^(-2i/dims), magnitude 1."""
    import math
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = torch.pow(torch.tensor(base, dtype=torch.float64), -2.0 * i / dims)
    if not yarn:
        return f, 1.0
    factor, original = float(yarn["factor"]), float(yarn["original"])

    def turn_dim(turns: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(turn_dim(float(yarn["fast"]))), 0)
    hi = min(math.ceil(turn_dim(float(yarn["slow"]))), dims - 1)
    ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


@register_part("position", "rope_interleaved")
class RotaryInterleaved(PositionEncoding):
    """Rotary encoding of neighbouring pairs: of a vector of `width` elements the pairs (2i, 2i+1), i < dims / 2, are
    rotated by the angle p * f_i at position p, (u, v) -> (u cos - v sin, v cos + u sin); the elements from `dims` on
    pass unchanged.  Frequencies and magnitude come from yarn_frequencies().  The part hands out float32 tables
    [positions, dims / 2] of cos and sin (magnitude included), built in float64 on the host and sized once by
    prepare(); the mixers' kernels apply them.  params: width, dims, base, yarn (dict or None), factor (default 1: every
    frequency is divided by it, the linear stretching of positions)."""
    capturable = True
    pair_layout = "neighbours"

    def __init__(self, spec, env):
        super().__init__(spec, env)
        p = spec.params
        self.width, self.dims, self.base = int(p["width"]), int(p["dims"]), float(p["base"])
        self.yarn = dict(p["yarn"]) if p.get("yarn") else None
        self.factor = float(p.get("factor", 1.0))
        if self.factor <= 0:
            raise ValueError(f"the frequencies' divisor must be positive, got {self.factor}")
        if self.dims % 2 or not (0 <= self.dims <= self.width):
            raise ValueError(f"rotated dimensions must be even and at most {self.width}, got {self.dims}")
        self._tables = None
        self._prepared = False

    def pair_tables(self, positions: int):
        """(cos, sin, dims), the tables float32 [rows >= positions, dims / 2]; None when nothing is rotated."""
        if self.dims == 0:
            return None
        if self._tables is None or self._tables[0].shape[0] < positions:
            if self._prepared:
                raise ValueError(f"position {positions - 1} lies beyond the {self._tables[0].shape[0]} positions the "
                                 f"rotary table was prepared for")
            rows = max(positions, 2 * (self._tables[0].shape[0] if self._tables is not None else 0))
            key = ("pairs", self.dims, self.base, tuple(sorted(self.yarn.items())) if self.yarn else None, str(self.env.device))
            if self.factor != 1.0:
                key += (self.factor,)
            have = _TABLES.get(key)
            if have is None or have[0].shape[0] < rows:
                f, mag = yarn_frequencies(self.dims, self.base, self.yarn)
                f = f / self.factor
                ang = torch.arange(rows, dtype=torch.float64)[:, None] * f[None, :]
                have = ((torch.cos(ang) * mag).to(torch.float32).to(self.env.device).contiguous(),
                        (torch.sin(ang) * mag).to(torch.float32).to(self.env.device).contiguous())
                _TABLES[key] = have
            self._tables = have
        return self._tables[0], self._tables[1], self.dims

    def prepare(self, max_positions):
        self._prepared = False
        self.pair_tables(max_positions)
        self._prepared = True

    def apply(self, qkv, num_heads, num_kv_heads, ctx):
        raise NotImplementedError("this encoding hands out pair_tables(); the mixers that take it rotate in their own kernels")
