from __future__ import annotations

import torch

from .. import kernels
from .base import Mixer, TensorDecl, register_part


@register_part("mixer", "min_gru")
class MinGRU(Mixer):
    """A recurrent mixer with one float32 number of memory per channel, kept in the cache's fixed-size state of the
    sequence (zero when the sequence starts) and carried from token to token.  Its gates read the current token only:

        z = sigmoid(Wz h + bz)                    c = u + 1/2 where u >= 0, sigmoid(u) below,  u = Wx h + bx
        S <- (1 - z) S + z c                      (element by element, `width` channels)
        out = Wo (S * silu(Wg h))

    The three input projections are one matrix product whose output stays float32 in both precisions; gates, candidates,
    the state and its sums are float32.  Since S is an affine function of the state before, a long prompt is cut into
    chunks that run side by side (kernels.mingru); single tokens and short portions run in one launch.

    params: hidden_size, width, names (local tensor names of z, z_bias, x, x_bias, g, o).
    """
    capturable = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        p = spec.params
        self.hidden, self.width = int(p["hidden_size"]), int(p["width"])
        if self.width <= 0:
            raise ValueError(f"the recurrence needs at least one channel, got {self.width}")
        self.names = dict({"z": "z", "z_bias": "z.b", "x": "x", "x_bias": "x.b", "g": "g", "o": "o"}, **(p.get("names") or {}))
        self.w_in = self.b_in = self.w_o = None

    def state_size(self):
        return self.width

    def tensors(self):
        n, D, W = self.names, self.hidden, self.width
        return {n["z"]: TensorDecl((W, D)), n["z_bias"]: TensorDecl((W,), use="vector"), n["x"]: TensorDecl((W, D)),
                n["x_bias"]: TensorDecl((W,), use="vector"), n["g"]: TensorDecl((W, D)), n["o"]: TensorDecl((D, W))}

    def load(self, tensors):
        n = self.names
        ts = [tensors[n[k]] for k in ("z", "x", "g")]
        dt = ts[0].dtype
        for t in ts[1:]:
            dt = torch.promote_types(dt, t.dtype)
        self.w_in = torch.cat([t.to(dt) for t in ts], dim=0).contiguous()                     # [z | x | g]
        zb, xb = tensors[n["z_bias"]].float(), tensors[n["x_bias"]].float()
        self.b_in = torch.cat([zb, xb, torch.zeros_like(zb)]).contiguous()
        self.w_o = tensors[n["o"]].contiguous()

    def forward(self, x, ctx, call):
        from .mlp import delta_dtype
        proj = kernels.linear(x, self.w_in, self.b_in, out_dtype=torch.float32)
        y = kernels.mingru(proj, self.width, ctx.state(call), ctx.seq_start, ctx.seq_slot, ctx.n_seqs, ctx.max_new, x.dtype)
        return kernels.linear(y, self.w_o, out_dtype=delta_dtype(y))
