from __future__ import annotations

import torch

from ..config.spec import PartSpec
from .base import Block, TensorDecl, register_part


@register_part("block", "pre_norm_residual")
class PreNormResidual(Block):
    """x -> norm -> part -> + for every sub-layer in turn; with a mixer and a feed-forward that is
    x -> norm -> mixer -> +x -> norm -> feed-forward -> +   (xsmccc/llaisys
    src/models/qwen2/layer.hpp:47-84).  A part that can add its result to the residual stream in its
    own last kernel does so (forward_into); otherwise the add is done by the norm that follows, so
    the block hands its last delta on to the next block (or to the final norm).  A sub-layer
    without a norm of its own gets the residual stream as it is (the pending delta added)."""
    capturable = True

    def forward(self, residual, pending, ctx, users):
        from .. import kernels
        if isinstance(pending, Deferred):
            pending = settle(residual, pending)
        mixers = iter(users)
        for sub in self.sublayers:
            if sub.norm is not None:
                h = sub.norm.forward(residual, pending)
            else:
                if pending is not None:
                    kernels.residual_add(residual, pending)
                h = residual.to(self.env.dtype)
            if sub.category == "mixer":
                call = next(mixers)
                pending = None if sub.part.forward_into(h, ctx, call, residual) else sub.part.forward(h, ctx, call)
            else:
                pending = None if sub.part.forward_into(h, ctx, residual) else sub.part.forward(h, ctx)
        return residual, pending


@register_part("block", "parallel_residual")
class ParallelResidual(Block):
    """x -> x + sum over the sub-layers of part(norm(x)): every sub-layer reads the same stream, each through a norm
    of its own.  The norms are computed first, all from one root mean square per row (they differ in their weights
    only) in one pass over the stream; after that the parts may add into the stream in any order, each in its own
    last kernel where it can.  Needs norms that are RMS norms with one eps."""
    capturable = True

    def forward(self, residual, pending, ctx, users):
        from .. import kernels
        if isinstance(pending, Deferred):
            pending = settle(residual, pending)
        if pending is not None:
            kernels.residual_add(residual, pending)
        norms = [sub.norm for sub in self.sublayers]
        if any(n is None or n.kind != "rms_norm" or n.eps != norms[0].eps for n in norms):
            raise ValueError("a parallel layer needs an RMS norm with the same eps ahead of every sub-layer")
        hs = []
        for i in range(0, len(norms), 2):
            hs += kernels.rmsnorm_multi(residual, [n.weight for n in norms[i:i + 2]], norms[0].eps, self.env.dtype)
        mixers = iter(users)
        for sub, h in zip(self.sublayers, hs):
            if sub.category == "mixer":
                call = next(mixers)
                if not sub.part.forward_into(h, ctx, call, residual):
                    kernels.residual_add(residual, sub.part.forward(h, ctx, call))
            elif not sub.part.forward_into(h, ctx, residual):
                kernels.residual_add(residual, sub.part.forward(h, ctx))
        return residual, None


@register_part("block", "sandwich_residual")
class SandwichResidual(Block):
    """x -> x + mult * post_norm(part(norm(x))) for every sub-layer in turn: each part sits between a norm of its input
    and a norm of its output, and the normed output is scaled by the layer's constant `mult` before it joins the float32
    stream.  Output norm, add and the next sub-layer's input norm are one pass over the row (Norm.forward_scaled_add);
    the layer's last part leaves its output pending with its norm, and the block after it (or the final norm) runs
    that pass, so a layer costs one norm launch per part.  params: mult."""
    capturable = True

    def __init__(self, sublayers, env, params=None):
        super().__init__(sublayers, env, params)
        self.mult = float(self.params.get("mult", 1.0))
        for sub in self.sublayers:
            if sub.norm is None or sub.post_norm is None:
                raise ValueError("every sub-layer of this arrangement has a norm before and a norm after its part")

    def forward(self, residual, pending, ctx, users):
        mixers = iter(users)
        h = None
        for i, sub in enumerate(self.sublayers):
            if i == 0:
                h = settle(residual, pending, sub.norm)
            if sub.category == "mixer":
                delta = sub.part.forward(h, ctx, next(mixers))
            else:
                delta = sub.part.forward(h, ctx)
            if i + 1 < len(self.sublayers):
                h = sub.post_norm.forward_scaled_add(residual, delta, self.mult, then=self.sublayers[i + 1].norm)
            else:
                pending = PendingNormed(delta, sub.post_norm, self.mult)
        return residual, pending


@register_part("block", "depth_averaged_residual")
class DepthAveragedResidual(Block):
    """x -> x + mult * part(norm(x)) for every sub-layer in turn, and then, as what the next layer (or the output norm)
    reads, a weighted sum over depth: with X_0 the embedding's output and X_(k+1) the result of the k-th layer of this
    kind (before any averaging), layer i hands on  sum_{j <= i+1} a_i[j] X_j,  a_i the layer's tensor of i + 2 weights.

    The results are kept for the step in one buffer of planes ([layers + 1, T, H] float32, made by the step's first
    layer of this kind): layer i works in plane i, which starts as what the layer before handed on and ends as
    X_(i+1).  Every pass over the stream is one launch (kernels.stream_update): the scaled add of a part's output with
    the next sub-layer's norm; at a layer's end the scaled add, the sum over depth into the next plane and the next
    layer's first norm, which the layer leaves pending (PendingDepthSum) for whoever reads the stream next.  A part that
    can add its scaled output to the stream itself (`scaled_into`) does.  Needs RMS norms.

    params: mult, index (which layer of this kind: 0, 1, ...), layers (how many there are), prefix, tensor (the weights'
    local name, default "dwa": the file's name is prefix.tensor)."""
    capturable = True

    def __init__(self, sublayers, env, params=None):
        super().__init__(sublayers, env, params)
        p = self.params
        self.mult, self.index, self.layers = float(p.get("mult", 1.0)), int(p["index"]), int(p["layers"])
        if not (0 <= self.index < self.layers):
            raise ValueError(f"layer {self.index} of {self.layers}")
        self.tensor = str(p.get("tensor", "dwa"))
        self.spec = PartSpec("depth_averaged_residual", p, prefix=str(p.get("prefix", "")))
        for sub in self.sublayers:
            if sub.norm is None or sub.norm.kind != "rms_norm":
                raise ValueError("every sub-layer of this arrangement sits behind an RMS norm")
        self.weights = None

    def tensors(self):
        n = self.index + 2
        return {self.tensor: TensorDecl((n,), init=f"mean:{1.0 / n}", use="vector")}

    def load(self, tensors):
        self.weights = tensors[self.tensor].float().contiguous()

    def forward(self, residual, pending, ctx, users):
        from .. import kernels
        first = self.sublayers[0].norm
        if isinstance(pending, PendingDepthSum):
            planes, x0 = pending.planes, pending.x0
            h = pending.settle(residual, first)
        else:
            # the step's first layer of this kind: what it is handed is X_0; it works on a copy in plane 0
            if isinstance(pending, Deferred):
                pending = settle(residual, pending)
            T, H = residual.shape
            planes = torch.empty((self.layers + 1, T, H), dtype=torch.float32, device=residual.device)
            x0 = residual
            h = kernels.stream_update(x0, pending, 1.0, dst=planes[0], weight=first.weight, eps=first.eps, out_dtype=self.env.dtype)
            residual = planes[0]
        mixers = iter(users)
        delta = None
        for i, sub in enumerate(self.sublayers):
            if i > 0:
                h = kernels.stream_update(residual, delta, self.mult, weight=sub.norm.weight, eps=sub.norm.eps, out_dtype=self.env.dtype)
            if sub.category == "mixer":
                delta = sub.part.forward(h, ctx, next(mixers))
            elif getattr(sub.part, "scaled_into", False) and sub.part.forward_into(h, ctx, residual, scale=self.mult):
                delta = None
            else:
                delta = sub.part.forward(h, ctx)
        return planes[self.index + 1], PendingDepthSum(residual, delta, self.mult, self.weights, x0, planes)


@register_part("block", "gated_residual")
class GatedResidual(Block):
    """x -> x + sigmoid(Wg h + bg) * part(h), h = norm(x), for every sub-layer in turn: a part's result passes, element by
    element, through a gate that is computed from the same normed input the part reads; every sub-layer has a gate matrix
    [H, H] and bias [H] of its own.  The gate's logits leave their matrix product in float32.  The gated add and the norm
    that follows are one pass over the row (kernels.stream_join); a layer's last part is left pending (PendingGated) for
    whoever reads the stream next, so a layer costs one pass per sub-layer.  Needs RMS norms.

    params: hidden_size, prefix, gates (the local names of the sub-layers' gate matrices, in order; a bias is the
    matrix's name + ".b")."""
    capturable = True

    def __init__(self, sublayers, env, params=None):
        super().__init__(sublayers, env, params)
        p = self.params
        self.hidden, self.gates = int(p["hidden_size"]), [str(g) for g in p["gates"]]
        if len(self.gates) != len(self.sublayers):
            raise ValueError(f"{len(self.sublayers)} sub-layers but {len(self.gates)} gates")
        self.spec = PartSpec("gated_residual", p, prefix=str(p.get("prefix", "")))
        for sub in self.sublayers:
            if sub.norm is None or sub.norm.kind != "rms_norm":
                raise ValueError("every sub-layer of this arrangement sits behind an RMS norm")
        self.w, self.b = [], []

    def tensors(self):
        t = {}
        for g in self.gates:
            t[g] = TensorDecl((self.hidden, self.hidden))
            t[g + ".b"] = TensorDecl((self.hidden,), use="vector")
        return t

    def load(self, tensors):
        self.w = [tensors[g].contiguous() for g in self.gates]
        self.b = [tensors[g + ".b"].float().contiguous() for g in self.gates]

    def forward(self, residual, pending, ctx, users):
        from .. import kernels
        mixers = iter(users)
        for i, sub in enumerate(self.sublayers):
            h = settle(residual, pending, sub.norm)
            gate = kernels.linear(h, self.w[i], self.b[i], out_dtype=torch.float32)
            if sub.category == "mixer":
                delta = sub.part.forward(h, ctx, next(mixers))
            else:
                delta = sub.part.forward(h, ctx)
            pending = PendingGated(delta, gate)
        return residual, pending


class Deferred:
    """What a block may leave for whoever reads the stream next (the next block's first norm, or the output norm)."""


class PendingGated(Deferred):
    """A part's output that has not joined the stream yet: it joins as sigmoid(gate) * delta (gate: float32 logits, None:
    as it is), together with `rows_add` (float32 [T, H]) and `vec_add` (float32 [H]) where given."""

    def __init__(self, delta=None, gate=None, rows_add=None, vec_add=None):
        self.delta, self.gate, self.rows_add, self.vec_add = delta, gate, rows_add, vec_add

    def settle(self, residual, norm=None, rows=None):
        from .. import kernels
        fused = norm is not None and rows is None and norm.kind == "rms_norm" and norm.weight.dtype == torch.float32
        h = kernels.stream_join(residual, self.delta, self.gate, rows_add=self.rows_add, vec_add=self.vec_add,
                                weight=norm.weight if fused else None, eps=norm.eps if fused else 0.0,
                                out_dtype=norm.env.dtype if fused else None)
        if norm is None or fused:
            return h
        return norm.forward(residual, None, rows=rows)


class PendingNormed(Deferred):
    """A part's output that has not joined the stream yet: it is to be normed by `norm`, scaled by `mult` and added."""

    def __init__(self, delta, norm, mult):
        self.delta, self.norm, self.mult = delta, norm, mult


class PendingDepthSum(Deferred):
    """The end of a depth-averaged layer that has not run yet: `cur` (the layer's plane) still lacks mult * delta, and
    the stream handed on is the weighted sum of x0, the planes before cur's and cur."""

    def __init__(self, cur, delta, mult, weights, x0, planes):
        self.cur, self.delta, self.mult, self.weights, self.x0, self.planes = cur, delta, mult, weights, x0, planes

    def settle(self, dst, norm=None, rows=None):
        """The sum into `dst` (the plane the next layer works on); returns norm of it (None without a norm).  With
        `rows` only those rows of the sum are formed and normed, and dst is not written."""
        from .. import kernels
        if norm is not None and norm.kind != "rms_norm":
            kernels.stream_update(self.cur, self.delta, self.mult, mix=self.weights, x0=self.x0, planes=self.planes, dst=dst)
            return norm.forward(dst, None, rows=rows)
        return kernels.stream_update(self.cur, self.delta, self.mult, mix=self.weights, x0=self.x0, planes=self.planes,
                                     dst=None if rows is not None else dst, rows=rows,
                                     weight=norm.weight if norm is not None else None,
                                     eps=norm.eps if norm is not None else 0.0, out_dtype=norm.env.dtype if norm is not None else None)


def settle(residual, pending, norm=None, rows=None):
    """Adds whatever the block before left pending to the float32 stream and returns `norm` of the result (None without
    a norm).  With `rows` only those rows are returned (the stream itself is still brought up to date)."""
    from .. import kernels
    if isinstance(pending, (PendingDepthSum, PendingGated)):
        return pending.settle(residual, norm, rows)
    if isinstance(pending, PendingNormed):
        if rows is None:
            try:
                return pending.norm.forward_scaled_add(residual, pending.delta, pending.mult, then=norm)
            except ValueError:
                pass                                    # norms of different kinds: two passes
        pending.norm.forward_scaled_add(residual, pending.delta, pending.mult)
        pending = None
    if norm is None:
        if pending is not None:
            kernels.residual_add(residual, pending)
        return None
    return norm.forward(residual, pending, rows=rows)
