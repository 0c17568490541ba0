from __future__ import annotations

import torch

from .. import kernels
from .base import FeedForward, TensorDecl, register_part


@register_part("ffn", "routed_experts")
class RoutedExperts(FeedForward):
    """A mixture of small feed-forward experts of which every token uses `top`, plus (optionally) a shared expert
    that every token uses.

      gates     g = sigmoid(Wr h), computed in float32
      choice    the `top` experts with the largest g + bias (`bias`: a per-expert correction that steers the choice
                only); ties go to the lower index
      weights   g of the chosen experts times route_scale, not renormalised
      expert    Wd act(Wu h), no biases; act = max(., 0)^2 ("relu_squared")
      output    sum over the chosen experts of weight * expert(h), plus shared(h)

    Variants.  `groups` = {count, keep}: the experts form `count` equal groups of neighbours; a group's score is the sum
    of its two largest choice scores, and only experts of the `keep` best groups can be chosen.  `renorm`: the chosen
    gates are divided by their sum (+ 1e-20) before route_scale is applied.  `act` "swish_clamped": a gated expert with a
    second matrix Wg (tensor `expert_gate`), g = min(Wg h, limit), u = clamp(Wu h, -limit, limit),
    expert = Wd (g sigmoid(alpha g) (u + 1)); gate and up matrices are kept as one, and the activation is a pass of its
    own between the two products.  `gate` "softmax_chosen": the `top` experts with the largest logits Wr h (+ bias) are chosen and their
    weights are the softmax over the chosen logits alone (times route_scale).  `act` "gelu": an expert is
    Wd gelu(Wu h) with the erf form of gelu.  `shared_gate`: the shared expert's output is multiplied by
    sigmoid(w_sg . h), one number per token (tensor `shared_gate`, [1, hidden]); its logit rides on the router's
    product as one more row of the matrix.

    The experts' matrices are kept stacked ([E, ff, H] and [E, H, ff]).  A step's (token, choice) pairs are grouped by
    expert on the device (kernels.moe_plan) and the two products run over those groups: in bfloat16 on tcgen05, the
    second one ending in the weighted add into the float32 residual stream (float32 atomics, arrival order); in float32
    (and for widths the tensor-core kernel does not take) on the CUDA cores with the weighted sum added in a fixed
    order.  Nothing is read back to the host, so a step can be captured.

    forward_into(..., scale=c) adds c times the part's output (the weights and the shared expert's activations carry the
    factor), for arrangements whose parts join the stream scaled.

    params: hidden_size, experts, top, expert_ff, route_scale, gate, act, limit, alpha, groups, renorm, shared_ff (None: no
    shared expert), shared_gate, use_bias, names (local tensor names: router, bias, expert_up, expert_down with {e} for the expert's index, shared_up,
    shared_down, shared_gate).
    """
    capturable = True
    scaled_into = True
    NAMES = {"router": "router", "bias": "correction", "expert_up": "e{e}.up", "expert_down": "e{e}.down", "expert_gate": "e{e}.gate",
             "shared_up": "shared.up", "shared_down": "shared.down", "shared_gate": "shared.sg"}

    def __init__(self, spec, env):
        super().__init__(spec, env)
        p = spec.params
        self.hidden, self.n_experts, self.top = int(p["hidden_size"]), int(p["experts"]), int(p["top"])
        self.ff = int(p["expert_ff"])
        self.route_scale = float(p.get("route_scale", 1.0))
        self.act = str(p.get("act", "relu_squared"))
        if self.act not in ("relu_squared", "gelu", "swish_clamped"):
            raise ValueError(f"expert activation {self.act!r} is not built (relu_squared, gelu, swish_clamped)")
        self.gated = self.act == "swish_clamped"
        self.limit, self.alpha = float(p.get("limit", 0.0)), float(p.get("alpha", 1.0))
        if self.gated and self.limit <= 0:
            raise ValueError(f"the clamped activation needs a positive limit, got {self.limit}")
        self.groups = (int(p["groups"]["count"]), int(p["groups"]["keep"])) if p.get("groups") else None
        self.renorm = bool(p.get("renorm", False))
        self.gate = str(p.get("gate", "sigmoid"))
        if self.gate not in kernels.ops.MOE_GATES:
            raise ValueError(f"unknown router gate {self.gate!r}; known: {sorted(kernels.ops.MOE_GATES)}")
        if not (1 <= self.top <= self.n_experts):
            raise ValueError(f"a token cannot use {self.top} of {self.n_experts} experts")
        if self.groups:
            count, keep = self.groups
            if count < 1 or self.n_experts % count or not (1 <= keep <= count) or keep * (self.n_experts // count) < self.top:
                raise ValueError(f"{self.n_experts} experts in {count} groups of which {keep} are kept cannot give {self.top} choices")
            if count == 1:
                self.groups = None
        self.shared_ff = int(p["shared_ff"]) if p.get("shared_ff") else None
        self.use_bias = bool(p.get("use_bias", True))
        self.shared_gate = bool(p.get("shared_gate", False)) and self.shared_ff is not None
        self.names = dict(self.NAMES, **(p.get("names") or {}))
        self.router = self.bias = self.up = self.down = self.shared_up = self.shared_down = None

    def tensors(self):
        n = self.names
        t = {n["router"]: TensorDecl((self.n_experts, self.hidden))}
        if self.use_bias:
            t[n["bias"]] = TensorDecl((self.n_experts,), use="vector")
        for e in range(self.n_experts):
            t[n["expert_up"].format(e=e)] = TensorDecl((self.ff, self.hidden))
            if self.gated:
                t[n["expert_gate"].format(e=e)] = TensorDecl((self.ff, self.hidden))
            t[n["expert_down"].format(e=e)] = TensorDecl((self.hidden, self.ff))
        if self.shared_ff:
            t[n["shared_up"]] = TensorDecl((self.shared_ff, self.hidden))
            t[n["shared_down"]] = TensorDecl((self.hidden, self.shared_ff))
        if self.shared_gate:
            t[n["shared_gate"]] = TensorDecl((1, self.hidden))
        return t

    def load(self, tensors):
        n = self.names
        self.router = tensors[n["router"]].contiguous()
        if self.shared_gate:
            # the shared expert's gate logit is one more row of the router's product
            sg = tensors[n["shared_gate"]].reshape(1, self.hidden)
            dt = torch.promote_types(self.router.dtype, sg.dtype)
            self.router = torch.cat([self.router.to(dt), sg.to(dt)], dim=0).contiguous()
        self.bias = tensors[n["bias"]].to(torch.float32).contiguous() if self.use_bias else None
        if self.gated:
            # [E, 2 ff, H]: an expert's gate rows, then its up rows
            self.up = torch.stack([torch.cat([tensors[n["expert_gate"].format(e=e)], tensors[n["expert_up"].format(e=e)]], dim=0)
                                   for e in range(self.n_experts)]).contiguous()
        else:
            self.up = torch.stack([tensors[n["expert_up"].format(e=e)] for e in range(self.n_experts)]).contiguous()
        self.down = torch.stack([tensors[n["expert_down"].format(e=e)] for e in range(self.n_experts)]).contiguous()
        if self.shared_ff:
            self.shared_up, self.shared_down = tensors[n["shared_up"]].contiguous(), tensors[n["shared_down"]].contiguous()

    def forward(self, x, ctx):
        out = torch.zeros((x.shape[0], self.hidden), dtype=torch.float32, device=x.device)
        self.forward_into(x, ctx, out)
        return out

    def forward_into(self, x, ctx, residual, scale: float = 1.0):
        idx, wgt, z = kernels.moe_route(x, self.router, self.bias, self.top, self.route_scale * scale, gate=self.gate,
                                        n_experts=self.n_experts, with_logits=True, groups=self.groups, renorm=self.renorm)
        tc = kernels.moe_tc_ok(x, self.up, self.down) and residual.stride(1) == 1
        plan = kernels.moe_plan(idx, self.n_experts, kernels.moe_tc_tile_rows(idx.numel(), self.n_experts) if tc else None)
        if tc:
            # tensor cores: the tokens' rows in slot order, the up projection with its activation, and the down
            # projection that ends in the weighted add into the stream
            act = kernels.moe_gemm_tc(kernels.moe_gather_rows(x, plan), self.up, plan, "store" if self.gated else self.act,
                                      out_dtype=x.dtype)
            if self.gated:
                act = kernels.glu(act, self.act, limit=self.limit, alpha=self.alpha)
            kernels.moe_gemm_tc(act, self.down, plan, "weighted_add", out=residual, wgt=wgt)
        else:
            act = kernels.moe_gemm(x, self.up, plan, gather=True, act=None if self.gated else self.act, out_dtype=x.dtype)
            if self.gated:
                act = kernels.glu(act, self.act, limit=self.limit, alpha=self.alpha)
            y = kernels.moe_gemm(act, self.down, plan, gather=False, act=None, out_dtype=torch.float32)
            kernels.moe_combine(residual, y, plan, wgt)
        if self.shared_ff:
            a = kernels.linear(x, self.shared_up)
            if self.shared_gate or scale != 1.0 or self.act != "relu_squared":
                kernels.act_rows_(a, self.act, z[:, self.n_experts] if self.shared_gate else None, scale)
            else:
                kernels.relu_squared_(a)
            if kernels.linear_into_ok(a, self.shared_down, None, residual):
                kernels.linear_into(a, self.shared_down, None, residual)
            else:
                kernels.residual_add(residual, kernels.linear(a, self.shared_down))
        return True
