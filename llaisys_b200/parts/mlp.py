from __future__ import annotations

import torch

from .. import kernels
from .base import FeedForward, TensorDecl, register_part


@register_part("ffn", "swiglu_mlp")
class SwiGLUMLP(FeedForward):
    """down(up(x) * silu(gate(x))), no biases (xsmccc/llaisys src/models/qwen2/mlp.hpp:18-39,
    src/ops/swiglu/cpu/swiglu_cpu.cpp:13-21).  The gate and up matrices are kept as one
    [2I, H] matrix so that one product serves both.  params: hidden_size, intermediate_size."""
    capturable = True


    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.hidden, self.inter = int(spec.params["hidden_size"]), int(spec.params["intermediate_size"])
        self.gate_up = self.down = None

    def tensors(self):
        return {"gate_proj.weight": TensorDecl((self.inter, self.hidden)),
                "up_proj.weight": TensorDecl((self.inter, self.hidden)),
                "down_proj.weight": TensorDecl((self.hidden, self.inter))}

    def load(self, tensors):
        g, u = tensors["gate_proj.weight"], tensors["up_proj.weight"]
        dt = torch.promote_types(g.dtype, u.dtype)
        self.gate_up = torch.cat([g.to(dt), u.to(dt)], dim=0).contiguous()
        self.down = tensors["down_proj.weight"].contiguous()

    def forward(self, x, ctx):
        return kernels.linear(kernels.linear_swiglu(x, self.gate_up), self.down)

    def forward_into(self, x, ctx, residual):
        # a few tokens (decode): the three matrices stream through one launch that ends in the residual add
        if kernels.mlp_fused_ok(x, self.gate_up, self.down, residual):
            kernels.mlp_fused(x, self.gate_up, self.down, residual)
            return True
        # more tokens: the down projection's tiles are added to the stream as they are finished
        if x.dtype == torch.bfloat16 and self.gate_up.dtype == torch.bfloat16 and x.shape[0] > 0:
            act = kernels.linear_swiglu(x, self.gate_up)
            if kernels.linear_into_ok(act, self.down, None, residual):
                kernels.linear_into(act, self.down, None, residual)
                return True
            kernels.residual_add(residual, kernels.linear(act, self.down))
            return True
        return False


@register_part("ffn", "gated_mlp")
class GatedMLP(FeedForward):
    """down(act(gate(x)) * up(x)) with the activation a parameter: "silu", "relu" or "gelu_tanh".  The gate
    and up matrices are kept as one [2I, H] matrix so that one product serves both; the activation and the product of
    the halves are one pass in float32.  With `bias` every projection has a bias (tensors named after the matrices with
    `bias_suffix`, default ".b").  The result is returned in float32 (it may be normed or scaled before it joins the
    stream).  params: hidden_size, intermediate_size, act, bias, bias_suffix, names (local tensor names of gate, up, down)."""
    capturable = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        p = spec.params
        self.hidden, self.inter, self.act = int(p["hidden_size"]), int(p["intermediate_size"]), str(p.get("act", "silu"))
        if self.act not in kernels.ops.GLU_ACTS:
            raise ValueError(f"unknown activation {self.act!r}; known: {sorted(kernels.ops.GLU_ACTS)}")
        self.names = dict({"gate": "gate_proj.weight", "up": "up_proj.weight", "down": "down_proj.weight"}, **(p.get("names") or {}))
        self.bias, self.bias_suffix = bool(p.get("bias", False)), str(p.get("bias_suffix", ".b"))
        self.gate_up = self.down = self.b_gate_up = self.b_down = None

    def tensors(self):
        n = self.names
        t = {n["gate"]: TensorDecl((self.inter, self.hidden)), n["up"]: TensorDecl((self.inter, self.hidden)),
             n["down"]: TensorDecl((self.hidden, self.inter))}
        if self.bias:
            t.update({n["gate"] + self.bias_suffix: TensorDecl((self.inter,), use="vector"),
                      n["up"] + self.bias_suffix: TensorDecl((self.inter,), use="vector"),
                      n["down"] + self.bias_suffix: TensorDecl((self.hidden,), use="vector")})
        return t

    def load(self, tensors):
        g, u = tensors[self.names["gate"]], tensors[self.names["up"]]
        dt = torch.promote_types(g.dtype, u.dtype)
        self.gate_up = torch.cat([g.to(dt), u.to(dt)], dim=0).contiguous()
        self.down = tensors[self.names["down"]].contiguous()
        if self.bias:
            b = self.bias_suffix
            self.b_gate_up = torch.cat([tensors[self.names["gate"] + b].float(), tensors[self.names["up"] + b].float()]).contiguous()
            self.b_down = tensors[self.names["down"] + b].float().contiguous()

    def forward(self, x, ctx):
        if self.act == "silu" and not self.bias:
            act = kernels.linear_swiglu(x, self.gate_up)
        else:
            act = kernels.glu(kernels.linear(x, self.gate_up, self.b_gate_up), self.act)
        return kernels.linear(act, self.down, self.b_down, out_dtype=delta_dtype(act))


def delta_dtype(x):
    """The dtype in which a part hands its output to a norm that follows it: float32 in both precisions, so that the
    norm reads the product unrounded (the product's accumulator is float32 anyway).  Measured with bfloat16 beyond 256
    tokens, which lets that product run on the paired-SM kernel: a twentieth of a prefill step gained, and the logits'
    distance from a float64 evaluation up by half for short prompts that share a step with long ones; not kept."""
    return torch.float32
