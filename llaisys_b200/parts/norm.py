from __future__ import annotations

from .. import kernels
from .base import Norm, TensorDecl, register_part


@register_part("norm", "rms_norm")
class RMSNorm(Norm):
    """y = x * w / sqrt(mean(x^2) + eps): eps inside the root, plain weight
    (xsmccc/llaisys src/ops/rms_norm/cpu/rms_norm_cpu.cpp:15-34), fused with the residual add
    that precedes it (src/models/qwen2/layer.hpp:60-71).  params: size, eps, tensor (the weight's local name, "weight" unless
    given; "" when the tensor carries the part's own name), offset (default 0: with an offset c the stored tensor is
    the weight's distance from c, y = x * (c + w) / ...; the sum is formed in float32 when the weights are loaded),
    scalar (default false: true when the stored weight is a single number for all coordinates; it is kept as a float32
    vector of `size` equal values).

    forward_scaled_add() is the same norm on a part's output on its way into the stream:
    residual += mult * norm(delta), and in the same pass the next norm of the new stream."""
    capturable = True


    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.size, self.eps = int(spec.params["size"]), float(spec.params["eps"])
        self.tensor = str(spec.params.get("tensor", "weight"))
        self.offset = float(spec.params.get("offset", 0.0))
        self.scalar = bool(spec.params.get("scalar", False))
        self.weight = None

    def tensors(self):
        return {self.tensor: TensorDecl(() if self.scalar else (self.size,), init="normal" if self.offset else "one_plus_normal",
                                        use="vector")}

    def load(self, tensors):
        w = tensors[self.tensor]
        if self.scalar:
            self.weight = (w.float().reshape(1) + self.offset).expand(self.size).contiguous()
            return
        # a weight stored as a distance from the offset: the sum would lose the stored bits in 16-bit arithmetic
        self.weight = (w.float() + self.offset).contiguous() if self.offset else w.contiguous()

    def forward(self, residual, delta=None, rows=None):
        return kernels.add_rmsnorm(residual, delta, self.weight, self.eps, self.env.dtype, rows=rows)

    def forward_scaled_add(self, residual, delta, mult, then=None):
        if then is not None and (then.kind != self.kind or then.eps != self.eps or then.weight.dtype != self.weight.dtype):
            raise ValueError("the norm that follows must be an RMS norm with the same eps")
        return kernels.scaled_norm_add(residual, delta, self.weight, float(mult), then.weight if then is not None else None,
                                       self.eps, 0.0, self.env.dtype)
