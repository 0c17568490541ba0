from __future__ import annotations

from .. import kernels
from .base import Part, TensorDecl, register_part


@register_part("embedding", "token_embedding")
class TokenEmbedding(Part):
    """x[t] = E[id[t]] (xsmccc/llaisys src/ops/embedding/cpu/embedding_cpu.cpp:16-22), written
    as the float32 residual stream.  An id outside the table is reported through ctx.err.
    params: vocab_size, hidden_size."""
    capturable = True


    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.vocab, self.hidden = int(spec.params["vocab_size"]), int(spec.params["hidden_size"])
        self.weight = None

    def tensors(self):
        return {"weight": TensorDecl((self.vocab, self.hidden))}

    def load(self, tensors):
        self.weight = tensors["weight"].contiguous()

    def forward(self, ctx):
        return kernels.embedding(ctx.tokens, self.weight, ctx.err)


@register_part("embedding", "scaled_pair_embedding")
class ScaledPairEmbedding(Part):
    """x[t] = E[id[t]] * scale + P[r[t]]: the token's row, scaled, plus a row of a second table that the token and
    the one before it in its sequence choose together: r = (id[t-1] * mul_prev + id[t] * mul_cur) mod buckets, and
    row `buckets` (the table's last) for a sequence's first token.  The token before a step's first one is carried
    from step to step on the device (two int32 per cache slot: the token and its position), so a step whose tokens
    are themselves taken from the device needs nothing from the host.  Without `pair` the part is a scaled embedding.
    params: vocab_size, hidden_size, scale, tensor, pair = {tensor, buckets, mul_prev, mul_cur} or None."""
    capturable = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        p = spec.params
        self.vocab, self.hidden, self.scale = int(p["vocab_size"]), int(p["hidden_size"]), float(p.get("scale", 1.0))
        self.tensor = str(p.get("tensor", "weight"))
        self.pair = dict(p["pair"]) if p.get("pair") else None
        if self.pair:
            self.buckets, self.mul_prev, self.mul_cur = (int(self.pair[k]) for k in ("buckets", "mul_prev", "mul_cur"))
            if self.buckets <= 0:
                raise ValueError(f"the pair table needs a positive number of buckets, got {self.buckets}")
        self.weight = self.pair_weight = None

    def token_state_ints(self) -> int:
        """int32 values per cache slot that the part carries from step to step."""
        return 2 if self.pair else 0

    def tensors(self):
        t = {self.tensor: TensorDecl((self.vocab, self.hidden))}
        if self.pair:
            t[self.pair["tensor"]] = TensorDecl((self.buckets + 1, self.hidden))
        return t

    def load(self, tensors):
        self.weight = tensors[self.tensor].contiguous()
        if self.pair:
            self.pair_weight = tensors[self.pair["tensor"]].to(self.weight.dtype).contiguous()

    def forward(self, ctx):
        if not self.pair:
            return kernels.embedding_pair(ctx, self.weight, self.scale)
        return kernels.embedding_pair(ctx, self.weight, self.scale, self.pair_weight, self.buckets, self.mul_prev,
                                      self.mul_cur, ctx.token_state())


@register_part("head", "lm_head")
class LMHead(Part):
    """logits = h W^T in float32, no bias (xsmccc/llaisys src/models/qwen2/qwen2.cpp:76-77).
    With params["tied_to"] set, W is the tensor of that name (the embedding table) and the part
    declares no tensor of its own.  params: vocab_size, hidden_size, tied_to, tensor (the matrix's local name,
    "weight" unless given), scale (default 1: the float32 logits are multiplied by it)."""
    capturable = True


    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.vocab, self.hidden = int(spec.params["vocab_size"]), int(spec.params["hidden_size"])
        self.tied_to = spec.params.get("tied_to")
        self.tensor = str(spec.params.get("tensor", "weight"))
        self.scale = float(spec.params.get("scale", 1.0))
        self.weight = None

    def tensors(self):
        return {} if self.tied_to else {self.tensor: TensorDecl((self.vocab, self.hidden))}

    def load(self, tensors):
        if not self.tied_to:
            self.weight = tensors[self.tensor].contiguous()

    def tie(self, weight):
        self.weight = weight

    def forward(self, h):
        import torch
        logits = kernels.linear(h, self.weight, out_dtype=torch.float32)
        return kernels.scale_(logits, self.scale) if self.scale != 1.0 else logits
