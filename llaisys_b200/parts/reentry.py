from __future__ import annotations

import torch

from .base import Part, TensorDecl, register_part


@register_part("reentry", "embedding_and_offset")
class EmbeddingAndOffset(Part):
    """What a pass over a repeated run of layers starts with: before pass t (0, 1, ...) the row t of a table of offsets
    [passes, H] is added to every token's stream, and before every pass but the first also the embedding's output as it
    was before the first layer.  The model asks for a copy of that output once a step (`remember`), and for the add where
    an entry of the run order opens a pass (`forward`); the add is left pending and runs in the next norm's pass over the
    stream.  params: hidden_size, passes, tensor (the table's name)."""
    capturable = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.hidden, self.passes = int(spec.params["hidden_size"]), int(spec.params["passes"])
        self.tensor = str(spec.params.get("tensor", "offset"))
        self.offsets = None

    def tensors(self):
        return {self.tensor: TensorDecl((self.passes, self.hidden), use="vector")}

    def load(self, tensors):
        self.offsets = tensors[self.tensor].float().contiguous()

    def remember(self, residual):
        """A copy of the embedding's output (the stream is changed in place by the layers); None when no pass needs it."""
        return residual.clone() if self.passes > 1 else None

    def forward(self, residual, pending, first, t: int):
        from .block import PendingGated, settle
        if not (0 <= t < self.passes):
            raise ValueError(f"pass {t} of {self.passes}")
        if pending is not None:
            if isinstance(pending, PendingGated) and pending.rows_add is None and pending.vec_add is None:
                # the part before it has not joined the stream yet: both adds go into the same pass over the rows
                pending.rows_add, pending.vec_add = (first if t > 0 else None), self.offsets[t]
                return residual, pending
            settle(residual, pending)
        return residual, PendingGated(rows_add=first if t > 0 else None, vec_add=self.offsets[t])
