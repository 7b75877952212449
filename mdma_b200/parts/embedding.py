"""Token embedding (x[t,:] = table[ids[t],:], src/backend/cpu.rs:370-384; times `scale` where an
architecture sets one) and
the output head (logits = h W^T over the wanted rows only,
src/model.rs:370-373, 462-467).  A tied head names the embedding's tensor."""
from __future__ import annotations

from .. import ops
from ..registry import EMBEDDINGS, HEADS
from ..spec import TensorSpec
from .base import Part
from .linear import Linear


@EMBEDDINGS.register("embedding")
class Embedding(Part):
    def __init__(self, spec):
        super().__init__(spec)
        self.vocab, self.width = int(self.params["vocab_size"]), int(self.params["width"])
        self.scale = float(self.params.get("scale", 1.0))      # the rows are multiplied by it, in float

    def tensor_specs(self):
        return {"weight": TensorSpec((self.vocab, self.width))}

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.weight = tensors["weight"]

    def forward(self, ctx, ids, x):
        ops.embed_rows(self.weight, ids, x, self.scale)

    def resident_tensors(self):
        return [self.weight]


@HEADS.register("lm_head")
class LMHead(Part):
    def __init__(self, spec):
        super().__init__(spec)
        self.vocab, self.width = int(self.params["vocab_size"]), int(self.params["width"])
        # `softcap` c: logits <- c * tanh(logits / c); None or 0: none
        self.softcap = float(self.params.get("softcap") or 0.0)
        if self.softcap < 0:
            raise ValueError("the logits' soft cap must be positive")

    def tensor_specs(self):
        return {"weight": TensorSpec((self.vocab, self.width))}

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.proj = Linear(tensors["weight"], rt)

    def forward(self, ctx, h_rows, logits, n_rows):
        self.proj.store(h_rows, logits, n_rows)
        if self.softcap:
            if not logits.is_contiguous():
                raise ops.KernelError("the soft cap takes contiguous logit rows")
            ops.softcap(logits, n_rows, self.softcap)

    def resident_tensors(self):
        return [self.proj.w]
