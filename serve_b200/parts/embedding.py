"""Token embedding and output head.

Embedding: a row gather (serve/model.py:157,220), written into the float32
residual stream. Head: logits = x W^T without bias (model.py:159,227,231), in
float32. A tied head uses the embedding's table (the reference copies it at
conversion, serve/hf_utils/convert_hf_checkpoint.py:146-147).
"""
from __future__ import annotations

import torch

from .base import Part, TensorDecl, register_part


@register_part("embedding", "table")
class TokenEmbedding(Part):
    """params: vocab, hidden, name."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.vocab = int(spec.params["vocab"])
        self.hidden = int(spec.params["hidden"])
        self.name = self.prefix + spec.params.get("name", "weight")
        self.table = None

    def tensor_decls(self):
        return [TensorDecl(self.name, (self.vocab, self.hidden))]

    def load(self, tensors):
        self.table = tensors[self.name]

    def forward(self, tokens, ctx):
        x = torch.empty((tokens.shape[0], self.hidden), dtype=torch.float32, device=self.rt.device)
        self.rt.kernels.embedding(tokens, self.table, x, getattr(ctx, "last_token", None))
        return x


@register_part("head", "linear")
class OutputHead(Part):
    """params: vocab, hidden, name; tied_to: name of the embedding table, or None."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.vocab = int(spec.params["vocab"])
        self.hidden = int(spec.params["hidden"])
        self.tied_to = spec.params.get("tied_to")
        self.own_name = self.prefix + spec.params.get("name", "weight")
        self.name = self.tied_to if self.tied_to else self.own_name
        self.weight = None

    def tensor_decls(self):
        return [TensorDecl(self.name, (self.vocab, self.hidden))]

    def ignorable_tensors(self):
        return [self.own_name] if self.tied_to else []

    def load(self, tensors):
        self.weight = tensors[self.name]

    def forward(self, h, ctx):
        logits = torch.empty((h.shape[0], self.vocab), dtype=torch.float32, device=self.rt.device)
        self.rt.kernels.linear(h, self.weight, logits)
        return logits
