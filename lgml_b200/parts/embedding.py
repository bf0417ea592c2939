"""Token embedding and the output head.

``x = get_rows(tok_embd, ids)`` with no scale (``lua/lgml/transformer.lua:2303-2306``);
``logits = output . norm(x)`` in float32 (``:2095-2096``, ``:2610``); the head falls
back to the embedding when the folder has no head of its own (``:408``).
"""
from __future__ import annotations

import torch

from .. import ops
from ..weights import MATRIX, TensorSpec
from .base import Part


class TokenEmbedding(Part):
    graph_safe = True
    def __init__(self, vocab: int, width: int, name: str = "model.embed_tokens.weight"):
        self.vocab, self.width, self.name = vocab, width, name
        self.table = None

    def tensor_specs(self, prefix=""):
        return [TensorSpec(self.name, (self.vocab, self.width), MATRIX)]

    def bind(self, prefix, tensors, rt):
        self.table = tensors[self.name]

    def forward(self, rt, token_ids):
        out = torch.empty((token_ids.numel(), self.width), dtype=torch.float32, device=token_ids.device)
        return ops.embed_rows(self.table, token_ids, out, rt.status)


class LMHead(Part):
    graph_safe = True
    def __init__(self, vocab: int, width: int, tied_to: TokenEmbedding = None, name: str = "lm_head.weight"):
        self.vocab, self.width, self.tied_to, self.name = vocab, width, tied_to, name
        self.weight = None

    def tensor_specs(self, prefix=""):
        # tied: the head's own tensor is optional and wins when the folder has it, as the
        # reference takes ``output.weight`` whenever it is there (``lua/lgml/transformer.lua:408``)
        return [TensorSpec(self.name, (self.vocab, self.width), MATRIX, optional=self.tied_to is not None)]

    def bind(self, prefix, tensors, rt):
        own = tensors.get(self.name)
        self.weight = own if own is not None or self.tied_to is None else self.tied_to.table
        if self.weight is None:
            raise KeyError(self.name)

    def forward(self, rt, h):
        """h [rows, width] in the compute type -> float32 logits [rows, vocab]."""
        return rt.linear(h, self.weight, out_dtype=torch.float32)
