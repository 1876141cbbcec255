"""Token embedding and the output head.

Embedding: x[t] = E[id_t], ids outside the table read row 0, no scale (src/model.c:6148-6162).
Head: logits = W_out . norm(x) at the wanted rows; when the model ties its head to the embedding
the same tensor serves both (src/model.c:2353-2354).
"""
from __future__ import annotations

import torch

from .. import kernels
from ..weights.loader import TensorSpec
from .base import Part
from .linear import Linear


class Embedding(Part):
    graph_safe = True
    def __init__(self, vocab: int, width: int, name: str):
        self.vocab, self.width, self.name = vocab, width, name
        self.table = None

    def tensors(self):
        return {self.name: TensorSpec((self.vocab, self.width), kind="matrix")}

    def bind(self, tensors, rt):
        self.table = tensors[self.name]

    def forward(self, ctx, ids: torch.Tensor, x: torch.Tensor) -> None:
        # ids below zero stand for tokens an earlier step left on the device (the step context's `token_feed`)
        kernels.embed(self.table, ids, x, getattr(ctx, "token_feed", None))


class Head(Part):
    graph_safe = True
    """`tied_to` set: no tensor of its own, multiplies by the embedding table."""

    def __init__(self, vocab: int, width: int, name: str = None, tied_to: Embedding = None):
        assert (name is None) != (tied_to is None)
        self.vocab, self.width, self.name, self.tied_to = vocab, width, name, tied_to
        self.linear = None

    def tensors(self):
        return {} if self.tied_to is not None else {self.name: TensorSpec((self.vocab, self.width), kind="matrix")}

    def bind(self, tensors, rt):
        # a tied head multiplies by the embedding table; the gather keeps reading the table as stored
        self.linear = Linear(self.tied_to.table if self.tied_to is not None else tensors[self.name]).prepare(
            rt, keep_plain=self.tied_to is not None)

    def weight_bytes(self):
        return self.linear.nbytes()

    def forward(self, ctx, h: torch.Tensor, logits: torch.Tensor) -> None:
        self.linear.forward(h, logits)
