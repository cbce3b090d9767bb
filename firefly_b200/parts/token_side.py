"""A per-layer input from the token itself, added to the stream at the end of a block (category ``tail``).

A table holds, for every token id, a row of ``table_cols`` numbers; this part reads ``dim`` of them from column
``col0`` on (a model gives each layer its own slice of one table):

    e = table[token][col0 : col0 + dim];   g = act(W_gate x) * e;   y = W_proj g;   x <- x + rms(y) * norm

with x the stream behind the block's feed-forward, act the tanh form of GELU (or SiLU), rms(y) = y / sqrt(mean(y^2) +
eps) and ``norm`` a plain weight.  The stream, the norm and the sum are 32-bit; the two products run in the engine's
type on a copy of the stream in that type, the second one writes 32-bit.

Parameters: hidden_size, dim, vocab_size, table (the table's full tensor name), table_cols, col0, eps, activation
("gelu_tanh"), gate_leaf ("gate"), proj_leaf ("proj"), norm_leaf ("norm").
"""
from __future__ import annotations

from typing import List, Mapping

import torch

from ..ops import kernels as K
from ..weights.loader import WeightSpec
from .base import Part, register_part
from .linear import apply_linear
from .norm import FoldedNorm


class TokenSide(Part):
    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.hidden = int(self.p("hidden_size"))
        self.dim = int(self.p("dim"))
        self.vocab = int(self.p("vocab_size"))
        self.table_name = str(self.p("table"))
        self.table_cols = int(self.p("table_cols", self.dim))
        self.col0 = int(self.p("col0", 0))
        self.eps = float(self.p("eps"))
        self.activation = str(self.p("activation", "gelu_tanh"))
        self.leaves = tuple(self.p(k, d) for k, d in (("gate_leaf", "gate"), ("proj_leaf", "proj"), ("norm_leaf", "norm")))
        if self.activation not in ("gelu_tanh", "silu"):
            raise ValueError(f"{self.prefix}: activation '{self.activation}' is not 'gelu_tanh' or 'silu'")
        if self.dim <= 0 or self.col0 < 0 or self.col0 + self.dim > self.table_cols:
            raise ValueError(f"{self.prefix}: columns {self.col0}..{self.col0 + self.dim} do not fit a table of {self.table_cols}")
        self.table = self.w_gate = self.w_proj = self.norm = None

    def weight_specs(self) -> List[WeightSpec]:
        g, p, n = (self.name(leaf) for leaf in self.leaves)
        return [WeightSpec(self.table_name, (self.vocab, self.table_cols)),
                WeightSpec(g, (self.dim, self.hidden)), WeightSpec(p, (self.hidden, self.dim)),
                WeightSpec(n, (self.hidden,), init="norm", as_float32=True)]

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        g, p, n = (self.name(leaf) for leaf in self.leaves)
        self.table = self._matrix(tensors[self.table_name])
        self.w_gate, self.w_proj = self._matrix(tensors[g]), self._matrix(tensors[p])
        if len({self.table.dtype, self.w_gate.dtype, self.w_proj.dtype}) != 1:
            self.table, self.w_gate, self.w_proj = (t.to(torch.float32) for t in (self.table, self.w_gate, self.w_proj))
        self.norm = self._vector32(tensors[n])

    def forward(self, residual: torch.Tensor, pending, ctx):
        if pending is not None and not isinstance(pending, FoldedNorm):
            K.residual_add(residual, pending)
        T, ws, dt = residual.shape[0], ctx.workspace, self.w_gate.dtype
        x = residual
        if dt != torch.float32:
            x = ws.get("side.x", (T, self.hidden), dt)
            K.cast(residual, x)
        gate = ws.get("side.gate", (T, self.dim), dt)
        apply_linear(x, self.w_gate, gate, ctx, "side.gate")
        g = ws.get("side.g", (T, self.dim), dt)
        K.act_mul_table_rows(gate, ctx.token_ids, self.table, self.col0, g, self.activation, ctx.status)
        y = ws.get("side.y", (T, self.hidden), torch.float32)
        apply_linear(g, self.w_proj, y, ctx, "side.y")
        K.norm_add(residual, y, self.norm, self.eps)
        return residual, None


register_part("tail", "token_side", TokenSide)
