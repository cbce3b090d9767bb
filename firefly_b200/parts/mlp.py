"""SwiGLU feed-forward: (silu(x Wg^T) * (x Wu^T)) Wd^T, silu(g) = g / (1 + exp(-g))
in 32-bit (src/model/qwen_model.cu:164-174, src/kernels/activation.cu:15-19 of the
reference, which runs gate and up as two products and the activation as a third
launch).  Gate and up are one product against the stacked matrix [2I, H].

Parameters: hidden_size, intermediate_size.
"""
from __future__ import annotations

from typing import List, Mapping

import torch

from ..ops import kernels as K
from ..weights.arena import FusedSpec, Piece
from ..weights.loader import WeightSpec
from .base import Part, register_part
from .linear import apply_linear, linear_into_residual, linear_swiglu


class SwiGLUMLP(Part):
    adds_into_residual = True        # forward(accumulate_into=...)
    folds_next_norm = True           # forward(then_norm=...)
    accepts_folded_norm = True       # its first operation is a product that can finish a folded norm

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.hidden = int(self.p("hidden_size"))
        self.inter = int(self.p("intermediate_size"))
        self.w_gate_up = self.w_down = None
        self.interleaved = False

    def weight_specs(self) -> List[WeightSpec]:
        return [WeightSpec(self.name("gate_proj.weight"), (self.inter, self.hidden)),
                WeightSpec(self.name("up_proj.weight"), (self.inter, self.hidden)),
                WeightSpec(self.name("down_proj.weight"), (self.hidden, self.inter))]

    def _interleaves(self, gate_dtype, up_dtype) -> bool:
        """bfloat16: rows of gate and up alternate in groups of 16, the layout the fused product's
        epilogue pairs up; else gate rows first, then up rows."""
        return gate_dtype == up_dtype == torch.bfloat16 and self.rt.dtype == torch.bfloat16 and self.inter % 16 == 0

    def fused_layout(self, dtype_of) -> List[FusedSpec]:
        g, u = self.name("gate_proj.weight"), self.name("up_proj.weight")
        if self._interleaves(dtype_of(g), dtype_of(u)):
            pieces = (Piece(g, 0, 16, 32), Piece(u, 16, 16, 32))
        else:
            pieces = (Piece(g, 0), Piece(u, self.inter))
        return [FusedSpec(self.name("gate_up_proj.weight"), (2 * self.inter, self.hidden), pieces)]

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        fused = self.name("gate_up_proj.weight")
        if fused in tensors:
            self.w_gate_up = self._matrix(tensors[fused])
            self.interleaved = self._interleaves(self.w_gate_up.dtype, self.w_gate_up.dtype)
        else:
            g = self._matrix(tensors[self.name("gate_proj.weight")])
            u = self._matrix(tensors[self.name("up_proj.weight")])
            if g.dtype != u.dtype:
                g, u = g.to(torch.float32), u.to(torch.float32)
            self.interleaved = self._interleaves(g.dtype, u.dtype)
            self.w_gate_up = K.interleave_gate_up(g, u) if self.interleaved else torch.cat([g, u], dim=0).contiguous()
        self.w_down = self._matrix(tensors[self.name("down_proj.weight")])

    def forward(self, x, ctx, accumulate_into=None, then_norm=None):
        """Returns the delta [T, hidden]; or None when it was added into ``accumulate_into`` (the
        32-bit residual) by the last product's epilogue; or a FoldedNorm when that epilogue also
        prepared the norm that follows (``then_norm``)."""
        act = linear_swiglu(x, self.w_gate_up, self.inter, self.interleaved, ctx)
        return linear_into_residual(act, self.w_down, accumulate_into, ctx, "mlp.down", then_norm)


class GatedMLP(Part):
    """W_down (act(W_gate x) * (W_up x)) with the activation as a parameter ("silu", "gelu_tanh", or
    "clamped_swish": min(g, limit) * sigmoid(1.702 min(g, limit)) * (clamp(u, -limit, limit) + 1)) and the
    tensors' leaves under the prefix as parameters (``gate_leaf``, ``up_leaf``, ``down_leaf``).  Gate and up are one
    product against the stacked matrix [gate rows | up rows]; the activation is a kernel of its own.  With
    ``bias`` every projection has a bias (leaf + ``bias_suffix``), added in 32-bit: gate's and up's where the
    activation reads them, down's into the 32-bit stream.  With SiLU and no biases it is the SwiGLU feed-forward under
    other tensor names, and runs as that one does: in bfloat16 the stacked matrix interleaves gate and up rows in groups
    of 16 and steps of few tokens take the activation in the product's epilogue.

    Parameters: hidden_size, intermediate_size, activation, limit, bias, bias_suffix."""

    adds_into_residual = True        # forward(accumulate_into=...)

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.hidden = int(self.p("hidden_size"))
        self.inter = int(self.p("intermediate_size"))
        self.activation = str(self.p("activation", "silu"))
        if self.activation not in K.GLU_ACTIVATIONS:
            raise ValueError(f"{self.prefix}: activation '{self.activation}' is not one of {sorted(K.GLU_ACTIVATIONS)}")
        self.leaves = tuple(self.p(k, d) for k, d in (("gate_leaf", "gate"), ("up_leaf", "up"), ("down_leaf", "down")))
        self.limit = float(self.p("limit", 0.0))
        self.has_bias = bool(self.p("bias", False))
        self.bias_suffix = str(self.p("bias_suffix", ".b"))
        if self.activation == "clamped_swish" and not (self.limit > 0):
            raise ValueError(f"{self.prefix}: the clamped activation needs a positive limit")
        self.w_gate_up = self.w_down = self.b_gate_up = self.b_down = None
        self.swiglu = self.activation == "silu" and not self.has_bias      # the fused SwiGLU path serves it
        self.interleaved = False

    def _interleaves(self, gate_dtype, up_dtype) -> bool:
        return self.swiglu and gate_dtype == up_dtype == torch.bfloat16 and self.rt.dtype == torch.bfloat16 \
            and self.inter % 16 == 0

    def weight_specs(self) -> List[WeightSpec]:
        g, u, d = (self.name(leaf) for leaf in self.leaves)
        out = [WeightSpec(g, (self.inter, self.hidden)), WeightSpec(u, (self.inter, self.hidden)),
               WeightSpec(d, (self.hidden, self.inter))]
        if self.has_bias:
            sfx = self.bias_suffix
            out += [WeightSpec(g + sfx, (self.inter,), init="zeros", as_float32=True),
                    WeightSpec(u + sfx, (self.inter,), init="zeros", as_float32=True),
                    WeightSpec(d + sfx, (self.hidden,), init="zeros", as_float32=True)]
        return out

    def fused_layout(self, dtype_of) -> List[FusedSpec]:
        g, u, _ = (self.name(leaf) for leaf in self.leaves)
        if self._interleaves(dtype_of(g), dtype_of(u)):
            pieces = (Piece(g, 0, 16, 32), Piece(u, 16, 16, 32))
        else:
            pieces = (Piece(g, 0), Piece(u, self.inter))
        return [FusedSpec(self.name("gate_up"), (2 * self.inter, self.hidden), pieces)]

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        g, u, d = (self.name(leaf) for leaf in self.leaves)
        if self.name("gate_up") in tensors:
            self.w_gate_up = self._matrix(tensors[self.name("gate_up")])
            self.interleaved = self._interleaves(self.w_gate_up.dtype, self.w_gate_up.dtype)
        else:
            a, b = self._matrix(tensors[g]), self._matrix(tensors[u])
            if a.dtype != b.dtype:
                a, b = a.to(torch.float32), b.to(torch.float32)
            self.interleaved = self._interleaves(a.dtype, b.dtype)
            self.w_gate_up = K.interleave_gate_up(a, b) if self.interleaved else torch.cat([a, b], dim=0).contiguous()
        self.w_down = self._matrix(tensors[d])
        if self.has_bias:
            sfx = self.bias_suffix
            self.b_gate_up = torch.cat([self._vector32(tensors[g + sfx]), self._vector32(tensors[u + sfx])]).contiguous()
            self.b_down = self._vector32(tensors[d + sfx])

    def forward(self, x, ctx, accumulate_into=None):
        T = x.shape[0]
        if self.swiglu:
            act = linear_swiglu(x, self.w_gate_up, self.inter, self.interleaved, ctx)
            return linear_into_residual(act, self.w_down, accumulate_into, ctx, "mlp.down")
        gu = ctx.workspace.get("mlp.gate_up", (T, 2 * self.inter), ctx.dtype)
        apply_linear(x, self.w_gate_up, gu, ctx, "mlp.gate_up")
        act = ctx.workspace.get("mlp.act", (T, self.inter), ctx.dtype)
        K.glu_act(gu, act, self.activation, self.b_gate_up, self.limit)
        left = linear_into_residual(act, self.w_down, accumulate_into, ctx, "mlp.down")
        if not self.has_bias:
            return left
        if left is None:                         # the product went into the 32-bit stream: so does its bias
            K.add_row_vector(accumulate_into, self.b_down)
            return None
        if left.dtype != torch.float32:          # a delta in the engine's type: widened, so that the bias is not rounded
            wide = ctx.workspace.get("mlp.down.f32", tuple(left.shape), torch.float32)
            K.cast(left, wide)
            left = wide
        K.add_row_vector(left, self.b_down)
        return left


register_part("feed_forward", "swiglu_mlp", SwiGLUMLP)
register_part("feed_forward", "gated_mlp", GatedMLP)
