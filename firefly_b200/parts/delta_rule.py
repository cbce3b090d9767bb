"""A recurrent mixer that writes into its state the error of its own prediction (the gated delta rule), with a
decay per head and key channel:

    q, k = silu(conv(W_q x)), silu(conv(W_k x))   [kv_heads, dim];   v = silu(conv(W_v x))   [heads, vdim]
    q, k <- unit vectors per head (x / sqrt(sum x^2 + 1e-6)), q also times dim^(-1/2)
    beta = sigmoid(W_b x)  [heads];   g = exp(-exp(A_log_h) softplus(W_a2 (W_a1 x) + dt_bias))   [heads, dim]
    per head (head h reads q/k head floor(h / (heads / kv_heads))), S [dim, vdim] starting at 0:
        S <- diag(g) S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q
    out  = W_o (rms_norm(o over each head's vdim) * norm * sigmoid(W_g2 (W_g1 x)))        norm [vdim] shared by the heads

The request's state slot holds S of every head in 32-bit (in the kernel's own order) and the last conv-1 rows of
the q | k | v projection; a portion of a prompt continues from both.  Unit norms, beta, the decay with its softplus
and exponentials, S and every sum of the recurrence, the head norm and the gate are 32-bit; the projections and
the convolution's output are in the engine's type.  The two second-step projections are one product against a
block-diagonal matrix [a2 0; 0 g2] that writes 32-bit.  Kernels: ``csrc/delta_rule.cu``, the convolution of
``csrc/ssm.cu``.

Parameters: hidden_size, heads, kv_heads, dim, vdim, conv, decay_rank, gate_rank, eps.
Tensors (leaves under the prefix): q, k [kv_heads*dim, W]; v [heads*vdim, W]; q.conv, k.conv, v.conv [channels, conv];
b [heads, W]; a1 [decay_rank, W], a2 [heads*dim, decay_rank], dt_bias [heads*dim], A_log [heads];
g1 [gate_rank, W], g2 [heads*vdim, gate_rank]; norm [vdim]; o [W, heads*vdim].

Further parameters, for designs that differ from the above (defaults: as above):
    decay            "channel" | "head": with "head" a head has one decay, g = exp(-exp(A_log_h) softplus(a_h + dt_bias_h)),
                     dt_bias [heads] and the decay's projection has `heads` rows
    decay_rank, gate_rank   None (both): the decay and the gate are single projections, ``a`` [heads or heads*dim, W]
                     and ``g`` [heads*vdim, W], run as one product that writes 32-bit
    gate_activation  "sigmoid" | "silu": what the gate's projection passes through
    scales_residual: the output may enter a 32-bit sum times a constant (``forward(residual_scale=)``), so that the
                     mixer can stand beside another one (``parallel``)
The kind ``gated_delta`` is this mixer with decay "head", single projections and a SiLU gate.
"""
from __future__ import annotations

from typing import List, Mapping

import torch

from ..cache.spec import StateSpec
from ..ops import kernels as K
from ..weights.arena import FusedSpec, Piece
from ..weights.loader import WeightSpec
from .base import Part, register_part
from .linear import apply_linear, linear_into_residual, scaled_linear_into_residual


class ChannelDeltaMixer(Part):
    adds_into_residual = True        # forward(accumulate_into=...)
    folds_next_norm = True           # forward(then_norm=...)
    scales_residual = True           # forward(residual_scale=...)
    DEFAULTS = dict(decay="channel", gate_activation="sigmoid")

    def __init__(self, spec, rt, position=None):
        super().__init__(spec, rt)
        self.hidden = int(self.p("hidden_size"))
        self.H, self.G = int(self.p("heads")), int(self.p("kv_heads"))
        self.D, self.V = int(self.p("dim")), int(self.p("vdim"))
        self.taps = int(self.p("conv"))
        self.decay = str(self.p("decay", self.DEFAULTS["decay"]))
        self.gate_act = str(self.p("gate_activation", self.DEFAULTS["gate_activation"]))
        if self.decay not in ("channel", "head") or self.gate_act not in ("sigmoid", "silu"):
            raise ValueError(f"{self.prefix}: decay '{self.decay}' / gate activation '{self.gate_act}'")
        ra, rg = self.p("decay_rank", None), self.p("gate_rank", None)
        if (ra is None) != (rg is None):
            raise ValueError(f"{self.prefix}: decay_rank and gate_rank are given both or neither")
        self.two_step = ra is not None
        self.ra, self.rg = (int(ra), int(rg)) if self.two_step else (0, 0)
        self.eps = float(self.p("eps"))
        if self.H % self.G or not (1 <= self.taps <= 16):
            raise ValueError(f"{self.prefix}: {self.H} heads on {self.G} q/k heads, {self.taps} taps")
        self.GD, self.HV = self.G * self.D, self.H * self.V
        self.HD = self.H * self.D if self.decay == "channel" else self.H      # decay inputs a token
        self.C = 2 * self.GD + self.HV
        self.state_floats = K.delta_state_floats_plan(self.H, self.D, self.V)
        self.w_in = self.w_low1 = self.w_low2 = self.w_o = None
        self.conv_w = self.dt_bias = self.a_log = self.norm = None

    def cache_spec(self):
        return StateSpec((self.state_floats + (self.taps - 1) * self.C,), torch.float32)

    def _wide(self):
        n = self.name
        return [(n("q"), self.GD), (n("k"), self.GD), (n("v"), self.HV), (n("b"), self.H)]

    def _low(self):
        if not self.two_step:
            return [(self.name("a"), self.HD), (self.name("g"), self.HV)]
        return [(self.name("a1"), self.ra), (self.name("g1"), self.rg)]

    def weight_specs(self) -> List[WeightSpec]:
        n = self.name
        out = [WeightSpec(name, (rows, self.hidden)) for name, rows in self._wide() + self._low()]
        if self.two_step:
            out += [WeightSpec(n("a2"), (self.HD, self.ra)), WeightSpec(n("g2"), (self.HV, self.rg))]
        out += [WeightSpec(n("o"), (self.hidden, self.HV)),
                WeightSpec(n("q.conv"), (self.GD, self.taps), as_float32=True),
                WeightSpec(n("k.conv"), (self.GD, self.taps), as_float32=True),
                WeightSpec(n("v.conv"), (self.HV, self.taps), as_float32=True),
                WeightSpec(n("dt_bias"), (self.HD,), init="zeros", as_float32=True),
                WeightSpec(n("A_log"), (self.H,), init="zeros", as_float32=True),
                WeightSpec(n("norm"), (self.V,), init="norm", as_float32=True)]
        return out

    def fused_layout(self, dtype_of) -> List[FusedSpec]:
        out = []
        for fused, sources in (("qkvb", self._wide()), ("a1g1" if self.two_step else "ag", self._low())):
            pieces, at = [], 0
            for name, rows in sources:
                pieces.append(Piece(name, at))
                at += rows
            out.append(FusedSpec(self.name(fused), (at, self.hidden), tuple(pieces)))
        return out

    def _stacked(self, tensors, fused: str, sources) -> torch.Tensor:
        if self.name(fused) in tensors:
            return self._matrix(tensors[self.name(fused)])
        mats = [self._matrix(tensors[name]) for name, _ in sources]
        if len({m.dtype for m in mats}) != 1:
            mats = [m.to(torch.float32) for m in mats]
        return torch.cat(mats, dim=0).contiguous()

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        n = self.name
        self.w_in = self._stacked(tensors, "qkvb", self._wide())
        self.w_low1 = self._stacked(tensors, "a1g1" if self.two_step else "ag", self._low())
        if self.two_step:
            a2, g2 = self._matrix(tensors[n("a2")]), self._matrix(tensors[n("g2")])
            if a2.dtype != g2.dtype:
                a2, g2 = a2.to(torch.float32), g2.to(torch.float32)
            low2 = torch.zeros((self.HD + self.HV, self.ra + self.rg), dtype=a2.dtype, device=a2.device)
            low2[: self.HD, : self.ra] = a2
            low2[self.HD:, self.ra:] = g2
            self.w_low2 = low2
            if self.w_low2.dtype != self.w_low1.dtype:
                self.w_low1, self.w_low2 = self.w_low1.to(torch.float32), self.w_low2.to(torch.float32)
        self.w_o = self._matrix(tensors[n("o")])
        self.conv_w = torch.cat([self._vector32(tensors[n(leaf)]) for leaf in ("q.conv", "k.conv", "v.conv")], dim=0).contiguous()
        self.dt_bias, self.a_log = self._vector32(tensors[n("dt_bias")]), self._vector32(tensors[n("A_log")])
        self.norm = self._vector32(tensors[n("norm")])

    def forward(self, x, ctx, slot: int, write_cache: bool, accumulate_into=None, then_norm=None,
                residual_scale: float = 1.0):
        T, ws = x.shape[0], ctx.workspace
        dt = self.w_in.dtype
        if x.dtype != dt:
            raise K.KernelError(f"{self.prefix}: activations {x.dtype} against matrices {dt}")
        state = ctx.state(slot)
        proj = ws.get("delta.proj", (T, self.C + self.H), dt)
        apply_linear(x, self.w_in, proj, ctx, "delta.proj")
        ag = ws.get("delta.ag", (T, self.HD + self.HV), torch.float32)
        if self.two_step:
            low = ws.get("delta.low", (T, self.ra + self.rg), self.w_low1.dtype)
            apply_linear(x, self.w_low1, low, ctx, "delta.low")
            apply_linear(low, self.w_low2, ag, ctx, "delta.ag")
        else:
            apply_linear(x, self.w_low1, ag, ctx, "delta.ag")
        qkv = ws.get("delta.qkv", (T, self.C), dt)
        K.causal_conv(proj, 0, self.C, self.conv_w, None, state, self.state_floats, ctx, qkv, silu=True)
        o = ws.get("delta.o", (T, self.HV), torch.float32)
        K.delta_rule_scan((qkv, 0), (qkv, self.GD), (qkv, 2 * self.GD), (proj, self.C), (ag, 0), self.dt_bias, self.a_log,
                          state, 0, ctx, o, self.H, self.D, self.V, heads_per_group=self.H // self.G,
                          q_scale=float(self.D) ** -0.5, unit_eps=1e-6, decay_per_head=self.decay == "head")
        y = ws.get("delta.y", (T, self.HV), dt)
        K.head_norm_gate(o, (ag, self.HD), self.norm, self.eps, y, self.H, self.V, self.gate_act)
        if residual_scale != 1.0:
            return scaled_linear_into_residual(y, self.w_o, accumulate_into, residual_scale, ctx, "delta.out")
        return linear_into_residual(y, self.w_o, accumulate_into, ctx, "delta.out", then_norm)


class GatedDeltaMixer(ChannelDeltaMixer):
    """The delta rule with one decay per head, single projections for the decay and the gate, and a SiLU gate."""

    DEFAULTS = dict(decay="head", gate_activation="silu")


register_part("mixer", "channel_delta", ChannelDeltaMixer)
register_part("mixer", "gated_delta", GatedDeltaMixer)
