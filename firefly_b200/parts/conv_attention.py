"""Grouped-query softmax attention whose projections pass a short causal convolution, with a norm over the whole
projection, a bias by distance inside a sliding window, values blended across layers and a sigmoid output gate:

    q, k, v = conv(W_q x), conv(W_k x), conv(W_v x)      per channel, `conv` taps, no bias, zeros in front of the sequence
    q, k    = rms_norm(q) * q.norm, rms_norm(k) * k.norm  each over its whole projection (all heads at once)
    v       = (1 - f) v + f v_first                        in layers that blend (f = `vmix`; v_first: the values, behind
                                                           their convolution, of the first such layer for the same token)
    s_ij    = q_i . k_j * scale - r1_h ln(1 + r2_h (i - j))      for 0 <= i - j < window; softmax over those keys
    out     = W_o (heads * sigmoid(W_g x))

No rotation: positions enter only through the bias and the window.  Query head h reads key/value head
floor(h / (heads / kv_heads)).  The blended v is what the cache holds.  The request's state slot holds the last
conv-1 rows of the q | k | v projection; keys and values lie in the paged cache, whose heads have
d = max(dim, vdim) elements rounded up to 16 (the shorter kind is filled up with zeros).  The convolution, the
norms, the blend, scores and softmax are 32-bit.  The bias is a table [heads, window] made once in 64-bit.
Kernels: ``csrc/conv_attention.cu`` and the paged attention kernels.

Parameters: hidden_size, heads, kv_heads, dim, vdim, conv, scale, window, eps, distance_bias (bool),
value_mix (None | "first" | "blend") and value_key (the name under which a step keeps the first layer's values).
Tensors (leaves under the prefix): q, k, v, g, o; q.conv, k.conv, v.conv; q.norm, k.norm; r1, r2 [heads]; vmix [].
"""
from __future__ import annotations

from typing import List, Mapping

import torch

from ..cache.spec import PagedKVSpec, StateSpec, sub_slot
from ..ops import kernels as K
from ..weights.arena import FusedSpec, Piece
from ..weights.loader import WeightSpec
from .base import Part, register_part
from .linear import apply_linear, linear_into_residual


class ConvGatedAttention(Part):
    adds_into_residual = True        # forward(accumulate_into=...)
    folds_next_norm = True           # forward(then_norm=...)

    def __init__(self, spec, rt, position=None):
        super().__init__(spec, rt)
        self.hidden = int(self.p("hidden_size"))
        self.H, self.G = int(self.p("heads")), int(self.p("kv_heads"))
        self.dk, self.dv = int(self.p("dim")), int(self.p("vdim"))
        self.taps = int(self.p("conv"))
        self.scale = float(self.p("scale"))
        self.window = int(self.p("window"))
        self.eps = float(self.p("eps"))
        self.has_bias = bool(self.p("distance_bias", True))
        self.value_mix = self.p("value_mix", None)
        self.value_key = str(self.p("value_key", "values"))
        if self.H % self.G or self.window <= 0 or not (1 <= self.taps <= 16):
            raise ValueError(f"{self.prefix}: {self.H} heads on {self.G} kv heads, window {self.window}, {self.taps} taps")
        if self.value_mix not in (None, "first", "blend"):
            raise ValueError(f"{self.prefix}: value_mix must be None, 'first' or 'blend'")
        self.d = -(-max(self.dk, self.dv) // 16) * 16
        if self.d > 256:
            raise ValueError(f"{self.prefix}: head size {self.d} > 256 is not supported by the attention kernels")
        self.Cq, self.Ck, self.Cv = self.H * self.dk, self.G * self.dk, self.G * self.dv
        self.C = self.Cq + self.Ck + self.Cv
        self.w_in = self.w_o = self.conv_w = self.conv_w_t = self.q_norm = self.k_norm = self.bias_table = self.mix_factor = None

    def cache_spec(self):
        return (PagedKVSpec(self.G, self.d, self.window),
                StateSpec((max(1, (self.taps - 1) * self.C),), torch.float32))

    def _sources(self):
        n = self.name
        return [(n("q"), self.Cq), (n("k"), self.Ck), (n("v"), self.Cv), (n("g"), self.H * self.dv)]

    def weight_specs(self) -> List[WeightSpec]:
        n = self.name
        out = [WeightSpec(name, (rows, self.hidden)) for name, rows in self._sources()]
        out += [WeightSpec(n("o"), (self.hidden, self.H * self.dv)),
                WeightSpec(n("q.conv"), (self.Cq, self.taps), as_float32=True),
                WeightSpec(n("k.conv"), (self.Ck, self.taps), as_float32=True),
                WeightSpec(n("v.conv"), (self.Cv, self.taps), as_float32=True),
                WeightSpec(n("q.norm"), (self.Cq,), init="norm", as_float32=True),
                WeightSpec(n("k.norm"), (self.Ck,), init="norm", as_float32=True),
                WeightSpec(n("vmix"), (), init="zeros", as_float32=True, optional=self.value_mix != "blend")]
        if self.has_bias:
            out += [WeightSpec(n("r1"), (self.H,), init="norm", as_float32=True),
                    WeightSpec(n("r2"), (self.H,), init="norm", as_float32=True)]
        return out

    def fused_layout(self, dtype_of) -> List[FusedSpec]:
        pieces, at = [], 0
        for name, rows in self._sources():
            pieces.append(Piece(name, at))
            at += rows
        return [FusedSpec(self.name("qkvg"), (at, self.hidden), tuple(pieces))]

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        n = self.name
        if n("qkvg") in tensors:
            self.w_in = self._matrix(tensors[n("qkvg")])
        else:
            mats = [self._matrix(tensors[name]) for name, _ in self._sources()]
            if len({m.dtype for m in mats}) != 1:
                mats = [m.to(torch.float32) for m in mats]
            self.w_in = torch.cat(mats, dim=0).contiguous()
        self.w_o = self._matrix(tensors[n("o")])
        self.conv_w = torch.cat([self._vector32(tensors[n(leaf)]) for leaf in ("q.conv", "k.conv", "v.conv")], dim=0).contiguous()
        self.conv_w_t = self.conv_w.t().contiguous()            # [taps, C]: what the kernel for sizes in steps of 8 reads
        self.q_norm, self.k_norm = self._vector32(tensors[n("q.norm")]), self._vector32(tensors[n("k.norm")])
        if self.value_mix == "blend":
            self.mix_factor = self._vector32(tensors[n("vmix")]).reshape(1)
        if self.has_bias:
            # b[h, dist] = r1_h ln(1 + r2_h dist) for the distances a window lets through, formed once in 64-bit
            r1 = tensors[n("r1")].to(torch.float64).view(-1, 1)
            r2 = tensors[n("r2")].to(torch.float64).view(-1, 1)
            dist = torch.arange(self.window, dtype=torch.float64, device=r1.device).view(1, -1)
            self.bias_table = (r1 * torch.log1p(r2 * dist)).to(torch.float32).contiguous()

    def forward(self, x, ctx, slot: int, write_cache: bool, accumulate_into=None, then_norm=None):
        if not write_cache:
            raise RuntimeError(f"{self.prefix}: this mixer always writes its own cache")
        T, ws = x.shape[0], ctx.workspace
        dt = self.w_in.dtype
        if x.dtype != dt:
            raise K.KernelError(f"{self.prefix}: activations {x.dtype} against matrices {dt}")
        proj = ws.get("cattn.proj", (T, self.C + self.H * self.dv), dt)
        apply_linear(x, self.w_in, proj, ctx, "cattn.proj")
        pages, table = ctx.kv(sub_slot(slot, 0))
        state = ctx.state(sub_slot(slot, 1))
        mix, shared = 0, None
        if self.value_mix is not None:
            key = ("shared_values", self.value_key)
            if self.value_mix == "first":
                shared = ctx.memo[key] = ws.get("cattn.values." + self.value_key, (T, self.Cv), torch.float32)
                mix = 1
            else:
                shared = ctx.memo.get(key)
                if shared is None or tuple(shared.shape) != (T, self.Cv):
                    raise RuntimeError(f"{self.prefix}: no layer in front kept values '{self.value_key}' of this size")
                mix = 2
        q = ws.get("cattn.q", (T, self.H * self.d), dt)
        K.conv_norm_store(proj, 0, self.conv_w, self.q_norm, self.k_norm, self.eps, state, 0, ctx, table, pages, q,
                          self.H, self.G, self.dk, self.dv, self.d, mix=mix, mix_factor=self.mix_factor, shared=shared,
                          conv_w_t=self.conv_w_t)
        K.conv_state_update(proj, 0, self.C, self.taps, state, 0, ctx)
        att = ws.get("cattn.att", (T, self.H * self.d), dt)
        K.paged_attention(q, self.H * self.d, pages, table, ctx, att, self.H, self.G, self.d, self.scale, self.window,
                          dist_bias=self.bias_table)
        y = ws.get("cattn.y", (T, self.H * self.dv), dt)
        K.head_gate(att, (proj, self.C), y, self.H, self.d, self.dv)
        return linear_into_residual(y, self.w_o, accumulate_into, ctx, "cattn.out", then_norm)


register_part("mixer", "conv_attention", ConvGatedAttention)
