"""Grouped-query attention over the paged cache.

Order of operations as in the reference's layer (src/model/qwen_model.cu:113-160):
q, k, v projections; RMSNorm of each q and k head over its ``head_dim`` elements
(weight [head_dim] shared by the heads, before the rotation, :124-128); rotary
encoding of q and k at the tokens' absolute positions (:136); k and v into the
cache (:139-143); attention with scale 1/sqrt(head_dim) where q head h reads kv
head h // (num_heads/num_kv_heads) (src/kernels/attention.cu:44,304,458);
output projection.  The three projections are one product against the
concatenated matrix; norm, rotation and cache write are one kernel.

Unlike the reference, whose prefill attends only inside the portion it is given
(src/model/qwen_model.cu:147-151), every query attends the cache from position 0
(or the start of its window) to itself, so a prompt may be cut anywhere.

Parameters: hidden_size, num_heads, num_kv_heads, head_dim, qk_norm (bool),
qk_norm_eps, window (None = all keys, W = the last W keys including the query's
own), scale (None = 1/sqrt(head_dim)), has_kv (False: the layer has no k/v
projections and only ever reads another run's cache), cache_block_size (tokens per
cache page if this layer wants a page size of its own; None: the engine's).

Further parameters, for designs that differ from the above (defaults: as above):
    value_dim       size of a value head if it is not head_dim.  The cache and the kernels keep heads of
                    max(head_dim, value_dim) elements; the shorter kind is filled up with zero rows (of W_q, W_k
                    or W_v) and zero columns (of W_o) when the matrices are bound, so nothing else changes
    chunk           C: a query sees key j <= i only if floor(i / C) = floor(j / C), chunks counted from position 0
                    of the sequence (not together with ``window``)
    unit_norm_after_rotation   q and k are divided by their root mean square over head_dim (no weight, eps =
                    qk_norm_eps) behind the rotation instead of a weighted norm in front of it; the rotation may
                    cover only the head's first elements and be rescaled (``position``'s parameters)
    q_leaf, k_leaf, v_leaf, o_leaf   the tensors' leaves under the prefix
    bias_suffix     q, k and v have biases (the tensor's leaf + this suffix), added in 32-bit by the kernel that
                    finishes the heads
    softcap         c > 0: the scaled score s becomes c tanh(s / c)
A position part whose ``pairing`` is "interleaved" (element 2i turns with element 2i + 1) is served by the same
head-finishing kernel as the unit norm, which forms the angles itself from the frequencies.
"""
from __future__ import annotations

import math
from typing import List, Mapping

import torch

from ..cache.spec import PagedKVSpec
from ..ops import kernels as K
from ..weights.arena import FusedSpec, Piece
from ..weights.loader import WeightSpec
from .base import Part, register_part
from .linear import apply_linear, linear_into_residual, scaled_linear_into_residual


class GQAttention(Part):
    adds_into_residual = True        # forward(accumulate_into=...)
    folds_next_norm = True           # forward(then_norm=...)
    accepts_folded_norm = True       # its first operation is a product that can finish a folded norm
    scales_residual = True           # forward(residual_scale=...)

    def __init__(self, spec, rt, position=None):
        super().__init__(spec, rt)
        self.hidden = int(self.p("hidden_size"))
        self.nq = int(self.p("num_heads"))
        self.nkv = int(self.p("num_kv_heads"))
        self.d = int(self.p("head_dim"))
        self.qk_norm = bool(self.p("qk_norm", False))
        self.eps = float(self.p("qk_norm_eps", 1e-6))
        self.window = self.p("window", None)
        scale = self.p("scale", None)
        self.scale = 1.0 / math.sqrt(self.d) if scale is None else float(scale)
        self.has_kv = bool(self.p("has_kv", True))
        self.cache_block_size = self.p("cache_block_size", None)
        self.position = position
        self.dv = int(self.p("value_dim", self.d))
        self.dk = self.d                                  # true size of a query / key head
        self.d = max(self.dk, self.dv)                    # size of a head in the projection, the cache and the kernels
        self.chunk = self.p("chunk", None)
        self.unit_norm = bool(self.p("unit_norm_after_rotation", False))
        self.leaf = {k: self.p(k + "_leaf", k + "_proj.weight") for k in "qkvo"}
        self.bias_suffix = self.p("bias_suffix", None)
        self.softcap = float(self.p("softcap", 0.0) or 0.0)
        if self.softcap < 0:
            raise ValueError("softcap must be positive (or absent)")
        interleaved = getattr(position, "pairing", "half") == "interleaved"
        # the kernel that forms the angles from the frequencies also adds biases and takes either pairing
        self.by_frequencies = self.unit_norm or interleaved or self.bias_suffix is not None
        if self.by_frequencies and self.qk_norm:
            raise ValueError("qk_norm (in front of the rotation) excludes biases, the interleaved pairing and the unit norm")
        if self.by_frequencies and position is not None and not hasattr(position, "frequencies"):
            raise ValueError("this attention needs a position encoding that gives its frequencies")
        self.interleaved = interleaved
        self.bias = None
        if self.chunk is not None and (self.window is not None or int(self.chunk) <= 0):
            raise ValueError("chunk must be positive and excludes window")
        if self.unit_norm and self.qk_norm:
            raise ValueError("qk_norm (in front of the rotation) and unit_norm_after_rotation exclude each other")
        if self.unit_norm and position is not None and not hasattr(position, "frequencies"):
            raise ValueError("unit_norm_after_rotation needs a position encoding that gives its frequencies")
        if self.nq % self.nkv:
            raise ValueError(f"num_heads {self.nq} is not a multiple of num_kv_heads {self.nkv}")
        if self.d > 256:
            raise ValueError(f"head_dim {self.d} > 256 is not supported by the attention kernels")
        if self.window is not None and int(self.window) <= 0:
            raise ValueError("window must be positive")
        self.w_qkv = self.w_o = self.q_norm_w = self.k_norm_w = None

    # -- cache ------------------------------------------------------------------
    def cache_spec(self):
        return PagedKVSpec(self.nkv, self.d, None if self.window is None else int(self.window),
                           None if self.cache_block_size is None else int(self.cache_block_size))

    # -- weights ------------------------------------------------------------------
    def weight_specs(self) -> List[WeightSpec]:
        L = self.leaf
        out = [WeightSpec(self.name(L["q"]), (self.nq * self.dk, self.hidden))]
        if self.has_kv:
            out += [WeightSpec(self.name(L["k"]), (self.nkv * self.dk, self.hidden)),
                    WeightSpec(self.name(L["v"]), (self.nkv * self.dv, self.hidden))]
        out.append(WeightSpec(self.name(L["o"]), (self.hidden, self.nq * self.dv)))
        if self.bias_suffix is not None:
            sfx = self.bias_suffix
            out.append(WeightSpec(self.name(L["q"]) + sfx, (self.nq * self.dk,), init="zeros", as_float32=True))
            if self.has_kv:
                out += [WeightSpec(self.name(L["k"]) + sfx, (self.nkv * self.dk,), init="zeros", as_float32=True),
                        WeightSpec(self.name(L["v"]) + sfx, (self.nkv * self.dv,), init="zeros", as_float32=True)]
        if self.qk_norm:
            out.append(WeightSpec(self.name("q_norm.weight"), (self.d,), init="norm", as_float32=True))
            if self.has_kv:
                out.append(WeightSpec(self.name("k_norm.weight"), (self.d,), init="norm", as_float32=True))
        return out

    def fused_layout(self, dtype_of) -> List[FusedSpec]:
        """q, k and v stacked into one matrix [(nq + 2 nkv) d, hidden], the three projections' rows
        in this order."""
        if not self.has_kv or self.dk != self.dv:       # heads that are filled up are put together when bound
            return []
        q_rows, kv_rows = self.nq * self.d, self.nkv * self.d
        return [FusedSpec(self.name("qkv_proj.weight"), (q_rows + 2 * kv_rows, self.hidden),
                          (Piece(self.name(self.leaf["q"]), 0), Piece(self.name(self.leaf["k"]), q_rows),
                           Piece(self.name(self.leaf["v"]), q_rows + kv_rows)))]

    def _filled(self, m: torch.Tensor, heads: int, size: int) -> torch.Tensor:
        """Rows of `heads` heads of `size` rows each, every head filled up to self.d rows with zeros."""
        if size == self.d:
            return m
        out = torch.zeros((heads, self.d, m.shape[1]), dtype=m.dtype, device=m.device)
        out[:, :size] = m.view(heads, size, m.shape[1])
        return out.view(heads * self.d, m.shape[1])

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        fused = self.name("qkv_proj.weight")
        if fused in tensors:
            self.w_qkv = self._matrix(tensors[fused])
        else:
            mats = [self._filled(self._matrix(tensors[self.name(self.leaf["q"])]), self.nq, self.dk)]
            if self.has_kv:
                mats += [self._filled(self._matrix(tensors[self.name(self.leaf["k"])]), self.nkv, self.dk),
                         self._filled(self._matrix(tensors[self.name(self.leaf["v"])]), self.nkv, self.dv)]
            if len({m.dtype for m in mats}) != 1:
                mats = [m.to(torch.float32) for m in mats]
            self.w_qkv = torch.cat(mats, dim=0).contiguous() if len(mats) > 1 else mats[0].contiguous()
        self.w_o = self._matrix(tensors[self.name(self.leaf["o"])])
        if self.dv != self.d:          # zero columns where the kernels' value heads are longer than the true ones
            wo = torch.zeros((self.hidden, self.nq, self.d), dtype=self.w_o.dtype, device=self.w_o.device)
            wo[:, :, : self.dv] = self.w_o.view(self.hidden, self.nq, self.dv)
            self.w_o = wo.view(self.hidden, self.nq * self.d).contiguous()
        if self.bias_suffix is not None:       # one row in the projection's layout, heads filled up with zeros
            sfx = self.bias_suffix
            parts = [(self.leaf["q"], self.nq, self.dk)]
            if self.has_kv:
                parts += [(self.leaf["k"], self.nkv, self.dk), (self.leaf["v"], self.nkv, self.dv)]
            rows = []
            for leaf, heads, size in parts:
                b = self._vector32(tensors[self.name(leaf) + sfx]).view(heads, size)
                full = torch.zeros((heads, self.d), dtype=torch.float32, device=b.device)
                full[:, :size] = b
                rows.append(full.view(-1))
            self.bias = torch.cat(rows).contiguous()
        if self.qk_norm:
            self.q_norm_w = self._vector32(tensors[self.name("q_norm.weight")])
            if self.has_kv:
                self.k_norm_w = self._vector32(tensors[self.name("k_norm.weight")])

    # -- run ------------------------------------------------------------------
    def _mask(self) -> int:
        """The kernels' one mask argument: W > 0 a window of W keys, -C < 0 chunks of C positions, 0 every key."""
        if self.chunk is not None:
            return -int(self.chunk)
        return 0 if self.window is None else int(self.window)

    def forward(self, x, ctx, slot: int, write_cache: bool, accumulate_into=None, then_norm=None,
                residual_scale: float = 1.0):
        T = x.shape[0]
        ws = ctx.workspace
        if write_cache and not self.has_kv:
            raise RuntimeError(f"{self.prefix}: a layer without k/v projections cannot write a cache")
        nkv_w = self.nkv if write_cache else 0
        width = (self.nq + 2 * nkv_w) * self.d
        w = self.w_qkv if (write_cache or not self.has_kv) else self.w_qkv[: self.nq * self.d]
        qkv = ws.get("attn.qkv", (T, width), ctx.dtype)
        apply_linear(x, w, qkv, ctx, "attn.qkv")
        pages, table = ctx.kv(slot)
        rot = self.position.rotary_table() if self.position is not None and not self.by_frequencies else None
        cos_sin, rotary_dim = rot if rot is not None else (None, 0)
        att = ws.get("attn.out", (T, self.nq * self.d), ctx.dtype)
        if self.by_frequencies:
            if self.position is not None:
                freq, mag = self.position.frequencies(), self.position.magnitude
            else:
                freq, mag = ctx.workspace.get("attn.no_freq", (0,), torch.float64), 1.0
            bias = self.bias if (self.bias is None or write_cache or not self.has_kv) else self.bias[: self.nq * self.d]
            K.rope_unit_norm_store(qkv, self.nq, nkv_w, self.d, self.dk, self.eps, freq, mag, ctx,
                                   table if write_cache else None, pages if write_cache else None,
                                   interleaved=self.interleaved, normalize=self.unit_norm, bias=bias)
            self._attend(qkv, width, pages, table, ctx, att)
        elif write_cache and self.chunk is None and not self.softcap and K.decode_finishes_heads(ctx, ctx.dtype, self.nq, self.nkv, self.d, rotary_dim):
            # a step of single tokens: the attention kernel finishes the heads itself
            K.attn_decode_heads(qkv, pages, table, ctx, att, self.nq, self.nkv, self.d, self.scale,
                                0 if self.window is None else int(self.window), self.q_norm_w,
                                self.k_norm_w, self.eps, cos_sin)
        else:
            K.qk_norm_rope_store(qkv, self.nq, nkv_w, self.d, self.q_norm_w,
                                 self.k_norm_w if write_cache else None, self.eps, cos_sin, rotary_dim,
                                 ctx.positions, ctx.token_seq, table if write_cache else None,
                                 pages if write_cache else None, ctx.status)
            self._attend(qkv, width, pages, table, ctx, att)
        if residual_scale != 1.0:
            return scaled_linear_into_residual(att, self.w_o, accumulate_into, residual_scale, ctx, "attn.proj")
        return linear_into_residual(att, self.w_o, accumulate_into, ctx, "attn.proj", then_norm)

    def _attend(self, qkv, width, pages, table, ctx, att) -> None:
        K.paged_attention(qkv, width, pages, table, ctx, att, self.nq, self.nkv, self.d, self.scale,
                          self._mask(), softcap=self.softcap)


register_part("mixer", "gqa_attention", GQAttention)
