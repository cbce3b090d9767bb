"""Arrangements: how a layer's parts are joined into a block.

``pre_norm`` is the reference's (src/model/qwen_model.cu:106-175):
    h += mixer(norm_0(h));  h += feed_forward(norm_1(h))
A block may hold an *input filter* (``LayerSpec.params["input_filter"]``, a PartSpec of category ``filter``): what
the mixer reads is then filter(norm_0(h)), e.g. a short causal convolution over time added to its own input.  The
filter's state lives under a cache id of its own per run (``cache.spec.filter_slot``).  A ``pre_norm`` block without
a feed-forward ends after the mixer.
A block may also hold a *tail* (``LayerSpec.params["tail"]``, a PartSpec of category ``tail``): a part that runs at the
block's end on the stream itself, e.g. an input that the token brings to every layer.
The residual stream ``h`` is 32-bit.  A part's output is not added at once: it is
handed on as ``pending`` and the next norm adds it while it reads the row, so
each sum is done once, in 32-bit, without a pass of its own.
"""
from __future__ import annotations

from typing import List, Mapping

import torch

from ..ops import kernels as K
from ..weights.loader import WeightSpec
from .base import Part, Runtime, build_part, declared, register_part


class Block:
    """Base of arrangements: owns the built parts of one layer."""

    n_norms = 2
    runs_tail = False            # an arrangement that runs ``params["tail"]`` at its end sets this

    def __init__(self, layer_spec, rt: Runtime):
        self.layer_spec = layer_spec
        self.position = build_part("position", layer_spec.position, rt) \
            if layer_spec.position is not None else None
        self.mixer = build_part("mixer", layer_spec.mixer, rt, position=self.position)
        self.feed_forward = build_part("feed_forward", layer_spec.feed_forward, rt) \
            if layer_spec.feed_forward is not None else None
        self.params = dict(getattr(layer_spec, "params", None) or {})
        self.input_filter = build_part("filter", self.params["input_filter"], rt) \
            if self.params.get("input_filter") is not None else None
        self.tail = build_part("tail", self.params["tail"], rt) if self.params.get("tail") is not None else None
        if self.tail is not None and not self.runs_tail:
            raise ValueError(f"arrangement '{layer_spec.arrangement}' has no place for a tail part")
        want_norms = self.n_norms if self.feed_forward is not None else self.n_norms - 1
        if len(layer_spec.norms) != want_norms:
            raise ValueError(f"arrangement '{layer_spec.arrangement}' needs {want_norms} norms, "
                             f"got {len(layer_spec.norms)}")
        self.norms = [build_part("norm", n, rt) for n in layer_spec.norms]
        # the parts' declared abilities (parts/base.py), checked here against their signatures:
        # adding into the 32-bit residual themselves, folding the norm that follows into their last
        # product, taking a folded norm as input
        self._mixer_fuses = declared(self.mixer, "adds_into_residual")
        has_ffn = self.feed_forward is not None
        self._ffn_fuses = has_ffn and declared(self.feed_forward, "adds_into_residual")
        self._mixer_folds = declared(self.mixer, "folds_next_norm")
        self._ffn_folds = has_ffn and declared(self.feed_forward, "folds_next_norm")
        self._mixer_defers = declared(self.mixer, "accepts_folded_norm")
        self._ffn_defers = has_ffn and declared(self.feed_forward, "accepts_folded_norm")
        self._mixer_scales = declared(self.mixer, "scales_residual")
        self._ffn_scales = has_ffn and declared(self.feed_forward, "scales_residual")
        self._norm_folds = [declared(nrm, "foldable") for nrm in self.norms]
        for k, nrm in enumerate(self.norms):
            if self._norm_folds[k]:
                nrm.fold_tag = f"fold.{k}"      # scratch of the folded form, one per norm of the block

    def parts(self) -> List[Part]:
        out = [p for p in (self.mixer, self.feed_forward, *self.norms, self.input_filter, self.tail) if p is not None]
        if self.position is not None:
            out.append(self.position)
        return out

    def filter_cache_spec(self):
        """What the input filter keeps per request (None: no filter, or one without state)."""
        return self.input_filter.cache_spec() if self.input_filter is not None else None

    def _filtered_norm(self, norm, residual, pending, ctx):
        """norm_0 followed by the input filter; the norm's rows stay 32-bit on the way where the filter wants that."""
        if getattr(self.input_filter, "wants_float32_input", False) and ctx.dtype != torch.float32:
            x = norm.forward(residual, pending, ctx, tag="normed.f32", out_dtype=torch.float32)
        else:
            x = norm.forward(residual, pending, ctx)
        return self.input_filter.forward(x, ctx, ctx.memo["filter_slot"])

    def weight_specs(self) -> List[WeightSpec]:
        return [w for p in self.parts() for w in p.weight_specs()]

    takes_next_norm = False      # an arrangement whose forward takes ``next_norm`` sets this

    def first_norm(self):
        """The norm a block in front of this one may fold into its last product (None: none)."""
        return None

    def fused_layout(self, dtype_of) -> list:
        # a part need not derive from ``Part``: one without the method wants nothing fused
        return [f for p in self.parts() if hasattr(p, "fused_layout") for f in p.fused_layout(dtype_of)]

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        for p in self.parts():
            p.bind(tensors)

    def cache_spec(self):
        return self.mixer.cache_spec()


class PreNormBlock(Block):
    takes_next_norm = True
    runs_tail = True

    def first_norm(self):
        """The norm a block in front of this one may fold into its last product (none when a filter reads the
        norm's rows: they must exist)."""
        return None if self.input_filter is not None else self.norms[0]

    def parts(self) -> list:
        """The parts this block holds."""
        return [p for p in (self.mixer, self.feed_forward, *self.norms, getattr(self, "position", None),
                            getattr(self, "input_filter", None), getattr(self, "tail", None)) if p is not None]

    def forward(self, residual: torch.Tensor, pending, ctx, slot: int, write_cache: bool, next_norm=None):
        # only a foldable norm knows ``may_defer`` (hand a folded norm on to a consumer that finishes it)
        has_ffn = self.feed_forward is not None
        if self.tail is not None:    # the tail reads the stream behind the last part: no norm is folded past it
            next_norm = None
        defer0 = {"may_defer": True} if self._norm_folds[0] and self._mixer_defers else {}
        defer1 = {"may_defer": True} if has_ffn and self._norm_folds[1] and self._ffn_defers else {}
        if self.input_filter is not None:
            x = self._filtered_norm(self.norms[0], residual, pending, ctx)
        else:
            x = self.norms[0].forward(residual, pending, ctx, **defer0)
        kw = {}
        if self._mixer_fuses:
            kw["accumulate_into"] = residual
            following = self.norms[1] if has_ffn else next_norm
            if self._mixer_folds and following is not None:
                kw["then_norm"] = following
        a = self.mixer.forward(x, ctx, slot, write_cache, **kw)
        if not has_ffn:              # a block of a mixer only: its delta (or folded norm) goes to the next block
            return (residual, a) if self.tail is None else self.tail.forward(residual, a, ctx)
        x = self.norms[1].forward(residual, a, ctx, **defer1)
        kw = {}
        if self._ffn_fuses:
            kw["accumulate_into"] = residual
            if self._ffn_folds:
                kw["then_norm"] = next_norm
        f = self.feed_forward.forward(x, ctx, **kw)
        return (residual, f) if self.tail is None else self.tail.forward(residual, f, ctx)


class ScaledPreNormBlock(Block):
    """h += m * mixer(norm_0(h));  h += m * feed_forward(norm_1(h))  with one multiplier m
    (``params["residual_mult"]``) on everything the parts add; a block without a feed-forward ends
    after the mixer.  Parts that declare ``scales_residual`` add their scaled output into the 32-bit
    stream themselves; another part's delta is added times m by the norm that follows (which must
    take ``delta_scale``) or, at the block's end, in a pass of its own."""

    def __init__(self, layer_spec, rt: Runtime):
        super().__init__(layer_spec, rt)
        self.mult = float(self.params.get("residual_mult", 1.0))
        if self.feed_forward is not None and not getattr(self.norms[1], "takes_delta_scale", False) \
                and not (self._mixer_fuses and (self._mixer_scales or self.mult == 1.0)):
            raise ValueError(f"arrangement '{layer_spec.arrangement}': the mixer leaves a delta and the second "
                             "norm cannot add it times a multiplier")

    def _run(self, part, fuses, scales, residual, *args):
        if fuses and scales:
            return part.forward(*args, accumulate_into=residual, residual_scale=self.mult)
        if fuses and self.mult == 1.0:
            return part.forward(*args, accumulate_into=residual)
        return part.forward(*args)

    def forward(self, residual: torch.Tensor, pending, ctx, slot: int, write_cache: bool):
        x = self.norms[0].forward(residual, pending, ctx)            # a delta handed over by another block is unscaled
        a = self._run(self.mixer, self._mixer_fuses, self._mixer_scales, residual, x, ctx, slot, write_cache)
        if self.feed_forward is None:
            if a is not None:
                residual.add_(a.to(torch.float32), alpha=self.mult)
            return residual, None
        x = self.norms[1].forward(residual, a, ctx, delta_scale=self.mult) if a is not None \
            else self.norms[1].forward(residual, None, ctx)
        f = self._run(self.feed_forward, self._ffn_fuses, self._ffn_scales, residual, x, ctx)
        if f is not None:
            residual.add_(f.to(torch.float32), alpha=self.mult)
        return residual, None


class OutputNormBlock(Block):
    """h += norm_0(mixer(h));  h += norm_1(feed_forward(h)): the norms sit on the parts' outputs and the parts
    read the stream itself (in the activation type: a copy of the 32-bit stream that the norm kernel keeps up to
    date; a 32-bit engine reads the stream).  A part that declares ``adds_into_residual`` adds its output into a
    zeroed 32-bit buffer, so that what the norm reads was never rounded; another part's delta is taken as it
    comes.  A block without a feed-forward ends after the mixer.  The norms must offer ``add_normed``."""

    def __init__(self, layer_spec, rt: Runtime):
        super().__init__(layer_spec, rt)
        for nrm in self.norms:
            if not hasattr(nrm, "add_normed"):
                raise ValueError(f"arrangement '{layer_spec.arrangement}': norm '{nrm.spec.kind}' cannot norm a part's output")

    def _stream_copy(self, residual, ctx):
        if ctx.dtype == torch.float32:
            return residual
        x = ctx.memo.get("stream_copy")
        if x is None:
            x = ctx.workspace.get("stream.copy", tuple(residual.shape), ctx.dtype)
            K.cast(residual, x)
            ctx.memo["stream_copy"] = x
        return x

    def _delta(self, part, fuses, ctx, residual, *args):
        if fuses:
            delta = ctx.workspace.get("block.delta", tuple(residual.shape), torch.float32)
            delta.zero_()
            left = part.forward(*args, accumulate_into=delta)
            return delta if left is None else left      # a part that could not add by itself hands its delta back
        return part.forward(*args)

    def forward(self, residual: torch.Tensor, pending, ctx, slot: int, write_cache: bool):
        if pending is not None:                  # handed over by a block of another arrangement
            from .norm import FoldedNorm
            if not isinstance(pending, FoldedNorm):
                K.residual_add(residual, pending)
            ctx.memo.pop("stream_copy", None)
        x = self._stream_copy(residual, ctx)
        copy = None if x is residual else x
        a = self._delta(self.mixer, self._mixer_fuses, ctx, residual, x, ctx, slot, write_cache)
        self.norms[0].add_normed(residual, a, ctx, copy)
        if self.feed_forward is not None:
            f = self._delta(self.feed_forward, self._ffn_fuses, ctx, residual, x, ctx)
            self.norms[1].add_normed(residual, f, ctx, copy)
        return residual, None


register_part("arrangement", "pre_norm", PreNormBlock)
register_part("arrangement", "output_norm", OutputNormBlock)
register_part("arrangement", "scaled_pre_norm", ScaledPreNormBlock)
