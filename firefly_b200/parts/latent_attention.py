"""Attention whose keys and values are re-made from a small cached latent vector.

Per token the cache holds c [kv_rank] (the first kv_rank outputs of the down projection W_dkv,
RMS-normed with a plain weight) and k_rot [rot_dim] (its last rot_dim outputs, rotated, one key part
shared by all heads).  Head h has key [W_uk[h] c | k_rot] and value W_uv[h] c; its query is laid out
[dim plain | rot_dim rotated]; score = (q_plain . k_plain + q_rot . k_rot) * scale; causal softmax
over all earlier tokens; the concatenated heads are multiplied by sigmoid(W_g x) and go through W_o.

The products with W_uk and W_uv are moved to the query side:  q_plain . (W_uk[h] c) = (W_uk[h]^T
q_plain) . c, and sum_j p_j W_uv[h] c_j = W_uv[h] (sum_j p_j c_j).  What remains over the cache is
attention with one key/value head of size kv_rank + rot_dim whose keys are the cache rows and whose
values are their first kv_rank elements: the paged attention kernels of the other mixers run it
(tcgen05 / mma.sync / plain, by size and type), prompts and decoding alike.  The rotation is
rotate-half over the rot_dim part, angle = position * base^(-2i/rot_dim), formed in double.

Parameters: hidden_size, heads, dim, rot_dim, vdim, kv_rank, scale, eps (of the latent's norm),
cache_block_size (optional).  Position part: ``rotary`` with head_dim = rot_dim and rotary_dim <= rot_dim
(the first rotary_dim elements of the rotated part turn, the rest pass unchanged).
Tensors: q [heads*(dim+rot_dim), W]; dkv [kv_rank+rot_dim, W]; dkv.norm [kv_rank];
uk [heads*dim, kv_rank]; uv [heads*vdim, kv_rank]; g [heads*vdim, W]; o [W, heads*vdim].

Further parameters, for designs that differ from the above (defaults: as above):
    q_rank        the queries go through a latent of their own: c_q = rms_norm(W_dq x) * dq.norm (32-bit, eps as
                  above), q = W_uq c_q; tensors dq [q_rank, W], dq.norm [q_rank], uq [heads*(dim+rot_dim), q_rank]
                  instead of q
    window        W: query i sees key j only when 0 <= i - j < W
    cache_window  the window the cache keeps (default: ``window``): at least the longest window of the layers that
                  read this layer's cache
    has_kv        False: the layer has no down projection and reads the cache rows that another run wrote (the
                  schedule points it at that run's cache slot), with its own up-projections, queries and window
    gate          "element" (g [heads*vdim, W]) | "head" (g [heads, W]: one gate a head)
The position part's ``pairing`` ("half" | "interleaved") says which elements of the rotated part turn together.
"""
from __future__ import annotations

from typing import List, Mapping

import torch

from ..cache.spec import PagedKVSpec
from ..ops import kernels as K
from ..weights.arena import FusedSpec, Piece
from ..weights.loader import WeightSpec
from .base import Part, register_part
from .linear import apply_linear, scaled_linear_into_residual


class LatentAttention(Part):
    adds_into_residual = True        # forward(accumulate_into=...)
    scales_residual = True           # forward(residual_scale=...)

    def __init__(self, spec, rt, position=None):
        super().__init__(spec, rt)
        self.hidden = int(self.p("hidden_size"))
        self.heads = int(self.p("heads"))
        self.dim = int(self.p("dim"))
        self.rot = int(self.p("rot_dim"))
        self.vdim = int(self.p("vdim"))
        self.rank = int(self.p("kv_rank"))
        self.scale = float(self.p("scale"))
        self.eps = float(self.p("eps"))
        self.cache_block_size = self.p("cache_block_size", None)
        self.position = position
        self.q_rank = self.p("q_rank", None)
        self.q_rank = None if self.q_rank is None else int(self.q_rank)
        self.window = self.p("window", None)
        self.window = None if self.window is None else int(self.window)
        cw = self.p("cache_window", None)
        self.cache_window = self.window if cw is None else int(cw)
        self.has_kv = bool(self.p("has_kv", True))
        self.gate = str(self.p("gate", "element"))
        self.interleaved = getattr(position, "pairing", "half") == "interleaved"
        if self.gate not in ("element", "head"):
            raise ValueError(f"{self.prefix}: gate '{self.gate}' is not 'element' or 'head'")
        if self.window is not None and (self.window <= 0 or self.cache_window is None or self.cache_window < self.window):
            raise ValueError(f"{self.prefix}: window {self.window} against a cache that keeps {self.cache_window}")
        self.d = self.rank + self.rot                      # size of a cache row and of a finished query head
        if self.rot and (position is None or not hasattr(position, "frequencies")):
            raise ValueError(f"{self.prefix}: needs a rotary position part")
        # the first rotary_dim elements of the rot_dim part turn (all of them unless the position part says fewer)
        self.rdims = int(getattr(position, "rotary_dim", 0)) if self.rot else 0
        if self.rdims % 2 or self.rdims > self.rot:
            raise ValueError(f"{self.prefix}: {self.rdims} rotated dimensions do not fit rot_dim {self.rot}")
        if self.d > 512:
            raise ValueError(f"{self.prefix}: kv_rank + rot_dim = {self.d} > 512 is not supported by the attention kernels")
        self.n_q, self.n_dkv = self.heads * (self.dim + self.rot), (self.d if self.has_kv else 0)
        self.n_g = self.heads * self.vdim if self.gate == "element" else self.heads
        self.n_v = self.heads * self.vdim
        self.w_in = self.w_uk = self.w_uv = self.w_o = self.c_norm = self.w_dq = self.w_uq = self.q_norm = None

    def cache_spec(self):
        # one vector per token in a cache of one plane: the attention kernels, built for such a cache, read it as
        # key and as value
        return PagedKVSpec(1, self.d, self.cache_window,
                           None if self.cache_block_size is None else int(self.cache_block_size), planes=1)

    def weight_specs(self) -> List[WeightSpec]:
        n, W = self.name, self.hidden
        out = [WeightSpec(n("q"), (self.n_q, W))] if self.q_rank is None else \
            [WeightSpec(n("dq"), (self.q_rank, W)), WeightSpec(n("dq.norm"), (self.q_rank,), init="norm", as_float32=True),
             WeightSpec(n("uq"), (self.n_q, self.q_rank))]
        if self.has_kv:
            out += [WeightSpec(n("dkv"), (self.n_dkv, W)),
                    WeightSpec(n("dkv.norm"), (self.rank,), init="norm", as_float32=True)]
        return out + [WeightSpec(n("uk"), (self.heads * self.dim, self.rank)),
                      WeightSpec(n("uv"), (self.n_v, self.rank)),
                      WeightSpec(n("g"), (self.n_g, W)), WeightSpec(n("o"), (W, self.n_v))]

    def _stacked(self):
        """The tensors that read the mixer's input through one product, in the order of their rows (a latent query's
        down projection has a product of its own, which writes 32-bit for its norm)."""
        return ([] if self.q_rank is not None else ["q"]) + (["dkv"] if self.has_kv else []) + ["g"]

    def fused_layout(self, dtype_of) -> List[FusedSpec]:
        """q, the down projection and the gate read the same input: one matrix, their rows in this order."""
        n = self.name
        rows = {"q": self.n_q, "dkv": self.n_dkv, "g": self.n_g}
        if len(self._stacked()) < 2:
            return []
        pieces, at = [], 0
        for leaf in self._stacked():
            pieces.append(Piece(n(leaf), at))
            at += rows[leaf]
        return [FusedSpec(n("_".join(self._stacked())), (at, self.hidden), tuple(pieces))]

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        n = self.name
        fused = n("_".join(self._stacked()))
        if fused in tensors and len(self._stacked()) > 1:
            self.w_in = self._matrix(tensors[fused])
        else:
            mats = [self._matrix(tensors[n(s)]) for s in self._stacked()]
            if len({m.dtype for m in mats}) != 1:
                mats = [m.to(torch.float32) for m in mats]
            self.w_in = torch.cat(mats, dim=0).contiguous() if len(mats) > 1 else mats[0]
        dt = self.w_in.dtype
        if self.q_rank is not None:
            self.w_dq, self.w_uq = self._matrix(tensors[n("dq")]).to(dt), self._matrix(tensors[n("uq")]).to(dt)
            self.q_norm = self._vector32(tensors[n("dq.norm")])
        # [heads, kv_rank, dim]: the transposed key up-projection, so that q_abs = q_plain @ it^T
        self.w_uk = self._matrix(tensors[n("uk")]).to(dt).view(self.heads, self.dim, self.rank).transpose(1, 2).contiguous()
        self.w_uv = self._matrix(tensors[n("uv")]).to(dt).view(self.heads, self.vdim, self.rank).contiguous()
        self.w_o = self._matrix(tensors[n("o")])
        self.c_norm = self._vector32(tensors[n("dkv.norm")]) if self.has_kv else torch.ones(1, dtype=torch.float32, device=self.w_o.device)

    def forward(self, x, ctx, slot: int, write_cache: bool, accumulate_into=None, residual_scale: float = 1.0):
        if write_cache != self.has_kv:
            raise RuntimeError(f"{self.prefix}: a layer with a down projection writes the cache it reads, one without "
                               "reads another run's")
        T, ws, H, d = x.shape[0], ctx.workspace, self.heads, self.d
        dt = self.w_in.dtype
        n_q = self.n_q if self.q_rank is None else 0            # q's columns in the stacked product
        proj = ws.get("lat.proj", (T, n_q + self.n_dkv + self.n_g), dt)
        apply_linear(x, self.w_in, proj, ctx, "lat.proj")
        if self.q_rank is None:
            q = proj[:, :n_q]
        else:
            # the queries' latent: the down projection in 32-bit, its norm, the up projection
            dq = ws.get("lat.dq", (T, self.q_rank), torch.float32)
            apply_linear(x, self.w_dq, dq, ctx, "lat.dq")
            cq = ws.get("lat.cq", (T, self.q_rank), dt)
            K.add_rms_norm(dq, None, self.q_norm, self.eps, cq)
            q = ws.get("lat.q", (T, self.n_q), dt)
            apply_linear(cq, self.w_uq, q, ctx, "lat.q")
        # W_uk[h]^T q_plain[h] for every head: the heads are the batch of one library product
        q_plain = q.view(T, H, self.dim + self.rot)[:, :, :self.dim].transpose(0, 1)
        q_abs = ws.get("lat.q_abs", (H, T, self.rank), dt)
        K.batched_linear(q_plain, self.w_uk, q_abs)
        pages, table = ctx.kv(slot)
        q_full = ws.get("lat.q_full", (T, H * d), dt)
        freq = self.position.frequencies() if self.rdims else torch.empty(0, dtype=torch.float64, device=x.device)
        dkv = proj[:, n_q:n_q + self.n_dkv] if self.has_kv else None
        K.latent_finish(q, dkv, q_abs, self.c_norm, self.eps, freq, ctx, table, pages, q_full,
                        H, self.dim, self.rot, self.rank, self.rdims, self.interleaved)
        att = ws.get("lat.att", (T, H * d), dt)
        K.paged_attention(q_full, H * d, pages, table, ctx, att, H, 1, d, self.scale,
                          0 if self.window is None else self.window)
        latent = att.view(T, H, d)[:, :, :self.rank].transpose(0, 1)
        val = ws.get("lat.val", (H, T, self.vdim), dt)
        K.batched_linear(latent, self.w_uv, val)
        y = ws.get("lat.y", (T, self.n_v), dt)
        K.latent_gate(val, proj[:, n_q + self.n_dkv:], y, H, self.vdim, per_head=self.gate == "head")
        return scaled_linear_into_residual(y, self.w_o, accumulate_into, residual_scale, ctx, "lat.out")


register_part("mixer", "latent_attention", LatentAttention)
