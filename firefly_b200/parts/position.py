"""Position encodings.

``rotary``: rotate-half rotary encoding, f_i = theta^(-2i/r) for i in [0, r/2),
angle = position * f_i, pairs (i, i + r/2) of the first ``rotary_dim`` = r
elements of a head (the reference rotates the whole head: src/kernels/rope.cu:68-95).
The reference evaluates powf/cosf/sinf per element under --use_fast_math; here
cosines and sines come from a table computed once on the host in double
precision and stored in 32-bit, one row per position up to ``max_positions``.

``scaling`` (a parameter of ``rotary``; None: none) = dict(factor, original, fast, slow) rescales the
frequencies in the YaRN manner: with where(n) = r ln(original / (2 pi n)) / (2 ln theta), lo = max(floor(where(fast)),
0), hi = min(ceil(where(slow)), r - 1) and ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), the frequency is
f_i / factor * ramp_i + f_i (1 - ramp_i), and cos and sin are multiplied by ``magnitude`` = 0.1 ln(factor) + 1.

``scaling`` = dict(kind="wavelength_bands", factor, low, high, original) rescales by the wavelength l = 2 pi / f_i:
f_i is kept where l < original / high, divided by ``factor`` where l > original / low, and between the two it is
(1 - s) f_i / factor + s f_i with s = (original / l - low) / (high - low); cos and sin keep magnitude 1.

``pairing`` (a parameter of ``rotary``): "half" (default) pairs element i with element i + r/2; "interleaved" pairs
element 2i with element 2i + 1.  The table of positions (`rotary_table`) is laid out for "half" only; the kernels
that form the angle themselves from `frequencies` take either.

``none``: no position information (a mixer that needs none).
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

from .base import Part, register_part


class PositionEncoding(Part):
    def rotary_table(self) -> Optional[Tuple[torch.Tensor, int]]:
        return None

    def apply_to_embedding(self, h: torch.Tensor, ctx) -> None:
        return None


class RotaryEncoding(PositionEncoding):
    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.head_dim = int(self.p("head_dim"))
        self.rotary_dim = int(self.p("rotary_dim", self.head_dim))
        self.theta = float(self.p("theta"))
        self.max_positions = int(self.p("max_positions", 0))     # 0: no table of positions (see `frequencies`)
        if self.rotary_dim % 2 or not (0 < self.rotary_dim <= self.head_dim):
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and within the head "
                             f"({self.head_dim})")
        sc = self.p("scaling", None)
        self.pairing = str(self.p("pairing", "half"))
        if self.pairing not in ("half", "interleaved"):
            raise ValueError(f"rotary pairing '{self.pairing}' is not 'half' or 'interleaved'")
        self.scaling_kind = str(sc.get("kind", "yarn")) if sc else None
        if self.scaling_kind not in (None, "yarn", "wavelength_bands"):
            raise ValueError(f"rotary scaling kind '{self.scaling_kind}' is not 'yarn' or 'wavelength_bands'")
        keys = ("factor", "original", "low", "high") if self.scaling_kind == "wavelength_bands" \
            else ("factor", "original", "fast", "slow")
        self.scaling = None if not sc else tuple(float(sc[k]) for k in keys)
        if self.scaling is not None and not (self.scaling[0] > 0 and self.scaling[1] > 0 and self.scaling[2] > 0
                                             and self.scaling[3] > 0):
            raise ValueError(f"rotary scaling {sc} must have positive {', '.join(keys)}")
        if self.scaling_kind == "wavelength_bands" and not (self.scaling[3] > self.scaling[2]):
            raise ValueError(f"rotary scaling {sc}: high must be above low")

    @property
    def magnitude(self) -> float:
        """The factor on cos and sin (1 without scaling)."""
        return 1.0 if self.scaling is None or self.scaling_kind != "yarn" else 0.1 * math.log(self.scaling[0]) + 1.0

    def _frequencies64(self) -> torch.Tensor:
        r = self.rotary_dim
        i = torch.arange(r // 2, dtype=torch.float64)
        freq = torch.pow(torch.tensor(self.theta, dtype=torch.float64), -2.0 * i / r)
        if self.scaling is None:
            return freq
        if self.scaling_kind == "wavelength_bands":
            factor, original, low, high = self.scaling
            wavelength = 2.0 * math.pi / freq
            s = (original / wavelength - low) / (high - low)
            blend = (1.0 - s) * freq / factor + s * freq
            return torch.where(wavelength < original / high, freq,
                               torch.where(wavelength > original / low, freq / factor, blend))
        factor, original, fast, slow = self.scaling

        def where(turns: float) -> float:
            return r * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(self.theta))
        lo = max(math.floor(where(fast)), 0)
        hi = min(math.ceil(where(slow)), r - 1)
        ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
        return freq / factor * ramp + freq * (1.0 - ramp)

    def rotary_table(self):
        if self.pairing != "half":
            raise ValueError("the table of positions serves the 'half' pairing only")
        key = ("rotary", self.rotary_dim, self.theta, self.max_positions, self.scaling_kind, self.scaling)
        table = self.rt.shared.get(key)
        if table is None:
            freq = self._frequencies64()
            ang = torch.arange(self.max_positions, dtype=torch.float64)[:, None] * freq[None, :]
            table = (torch.stack([torch.cos(ang), torch.sin(ang)], dim=-1) * self.magnitude).to(torch.float32)
            table = table.contiguous().to(self.rt.device)
            self.rt.shared[key] = table
        return table, self.rotary_dim


    def frequencies(self) -> torch.Tensor:
        """f_i = theta^(-2i/r), i in [0, r/2) (rescaled when ``scaling`` is given), as a 64-bit table on the
        device: for kernels that form the angle position * f_i themselves (in double, so no table of positions
        and no longest position).  Such a kernel multiplies cos and sin by ``magnitude``."""
        key = ("rotary_freq", self.rotary_dim, self.theta, self.scaling_kind, self.scaling)
        freq = self.rt.shared.get(key)
        if freq is None:
            freq = self._frequencies64().contiguous().to(self.rt.device)
            self.rt.shared[key] = freq
        return freq


class NoPosition(PositionEncoding):
    pass


register_part("position", "rotary", RotaryEncoding)
register_part("position", "none", NoPosition)
