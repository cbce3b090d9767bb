"""Typed configuration of the Papusun design.

``config.json`` names the design under ``architecture`` and gives every size and constant:

    vocab, width, norm.eps, logit_scale, token_side {dim}
    layers[i]: type ("parallel" | "latent_attention"), mixer {...}, mlp {kind "dense", ff} | null
        parallel mixer:  left {heads, kv_heads, dim, vdim, scale, softcap, rot {base, dims, scaling {factor, low, high,
                         original} | absent}}, right {heads, kv_heads, dim, vdim, conv}, left_scale, right_scale
        latent_attention mixer:  heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, mask {size}, rot {base, dims},
                         kv_from: j (optional: the layer has no down projection and reads layer j's cache rows)

The nested objects are kept as they are and checked here, so that a wrong or missing key is told by name before
anything is built.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, ClassVar, Dict, Mapping, Optional, Tuple

from .base import ConfigError, ModelConfig
from .pepolorn import _need

MIXERS = ("parallel", "latent_attention")


def _check_rot(rot, where: str, within: int) -> None:
    _need(rot, "base", float, where)
    dims = _need(rot, "dims", int, where)
    if dims % 2 or dims > within:
        raise ConfigError(f"config.json: {where}.dims {dims} must be even and at most {within}")
    sc = rot.get("scaling")
    if sc is not None:
        for key in ("factor", "low", "high", "original"):
            if not (_need(sc, key, float, where + ".scaling") > 0):
                raise ConfigError(f"config.json: {where}.scaling.{key} must be positive")
        if not (float(sc["high"]) > float(sc["low"])):
            raise ConfigError(f"config.json: {where}.scaling.high must be above low")


def _check_parallel(mx, where: str) -> None:
    left, right = _need(mx, "left", None, where), _need(mx, "right", None, where)
    _need(mx, "left_scale", float, where)
    _need(mx, "right_scale", float, where)
    for key in ("heads", "kv_heads", "dim", "vdim"):
        _need(left, key, int, where + ".left")
        _need(right, key, int, where + ".right")
    _need(left, "scale", float, where + ".left")
    if left.get("softcap") is not None and not (_need(left, "softcap", float, where + ".left") > 0):
        raise ConfigError(f"config.json: {where}.left.softcap must be positive")
    _check_rot(_need(left, "rot", None, where + ".left"), where + ".left.rot", int(left["dim"]))
    if _need(right, "conv", int, where + ".right") > 16:
        raise ConfigError(f"config.json: {where}.right.conv {right['conv']}: at most 16 taps")
    for side, part in (("left", left), ("right", right)):
        if part["heads"] % part["kv_heads"]:
            raise ConfigError(f"config.json: {where}.{side}.heads must be a multiple of kv_heads")


def _check_latent(mx, where: str) -> None:
    for key in ("heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank"):
        _need(mx, key, int, where)
    _need(mx, "scale", float, where)
    if mx.get("mask") is not None:
        _need(mx["mask"], "size", int, where + ".mask")
    _check_rot(_need(mx, "rot", None, where), where + ".rot", int(mx["rot_dim"]))


@dataclass(frozen=True)
class PapusunConfig(ModelConfig):
    architecture: ClassVar[str] = "Papusun"

    vocab: int
    width: int
    norm_eps: float
    logit_scale: float
    side_dim: int                     # 0: no per-layer token input
    layers: Tuple[Mapping[str, Any], ...]

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "PapusunConfig":
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        side = raw.get("token_side")
        cfg = cls(vocab=cls._get(raw, "vocab", int), width=cls._get(raw, "width", int),
                  norm_eps=_need(raw.get("norm") or {}, "eps", float, "norm"),
                  logit_scale=cls._get(raw, "logit_scale", float, 1.0),
                  side_dim=_need(side, "dim", int, "token_side") if side else 0, layers=tuple(layers))
        cfg.validate()
        return cfg

    def to_dict(self) -> Dict[str, Any]:
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
               "norm": {"eps": self.norm_eps}, "logit_scale": self.logit_scale,
               "layers": [dict(L) for L in self.layers]}
        if self.side_dim:
            out["token_side"] = {"dim": self.side_dim}
        return out

    def kv_source(self, i: int) -> Optional[int]:
        """The layer whose cache rows latent-attention layer i reads (None: its own)."""
        src = self.layers[i]["mixer"].get("kv_from")
        return None if src is None else int(src)

    def cache_window(self, i: int) -> Optional[int]:
        """The window that the cache of latent-attention layer i keeps: the longest window among the layer and the
        layers that read its rows (None: one of them sees every key)."""
        sizes = []
        for j, L in enumerate(self.layers):
            if L["type"] == "latent_attention" and (j == i or self.kv_source(j) == i):
                mask = L["mixer"].get("mask")
                if mask is None:
                    return None
                sizes.append(int(mask["size"]))
        return max(sizes)

    def validate(self) -> None:
        if self.vocab <= 0 or self.width <= 0:
            raise ConfigError("config.json: 'vocab' and 'width' must be positive")
        if not (self.norm_eps > 0):
            raise ConfigError(f"config.json: norm.eps must be > 0, got {self.norm_eps}")
        for i, L in enumerate(self.layers):
            where = f"layers[{i}]"
            kind = _need(L, "type", str, where)
            if kind not in MIXERS:
                raise ConfigError(f"config.json: {where}.type '{kind}' is not one of {MIXERS}")
            mx = _need(L, "mixer", None, where)
            if kind == "parallel":
                _check_parallel(mx, where + ".mixer")
            else:
                _check_latent(mx, where + ".mixer")
                src = mx.get("kv_from")
                if src is not None:
                    if isinstance(src, bool) or not isinstance(src, int) or not (0 <= src < i):
                        raise ConfigError(f"config.json: {where}.mixer.kv_from must name an earlier layer")
                    S = self.layers[src]
                    if S.get("type") != "latent_attention" or S["mixer"].get("kv_from") is not None:
                        raise ConfigError(f"config.json: {where}.mixer.kv_from: layer {src} has no cache rows of its own")
                    for key in ("kv_rank", "rot_dim"):
                        if int(S["mixer"][key]) != int(mx[key]):
                            raise ConfigError(f"config.json: {where}.mixer.{key} differs from layer {src}'s")
            ml = L.get("mlp")
            if ml is not None:
                if _need(ml, "kind", str, where + ".mlp") != "dense":
                    raise ConfigError(f"config.json: {where}.mlp.kind '{ml['kind']}' is not 'dense'")
                _need(ml, "ff", int, where + ".mlp")
