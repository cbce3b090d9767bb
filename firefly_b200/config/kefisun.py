"""Typed configuration of the Kefisun design.

``config.json`` names the design under ``architecture`` and gives every size and constant:

    vocab, width, norm.eps, canon.taps, embedding.scale, logit_scale
    layers[i]: type ("attention" | "channel_delta"), mixer {...}, mlp {...} | null
        attention mixer:      heads, kv_heads, dim, vdim, conv, scale, mask {size}, v_mix (optional, false)
        channel_delta mixer:  heads, kv_heads, dim, vdim, conv
        mlp kind "dense":     ff, limit

Two sizes of a channel_delta mixer come from the checkpoint's tensor shapes, which is where they are written:
the inner sizes of its two-step projections (``decay_rank``: rows of ``a1``; ``gate_rank``: rows of ``g1``).
The nested objects are kept as they are and checked here, so that a wrong or missing key is told by name before
anything is built.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, ClassVar, Dict, Mapping, Tuple

from .base import ConfigError, ModelConfig
from .pepolorn import _need

MIXERS = ("attention", "channel_delta")
DEFAULT_RANK = 16          # inner size of the two-step projections when neither the configuration nor a file says


def _check_mixer(kind: str, mx, where: str) -> None:
    for key in ("heads", "kv_heads", "dim", "vdim", "conv"):
        _need(mx, key, int, where)
    if mx["heads"] % mx["kv_heads"]:
        raise ConfigError(f"config.json: {where}.heads must be a multiple of kv_heads")
    if kind == "attention":
        _need(mx, "scale", float, where)
        _need(_need(mx, "mask", None, where), "size", int, where + ".mask")
        if not isinstance(mx.get("v_mix", False), bool):
            raise ConfigError(f"config.json: {where}.v_mix must be true or false")
    else:
        for key in ("decay_rank", "gate_rank"):
            if key in mx:
                _need(mx, key, int, where)


@dataclass(frozen=True)
class KefisunConfig(ModelConfig):
    architecture: ClassVar[str] = "Kefisun"

    vocab: int
    width: int
    norm_eps: float
    canon_taps: int
    embedding_scale: float
    logit_scale: float
    layers: Tuple[Mapping[str, Any], ...]

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "KefisunConfig":
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        cfg = cls(vocab=cls._get(raw, "vocab", int), width=cls._get(raw, "width", int),
                  norm_eps=_need(raw.get("norm") or {}, "eps", float, "norm"),
                  canon_taps=_need(raw.get("canon") or {}, "taps", int, "canon"),
                  embedding_scale=_need(raw.get("embedding") or {}, "scale", float, "embedding"),
                  logit_scale=cls._get(raw, "logit_scale", float), layers=tuple(layers))
        cfg.validate()
        return cfg

    def to_dict(self) -> Dict[str, Any]:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "norm": {"eps": self.norm_eps}, "canon": {"taps": self.canon_taps},
                "embedding": {"scale": self.embedding_scale}, "logit_scale": self.logit_scale,
                "layers": [dict(L) for L in self.layers]}

    def first_value_mixer(self) -> int:
        """The first layer whose values the later value-mixing layers blend in (-1: no layer mixes values)."""
        for i, L in enumerate(self.layers):
            if L["type"] == "attention" and L["mixer"].get("v_mix", False):
                return i
        return -1

    def validate(self) -> None:
        if self.vocab <= 0 or self.width <= 0:
            raise ConfigError("config.json: 'vocab' and 'width' must be positive")
        if not (self.norm_eps > 0):
            raise ConfigError(f"config.json: norm.eps must be > 0, got {self.norm_eps}")
        if self.canon_taps > 16:
            raise ConfigError(f"config.json: canon.taps {self.canon_taps}: at most 16 taps")
        shared = None
        for i, L in enumerate(self.layers):
            where = f"layers[{i}]"
            kind = _need(L, "type", str, where)
            if kind not in MIXERS:
                raise ConfigError(f"config.json: {where}.type '{kind}' is not one of {MIXERS}")
            mx = _need(L, "mixer", None, where)
            _check_mixer(kind, mx, where + ".mixer")
            if mx["conv"] > 16:
                raise ConfigError(f"config.json: {where}.mixer.conv {mx['conv']}: at most 16 taps")
            if kind == "attention" and mx.get("v_mix", False):
                size = int(mx["kv_heads"]) * int(mx["vdim"])
                if shared is not None and shared != size:
                    raise ConfigError(f"config.json: {where}.mixer mixes values of {size} channels with the first "
                                      f"such layer's {shared}")
                shared = size
            ml = L.get("mlp")
            if ml is not None:
                if _need(ml, "kind", str, where + ".mlp") != "dense":
                    raise ConfigError(f"config.json: {where}.mlp.kind '{ml['kind']}' is not 'dense'")
                _need(ml, "ff", int, where + ".mlp")
                if not (_need(ml, "limit", float, where + ".mlp") > 0):
                    raise ConfigError(f"config.json: {where}.mlp.limit must be positive")


def file_hints(raw: Mapping[str, Any], shapes: Mapping[str, Tuple[int, ...]]) -> Mapping[str, Any]:
    """Sizes that only the tensors' shapes give: the inner sizes of each channel_delta mixer's two-step projections."""
    layers = raw.get("layers")
    if not isinstance(layers, list):
        return raw
    out = []
    for i, L in enumerate(layers):
        if isinstance(L, dict) and L.get("type") == "channel_delta" and isinstance(L.get("mixer"), dict):
            mx = dict(L["mixer"])
            for key, leaf in (("decay_rank", "a1"), ("gate_rank", "g1")):
                name = f"l{i}.mix.{leaf}"
                if key not in mx and name in shapes and len(shapes[name]) == 2:
                    mx[key] = int(shapes[name][0])
            L = dict(L, mixer=mx)
        out.append(L)
    return dict(raw, layers=out)
