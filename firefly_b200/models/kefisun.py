"""Kefisun as data: a ``ModelSpec`` made of registered parts.

Pre-norm blocks (``pre_norm``) whose norms are RMS norms with a weight stored around zero (multiplier 1 + w) and
whose mixer reads its normed input through a short causal convolution added to that input (the block's input
filter, ``causal_conv_filter``).  A layer's mixer is softmax attention behind short convolutions with a norm over
the whole projection, a bias by distance inside a sliding window, values blended with the first blending layer's
and a sigmoid output gate (``conv_attention``), or a gated delta rule with a decay per key channel
(``channel_delta``).  Its feed-forward is a gated MLP with biases and a clamped activation, or nothing.  The
embedding rows enter the stream times a constant; the output is the same kind of norm and the embedding table as
the head, the logits times a constant.
Tensor names: ``embed``, ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.canon1``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``.
"""
from __future__ import annotations

from ..config.base import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from ..config.kefisun import DEFAULT_RANK, KefisunConfig, file_hints
from .registry import register_architecture

# The design has no longest position (windows and states have no length); the engine's block tables and its cache
# sizing still want a bound on a request's length.
MAX_POSITIONS = 1 << 20


def _norm(cfg: KefisunConfig, tensor: str) -> PartSpec:
    return PartSpec("rms_norm", dict(size=cfg.width, eps=cfg.norm_eps, weight_offset=1.0, tensor=tensor))


def _mixer(cfg: KefisunConfig, i: int, L, first_mixer: int) -> PartSpec:
    W, mx, p = cfg.width, L["mixer"], f"l{i}.mix"
    if L["type"] == "attention":
        mix = None
        if mx.get("v_mix", False):
            mix = "first" if i == first_mixer else "blend"
        return PartSpec("conv_attention", dict(
            hidden_size=W, heads=int(mx["heads"]), kv_heads=int(mx["kv_heads"]), dim=int(mx["dim"]), vdim=int(mx["vdim"]),
            conv=int(mx["conv"]), scale=float(mx["scale"]), window=int(mx["mask"]["size"]), eps=cfg.norm_eps,
            distance_bias=True, value_mix=mix, value_key="v_first"), prefix=p)
    return PartSpec("channel_delta", dict(
        hidden_size=W, heads=int(mx["heads"]), kv_heads=int(mx["kv_heads"]), dim=int(mx["dim"]), vdim=int(mx["vdim"]),
        conv=int(mx["conv"]), decay_rank=int(mx.get("decay_rank", DEFAULT_RANK)),
        gate_rank=int(mx.get("gate_rank", DEFAULT_RANK)), eps=cfg.norm_eps), prefix=p)


def _feed_forward(cfg: KefisunConfig, ml, p: str):
    if ml is None:
        return None
    return PartSpec("gated_mlp", dict(hidden_size=cfg.width, intermediate_size=int(ml["ff"]), activation="clamped_swish",
                                      limit=float(ml["limit"]), bias=True, bias_suffix=".b"), prefix=f"{p}.mlp")


def kefisun_spec(cfg: KefisunConfig) -> ModelSpec:
    layers = []
    first_mixer = cfg.first_value_mixer()
    for i, L in enumerate(cfg.layers):
        p = f"l{i}"
        ff = _feed_forward(cfg, L.get("mlp"), p)
        norms = (_norm(cfg, f"{p}.norm1"),) + ((_norm(cfg, f"{p}.norm2"),) if ff is not None else ())
        canon = PartSpec("causal_conv_filter", dict(size=cfg.width, taps=cfg.canon_taps, tensor=f"{p}.canon1"))
        layers.append(LayerSpec("pre_norm", _mixer(cfg, i, L, first_mixer), ff, norms, params=dict(input_filter=canon)))
    return ModelSpec(
        vocab_size=cfg.vocab, hidden_size=cfg.width, max_positions=MAX_POSITIONS,
        embedding=PartSpec("token_embedding", dict(vocab_size=cfg.vocab, hidden_size=cfg.width, tensor="embed",
                                                   scale=cfg.embedding_scale)),
        layers=tuple(layers), schedule=tuple(ScheduleEntry(i) for i in range(len(layers))),
        final_norm=_norm(cfg, "final.norm"),
        head=PartSpec("lm_head", dict(vocab_size=cfg.vocab, hidden_size=cfg.width, tied_to="embed", tensor="head",
                                      scale=cfg.logit_scale)),
    )


register_architecture("Kefisun", KefisunConfig, kefisun_spec, file_hints=file_hints)
