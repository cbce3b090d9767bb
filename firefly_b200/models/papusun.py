"""Papusun as data: a ``ModelSpec`` made of registered parts.

Pre-norm blocks (``pre_norm``) whose norms are layer norms with a weight and no bias, and whose last step is an
input from the token itself (the block's tail, ``token_side``): every layer reads its own slice of one table of
rows per token id.  A layer's mixer is either two mixers side by side (``parallel``): grouped-query softmax attention
over every earlier key with biases, a partly rotated head (interleaved pairs, frequencies rescaled by wavelength
bands) and capped scores (``gqa_attention`` with its parameters), beside a gated delta rule with one decay per head
(``gated_delta``); or attention over a cached latent vector inside a sliding window, its queries made through a
latent of their own and its heads gated one by one (``latent_attention`` with its parameters).  A latent-attention
layer may read the cache rows of an earlier one: its run of the schedule then points at that run's cache slot and
writes nothing.  The feed-forward is SwiGLU (``gated_mlp``) or nothing.  The output is the same kind of norm and a
head of its own, the logits times a constant.
Tensor names: ``embed``, ``side.embed``, ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.*``, ``l<i>.mlp.*``,
``l<i>.side.*``, ``final.norm``, ``head``.
"""
from __future__ import annotations

from ..config.base import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from ..config.papusun import PapusunConfig
from .registry import register_architecture

# The design has no longest position (angles are formed from the position, windows and states have no length); the
# engine's block tables and its cache sizing still want a bound on a request's length.
MAX_POSITIONS = 1 << 20


def _norm(cfg: PapusunConfig, prefix: str) -> PartSpec:
    return PartSpec("layer_norm", dict(size=cfg.width, eps=cfg.norm_eps, weight_leaf="", bias_leaf=None), prefix=prefix)


def _rotary(rot, head_dim: int) -> PartSpec:
    sc = rot.get("scaling")
    scaling = dict(kind="wavelength_bands", factor=float(sc["factor"]), low=float(sc["low"]), high=float(sc["high"]),
                   original=float(sc["original"])) if sc else None
    return PartSpec("rotary", dict(head_dim=head_dim, rotary_dim=int(rot["dims"]), theta=float(rot["base"]),
                                   max_positions=0, pairing="interleaved", scaling=scaling))


def _mixer(cfg: PapusunConfig, i: int, L):
    """(mixer, its position part or None)."""
    W, mx, p = cfg.width, L["mixer"], f"l{i}.mix"
    if L["type"] == "parallel":
        left, right = mx["left"], mx["right"]
        attention = PartSpec("gqa_attention", dict(
            hidden_size=W, num_heads=int(left["heads"]), num_kv_heads=int(left["kv_heads"]), head_dim=int(left["dim"]),
            value_dim=int(left["vdim"]), scale=float(left["scale"]), softcap=float(left.get("softcap") or 0.0),
            bias_suffix=".b", q_leaf="q", k_leaf="k", v_leaf="v", o_leaf="o"), prefix=f"{p}.left")
        delta = PartSpec("gated_delta", dict(
            hidden_size=W, heads=int(right["heads"]), kv_heads=int(right["kv_heads"]), dim=int(right["dim"]),
            vdim=int(right["vdim"]), conv=int(right["conv"]), eps=cfg.norm_eps), prefix=f"{p}.right")
        return PartSpec("parallel", dict(mixers=(attention, delta), positions=(_rotary(left["rot"], int(left["dim"])), None),
                                         scales=(float(mx["left_scale"]), float(mx["right_scale"]))), prefix=p), None
    src = cfg.kv_source(i)
    mask = mx.get("mask")
    mixer = PartSpec("latent_attention", dict(
        hidden_size=W, heads=int(mx["heads"]), dim=int(mx["dim"]), rot_dim=int(mx["rot_dim"]), vdim=int(mx["vdim"]),
        kv_rank=int(mx["kv_rank"]), q_rank=int(mx["q_rank"]), scale=float(mx["scale"]), eps=cfg.norm_eps,
        window=int(mask["size"]) if mask else None, cache_window=cfg.cache_window(i if src is None else src),
        has_kv=src is None, gate="head"), prefix=p)
    return mixer, _rotary(mx["rot"], int(mx["rot_dim"]))


def papusun_spec(cfg: PapusunConfig) -> ModelSpec:
    layers, runs = [], []
    n = len(cfg.layers)
    for i, L in enumerate(cfg.layers):
        p = f"l{i}"
        ml = L.get("mlp")
        ff = PartSpec("gated_mlp", dict(hidden_size=cfg.width, intermediate_size=int(ml["ff"]), activation="silu"),
                      prefix=f"{p}.mlp") if ml is not None else None
        norms = (_norm(cfg, f"{p}.norm1"),) + ((_norm(cfg, f"{p}.norm2"),) if ff is not None else ())
        params = {}
        if cfg.side_dim:
            params["tail"] = PartSpec("token_side", dict(
                hidden_size=cfg.width, dim=cfg.side_dim, vocab_size=cfg.vocab, table="side.embed",
                table_cols=n * cfg.side_dim, col0=i * cfg.side_dim, eps=cfg.norm_eps, activation="gelu_tanh"),
                prefix=f"{p}.side")
        mixer, position = _mixer(cfg, i, L)
        layers.append(LayerSpec("pre_norm", mixer, ff, norms, position, params=params))
        src = cfg.kv_source(i) if L["type"] == "latent_attention" else None
        runs.append(ScheduleEntry(i) if src is None else ScheduleEntry(i, cache=src, write_cache=False))
    return ModelSpec(
        vocab_size=cfg.vocab, hidden_size=cfg.width, max_positions=MAX_POSITIONS,
        embedding=PartSpec("token_embedding", dict(vocab_size=cfg.vocab, hidden_size=cfg.width, tensor="embed")),
        layers=tuple(layers), schedule=tuple(runs), final_norm=_norm(cfg, "final.norm"),
        head=PartSpec("lm_head", dict(vocab_size=cfg.vocab, hidden_size=cfg.width, tensor="head", scale=cfg.logit_scale)),
    )


register_architecture("Papusun", PapusunConfig, papusun_spec)
