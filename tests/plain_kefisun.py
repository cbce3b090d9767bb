"""A plain, slow implementation of the Kefisun design, one function per mechanism, written from the design's
equations and sharing no code with the package.  Everything runs on whole sequences in one floating type
(float64 by default), on the CPU; the tests hold the engine against it in every cutting of a prompt.

Notation: W the width, T the tokens of one sequence, rms(v) = v / sqrt(mean(v^2) + eps).

    x0      = E[token] * embedding_scale
    layer:    h = (1 + n1) rms(x);  h <- h + conv_c(h);  x <- x + mixer(h);  x <- x + ff((1 + n2) rms(x))
    logits  = E ((1 + nf) rms(x)) * logit_scale

conv_w(u)_t = sum_j w[:, j] u_(t - taps + 1 + j) per channel, zeros in front of the sequence.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def rms(v: torch.Tensor, eps: float) -> torch.Tensor:
    return v / torch.sqrt((v * v).mean(dim=-1, keepdim=True) + eps)


def offset_norm(x, w, eps):
    """RMS norm whose weight is stored around zero."""
    return rms(x, eps) * (1.0 + w)


def causal_conv(u: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """u [T, C], w [C, taps]; the last column weighs the current token; zeros in front of the sequence."""
    T, C = u.shape
    taps = w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=u.dtype), u], dim=0)
    out = torch.zeros_like(u)
    for j in range(taps):
        out = out + padded[j:j + T] * w[:, j]
    return out


def distance_bias(r1: torch.Tensor, r2: torch.Tensor, T: int) -> torch.Tensor:
    """[heads, T, T]: r1_h * ln(1 + r2_h * (i - j)) where i >= j (0 elsewhere; those keys are masked)."""
    i = torch.arange(T).view(T, 1)
    j = torch.arange(T).view(1, T)
    dist = (i - j).clamp(min=0).to(r1.dtype)
    return r1.view(-1, 1, 1) * torch.log(1.0 + r2.view(-1, 1, 1) * dist)


def window_mask(T: int, size: int) -> torch.Tensor:
    """[T, T] bool: query i sees key j when 0 <= i - j < size."""
    i = torch.arange(T).view(T, 1)
    j = torch.arange(T).view(1, T)
    return (i - j >= 0) & (i - j < size)


def attention_values(h, w, p, mx):
    """The values a layer caches before any mixing: projection, then the short convolution."""
    return causal_conv(h @ w[p + ".v"].T, w[p + ".v.conv"])


def attention_mixer(h, w: Dict[str, torch.Tensor], p: str, mx, eps: float, v_first: Optional[torch.Tensor]):
    """Returns (output [T, W], this layer's values before mixing).  ``v_first`` None: this layer is the first of
    those that mix values (or mixes none)."""
    T = h.shape[0]
    H, G, D, V = int(mx["heads"]), int(mx["kv_heads"]), int(mx["dim"]), int(mx["vdim"])
    q = causal_conv(h @ w[p + ".q"].T, w[p + ".q.conv"])
    k = causal_conv(h @ w[p + ".k"].T, w[p + ".k.conv"])
    v = attention_values(h, w, p, mx)
    v_own = v
    q = rms(q, eps) * w[p + ".q.norm"]            # over the whole projection, all heads at once
    k = rms(k, eps) * w[p + ".k.norm"]
    if mx.get("v_mix") and v_first is not None:
        lam = w[p + ".vmix"]
        v = (1.0 - lam) * v + lam * v_first
    q = q.view(T, H, D).transpose(0, 1)            # [H, T, D]
    k = k.view(T, G, D).transpose(0, 1)
    v = v.view(T, G, V).transpose(0, 1)
    rep = H // G
    k = k.repeat_interleave(rep, dim=0)
    v = v.repeat_interleave(rep, dim=0)
    s = q @ k.transpose(1, 2) * float(mx["scale"]) - distance_bias(w[p + ".r1"], w[p + ".r2"], T)
    s = s.masked_fill(~window_mask(T, int(mx["mask"]["size"])), float("-inf"))
    a = torch.softmax(s, dim=-1)
    o = (a @ v).transpose(0, 1).reshape(T, H * V)
    o = o * torch.sigmoid(h @ w[p + ".g"].T)
    return o @ w[p + ".o"].T, v_own


def silu(z):
    return z * torch.sigmoid(z)


def unit(v):
    return v / torch.sqrt((v * v).sum(dim=-1, keepdim=True) + 1e-6)


def delta_recurrence(q, k, v, beta, g):
    """One head.  q, k, g [T, D]; v [T, V]; beta [T].  S [D, V] starts at zero.
    S <- diag(g_t) S;  u = beta_t (v_t - S^T k_t);  S <- S + k_t u^T;  o_t = S^T q_t."""
    T, D = q.shape
    V = v.shape[1]
    S = torch.zeros(D, V, dtype=q.dtype)
    out = []
    for t in range(T):
        S = g[t].view(D, 1) * S
        u = beta[t] * (v[t] - S.T @ k[t])
        S = S + torch.outer(k[t], u)
        out.append(S.T @ q[t])
    return torch.stack(out) if out else torch.zeros(0, V, dtype=q.dtype)


def channel_delta_mixer(h, w: Dict[str, torch.Tensor], p: str, mx, eps: float):
    T = h.shape[0]
    H, G, D, V = int(mx["heads"]), int(mx["kv_heads"]), int(mx["dim"]), int(mx["vdim"])
    q = silu(causal_conv(h @ w[p + ".q"].T, w[p + ".q.conv"])).view(T, G, D)
    k = silu(causal_conv(h @ w[p + ".k"].T, w[p + ".k.conv"])).view(T, G, D)
    v = silu(causal_conv(h @ w[p + ".v"].T, w[p + ".v.conv"])).view(T, H, V)
    q = unit(q) * D ** -0.5
    k = unit(k)
    beta = torch.sigmoid(h @ w[p + ".b"].T)                                     # [T, H]
    step = torch.nn.functional.softplus((h @ w[p + ".a1"].T) @ w[p + ".a2"].T + w[p + ".dt_bias"])
    g = torch.exp(-torch.exp(w[p + ".A_log"]).view(1, H, 1) * step.view(T, H, D))
    gate = torch.sigmoid((h @ w[p + ".g1"].T) @ w[p + ".g2"].T).view(T, H, V)
    rep = H // G
    heads = []
    for hd in range(H):
        o = delta_recurrence(q[:, hd // rep], k[:, hd // rep], v[:, hd], beta[:, hd], g[:, hd])
        heads.append(rms(o, eps) * w[p + ".norm"] * gate[:, hd])
    return torch.cat(heads, dim=-1) @ w[p + ".o"].T


def dense_ff(h, w: Dict[str, torch.Tensor], p: str, ml):
    limit = float(ml["limit"])
    g = (h @ w[p + ".gate"].T + w[p + ".gate.b"]).clamp(max=limit)
    u = (h @ w[p + ".up"].T + w[p + ".up.b"]).clamp(min=-limit, max=limit)
    y = g * torch.sigmoid(1.702 * g) * (u + 1.0)
    return y @ w[p + ".down"].T + w[p + ".down.b"]


def forward(config: dict, weights: Dict[str, torch.Tensor], tokens: List[int], dtype=torch.float64,
            layer_outputs: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence.  ``layer_outputs``: a list that receives the stream after every layer."""
    w = {k: (t.to(dtype) if t.is_floating_point() else t) for k, t in weights.items()}
    eps = float(config["norm"]["eps"])
    x = w["embed"][torch.tensor(tokens, dtype=torch.long)] * float(config["embedding"]["scale"])
    v_first = None
    for i, L in enumerate(config["layers"]):
        p = f"l{i}"
        h = offset_norm(x, w[p + ".norm1"], eps)
        h = h + causal_conv(h, w[p + ".canon1"])
        if L["type"] == "attention":
            delta, v_own = attention_mixer(h, w, p + ".mix", L["mixer"], eps, v_first)
            if L["mixer"].get("v_mix") and v_first is None:
                v_first = v_own
        elif L["type"] == "channel_delta":
            delta = channel_delta_mixer(h, w, p + ".mix", L["mixer"], eps)
        else:
            raise ValueError(L["type"])
        x = x + delta
        if L.get("mlp") is not None:
            x = x + dense_ff(offset_norm(x, w[p + ".norm2"], eps), w, p + ".mlp", L["mlp"])
        if layer_outputs is not None:
            layer_outputs.append(x.clone())
    return (offset_norm(x, w["final.norm"], eps) @ w["embed"].T) * float(config["logit_scale"])


def tensor_shapes(config: dict, ranks: Optional[dict] = None) -> Dict[str, tuple]:
    """Names and shapes of a model's tensors.  ``ranks``: {"a": r, "g": r} inner sizes of the channel_delta mixer's
    two-step projections (config.json does not give them; a checkpoint's shapes do)."""
    ranks = ranks or {"a": 8, "g": 8}
    W, taps = int(config["width"]), int(config["canon"]["taps"])
    out = {"embed": (int(config["vocab"]), W), "final.norm": (W,)}
    for i, L in enumerate(config["layers"]):
        p, mx = f"l{i}", L["mixer"]
        out[p + ".norm1"] = (W,)
        out[p + ".canon1"] = (W, taps)
        H, G, D, V, c = int(mx["heads"]), int(mx["kv_heads"]), int(mx["dim"]), int(mx["vdim"]), int(mx["conv"])
        m = p + ".mix"
        if L["type"] == "attention":
            out.update({m + ".q": (H * D, W), m + ".k": (G * D, W), m + ".v": (G * V, W),
                        m + ".q.norm": (H * D,), m + ".k.norm": (G * D,),
                        m + ".q.conv": (H * D, c), m + ".k.conv": (G * D, c), m + ".v.conv": (G * V, c),
                        m + ".vmix": (), m + ".r1": (H,), m + ".r2": (H,), m + ".g": (H * V, W), m + ".o": (W, H * V)})
        else:
            out.update({m + ".q": (G * D, W), m + ".q.conv": (G * D, c), m + ".k": (G * D, W), m + ".k.conv": (G * D, c),
                        m + ".v": (H * V, W), m + ".v.conv": (H * V, c), m + ".b": (H, W), m + ".A_log": (H,),
                        m + ".norm": (V,), m + ".a1": (ranks["a"], W), m + ".a2": (H * D, ranks["a"]),
                        m + ".dt_bias": (H * D,), m + ".g1": (ranks["g"], W), m + ".g2": (H * V, ranks["g"]),
                        m + ".o": (W, H * V)})
        if L.get("mlp") is not None:
            F = int(L["mlp"]["ff"])
            out[p + ".norm2"] = (W,)
            f = p + ".mlp"
            out.update({f + ".gate": (F, W), f + ".gate.b": (F,), f + ".up": (F, W), f + ".up.b": (F,),
                        f + ".down": (W, F), f + ".down.b": (W,)})
    return out


def random_weights(config: dict, seed: int = 0, ranks: Optional[dict] = None) -> Dict[str, torch.Tensor]:
    """Random tensors of a size that keeps every mechanism alive: matrices ~ 1/sqrt(columns), norm weights and
    biases around zero, plain norm weights around one, positive distance constants, a mix factor inside (0, 1).
    Values are rounded to bfloat16 so that a bfloat16 engine holds the same numbers."""
    gen = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(config, ranks).items():
        leaf = name.split(".", 1)[1] if name.startswith("l") and "." in name else name
        if name == "embed":
            t = torch.randn(shape, generator=gen) * 0.5
        elif leaf in ("norm1", "norm2") or name == "final.norm":
            t = torch.randn(shape, generator=gen) * 0.1
        elif leaf == "canon1" or leaf.endswith(".conv"):
            t = torch.randn(shape, generator=gen) * 0.4
        elif leaf.endswith("q.norm") or leaf.endswith("k.norm") or leaf == "mix.norm":
            t = 1.0 + torch.randn(shape, generator=gen) * 0.1
        elif leaf == "mix.vmix":
            t = torch.tensor(0.35)
        elif leaf == "mix.r1":
            t = 0.3 + torch.rand(shape, generator=gen)
        elif leaf == "mix.r2":
            t = 0.2 + torch.rand(shape, generator=gen)
        elif leaf == "mix.A_log":
            t = torch.randn(shape, generator=gen) * 0.5 - 1.0
        elif leaf == "mix.dt_bias" or leaf.endswith(".b") and len(shape) == 1:
            t = torch.randn(shape, generator=gen) * 0.3
        else:
            t = torch.randn(shape, generator=gen) / math.sqrt(shape[-1])
            if leaf.endswith(".q") or leaf.endswith(".k") or leaf.endswith(".v"):
                t = t * 2.0
        out[name] = t.to(torch.bfloat16).to(torch.float32)
    return out
