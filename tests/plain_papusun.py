"""A plain, slow implementation of the Papusun design, one function per mechanism, written from the design's
equations and sharing no code with the package.  Everything runs on whole sequences in one floating type
(float64 by default), on the CPU; the tests hold the engine against it in every cutting of a prompt.

Notation: W the width, T the tokens of one sequence, ln(v) = (v - mean) / sqrt(var + eps) * w,
rms(v) = v / sqrt(mean(v^2) + eps).

    x0      = E[token]
    layer i:  x <- x + mixer(ln1(x));  x <- x + ff(ln2(x));
              e = S[token][i d : (i+1) d];  y = P (gelu_tanh(G x) * e);  x <- x + rms(y) * n
    logits  = H lnf(x) * logit_scale
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def rms(v: torch.Tensor, eps: float) -> torch.Tensor:
    return v / torch.sqrt((v * v).mean(dim=-1, keepdim=True) + eps)


def layer_norm(x, w, eps):
    mu = x.mean(dim=-1, keepdim=True)
    var = ((x - mu) ** 2).mean(dim=-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def causal_conv(u: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """u [T, C], w [C, taps]; the last column weighs the current token; zeros in front of the sequence."""
    T, C = u.shape
    taps = w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=u.dtype), u], dim=0)
    out = torch.zeros_like(u)
    for j in range(taps):
        out = out + padded[j:j + T] * w[:, j]
    return out


def rotary_frequencies(rot: dict, dtype=torch.float64) -> torch.Tensor:
    """f_i = base^(-2i/dims), rescaled by wavelength bands when ``scaling`` is given."""
    dims = int(rot["dims"])
    f = torch.tensor([float(rot["base"]) ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=dtype)
    sc = rot.get("scaling")
    if not sc:
        return f
    factor, low, high, original = float(sc["factor"]), float(sc["low"]), float(sc["high"]), float(sc["original"])
    out = []
    for fi in f.tolist():
        wavelength = 2.0 * math.pi / fi
        if wavelength < original / high:
            out.append(fi)
        elif wavelength > original / low:
            out.append(fi / factor)
        else:
            s = (original / wavelength - low) / (high - low)
            out.append((1.0 - s) * fi / factor + s * fi)
    return torch.tensor(out, dtype=dtype)


def rotate_pairs(x: torch.Tensor, freq: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
    """x [T, heads, n]: the first 2 len(freq) elements of every head turn, element 2i with element 2i+1."""
    r = 2 * freq.numel()
    ang = positions.to(x.dtype).view(-1, 1, 1) * freq.to(x.dtype).view(1, 1, -1)
    c, s = torch.cos(ang), torch.sin(ang)
    u, v = x[..., 0:r:2], x[..., 1:r:2]
    out = x.clone()
    out[..., 0:r:2] = u * c - v * s
    out[..., 1:r:2] = v * c + u * s
    return out


def visible(T: int, window: Optional[int]) -> torch.Tensor:
    """[T, T] bool: query i sees key j when j <= i (and i - j < window where there is one)."""
    i = torch.arange(T).view(T, 1)
    j = torch.arange(T).view(1, T)
    ok = j <= i
    if window is not None:
        ok = ok & (i - j < window)
    return ok


def softmax_attention(q, k, v, scale, mask, softcap=None):
    """q [T, H, d], k [T, H, d], v [T, H, dv] (already one key/value head per query head) -> [T, H, dv]."""
    s = torch.einsum("ihd,jhd->hij", q, k) * scale
    if softcap:
        s = softcap * torch.tanh(s / softcap)
    s = s.masked_fill(~mask.unsqueeze(0), float("-inf"))
    p = torch.softmax(s, dim=-1)
    return torch.einsum("hij,jhd->ihd", p, v)


def capped_attention(h, w, p, mx, positions):
    """Grouped-query softmax attention with biases, a partly rotated head and capped scores."""
    T = h.shape[0]
    H, G, d, dv = int(mx["heads"]), int(mx["kv_heads"]), int(mx["dim"]), int(mx["vdim"])
    q = (h @ w[p + ".q"].T + w[p + ".q.b"]).view(T, H, d)
    k = (h @ w[p + ".k"].T + w[p + ".k.b"]).view(T, G, d)
    v = (h @ w[p + ".v"].T + w[p + ".v.b"]).view(T, G, dv)
    freq = rotary_frequencies(mx["rot"], h.dtype)
    q, k = rotate_pairs(q, freq, positions), rotate_pairs(k, freq, positions)
    rep = H // G
    k, v = k.repeat_interleave(rep, dim=1), v.repeat_interleave(rep, dim=1)
    o = softmax_attention(q, k, v, float(mx["scale"]), visible(T, None), mx.get("softcap"))
    return o.reshape(T, H * dv) @ w[p + ".o"].T


def delta_rule(h, w, p, mx, eps):
    """The gated delta rule with one decay per head; the read-out sees the current token's write."""
    T = h.shape[0]
    H, G, d, dv = int(mx["heads"]), int(mx["kv_heads"]), int(mx["dim"]), int(mx["vdim"])
    q = silu(causal_conv(h @ w[p + ".q"].T, w[p + ".q.conv"])).view(T, G, d)
    k = silu(causal_conv(h @ w[p + ".k"].T, w[p + ".k.conv"])).view(T, G, d)
    v = silu(causal_conv(h @ w[p + ".v"].T, w[p + ".v.conv"])).view(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w[p + ".b"].T)                                                   # [T, H]
    g = torch.exp(-torch.exp(w[p + ".A_log"]) * softplus(h @ w[p + ".a"].T + w[p + ".dt_bias"]))   # [T, H]
    rep = H // G
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for a in range(H):
        S = torch.zeros(d, dv, dtype=h.dtype)
        for t in range(T):
            kt, qt = k[t, a // rep], q[t, a // rep]
            S = g[t, a] * S
            u = beta[t, a] * (v[t, a] - S.T @ kt)
            S = S + torch.outer(kt, u)
            out[t, a] = S.T @ qt
    out = rms(out, eps) * w[p + ".norm"]
    gate = silu(h @ w[p + ".g"].T).view(T, H, dv)
    return (out * gate).reshape(T, H * dv) @ w[p + ".o"].T


def parallel_mixer(h, w, p, mx, positions, eps):
    return float(mx["left_scale"]) * capped_attention(h, w, p + ".left", mx["left"], positions) \
        + float(mx["right_scale"]) * delta_rule(h, w, p + ".right", mx["right"], eps)


def latent_rows(h, w, p, mx, positions, eps):
    """What the cache of a latent-attention layer holds per token: (c [T, kv_rank], rotated key part [T, rot_dim])."""
    r = int(mx["kv_rank"])
    dkv = h @ w[p + ".dkv"].T
    c = rms(dkv[:, :r], eps) * w[p + ".dkv.norm"]
    kr = rotate_pairs(dkv[:, r:].unsqueeze(1), rotary_frequencies(mx["rot"], h.dtype), positions).squeeze(1)
    return c, kr


def latent_attention(h, w, p, mx, positions, eps, rows):
    """``rows``: (c, rotated key part) of this layer or of the layer it takes them from."""
    T = h.shape[0]
    H, d, rd, dv = int(mx["heads"]), int(mx["dim"]), int(mx["rot_dim"]), int(mx["vdim"])
    c, kr = rows
    cq = rms(h @ w[p + ".dq"].T, eps) * w[p + ".dq.norm"]
    q = (cq @ w[p + ".uq"].T).view(T, H, d + rd)
    q_rot = rotate_pairs(q[..., d:], rotary_frequencies(mx["rot"], h.dtype), positions)
    q = torch.cat([q[..., :d], q_rot], dim=-1)
    k_plain = (c @ w[p + ".uk"].T).view(T, H, d)
    k = torch.cat([k_plain, kr.unsqueeze(1).expand(T, H, rd)], dim=-1)
    v = (c @ w[p + ".uv"].T).view(T, H, dv)
    window = int(mx["mask"]["size"]) if mx.get("mask") else None
    o = softmax_attention(q, k, v, float(mx["scale"]), visible(T, window))
    o = o * torch.sigmoid(h @ w[p + ".g"].T).unsqueeze(-1)
    return o.reshape(T, H * dv) @ w[p + ".o"].T


def dense_ff(h, w, p):
    return (silu(h @ w[p + ".gate"].T) * (h @ w[p + ".up"].T)) @ w[p + ".down"].T


def token_side(x, tokens, w, i, dim, eps):
    """The per-layer token input, added to the stream behind the feed-forward."""
    p = f"l{i}.side"
    e = w["side.embed"][tokens][:, i * dim:(i + 1) * dim]
    y = (gelu_tanh(x @ w[p + ".gate"].T) * e) @ w[p + ".proj"].T
    return x + rms(y, eps) * w[p + ".norm"]


def forward(config: dict, weights: Dict[str, torch.Tensor], tokens: List[int], dtype=torch.float64,
            streams: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence; ``streams`` (a list) receives the stream after every layer."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    eps = float(config["norm"]["eps"])
    tok = torch.tensor(tokens, dtype=torch.long)
    T = len(tokens)
    positions = torch.arange(T)
    x = w["embed"][tok]
    side_dim = int(config["token_side"]["dim"]) if config.get("token_side") else 0
    kept = {}
    for i, L in enumerate(config["layers"]):
        p, mx = f"l{i}", L["mixer"]
        h = layer_norm(x, w[p + ".norm1"], eps)
        if L["type"] == "parallel":
            x = x + parallel_mixer(h, w, p + ".mix", mx, positions, eps)
        else:
            src = mx.get("kv_from")
            if src is None:
                kept[i] = latent_rows(h, w, p + ".mix", mx, positions, eps)
                src = i
            x = x + latent_attention(h, w, p + ".mix", mx, positions, eps, kept[int(src)])
        if L.get("mlp") is not None:
            x = x + dense_ff(layer_norm(x, w[p + ".norm2"], eps), w, p + ".mlp")
        if side_dim:
            x = token_side(x, tok, w, i, side_dim, eps)
        if streams is not None:
            streams.append(x.clone())
    return (layer_norm(x, w["final.norm"], eps) @ w["head"].T) * float(config["logit_scale"])


def greedy_generate(config: dict, weights: Dict[str, torch.Tensor], prompt: List[int], n: int) -> List[int]:
    toks, out = list(prompt), []
    for _ in range(n):
        nxt = int(torch.argmax(forward(config, weights, toks)[-1]))
        out.append(nxt)
        toks.append(nxt)
    return out


def tensor_shapes(config: dict) -> Dict[str, tuple]:
    """Names and shapes of a model's tensors."""
    W, vocab, n = int(config["width"]), int(config["vocab"]), len(config["layers"])
    side = int(config["token_side"]["dim"]) if config.get("token_side") else 0
    out = {"embed": (vocab, W), "final.norm": (W,), "head": (vocab, W)}
    if side:
        out["side.embed"] = (vocab, n * side)
    for i, L in enumerate(config["layers"]):
        p, mx, m = f"l{i}", L["mixer"], f"l{i}.mix"
        out[p + ".norm1"] = (W,)
        if L["type"] == "parallel":
            a, b = mx["left"], mx["right"]
            H, G, D, V = int(a["heads"]), int(a["kv_heads"]), int(a["dim"]), int(a["vdim"])
            out.update({m + ".left.q": (H * D, W), m + ".left.q.b": (H * D,), m + ".left.k": (G * D, W),
                        m + ".left.k.b": (G * D,), m + ".left.v": (G * V, W), m + ".left.v.b": (G * V,),
                        m + ".left.o": (W, H * V)})
            H, G, D, V, c = int(b["heads"]), int(b["kv_heads"]), int(b["dim"]), int(b["vdim"]), int(b["conv"])
            r = m + ".right"
            out.update({r + ".q": (G * D, W), r + ".q.conv": (G * D, c), r + ".k": (G * D, W), r + ".k.conv": (G * D, c),
                        r + ".v": (H * V, W), r + ".v.conv": (H * V, c), r + ".b": (H, W), r + ".A_log": (H,),
                        r + ".norm": (V,), r + ".a": (H, W), r + ".dt_bias": (H,), r + ".g": (H * V, W),
                        r + ".o": (W, H * V)})
        else:
            H, D, R, V = int(mx["heads"]), int(mx["dim"]), int(mx["rot_dim"]), int(mx["vdim"])
            kr, qr = int(mx["kv_rank"]), int(mx["q_rank"])
            out.update({m + ".dq": (qr, W), m + ".dq.norm": (qr,), m + ".uq": (H * (D + R), qr), m + ".uk": (H * D, kr),
                        m + ".uv": (H * V, kr), m + ".g": (H, W), m + ".o": (W, H * V)})
            if mx.get("kv_from") is None:
                out.update({m + ".dkv": (kr + R, W), m + ".dkv.norm": (kr,)})
        if L.get("mlp") is not None:
            F = int(L["mlp"]["ff"])
            out.update({p + ".norm2": (W,), p + ".mlp.gate": (F, W), p + ".mlp.up": (F, W), p + ".mlp.down": (W, F)})
        if side:
            out.update({p + ".side.gate": (side, W), p + ".side.proj": (W, side), p + ".side.norm": (W,)})
    return out


def random_weights(config: dict, seed: int = 0) -> Dict[str, torch.Tensor]:
    """Random tensors of a size that keeps every mechanism alive: matrices ~ 1/sqrt(columns), norm weights around
    one, biases around zero.  Values are rounded to bfloat16 so that a bfloat16 engine holds the same numbers."""
    gen = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(config).items():
        leaf = name.rsplit(".", 1)[-1]
        if name in ("embed", "side.embed"):
            t = torch.randn(shape, generator=gen) * 0.7
        elif leaf in ("norm1", "norm2", "norm"):
            t = 1.0 + torch.randn(shape, generator=gen) * 0.2
        elif leaf == "conv":
            t = torch.randn(shape, generator=gen) * 0.5
        elif leaf == "A_log":
            t = torch.randn(shape, generator=gen) * 0.5 - 1.0
        elif leaf == "dt_bias" or (leaf == "b" and len(shape) == 1):
            t = torch.randn(shape, generator=gen) * 0.3
        else:
            t = torch.randn(shape, generator=gen) / math.sqrt(shape[-1])
            if leaf in ("q", "k", "v", "uq"):
                t = t * 2.0
        out[name] = t.to(torch.bfloat16).to(torch.float32)
    return out
