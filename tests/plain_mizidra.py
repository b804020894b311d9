"""Plain, slow implementation of the Mizidra decoder: whole sequences, no cache, one function per
mechanism, ordinary tensor arithmetic in float64.  It reads ``config.json`` and ``model.safetensors``
on its own and shares no code with the engine package.

Notation: ``L`` tokens of one sequence, ``t`` a position from 0, ``h`` the input of a sublayer (the
residual stream after the sublayer's norm), ``W[name]`` a tensor stored ``(out, in)``.

* stream: ``x_t = nrm(E[token_t]; embed.norm)``; every layer ``x += mixer(nrm(x; norm1))`` and, if the
  layer has a feed-forward, ``x += ff(nrm(x; norm2))``; ``nrm(x; w) = x * (mean(x^2) + eps)^-1/2 * w``;
  logits ``head @ nrm(x; final.norm)``.
* mixer ``delta``: a matrix state per head that forgets with one factor per head and token, and is
  corrected towards the token's value along the token's key (``delta_mixer``).
* mixer ``latent_attention``: keys and values of all heads are expanded from one small vector per
  token; a slice of query and key is rotated by position (long-context frequency rescaling); the
  softmax has one extra, keyless term per head (``latent_attention_mixer``).
* mixer ``lightning``: a matrix state per head with a constant forgetting factor, no softmax
  (``lightning_mixer``).
* feed-forward: routed experts with a group-limited choice, plus an always-on expert behind a scalar
  gate (``routed_ff``).
"""
from __future__ import annotations

import json
import math
import os

import torch

F64 = torch.float64


def read_config(folder: str) -> dict:
    with open(os.path.join(folder, "config.json")) as f:
        return json.load(f)


def read_weights(folder: str, dtype=F64) -> dict:
    from safetensors.torch import load_file
    return {k: v.to(dtype) for k, v in load_file(os.path.join(folder, "model.safetensors")).items()}


# --------------------------------------------------------------------------------------
# small pieces
# --------------------------------------------------------------------------------------

def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def nrm(x, w, eps):
    return rms(x, eps) * w


def silu(x):
    return x * torch.sigmoid(x)


def causal_conv(u, w):
    """u (L, C), w (C, taps): y_t = sum_j w[:, j] u_(t - (taps - 1) + j), u = 0 before the sequence."""
    L, C = u.shape
    taps = w.shape[1]
    y = torch.zeros_like(u)
    for j in range(taps):
        back = taps - 1 - j
        if back < L:
            y[back:] += w[:, j] * u[: L - back]
    return y


# --------------------------------------------------------------------------------------
# rotation by position with rescaled frequencies
# --------------------------------------------------------------------------------------

def rotary_frequencies(rot: dict):
    """(frequencies (dims/2,), magnitude) of a rotation over ``dims`` channels.  Plain frequencies are
    base^(-2i/dims).  With ``scaling`` = {factor, original, fast, slow}: the channel index at which a
    wave turns ``r`` times over ``original`` positions is c(r) = dims ln(original / (2 pi r)) / (2 ln base);
    channels below lo = floor(c(fast)) keep their frequency, channels above hi = ceil(c(slow)) have it divided
    by factor, between them the two are blended linearly; cos and sin are both scaled by 0.1 ln(factor) + 1."""
    dims, base = rot["dims"], float(rot["base"])
    half = dims // 2
    i = torch.arange(half, dtype=F64)
    f = base ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, orig = float(sc["factor"]), float(sc["original"])

    def c(r):
        return dims * math.log(orig / (2.0 * math.pi * r)) / (2.0 * math.log(base))

    lo = max(math.floor(c(float(sc["fast"]))), 0)
    hi = min(math.ceil(c(float(sc["slow"]))), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    f = f / factor * ramp + f * (1.0 - ramp)
    return f, 0.1 * math.log(factor) + 1.0


def rotate(x, positions, rot: dict):
    """x (L, ..., dims): channel i pairs with channel i + dims/2; the pair turns by positions * f_i."""
    f, mag = rotary_frequencies(rot)
    half = rot["dims"] // 2
    ang = positions.to(F64)[:, None] * f[None, :]
    shape = (x.shape[0],) + (1,) * (x.dim() - 2) + (half,)
    cos, sin = (torch.cos(ang) * mag).view(shape), (torch.sin(ang) * mag).view(shape)
    a, b = x[..., :half], x[..., half:2 * half]
    return torch.cat([a * cos - b * sin, b * cos + a * sin, x[..., 2 * half:]], dim=-1)


# --------------------------------------------------------------------------------------
# mixers
# --------------------------------------------------------------------------------------

def delta_mixer(h, W, p, m, eps):
    L = h.shape[0]
    H, G, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(causal_conv(h @ W[p + "q"].T, W[p + "q.conv"])).view(L, G, dim)
    k = silu(causal_conv(h @ W[p + "k"].T, W[p + "k.conv"])).view(L, G, dim)
    v = silu(causal_conv(h @ W[p + "v"].T, W[p + "v.conv"])).view(L, H, vdim)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dim ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    q = q.repeat_interleave(H // G, dim=1)
    k = k.repeat_interleave(H // G, dim=1)
    beta = torch.sigmoid(h @ W[p + "b"].T)                                        # (L, H)
    forget = torch.exp(-torch.exp(W[p + "A_log"]) * torch.nn.functional.softplus(h @ W[p + "a"].T + W[p + "dt_bias"]))
    S = torch.zeros((H, dim, vdim), dtype=h.dtype)
    o = torch.zeros((L, H, vdim), dtype=h.dtype)
    for t in range(L):
        S = forget[t][:, None, None] * S
        u = beta[t][:, None] * (v[t] - torch.einsum("hdv,hd->hv", S, k[t]))
        S = S + k[t][:, :, None] * u[:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    o = rms(o, eps) * W[p + "norm"] * silu(h @ W[p + "g"].T).view(L, H, vdim)
    return o.reshape(L, H * vdim) @ W[p + "o"].T


def attend_with_sink(q, k, v, scale, sink):
    """q, k (L, H, dk), v (L, H, dv), sink (H,) or None: causal softmax attention whose denominator holds one more
    term per head, exp(sink), that has no key and no value (it is not scaled)."""
    L, H = q.shape[0], q.shape[1]
    s = torch.einsum("ihd,jhd->hij", q, k) * scale
    s = s.masked_fill(torch.triu(torch.ones(L, L, dtype=torch.bool), 1), -math.inf)
    if sink is not None:
        s = torch.cat([s, sink.view(H, 1, 1).expand(H, L, 1).to(s.dtype)], dim=-1)
    w = torch.softmax(s, dim=-1)[..., :L]
    return torch.einsum("hij,jhd->ihd", w, v)


def latent_attention_mixer(h, W, p, m, eps, positions=None):
    L = h.shape[0]
    H, dim, rd, vdim, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(L) if positions is None else positions
    q = (h @ W[p + "q"].T).view(L, H, dim + rd)
    q_flat, q_rot = q[..., :dim], rotate(q[..., dim:], pos, m["rot"])
    down = h @ W[p + "dkv"].T
    c = nrm(down[:, :rank], W[p + "dkv.norm"], eps)
    k_rot = rotate(down[:, rank:], pos, m["rot"])                                  # (L, rd), the same for every head
    k_flat = (c @ W[p + "uk"].T).view(L, H, dim)
    v = (c @ W[p + "uv"].T).view(L, H, vdim)
    q_all = torch.cat([q_flat, q_rot], dim=-1)
    k_all = torch.cat([k_flat, k_rot[:, None, :].expand(L, H, rd)], dim=-1)
    o = attend_with_sink(q_all, k_all, v, m["scale"], W[p + "sink"])
    return o.reshape(L, H * vdim) @ W[p + "o"].T


def lightning_mixer(h, W, p, m, eps):
    L = h.shape[0]
    H, dim, vdim = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ W[p + "q"].T).view(L, H, dim)
    k = silu(h @ W[p + "k"].T).view(L, H, dim)
    v = silu(h @ W[p + "v"].T).view(L, H, vdim)
    keep = torch.tensor(m["decay"], dtype=h.dtype)
    S = torch.zeros((H, dim, vdim), dtype=h.dtype)
    o = torch.zeros((L, H, vdim), dtype=h.dtype)
    for t in range(L):
        S = keep[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    o = nrm(o.reshape(L, H * vdim), W[p + "norm"], eps) * torch.sigmoid(h @ W[p + "g"].T)
    return o @ W[p + "o"].T


# --------------------------------------------------------------------------------------
# feed-forward
# --------------------------------------------------------------------------------------

def gated_unit(h, W, p):
    return (silu(h @ W[p + "gate"].T) * (h @ W[p + "up"].T)) @ W[p + "down"].T


def route(h, W, p, router: dict):
    """(chosen experts (L, top), their weights (L, top))."""
    E, top = router["experts"], router["top"]
    s = torch.sigmoid(h @ W[p + "router"].T)                                       # (L, E)
    pick = s + W[p + "correction"]
    groups = router.get("groups")
    if groups:
        n, keep = groups["count"], groups["keep"]
        per = pick.view(-1, n, E // n)
        strength = per.topk(min(2, E // n), dim=-1).values.sum(-1)                  # (L, n)
        best = strength.topk(keep, dim=-1).indices
        allowed = torch.zeros_like(strength, dtype=torch.bool).scatter_(1, best, True)
        pick = per.masked_fill(~allowed[:, :, None], -math.inf).reshape(-1, E)
    idx = pick.topk(top, dim=-1).indices
    w = s.gather(1, idx)
    return idx, w / (w.sum(-1, keepdim=True) + 1e-20)


def routed_ff(h, W, p, f):
    idx, w = route(h, W, p, f["router"])
    out = torch.zeros_like(h)
    for e in range(f["router"]["experts"]):
        share = (w * (idx == e)).sum(-1, keepdim=True)                             # 0 where e was not chosen
        rows = share[:, 0] != 0
        if rows.any():
            out[rows] += share[rows] * gated_unit(h[rows], W, f"{p}e{e}.")
    if f.get("shared"):
        out = out + torch.sigmoid(h @ W[p + "shared.sg"].T) * gated_unit(h, W, p + "shared.")
    return out


# --------------------------------------------------------------------------------------
# the model
# --------------------------------------------------------------------------------------

MIXERS = {"delta": delta_mixer, "latent_attention": latent_attention_mixer, "lightning": lightning_mixer}


def plain_forward(c: dict, W: dict, tokens, return_layers: bool = False):
    eps = c["norm"]["eps"]
    x = nrm(W["embed"][torch.as_tensor(tokens, dtype=torch.long)], W["embed.norm"], eps)
    layers = []
    for i, layer in enumerate(c["layers"]):
        p = f"l{i}."
        x = x + MIXERS[layer["type"]](nrm(x, W[p + "norm1"], eps), W, p + "mix.", layer["mixer"], eps)
        if layer.get("mlp"):
            x = x + routed_ff(nrm(x, W[p + "norm2"], eps), W, p + "mlp.", layer["mlp"])
        layers.append(x.clone())
    logits = nrm(x, W["final.norm"], eps) @ W["head"].T
    if return_layers:
        return logits, torch.stack(layers)
    return logits
