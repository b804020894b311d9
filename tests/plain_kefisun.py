"""Plain, slow implementation of the Kefisun decoder: whole sequences, no cache, one
function per mechanism, ordinary tensor arithmetic in float64.  It reads ``config.json``
and ``model.safetensors`` on its own and shares no code with the engine package.

The design, layer by layer (``h`` is a sublayer's input after the norm, ``t`` a position
counted from 0 in its sequence):

* embedding: ``x_t = E[token_t] * embedding.scale``;
* a layer: ``x += mixer(filter(norm1(x)))``, then, when it has a feed-forward,
  ``x += ff(norm2(x))``; norm: ``x / sqrt(mean(x^2) + eps) * (1 + w)``;
* filter: ``h_t + sum_j c[:, j] * h_(t - taps + 1 + j)`` (h is 0 at negative t);
* mixer ``attention``: projections, a short causal convolution of q, k and v, an RMS norm over
  the whole of q and of k, ``softmax(q.k * scale - r1 * ln(1 + r2 * distance))`` over a window,
  values mixed with those of the first such layer, a sigmoid gate, the output projection;
* mixer ``channel_delta``: the delta rule with a decay per key channel;
* feed-forward: clamped gate and up, ``g * sigmoid(1.702 g) * (u + 1)``, down; all with biases;
* output: norm, then ``E x * logit_scale``.
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
# mechanisms
# --------------------------------------------------------------------------------------

def rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm_one_plus(x, w, eps):
    return rms(x, eps) * (1.0 + w)


def causal_conv(u, w):
    """u (L, C), w (C, taps): y_t = sum_j w[:, j] * u_(t - taps + 1 + j); column taps-1 multiplies u_t itself,
    u is 0 at negative t."""
    L, C = u.shape
    taps = w.shape[1]
    y = torch.zeros_like(u)
    for j in range(taps):
        back = taps - 1 - j
        if back < L:
            y[back:] += w[:, j] * u[: L - back]
    return y


def input_filter(h, w):
    return h + causal_conv(h, w)


def silu(x):
    return x * torch.sigmoid(x)


def distance_bias(r1, r2, L):
    """(H, L, L): r1_h * ln(1 + r2_h * (i - j)) for j <= i (0 elsewhere)."""
    i = torch.arange(L)
    d = (i[:, None] - i[None, :]).clamp(min=0).to(F64)
    return r1[:, None, None] * torch.log1p(r2[:, None, None] * d)


def window_mask(L, size):
    """(L, L) True where position i sees j: 0 <= i - j < size (size None: every earlier key)."""
    i = torch.arange(L)
    d = i[:, None] - i[None, :]
    m = d >= 0
    if size is not None:
        m &= d < size
    return m


def attention_mixer(h, W, p, m, eps, v_first):
    """h (L, width).  Returns (update, the values this layer caches, its unmixed values)."""
    L = h.shape[0]
    H, G, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = h @ W[p + "q"].T
    k = h @ W[p + "k"].T
    v = h @ W[p + "v"].T
    if p + "q.conv" in W:
        q, k, v = causal_conv(q, W[p + "q.conv"]), causal_conv(k, W[p + "k.conv"]), causal_conv(v, W[p + "v.conv"])
    q = rms(q, eps) * W[p + "q.norm"]
    k = rms(k, eps) * W[p + "k.norm"]
    own_v = v
    if v_first is not None:
        lam = W[p + "vmix"]
        v = (1.0 - lam) * v + lam * v_first
    qh = q.view(L, H, dim).transpose(0, 1)                       # (H, L, dim)
    kh = k.view(L, G, dim).transpose(0, 1).repeat_interleave(H // G, dim=0)
    vh = v.view(L, G, vdim).transpose(0, 1).repeat_interleave(H // G, dim=0)
    s = qh @ kh.transpose(1, 2) * m["scale"] - distance_bias(W[p + "r1"], W[p + "r2"], L)
    size = m["mask"]["size"] if m.get("mask") else None
    s = s.masked_fill(~window_mask(L, size), float("-inf"))
    o = torch.softmax(s, dim=-1) @ vh                            # (H, L, vdim)
    o = o.transpose(0, 1).reshape(L, H * vdim)
    o = o * torch.sigmoid(h @ W[p + "g"].T)
    return o @ W[p + "o"].T, v, own_v


def delta_mixer(h, W, p, m, eps):
    """The gated delta rule with one decay per head and key channel, token by token."""
    L = h.shape[0]
    H, G, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(causal_conv(h @ W[p + "q"].T, W[p + "q.conv"])).view(L, G, dim)
    k = silu(causal_conv(h @ W[p + "k"].T, W[p + "k.conv"])).view(L, G, dim)
    v = silu(causal_conv(h @ W[p + "v"].T, W[p + "v.conv"])).view(L, H, vdim)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dim ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    q = q.repeat_interleave(H // G, dim=1)
    k = k.repeat_interleave(H // G, dim=1)
    beta = torch.sigmoid(h @ W[p + "b"].T)                        # (L, H)
    a = (h @ W[p + "a1"].T) @ W[p + "a2"].T + W[p + "dt_bias"]
    decay = torch.exp(-torch.exp(W[p + "A_log"])[None, :, None] * torch.nn.functional.softplus(a.view(L, H, dim)))
    S = torch.zeros((H, dim, vdim), dtype=h.dtype)
    o = torch.zeros((L, H, vdim), dtype=h.dtype)
    for t in range(L):
        S = decay[t][:, :, None] * S
        u = beta[t][:, None] * (v[t] - torch.einsum("hdv,hd->hv", S, k[t]))
        S = S + k[t][:, :, None] * u[:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    gate = torch.sigmoid((h @ W[p + "g1"].T) @ W[p + "g2"].T).view(L, H, vdim)
    o = rms(o, eps) * W[p + "norm"] * gate
    return o.reshape(L, H * vdim) @ W[p + "o"].T


def dense_ff(h, W, p, f):
    lim = f["limit"]
    g = (h @ W[p + "gate"].T + W[p + "gate.b"]).clamp(max=lim)
    u = (h @ W[p + "up"].T + W[p + "up.b"]).clamp(min=-lim, max=lim)
    y = g * torch.sigmoid(1.702 * g) * (u + 1.0)
    return y @ W[p + "down"].T + W[p + "down.b"]


# --------------------------------------------------------------------------------------
# the model
# --------------------------------------------------------------------------------------

def plain_forward(c: dict, W: dict, tokens, return_layers: bool = False):
    """Logits (L, vocab) of one sequence; with ``return_layers`` also the residual stream after
    every layer, (layers, L, width)."""
    eps = c["norm"]["eps"]
    x = W["embed"][torch.as_tensor(tokens, dtype=torch.long)] * c["embedding"]["scale"]
    v_first = None
    seen_first = False
    layers = []
    for i, layer in enumerate(c["layers"]):
        p = f"l{i}."
        h = norm_one_plus(x, W[p + "norm1"], eps)
        if p + "canon1" in W:
            h = input_filter(h, W[p + "canon1"])
        m = layer["mixer"]
        if layer["type"] == "attention":
            mixes = bool(m.get("v_mix"))
            upd, _, own_v = attention_mixer(h, W, p + "mix.", m, eps, v_first if (mixes and seen_first) else None)
            if mixes and not seen_first:
                v_first, seen_first = own_v, True
        elif layer["type"] == "channel_delta":
            upd = delta_mixer(h, W, p + "mix.", m, eps)
        else:
            raise ValueError(layer["type"])
        x = x + upd
        if layer.get("mlp"):
            x = x + dense_ff(norm_one_plus(x, W[p + "norm2"], eps), W, p + "mlp.", layer["mlp"])
        layers.append(x.clone())
    logits = norm_one_plus(x, W["final.norm"], eps) @ W["embed"].T * c["logit_scale"]
    if return_layers:
        return logits, torch.stack(layers)
    return logits
