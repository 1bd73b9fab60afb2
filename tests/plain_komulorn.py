"""Plain, slow Komulorn decoder: whole sequences, no cache, one function per mechanism.

The oracle that the engine's Komulorn model is compared with.  It shares no code with the package: the
configuration is a plain dict (config.json as parsed), the weights a dict of name -> tensor, and every
mechanism is written out with elementary torch operations on the CPU in float64 (stored bfloat16 weights
are exact there).

Notation.  x: the residual stream [T, W].  n(x) = x / sqrt(mean(x^2) + eps) * w.  A layer is
x += mixer(n1(x)); x += ff(n2(x)) (the second line only where the layer has a feed-forward).
Logits = cap * tanh(head(n_final(x)) / cap).
"""
from __future__ import annotations

import math

import torch

F = torch.float64


def rms_norm(x, w, eps):
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * w


def rotary_frequencies(rot):
    """(frequencies [dims/2], the factor on cos and sin).  Plain frequencies base^(-2i/dims); with ``scaling`` each
    is blended between itself and itself / factor by a ramp over the index i, and cos / sin grow by 0.1 ln(factor) + 1."""
    dims, base = int(rot["dims"]), float(rot["base"])
    i = torch.arange(dims // 2, dtype=F)
    f = base ** (-2.0 * i / dims)
    s = rot.get("scaling")
    if not s:
        return f, 1.0
    factor, original = float(s["factor"]), float(s["original"])

    def index_of(turns):            # the index whose wavelength makes ``turns`` turns over the original length
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(index_of(float(s["fast"]))), 0)
    hi = min(math.ceil(index_of(float(s["slow"]))), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(x, positions, rot):
    """x [T, heads, d]: the first rot.dims channels of every head are rotated in pairs (i, i + dims/2).  No ``rot``:
    nothing is rotated."""
    if not rot or not rot.get("dims"):
        return x
    dims = int(rot["dims"])
    f, grow = rotary_frequencies(rot)
    a = torch.as_tensor(positions, dtype=F)[:, None] * f[None, :]              # [T, dims/2]
    cos, sin = (torch.cos(a) * grow)[:, None, :], (torch.sin(a) * grow)[:, None, :]
    u, v = x[..., :dims // 2], x[..., dims // 2:dims]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, x[..., dims:]], dim=-1)


def causal_softmax_attention(q, k, v, scale):
    """q [T, H, d], k [S, G, d], v [S, G, dv] with S >= T: the queries are the last T positions.  Query head h reads
    key/value head h // (H / G).  Returns [T, H, dv]."""
    T, H, _ = q.shape
    S, G, _ = k.shape
    out = torch.empty((T, H, v.shape[-1]), dtype=F)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale                                         # [T, S]
        i = torch.arange(T)[:, None] + (S - T)
        j = torch.arange(S)[None, :]
        s = s.masked_fill(j > i, float("-inf"))
        out[:, h] = torch.softmax(s, dim=-1) @ v[:, g]
    return out


def attention_keys_values(h, w, pre, m, positions):
    """The rotated keys [T, G, d] and the values [T, G, dv] a layer with projections of its own makes."""
    T, G, d, dv = h.shape[0], m["kv_heads"], m["dim"], m["vdim"]
    k = (h @ w[pre + "k"].to(F).T + w[pre + "k.b"].to(F)).view(T, G, d)
    v = (h @ w[pre + "v"].to(F).T + w[pre + "v.b"].to(F)).view(T, G, dv)
    return rotate(k, positions, m.get("rot")), v


def attention_mixer(h, w, pre, m, positions, keys_values):
    """``keys_values``: (k, v) of the layer whose cache this one reads (its own, or another layer's)."""
    T, H, d = h.shape[0], m["heads"], m["dim"]
    q = rotate((h @ w[pre + "q"].to(F).T + w[pre + "q.b"].to(F)).view(T, H, d), positions, m.get("rot"))
    k, v = keys_values
    o = causal_softmax_attention(q, k, v, float(m["scale"]))
    gate = torch.sigmoid(h @ w[pre + "g"].to(F).T)                                # [T, H]
    o = o * gate[:, :, None]
    return o.reshape(T, -1) @ w[pre + "o"].to(F).T


def squared_relu_expert(x, up, down):
    return torch.relu(x @ up.to(F).T) ** 2 @ down.to(F).T


def router_choice(h, w_router, top):
    """(ids [T, top], scores [T, top]): sigmoid scores, the largest ``top`` (ties to the lower index), not renormalised."""
    s = torch.sigmoid(h @ w_router.to(F).T)
    order = torch.sort(s, dim=-1, descending=True, stable=True).indices[:, :top]
    return order, torch.gather(s, 1, order)


def mixture_of_experts(h, w, pre, mlp, choice=None):
    """sum over the chosen experts of expert(score * h), plus sigmoid(sg . h) * shared(h)."""
    top = mlp["router"]["top"]
    ids, scores = choice if choice is not None else router_choice(h, w[pre + "router"], top)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(top):
            e = int(ids[t, j])
            out[t] += squared_relu_expert(scores[t, j] * h[t], w[f"{pre}e{e}.up"], w[f"{pre}e{e}.down"])
    if mlp.get("shared"):
        gate = torch.sigmoid(h @ w[pre + "shared.sg"].to(F).T)                    # [T, 1]
        out = out + gate * squared_relu_expert(h, w[pre + "shared.up"], w[pre + "shared.down"])
    return out


def forward(config, w, tokens, trace=None, choices=None):
    """Logits [T, vocab] (float64) of one whole sequence.  ``trace``: a list that receives the stream after every layer.
    ``choices``: {layer: (ids, scores)} to force the experts (for comparisons that a near-tie would spoil)."""
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    positions = torch.arange(len(tokens))
    eps = float(config["norm"]["eps"])
    x = w["embed"].to(F)[tokens]
    kept = {}
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        m = layer["mixer"]
        h = rms_norm(x, w[p + "norm1"].to(F), eps)
        if m.get("kv_from") is None:
            kept[i] = attention_keys_values(h, w, p + "mix.", m, positions)
            kv = kept[i]
        else:
            kv = kept[int(m["kv_from"])]
        x = x + attention_mixer(h, w, p + "mix.", m, positions, kv)
        if layer.get("mlp"):
            h = rms_norm(x, w[p + "norm2"].to(F), eps)
            x = x + mixture_of_experts(h, w, p + "mlp.", layer["mlp"], None if choices is None else choices.get(i))
        if trace is not None:
            trace.append(x.clone())
    z = rms_norm(x, w["final.norm"].to(F), eps) @ w["head"].to(F).T
    cap = config.get("logit_softcap")
    return float(cap) * torch.tanh(z / float(cap)) if cap else z
