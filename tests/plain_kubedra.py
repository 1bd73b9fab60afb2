"""Plain, slow Kubedra decoder: whole sequences, no cache, one function per mechanism.

The oracle that the engine's Kubedra model is compared with.  It shares no code with the package:
the configuration is a plain dict, the weights a dict of name -> tensor, and every mechanism is
written out with elementary torch operations on the CPU in float64 (the stored bfloat16 weights
are exact there).

Notation.  x: the residual stream [T, W].  rms(x) = x / sqrt(mean(x^2) + eps).  A layer is
x += n1b(mixer(n1(x))); x += n2b(ff(n2(x))) with n(x) = rms(x) * (1 + w).  Layers ``start`` to
``stop - 1`` of the ``loop`` block run ``times`` times with the same weights; before every pass but
the first the embedding output is added to x.
"""
from __future__ import annotations

import math

import torch

F = torch.float64


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def offset_norm(x, w, eps):
    """rms(x) * (1 + w): the gain is stored around zero."""
    return rms(x, eps) * (1.0 + w)


def plain_norm(x, w, eps):
    """rms(x) * w: the gain is used as it is."""
    return rms(x, eps) * w


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def embed(weights, tokens):
    """x[t] = E[token t] + P[t], positions from 0."""
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    return weights["embed"].to(F)[tokens] + weights["pos"].to(F)[:len(tokens)]


def windowed_softmax_attention(q, k, v, scale, window):
    """q, k [T, H, d], v [T, H, dv] -> [T, H, dv].  Query i sees key j when 0 <= i - j < window
    (window None: every earlier key and itself)."""
    T = q.shape[0]
    s = torch.einsum("ihd,jhd->hij", q, k) * scale
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    seen = (j <= i) if window is None else ((j <= i) & (i - j < window))
    s = s.masked_fill(~seen, float("-inf"))
    p = torch.softmax(s, dim=-1)
    return torch.einsum("hij,jhd->ihd", p, v)


def latent_attention(h, w, pre, m, eps):
    """Queries through a normed latent, keys and values from one normed latent per token."""
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    cq = plain_norm(h @ w[pre + "dq"].to(F).T, w[pre + "dq.norm"].to(F), eps)
    q = (cq @ w[pre + "uq"].to(F).T).view(T, H, d)
    c = plain_norm(h @ w[pre + "dkv"].to(F).T, w[pre + "dkv.norm"].to(F), eps)
    k = (c @ w[pre + "uk"].to(F).T).view(T, H, d)
    v = (c @ w[pre + "uv"].to(F).T).view(T, H, dv)
    window = (m.get("mask") or {}).get("size")
    scale = m.get("scale", d ** -0.5)
    o = windowed_softmax_attention(q, k, v, scale, window)
    return o.reshape(T, H * dv) @ w[pre + "o"].to(F).T


def gla_decay(h, w, pre, m):
    """alpha = sigmoid(z)^(1/tau), z = A2 (A1 h) + b, one per key channel [T, H, d]."""
    z = (h @ w[pre + "a1"].to(F).T) @ w[pre + "a2"].to(F).T + w[pre + "a2.b"].to(F)
    return torch.sigmoid(z).pow(1.0 / m["tau"]).view(h.shape[0], m["heads"], m["dim"])


def gla_recurrence(q, k, v, alpha, state=None):
    """S_t = diag(alpha_t) S_{t-1} + k_t v_t^T; o_t = S_t^T q_t, token by token.
    q, k, alpha [T, H, d]; v [T, H, dv]; state [H, d, dv] or None (zero).  Returns (o [T, H, dv], state)."""
    T, H, d = q.shape
    dv = v.shape[-1]
    S = torch.zeros(H, d, dv, dtype=q.dtype) if state is None else state.clone()
    out = []
    for t in range(T):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        out.append(torch.einsum("hdv,hd->hv", S, q[t]))
    return torch.stack(out) if out else torch.zeros(0, H, dv, dtype=q.dtype), S


def gla(h, w, pre, m, eps):
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = (h @ w[pre + "q"].to(F).T).view(T, H, d) * d ** -0.5
    k = (h @ w[pre + "k"].to(F).T).view(T, H, d)
    v = (h @ w[pre + "v"].to(F).T).view(T, H, dv)
    o, _ = gla_recurrence(q, k, v, gla_decay(h, w, pre, m))
    o = plain_norm(o, w[pre + "norm"].to(F), eps).reshape(T, H * dv)
    g = h @ w[pre + "g"].to(F).T
    return (o * torch.nn.functional.silu(g)) @ w[pre + "o"].to(F).T


def dense_ff(h, w, pre):
    return (gelu_tanh(h @ w[pre + "gate"].to(F).T) * (h @ w[pre + "up"].to(F).T)) @ w[pre + "down"].to(F).T


def clamped_expert(h, w, pre, limit):
    """g = min(G h, limit); u = clamp(U h, -limit, limit); D (g sigmoid(1.702 g) (u + 1))."""
    g = (h @ w[pre + "gate"].to(F).T).clamp(max=limit)
    u = (h @ w[pre + "up"].to(F).T).clamp(-limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[pre + "down"].to(F).T


def route(h, w, pre, top):
    """The ``top`` largest router logits per token and the softmax over those alone."""
    z = h @ w[pre + "router"].to(F).T + w[pre + "router.b"].to(F)
    values, chosen = torch.topk(z, top, dim=-1)
    return chosen, torch.softmax(values, dim=-1)


def moe_ff(h, w, pre, mlp):
    chosen, weight = route(h, w, pre, mlp["router"]["top"])
    out = torch.zeros(h.shape[0], w[pre + "e0.down"].shape[0], dtype=F)
    for t in range(h.shape[0]):
        for e, g in zip(chosen[t].tolist(), weight[t]):
            out[t] += g * clamped_expert(h[t:t + 1], w, f"{pre}e{e}.", mlp["expert"]["limit"])[0]
    if mlp.get("shared"):
        out = out + clamped_expert(h, w, pre + "shared.", mlp["shared"]["limit"])
    return out


def layer(x, w, i, cfg):
    spec = cfg["layers"][i]
    eps = cfg["norm"]["eps"]
    p = f"l{i}."
    h = offset_norm(x, w[p + "norm1"].to(F), eps)
    if spec["type"] == "gla":
        a = gla(h, w, p + "mix.", spec["mixer"], eps)
    elif spec["type"] == "latent_attention":
        a = latent_attention(h, w, p + "mix.", spec["mixer"], eps)
    else:
        raise ValueError(spec["type"])
    x = x + offset_norm(a, w[p + "norm1b"].to(F), eps)
    mlp = spec.get("mlp")
    if mlp:
        h = offset_norm(x, w[p + "norm2"].to(F), eps)
        f = dense_ff(h, w, p + "mlp.") if mlp["kind"] == "dense" else moe_ff(h, w, p + "mlp.", mlp)
        x = x + offset_norm(f, w[p + "norm2b"].to(F), eps)
    return x


def layer_order(cfg):
    """(layer index, whether the embedding output is added before it) for every layer run."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    start, stop, times = loop["start"], loop["stop"], loop["times"]
    order = [(i, False) for i in range(start)]
    for p in range(times):
        order += [(i, p > 0 and i == start) for i in range(start, stop)]
    return order + [(i, False) for i in range(stop, n)]


def forward(cfg, w, tokens, return_layers=False):
    """Logits [T, vocab] of one whole sequence (float64)."""
    x0 = embed(w, tokens)
    x = x0
    after = []
    for i, add in layer_order(cfg):
        if add:
            x = x + x0
        x = layer(x, w, i, cfg)
        after.append(x)
    logits = offset_norm(x, w["final.norm"].to(F), cfg["norm"]["eps"]) @ w["embed"].to(F).T
    return (logits, torch.stack(after)) if return_layers else logits
