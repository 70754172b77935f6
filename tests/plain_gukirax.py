"""A plain, slow implementation of the Gukirax decoder: whole sequences, no cache, float64, one function per
mechanism.  It shares no code with the package; the tests compare the engine with it.

Notation: ``x [T, W]`` the residual stream of one sequence, ``w`` a dict of float64 tensors by checkpoint name,
``cfg`` the dict of ``config.json``.  Linear maps are stored ``[out, in]``.
"""

from __future__ import annotations

import math

import torch


def layer_norm(x, weight, eps):
    """Mean off, divided by the root of (mean squared deviation + eps), times a weight; no bias."""
    c = x - x.mean(-1, keepdim=True)
    return c / torch.sqrt(c.pow(2).mean(-1, keepdim=True) + eps) * weight


def unit_rms(x, eps):
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def turn_split_pairs(x, positions, dims, base):
    """``x [T, heads, d]``: of the first ``dims`` numbers of a head, number i and number i + dims/2 form a pair that
    turns by the angle position * base^(-2i/dims); the other numbers stay."""
    if dims == 0:
        return x
    half = dims // 2
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=torch.float64)
    ang = positions.double()[:, None, None] * freq[None, None, :]
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat([a * ang.cos() - b * ang.sin(), b * ang.cos() + a * ang.sin(), x[..., dims:]], dim=-1)


def talking_attention(h, w, p, m, eps, positions=None):
    """Queries and keys from ``h``; values = the keys' projections before anything else happens to them; rotation,
    then unit RMS per head; scaled scores mixed over the heads; causal softmax with a sink; output projection."""
    t = h.shape[0]
    nh, nkv, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    positions = torch.arange(t) if positions is None else positions
    q = (h @ w[p + "q"].T).view(t, nh, d)
    k = (h @ w[p + "k"].T).view(t, nkv, d)
    v = k[..., :dv]
    q = unit_rms(turn_split_pairs(q, positions, m["rot"]["dims"], m["rot"]["base"]), eps)
    k = unit_rms(turn_split_pairs(k, positions, m["rot"]["dims"], m["rot"]["base"]), eps)
    per = nh // nkv
    scores = torch.stack([q[:, g] @ k[:, g // per].T for g in range(nh)]) * m["scale"]  # [source head, query, key]
    mixed = torch.einsum("hg,gij->hij", w[p + "talk"], scores)
    out = torch.zeros(t, nh, dv, dtype=torch.float64)
    for hd in range(nh):
        for i in range(t):
            s = mixed[hd, i, : i + 1]
            top = max(float(s.max()), float(w[p + "sink"][hd]))
            e = torch.exp(s - top)
            weights = e / (e.sum() + math.exp(float(w[p + "sink"][hd]) - top))  # the sink: in the sum, nowhere else
            out[i, hd] = weights @ v[: i + 1, hd // per]
    return out.reshape(t, nh * dv) @ w[p + "o"].T


def softplus(x):
    return math.log1p(math.exp(x))


def xielu(z, p, q):
    pos = softplus(p) * z * z + z / 2
    neg = (0.5 + softplus(q)) * (torch.exp(torch.clamp(z, max=0.0)) - 1 - z) + z / 2
    return torch.where(z > 0, pos, neg)


def dense_ff(h, w, p):
    return xielu(h @ w[p + "up"].T, float(w[p + "act"][0]), float(w[p + "act"][1])) @ w[p + "down"].T


def relu2_ff(h, w, p):
    return torch.relu(h @ w[p + "up"].T).pow(2) @ w[p + "down"].T


def route(h, w, p, top):
    """Softmax over all experts; the ``top`` largest are chosen (the lower index at a tie); their weights are their
    scores as they are.  Returns (ids [T, top], weights [T, top])."""
    s = torch.softmax(h @ w[p + "router"].T, dim=-1)
    ids, wts = [], []
    for row in s:
        order = sorted(range(len(row)), key=lambda e: (-float(row[e]), e))[:top]
        ids.append(order)
        wts.append([float(row[e]) for e in order])
    return torch.tensor(ids), torch.tensor(wts, dtype=torch.float64)


def experts_ff(h, w, p, m):
    ids, wts = route(h, w, p, m["router"]["top"])
    out = torch.zeros_like(h)
    for n in range(h.shape[0]):
        for e, g in zip(ids[n].tolist(), wts[n]):
            out[n] += g * relu2_ff(h[n : n + 1], w, f"{p}e{e}.")[0]
    if m.get("shared"):
        out = out + relu2_ff(h, w, p + "shared.")
    return out


def feed_forward(h, w, p, m):
    return dense_ff(h, w, p) if m["kind"] == "dense" else experts_ff(h, w, p, m)


def layer(x, w, i, ly, eps):
    """Norm before and after each sublayer; the sublayer's result is gated by a logistic function of a linear map of
    the sublayer's input before the second norm."""
    p = f"l{i}."
    h = layer_norm(x, w[p + "norm1"], eps)
    y = talking_attention(h, w, p + "mix.", ly["mixer"], eps) * torch.sigmoid(h @ w[p + "rg1"].T + w[p + "rg1.b"])
    x = x + layer_norm(y, w[p + "norm1b"], eps)
    if ly["mlp"] is not None:
        h = layer_norm(x, w[p + "norm2"], eps)
        y = feed_forward(h, w, p + "mlp.", ly["mlp"]) * torch.sigmoid(h @ w[p + "rg2"].T + w[p + "rg2.b"])
        x = x + layer_norm(y, w[p + "norm2b"], eps)
    return x


def run_order(cfg):
    """(layer, starts a pass) in the order the layers run."""
    n, lp = len(cfg["layers"]), cfg.get("loop")
    if not lp:
        return [(i, False) for i in range(n)]
    order = [(i, False) for i in range(lp["start"])]
    for _ in range(lp["times"]):
        order += [(i, i == lp["start"]) for i in range(lp["start"], lp["stop"])]
    return order + [(i, False) for i in range(lp["stop"], n)]


def hidden(cfg, w, tokens, trace=None):
    eps = cfg["norm"]["eps"]
    x0 = layer_norm(w["embed"][torch.tensor(tokens)], w["embed.norm"], eps)
    x = x0
    for i, first in run_order(cfg):
        if first:
            x = torch.cat([x, x0], dim=-1) @ w["loop.in"].T
        x = layer(x, w, i, cfg["layers"][i], eps)
        if trace is not None:
            trace.append(x)
    return x


def logits(cfg, w, tokens):
    x = layer_norm(hidden(cfg, w, tokens), w["final.norm"], cfg["norm"]["eps"])
    z = x @ w["embed"].T * cfg.get("logit_scale", 1.0)
    cap = cfg.get("logit_softcap")
    return cap * torch.tanh(z / cap) if cap else z


def greedy(cfg, w, prompt, n):
    toks, out = list(prompt), []
    for _ in range(n):
        nxt = int(logits(cfg, w, toks)[-1].argmax())
        out.append(nxt)
        toks.append(nxt)
    return out
