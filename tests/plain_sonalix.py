"""A plain, slow implementation of the Sonalix decoder: whole sequences, no cache, no batching,
one function per mechanism, written from the design's equations.  It shares no code with the
package and is what the package's kernels are compared with.

Notation: ``T`` tokens, ``W`` model width, ``H`` heads, ``G`` key heads, ``dk`` / ``dv`` the key
and value sizes of a head.  Weights are a dict name -> tensor with the checkpoint's names; ``cfg``
is the parsed ``config.json``.  Everything runs in the dtype of the weights (float32 or float64)
on the CPU.
"""

from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import torch


# ---------------------------------------------------------------- reading a folder


def read_folder(folder, dtype=torch.float64):
    """(config dict, weights dict) of a model folder; floats widened to ``dtype``."""
    folder = Path(folder)
    cfg = json.loads((folder / "config.json").read_text())
    raw = (folder / "model.safetensors").read_bytes()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8 : 8 + n])
    kinds = {"BF16": torch.bfloat16, "F32": torch.float32, "F16": torch.float16, "I32": torch.int32, "F64": torch.float64}
    weights = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        a, b = info["data_offsets"]
        t = torch.frombuffer(bytearray(raw[8 + n + a : 8 + n + b]), dtype=kinds[info["dtype"]]).reshape(info["shape"])
        weights[name] = t.to(dtype) if t.is_floating_point() else t
    return cfg, weights


# ---------------------------------------------------------------- small pieces


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def tanh_norm(x, w, p: str):
    """The layers' and the model's norm: no statistics, ``tanh(alpha x) w + b``."""
    return torch.tanh(w[p + ".alpha"] * x) * w[p] + w[p + ".b"]


def silu(z):
    return z * torch.sigmoid(z)


def turn_halves(x, positions, dims: int, base: float):
    """``x [T, ..., d]``: dim ``i`` and dim ``i + dims/2`` (``i < dims/2``) turn together by the angle
    ``p * base^(-2i/dims)``; dims from ``dims`` on are left as they are."""
    half = dims // 2
    freqs = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=torch.float64)
    ang = positions.to(torch.float64)[:, None] * freqs[None, :]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [half]
    cos, sin = ang.cos().to(x.dtype).reshape(shape), ang.sin().to(x.dtype).reshape(shape)
    u, v = x[..., :half], x[..., half:dims]
    y = x.clone()
    y[..., :half] = u * cos - v * sin
    y[..., half:dims] = v * cos + u * sin
    return y


# ---------------------------------------------------------------- mixers


def windowed_attention(h, w, p: str, m: dict, eps: float, carried: dict):
    """Grouped-query attention: normed heads, rotation of half pairs, capped scores, a sliding window,
    a sink in the softmax's denominator, values mixed with those of the first layer that mixes values.
    ``carried`` holds that layer's values between the layers of one pass over the model."""
    t = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(t)
    q = (h @ w[p + "q"].T).reshape(t, H, dk)
    k = (h @ w[p + "k"].T).reshape(t, G, dk)
    v = (h @ w[p + "v"].T).reshape(t, G, dv)
    q = unit_rms(q, eps) * w[p + "q.norm"]
    k = unit_rms(k, eps) * w[p + "k.norm"]
    rot = m.get("rot")
    if rot:
        q = turn_halves(q, pos, rot["dims"], rot["base"])
        k = turn_halves(k, pos, rot["dims"], rot["base"])
    if m.get("v_mix"):
        if "v_first" in carried:
            lam = w[p + "vmix"]
            v = (1.0 - lam) * v + lam * carried["v_first"]
        else:
            carried["v_first"] = v
    i = torch.arange(t)[:, None]
    j = torch.arange(t)[None, :]
    visible = j <= i
    if m.get("mask"):
        visible = visible & (i - j < m["mask"]["size"])
    cap = m.get("softcap")
    out = h.new_zeros(t, H, dv)
    for head in range(H):
        g = head // (H // G)
        s = (q[:, head] @ k[:, g].T) * m["scale"]
        if cap:
            s = cap * torch.tanh(s / cap)
        s = s.masked_fill(~visible, float("-inf"))
        if p + "sink" in w:
            sink = w[p + "sink"][head]
            top = torch.maximum(s.max(-1, keepdim=True).values, sink)
            e = torch.exp(s - top)
            a = e / (e.sum(-1, keepdim=True) + torch.exp(sink - top))
        else:
            a = torch.softmax(s, dim=-1)
        out[:, head] = a @ v[:, g]
    return out.reshape(t, H * dv) @ w[p + "o"].T


def retention(h, w, p: str, m: dict, eps: float, carried: dict):
    """Linear attention with one fixed decay a head and no softmax: ``S_t = a S_(t-1) + k_t v_t^T``,
    ``o_t = S_t^T q_t``; every head's ``o`` is divided by its root mean square, the heads are gated by
    ``silu(W_g h)`` and projected."""
    t = h.shape[0]
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    pos = torch.arange(t)
    q = (h @ w[p + "q"].T).reshape(t, H, dk)
    k = (h @ w[p + "k"].T).reshape(t, H, dk)
    v = (h @ w[p + "v"].T).reshape(t, H, dv)
    rot = m.get("rot")
    if rot:
        q = turn_halves(q, pos, rot["dims"], rot["base"])
        k = turn_halves(k, pos, rot["dims"], rot["base"])
    k = k * dk**-0.5
    o = h.new_zeros(t, H, dv)
    for head in range(H):
        a = float(m["decay"][head])
        state = h.new_zeros(dk, dv)
        for s in range(t):
            state = a * state + k[s, head][:, None] * v[s, head][None, :]
            o[s, head] = state.T @ q[s, head]
    o = unit_rms(o, eps).reshape(t, H * dv)
    return (o * silu(h @ w[p + "g"].T)) @ w[p + "o"].T


def latent_attention(h, w, p: str, m: dict, eps: float, carried: dict):
    """Attention whose queries come through a normed latent and whose keys and values are made from one
    small normed latent per token, with a rotated key part shared by all heads, every earlier key
    visible, and a logistic gate on every output channel."""
    t = h.shape[0]
    H, dk, dr, dv, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(t)
    cq = unit_rms(h @ w[p + "dq"].T, eps) * w[p + "dq.norm"]
    q = (cq @ w[p + "uq"].T).reshape(t, H, dk + dr)
    q_plain, q_rot = q[..., :dk], q[..., dk:]
    down = h @ w[p + "dkv"].T
    c = unit_rms(down[:, :r], eps) * w[p + "dkv.norm"]
    k_rot = down[:, r:]
    rot = m["rot"]
    q_rot = turn_halves(q_rot, pos, rot["dims"], rot["base"])
    k_rot = turn_halves(k_rot, pos, rot["dims"], rot["base"])
    k_plain = (c @ w[p + "uk"].T).reshape(t, H, dk)
    v = (c @ w[p + "uv"].T).reshape(t, H, dv)
    visible = torch.arange(t)[None, :] <= torch.arange(t)[:, None]
    out = h.new_zeros(t, H, dv)
    for head in range(H):
        s = (q_plain[:, head] @ k_plain[:, head].T + q_rot[:, head] @ k_rot.T) * m["scale"]
        out[:, head] = torch.softmax(s.masked_fill(~visible, float("-inf")), dim=-1) @ v[:, head]
    gate = torch.sigmoid(h @ w[p + "g"].T)
    return (out.reshape(t, H * dv) * gate) @ w[p + "o"].T


MIXERS = {"attention": windowed_attention, "retention": retention, "latent_attention": latent_attention}


# ---------------------------------------------------------------- feed-forward


def dense_feed_forward(h, w, p: str, mlp: dict):
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def route(h, w, p: str, r: dict):
    """(chosen experts ``[T, top]``, their weights ``[T, top]``): the largest logits, softmax over them alone."""
    z = h @ w[p + "router"].T + w[p + "router.b"]
    best = z.topk(r["top"], dim=-1)
    return best.indices, torch.softmax(best.values, dim=-1)


def expert(h, w, p: str, limit: float):
    g = (h @ w[p + "gate"].T).clamp(max=limit)
    u = (h @ w[p + "up"].T).clamp(min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].T


def mixture_of_experts(h, w, p: str, mlp: dict):
    chosen, weights = route(h, w, p, mlp["router"])
    out = torch.zeros(h.shape[0], w[p + "e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for e, g in zip(chosen[t].tolist(), weights[t]):
            out[t] += g * expert(h[t], w, f"{p}e{e}.", mlp["expert"]["limit"])
    return out


def feed_forward(h, w, p: str, mlp: dict):
    return dense_feed_forward(h, w, p, mlp) if mlp["kind"] == "dense" else mixture_of_experts(h, w, p, mlp)


# ---------------------------------------------------------------- the model


def residual_after_every_layer(cfg, w, tokens) -> list[torch.Tensor]:
    eps = cfg["norm"]["eps"]
    mult = cfg.get("residual_mult", 1.0)
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)] * (cfg.get("embedding") or {}).get("scale", 1.0)
    out = []
    carried: dict = {}
    for i, layer in enumerate(cfg["layers"]):
        h = tanh_norm(x, w, f"l{i}.norm1")
        x = x + mult * MIXERS[layer["type"]](h, w, f"l{i}.mix.", layer["mixer"], eps, carried)
        if layer.get("mlp") is not None:
            h = tanh_norm(x, w, f"l{i}.norm2")
            x = x + mult * feed_forward(h, w, f"l{i}.mlp.", layer["mlp"])
        out.append(x)
    return out


def logits(cfg, w, tokens) -> torch.Tensor:
    x = residual_after_every_layer(cfg, w, tokens)[-1]
    return tanh_norm(x, w, "final.norm") @ w["head"].T


def greedy(cfg, w, prompt, n_new: int) -> list[int]:
    ids = list(prompt)
    for _ in range(n_new):
        ids.append(int(logits(cfg, w, ids)[-1].argmax()))
    return ids[len(prompt) :]
