"""Small Gukirax configurations for the tests, model folders with random weights made here (not by the
package's random-weights mode), and the plain implementation's logits for them.

The configurations differ from one another in every size and option: heads and key heads (equal, several
heads a key head, a single key head), head sizes (8 to 128, and sizes that are no multiple of 8), value sizes (equal to the key's and smaller), how
many dims turn (none, some, all), layers with a dense feed-forward, with experts (one a token, several; with
and without a shared expert) and without any, a loop from the first layer, in the middle, to the last layer,
over a single layer, and none, logits scaled and capped or neither.
"""

from __future__ import annotations

import random

import torch

import plain_gukirax as plain
from mopilorn_cases import row_error, write_folder  # noqa: F401  (the folder writer and the error measure are the same)


def attention(heads, kv_heads, dim, rot, vdim=None, base=10000.0, scale=None):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim if vdim is not None else dim, "rot": {"dims": rot, "base": base},
            "scale": scale if scale is not None else dim**-0.5}  # fmt: skip


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, shared=None):
    out = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared:
        out["shared"] = {"ff": shared}
    return out


def layer(mixer, mlp):
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


CASES: dict[str, dict] = {
    # a loop in the middle; a dense layer first; two heads a key head; half of a head's dims turn
    "a": {
        "config": {
            "architecture": "Gukirax", "vocab": 131, "width": 64, "norm": {"eps": 1e-5}, "logit_scale": 0.5, "logit_softcap": 20.0,
            "loop": {"start": 1, "stop": 3, "times": 2},
            "layers": [
                layer(attention(4, 2, 16, 8), dense(80)),
                layer(attention(4, 2, 16, 8), moe(6, 2, 40, 24)),
                layer(attention(2, 1, 24, 24, base=500.0), moe(6, 2, 40, 24)),
                layer(attention(4, 4, 16, 4, vdim=8), None),
            ],
        },
        "block_size": 16,
    },
    # looped from the first layer, a single layer three times; one expert a token, no shared expert; as many key heads
    # as heads; a value smaller than its key; no cap on the logits
    "b": {
        "config": {
            "architecture": "Gukirax", "vocab": 97, "width": 48, "norm": {"eps": 1e-6}, "logit_scale": 1.0,
            "loop": {"start": 0, "stop": 1, "times": 3},
            "layers": [
                layer(attention(3, 3, 24, 12, vdim=16), moe(4, 1, 32)),
                layer(attention(6, 2, 8, 8), dense(56)),
                layer(attention(5, 1, 16, 0), None),
            ],
        },
        "block_size": 8,
    },
    # no loop; a single key head for eight heads; three experts a token; pages of four tokens
    "c": {
        "config": {
            "architecture": "Gukirax", "vocab": 150, "width": 40, "norm": {"eps": 1e-6}, "logit_scale": 2.0, "logit_softcap": 50.0,
            "layers": [
                layer(attention(8, 1, 16, 16), moe(8, 3, 24, 16)),
                layer(attention(2, 2, 40, 20, scale=0.3), dense(72)),
            ],
        },
        "block_size": 4,
    },
    # the loop runs to the last layer; heads of 64 and of 128; many experts; pages of 32 tokens
    "d": {
        "config": {
            "architecture": "Gukirax", "vocab": 211, "width": 96, "norm": {"eps": 1e-5}, "logit_scale": 0.25, "logit_softcap": 30.0,
            "loop": {"start": 1, "stop": 3, "times": 2},
            "layers": [
                layer(attention(8, 2, 64, 32), dense(128)),
                layer(attention(4, 2, 128, 64, base=1e6), moe(16, 4, 64, 32)),
                layer(attention(8, 2, 64, 32), moe(16, 4, 64)),
            ],
        },
        "block_size": 32,
    },
    # heads whose sizes are no multiple of 8 (12, 20 and 36 numbers), of which 6, 10 and all turn; a width that is one neither
    "e": {
        "config": {
            "architecture": "Gukirax", "vocab": 77, "width": 52, "norm": {"eps": 1e-5}, "logit_scale": 0.7, "logit_softcap": 15.0,
            "loop": {"start": 0, "stop": 2, "times": 2},
            "layers": [
                layer(attention(3, 3, 12, 6), moe(5, 2, 20, 12)),
                layer(attention(4, 2, 20, 10, base=1000.0), dense(44)),
                layer(attention(2, 1, 36, 36), None),
            ],
        },
        "block_size": 8,
    },
}  # fmt: skip


def tensor_shapes(config: dict) -> dict[str, tuple[int, ...]]:
    """Checkpoint name -> shape, from the design's naming alone."""
    w = config["width"]
    out = {"embed": (config["vocab"], w), "embed.norm": (w,), "final.norm": (w,)}
    if config.get("loop"):
        out["loop.in"] = (w, 2 * w)
    for i, ly in enumerate(config["layers"]):
        p, m = f"l{i}.", ly["mixer"]
        h, g, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        out.update({p + "norm1": (w,), p + "norm1b": (w,), p + "rg1": (w, w), p + "rg1.b": (w,)})
        q = p + "mix."
        out.update({q + "q": (h * d, w), q + "k": (g * d, w), q + "talk": (h, h), q + "sink": (h,), q + "o": (w, h * dv)})
        f = ly["mlp"]
        if f is None:
            continue
        out.update({p + "norm2": (w,), p + "norm2b": (w,), p + "rg2": (w, w), p + "rg2.b": (w,)})
        q = p + "mlp."
        if f["kind"] == "dense":
            out.update({q + "up": (f["ff"], w), q + "down": (w, f["ff"]), q + "act": (2,)})
        else:
            out[q + "router"] = (f["router"]["experts"], w)
            for k in range(f["router"]["experts"]):
                out.update({f"{q}e{k}.up": (f["expert"]["ff"], w), f"{q}e{k}.down": (w, f["expert"]["ff"])})
            if f.get("shared"):
                out.update({q + "shared.up": (f["shared"]["ff"], w), q + "shared.down": (w, f["shared"]["ff"])})
    return out


def random_tensors(config: dict, seed: int, router_spread: float = 1.5) -> dict[str, torch.Tensor]:
    """Weights of order one where it matters, rounded to bfloat16 (what the files hold), as float32.  The mixing
    matrices of the heads are far from the identity and the sinks of the order of the scores, so that leaving
    either out shows.  ``router_spread``: the router's logits are of this order; a wide spread makes the choice of
    experts robust against rounding (a token's last chosen experts then carry little weight)."""
    g = torch.Generator().manual_seed(seed)
    w = config["width"]
    out = {}
    for name, shape in tensor_shapes(config).items():
        leaf = name.rsplit(".", 1)[-1]
        r = torch.randn(shape, generator=g)
        if name == "embed":
            t = r
        elif leaf in ("norm", "norm1", "norm2", "norm1b", "norm2b"):
            t = 1.0 + 0.2 * r
        elif leaf == "talk":
            t = torch.eye(shape[0]) * 0.8 + 0.5 * r
        elif leaf == "sink":
            t = 1.0 + r
        elif leaf == "act":
            t = 0.5 * r
        elif leaf == "b":
            t = 0.5 * r
        elif leaf == "router":
            t = r * router_spread / shape[-1] ** 0.5
        elif leaf == "in":
            t = torch.cat([torch.eye(w), 0.3 * torch.eye(w)], dim=1) + 0.5 * r / w**0.5
        else:
            t = r * (1.5 if leaf in ("q", "k") else 1.0) / shape[-1] ** 0.5
        out[name] = t.to(torch.bfloat16).to(torch.float32)
    return out


def plain_logits(config: dict, tensors: dict[str, torch.Tensor], tokens: list[int]) -> torch.Tensor:
    w = {k: v.double() for k, v in tensors.items()}
    return plain.logits(config, w, tokens)


def random_config(seed: int) -> dict:
    """A configuration drawn at random: widths that are and are not multiples of 16, one to twenty heads in any
    grouping, head sizes from 8 to 128 (multiples of 8 and not), values as wide as keys or narrower, any even number of turning dims, dense
    layers, experts with and without a shared one, layers without a feed-forward, a loop over any stretch (or none)
    with one to three passes."""
    rng = random.Random(seed)
    m8 = lambda lo, hi: 8 * rng.randint(lo, hi)  # noqa: E731
    width = rng.choice([m8(5, 24), 104, 136])
    n_layers = rng.randint(1, 5)
    experts = rng.choice([2, 4, 6, 9, 16, 24])
    layers = []
    for _ in range(n_layers):
        kv = rng.choice([1, 2, 3, 4])
        heads = kv * rng.choice([1, 2, 3, 5])
        dim = rng.choice([8, 12, 16, 20, 24, 40, 64, 96, 128])
        vdim = dim if rng.random() < 0.6 else 8 * rng.randint(1, dim // 8)
        rot = 2 * rng.randint(0, dim // 2)
        mixer = attention(heads, kv, dim, rot, vdim, base=rng.choice([100.0, 10000.0, 1e6]), scale=rng.uniform(0.05, 0.4))
        u = rng.random()
        if u < 0.2:
            mlp = None
        elif u < 0.5:
            mlp = dense(m8(2, 20))
        else:
            mlp = moe(experts, rng.randint(1, min(experts, 5)), m8(2, 12), m8(1, 8) if rng.random() < 0.6 else None)
        layers.append(layer(mixer, mlp))
    config = {"architecture": "Gukirax", "vocab": rng.randint(30, 300), "width": width, "norm": {"eps": rng.choice([1e-5, 1e-6])},
              "logit_scale": rng.uniform(0.2, 2.0), "layers": layers}  # fmt: skip
    if rng.random() < 0.7:
        config["logit_softcap"] = rng.uniform(10.0, 60.0)
    if rng.random() < 0.7:
        start = rng.randint(0, n_layers - 1)
        config["loop"] = {"start": start, "stop": rng.randint(start + 1, n_layers), "times": rng.randint(1, 3)}
    return config
