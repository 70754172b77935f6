"""Small Sonalix configurations for the tests, model folders with random weights made here (not by
the package's random-weights mode), and the plain implementation's logits for them.

The configurations differ from one another in every size and option: the order of the layers (each
kind of mixer first, last, twice in a row), heads and key heads (as many key heads as heads, a single
key head), key and value sizes (equal and not), how many dims turn (all, some), windows (shorter than a
page, longer than several, none), caps, layers that mix values and layers that do not, one decay or
several, latents of the queries and of the keys of many sizes, dense and routed feed-forwards and none,
one expert a token and several, inner sizes that are no multiple of 8, and a residual constant of one.
"""

from __future__ import annotations

import random

import torch

import plain_sonalix as plain
from mopilorn_cases import row_error, write_folder  # noqa: F401  (the folder writer and the error measure are the same)


def attention(heads, kv_heads, dim, vdim, window=None, softcap=None, rot=None, base=10000.0, v_mix=True, scale=None):
    out = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else dim**-0.5, "v_mix": v_mix}
    if window is not None:
        out["mask"] = {"size": window}
    if softcap is not None:
        out["softcap"] = softcap
    if rot != 0:
        out["rot"] = {"dims": rot or dim, "base": base}
    return out


def retention(heads, dim, vdim, decay, rot=None, base=10000.0):
    out = {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}
    if rot != 0:
        out["rot"] = {"dims": rot or dim, "base": base}
    return out


def latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, base=10000.0, scale=None, rot=None):
    return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
            "rot": {"dims": rot or rot_dim, "base": base}, "scale": scale if scale is not None else (dim + rot_dim) ** -0.5}  # fmt: skip


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, limit=2.5):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}


def layer(kind, mixer, mlp):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


def model(vocab, width, layers, eps=1e-6, scale=4.0, mult=0.75):
    return {"architecture": "Sonalix", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": scale}, "residual_mult": mult, "layers": layers}


CASES: dict[str, dict] = {
    # retention first; two attention layers that mix values around a latent layer; a window shorter than a page; some dims turn
    "a": {
        "config": model(131, 64, [
            layer("retention", retention(2, 16, 24, [0.9, 0.99]), moe(6, 2, 40)),
            layer("attention", attention(4, 2, 16, 24, window=11, softcap=8.0, rot=8), dense(72)),
            layer("latent_attention", latent(3, 16, 8, 24, 24, 40), moe(6, 2, 40)),
            layer("attention", attention(4, 2, 16, 24, window=11, softcap=8.0, rot=8), None),
        ], eps=1e-5, scale=3.0, mult=0.6),
        "block_size": 16,
    },
    # latent attention first and last; as many key heads as heads; an attention layer that mixes no values between two that do,
    # with another window (a cache group of its own); one expert a token; an inner size of the experts that is no multiple of 8
    "b": {
        "config": model(97, 48, [
            layer("latent_attention", latent(2, 8, 16, 8, 40, 16, base=500.0), moe(4, 1, 20, limit=1.0)),
            layer("attention", attention(3, 3, 24, 8, window=37, softcap=5.0, base=300.0), moe(4, 1, 20, limit=1.0)),
            layer("attention", attention(3, 3, 24, 8, window=5, softcap=5.0, base=300.0, v_mix=False), dense(50)),
            layer("retention", retention(3, 8, 8, [0.5, 0.9375, 1.0], rot=4), None),
            layer("attention", attention(3, 3, 24, 8, window=37, softcap=5.0, base=300.0), moe(4, 1, 20, limit=1.0)),
            layer("latent_attention", latent(4, 16, 8, 16, 16, 24, rot=4), dense(64)),
        ], scale=1.0, mult=1.0),
        "block_size": 8,
    },
    # attention that sees every key (no mask, no cap) with a single key head and no rotation; two retention layers in a row
    # with one head; three experts a token; pages of four tokens
    "c": {
        "config": model(150, 40, [
            layer("attention", attention(4, 1, 16, 16, rot=0, v_mix=False), moe(8, 3, 24, limit=3.5)),
            layer("retention", retention(1, 32, 8, [0.97], rot=0), moe(8, 3, 24, limit=3.5)),
            layer("retention", retention(1, 32, 8, [0.97], rot=0), dense(24)),
            layer("attention", attention(2, 2, 8, 16, window=6, softcap=30.0), moe(8, 3, 24, limit=3.5)),
        ], scale=0.5, mult=1.3),
        "block_size": 4,
    },
    # heads of 64 and 128, four heads a key head; a latent wider than a head; retention with keys of 128; many experts
    "d": {
        "config": model(211, 96, [
            layer("attention", attention(8, 2, 64, 64, window=48, softcap=25.0), moe(16, 4, 64)),
            layer("retention", retention(2, 128, 64, [0.984375, 0.998]), moe(16, 4, 64)),
            layer("latent_attention", latent(4, 32, 32, 48, 64, 96), moe(16, 4, 64)),
            layer("attention", attention(8, 2, 64, 64, window=48, softcap=25.0), dense(160)),
            layer("retention", retention(4, 64, 128, [0.9, 0.95, 0.99, 0.999], rot=32), None),
        ], eps=1e-5, scale=9.0, mult=0.5),
        "block_size": 16,
    },
}  # fmt: skip


def tensor_shapes(config: dict) -> dict[str, tuple[int, ...]]:
    """Checkpoint name -> shape, from the design's naming alone."""
    w = config["width"]
    out = {"embed": (config["vocab"], w), "head": (config["vocab"], w)}

    def norm(name):
        out.update({name: (w,), name + ".b": (w,), name + ".alpha": ()})

    norm("final.norm")
    for i, ly in enumerate(config["layers"]):
        p, m = f"l{i}.", ly["mixer"]
        norm(p + "norm1")
        q = p + "mix."
        if ly["type"] == "attention":
            h, g, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            out.update({q + "q": (h * dk, w), q + "k": (g * dk, w), q + "v": (g * dv, w), q + "q.norm": (dk,), q + "k.norm": (dk,),
                        q + "sink": (h,), q + "o": (w, h * dv)})  # fmt: skip
            if m.get("v_mix"):
                out[q + "vmix"] = ()
        elif ly["type"] == "retention":
            h, dk, dv = m["heads"], m["dim"], m["vdim"]
            out.update({q + "q": (h * dk, w), q + "k": (h * dk, w), q + "v": (h * dv, w), q + "g": (h * dv, w), q + "o": (w, h * dv)})
        else:
            h, dk, dr, dv, r, qr = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
            out.update({q + "dq": (qr, w), q + "dq.norm": (qr,), q + "uq": (h * (dk + dr), qr), q + "dkv": (r + dr, w), q + "dkv.norm": (r,),
                        q + "uk": (h * dk, r), q + "uv": (h * dv, r), q + "g": (h * dv, w), q + "o": (w, h * dv)})  # fmt: skip
        mlp = ly["mlp"]
        if mlp:
            norm(p + "norm2")
            q = p + "mlp."
            if mlp["kind"] == "dense":
                out.update({q + "gate": (mlp["ff"], w), q + "up": (mlp["ff"], w), q + "down": (w, mlp["ff"])})
            else:
                e, ff = mlp["router"]["experts"], mlp["expert"]["ff"]
                out.update({q + "router": (e, w), q + "router.b": (e,)})
                for k in range(e):
                    out.update({f"{q}e{k}.gate": (ff, w), f"{q}e{k}.up": (ff, w), f"{q}e{k}.down": (w, ff)})
    return out


def random_tensors(config: dict, seed: int, fixed_choice: bool = False) -> dict[str, torch.Tensor]:
    """Weights of order one where it matters, rounded to bfloat16 (what the files hold), as float32.
    ``fixed_choice``: the router's biases lie so far apart that they alone decide which experts a token uses
    (the weights of the chosen experts still follow the token): rounding cannot change the choice then."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(config).items():
        leaf = name.rsplit(".", 1)[-1]
        r = torch.randn(shape, generator=g)
        if name == "embed":
            t = r
        elif leaf == "alpha":
            t = 0.4 + 0.1 * r
        elif leaf == "vmix":
            t = 0.3 + 0.1 * r
        elif leaf == "sink":
            t = 1.0 + r
        elif leaf in ("norm1", "norm2") or name == "final.norm" or (leaf == "norm" and "mix." in name):
            t = 1.0 + 0.2 * r
        elif name.endswith("router.b"):
            t = 0.9 * torch.randperm(shape[0], generator=g).float() if fixed_choice else 0.3 * r
        elif leaf == "b":
            t = 0.1 * r
        elif leaf == "router":
            t = r * (0.3 if fixed_choice else 1.5) / shape[-1] ** 0.5
        else:
            t = r * (1.5 if leaf in ("q", "k", "dkv", "uk", "dq", "uq", "gate", "up") else 1.0) / shape[-1] ** 0.5
        out[name] = t.to(torch.bfloat16).to(torch.float32)
    return out


def plain_logits(config: dict, tensors: dict[str, torch.Tensor], tokens: list[int]) -> torch.Tensor:
    w = {k: v.double() for k, v in tensors.items()}
    return plain.logits(config, w, tokens)


def random_config(seed: int) -> dict:
    """A configuration drawn at random: widths that are and are not multiples of 8, one to twelve heads, one key head or
    several, key and value sizes from 8 to 128, some or all dims turning, windows of 1 to 100 tokens or none, with and
    without a cap, latents of 8 to 160 numbers, 4 to 24 experts, inner sizes that are no multiple of 8, layers without a
    feed-forward, a residual constant around one."""
    rng = random.Random(seed)
    m8 = lambda lo, hi: 8 * rng.randint(lo, hi)  # noqa: E731
    width = rng.choice([m8(5, 20), 100, 132])
    n_layers = rng.randint(2, 5)
    experts = rng.choice([4, 6, 9, 10, 16, 24])
    kv = rng.choice([1, 2, 3])
    mixed_vdim = rng.choice([8, 16, 48, 72])  # layers that mix values share the shape of their values
    layers = []
    for _ in range(n_layers):
        kind = rng.choice(["attention", "retention", "latent_attention"])
        if kind == "attention":
            v_mix = rng.random() < 0.7
            g = kv if v_mix else rng.choice([1, 2])
            heads = g * rng.choice([1, 2, 3, 5])
            dim = rng.choice([8, 16, 24, 40, 64, 128])
            vdim = mixed_vdim if v_mix else rng.choice([8, 24, 64])
            mixer = attention(heads, g, dim, vdim, window=rng.choice([None, rng.randint(1, 90)]), softcap=rng.choice([None, rng.uniform(3.0, 40.0)]),
                              rot=rng.choice([0, dim, 2 * rng.randint(1, dim // 2)]), base=rng.choice([100.0, 10000.0, 1e6]), v_mix=v_mix,
                              scale=rng.uniform(0.05, 0.3))  # fmt: skip
        elif kind == "retention":
            heads, dim = rng.choice([1, 2, 3, 6]), rng.choice([8, 16, 20, 48, 64, 96])
            mixer = retention(heads, dim, rng.choice([8, 12, 32, 40, 100]), [rng.choice([0.5, 0.9, 0.9375, 0.99, 0.9995]) for _ in range(heads)],
                              rot=rng.choice([0, dim, 2 * rng.randint(1, dim // 2)]), base=rng.choice([100.0, 1e6]))  # fmt: skip
        else:
            heads, dim, rot = rng.choice([1, 2, 5, 8, 12]), rng.choice([8, 16, 32]), rng.choice([8, 16, 32, 64])
            mixer = latent(heads, dim, rot, rng.choice([8, 24, 40]), rng.choice([8, 24, 32, 48, 64, 96, 128, 160]), rng.choice([8, 24, 56, 128]),
                           base=rng.choice([100.0, 10000.0, 1e6]), scale=rng.uniform(0.05, 0.3), rot=rng.choice([rot, 2 * rng.randint(1, rot // 2)]))  # fmt: skip
        which = rng.random()
        mlp = None if which < 0.15 else dense(rng.choice([m8(2, 12), 36, 50])) if which < 0.4 else moe(experts, rng.randint(1, min(experts, 5)), rng.choice([m8(2, 10), 20, 36]), rng.choice([1.0, 2.0, 7.0]))
        layers.append(layer(kind, mixer, mlp))
    return model(rng.randint(30, 300), width, layers, eps=rng.choice([1e-5, 1e-6]), scale=rng.uniform(0.5, 12), mult=rng.choice([1.0, rng.uniform(0.4, 1.4)]))
