"""Typed configuration of the Gukirax decoder, read from its ``config.json``.

The file gives every size and every constant that differs between models of the design::

    {"architecture": "Gukirax", "vocab": V, "width": W, "norm": {"eps": e}, "logit_scale": s, "logit_softcap": c,
     "loop": {"start": a, "stop": b, "times": t} | absent,
     "layers": [{"type": "attention", "mixer": {...}, "mlp": {...} | null}, ...]}

An ``attention`` mixer: ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale`` and ``rot.{dims, base}``.  A
feed-forward: ``kind`` ``"dense"`` with ``ff``, or ``kind`` ``"moe"`` with ``expert.ff``, ``router.{experts, top}``
and, where every token also passes a shared expert, ``shared.ff``.  Nothing here has a default that stands for a
size.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

from .model_config import ConfigError

ARCHITECTURE = "Gukirax"


def _need(d, key: str, where: str):
    if not isinstance(d, dict) or key not in d:
        raise ConfigError(f"config.json lacks {where}{key}")
    return d[key]


@dataclass(frozen=True)
class TalkingAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot_dims: int
    rot_base: float

    @classmethod
    def from_dict(cls, d: dict, where: str) -> TalkingAttentionConfig:
        rot = d.get("rot") or {}
        dims = int(rot.get("dims", 0))
        out = cls(
            heads=int(_need(d, "heads", where)), kv_heads=int(_need(d, "kv_heads", where)), dim=int(_need(d, "dim", where)),
            vdim=int(_need(d, "vdim", where)), scale=float(_need(d, "scale", where)), rot_dims=dims,
            rot_base=float(_need(rot, "base", where + "rot.")) if dims else 10000.0,
        )  # fmt: skip
        if out.kv_heads <= 0 or out.heads % out.kv_heads:
            raise ConfigError(f"{where}heads must be a multiple of kv_heads")
        if out.rot_dims % 2 or not 0 <= out.rot_dims <= out.dim:
            raise ConfigError(f"{where}rot.dims must be even and at most dim")
        if not 0 < out.vdim <= out.dim:
            raise ConfigError(f"{where}vdim must be at most dim: the values are the keys as projected")
        return out


@dataclass(frozen=True)
class FeedForwardConfig:
    kind: str  # "dense" or "moe"
    ff: int  # inner size of the dense layer, or of one expert
    experts: int = 0
    top: int = 0
    shared_ff: int | None = None

    @classmethod
    def from_dict(cls, d: dict, where: str) -> FeedForwardConfig:
        kind = _need(d, "kind", where)
        if kind == "dense":
            return cls("dense", int(_need(d, "ff", where)))
        if kind != "moe":
            raise ConfigError(f"{where}kind {kind!r} is not a feed-forward of this design ('dense', 'moe')")
        r = _need(d, "router", where)
        shared = d.get("shared")
        out = cls(
            "moe", int(_need(_need(d, "expert", where), "ff", where + "expert.")), int(_need(r, "experts", where + "router.")),
            int(_need(r, "top", where + "router.")), int(_need(shared, "ff", where + "shared.")) if shared else None,
        )  # fmt: skip
        if not 0 < out.top <= out.experts:
            raise ConfigError(f"{where}router: 'top' must be between 1 and the number of experts")
        return out


@dataclass(frozen=True)
class LayerConfig:
    type: str  # "attention"
    mixer: TalkingAttentionConfig
    mlp: FeedForwardConfig | None


@dataclass(frozen=True)
class LoopConfig:
    start: int
    stop: int
    times: int


@dataclass
class GukiraxConfig:
    vocab_size: int
    hidden_size: int
    eps: float
    logit_scale: float
    logit_softcap: float
    layers: list[LayerConfig]
    loop: LoopConfig | None = None
    architectures: list[str] = field(default_factory=lambda: [ARCHITECTURE])
    raw: dict[str, Any] = field(default_factory=dict, repr=False)

    @property
    def architecture(self) -> str:
        return self.architectures[0]

    @property
    def num_layers(self) -> int:
        return len(self.layers)

    @property
    def max_position_embeddings(self) -> int:
        return 1 << 30  # the design names no longest sequence

    @classmethod
    def from_dict(cls, d: dict[str, Any]) -> GukiraxConfig:
        layers = []
        for i, ld in enumerate(_need(d, "layers", "")):
            where = f"layers[{i}]."
            kind = _need(ld, "type", where)
            if kind != "attention":
                raise ConfigError(f"{where}type {kind!r} is not a mixer of this design ('attention')")
            mlp = ld.get("mlp")
            layers.append(
                LayerConfig(kind, TalkingAttentionConfig.from_dict(_need(ld, "mixer", where), where + "mixer."),
                            FeedForwardConfig.from_dict(mlp, where + "mlp.") if mlp is not None else None)
            )  # fmt: skip
        loop = d.get("loop")
        if loop:
            loop = LoopConfig(int(_need(loop, "start", "loop.")), int(_need(loop, "stop", "loop.")), int(_need(loop, "times", "loop.")))
            if not 0 <= loop.start < loop.stop <= len(layers) or loop.times < 1:
                raise ConfigError("loop: start < stop within the layers and at least one pass are needed")
        cap = d.get("logit_softcap")
        scale = d.get("logit_scale")
        return cls(
            vocab_size=int(_need(d, "vocab", "")), hidden_size=int(_need(d, "width", "")),
            eps=float(_need(_need(d, "norm", ""), "eps", "norm.")), logit_scale=float(scale) if scale is not None else 1.0,
            logit_softcap=float(cap) if cap else 0.0, layers=layers, loop=loop or None, raw=dict(d),
        )  # fmt: skip

    def to_hf_dict(self) -> dict[str, Any]:
        """The ``config.json`` of this configuration."""
        layers = []
        for lc in self.layers:
            m = lc.mixer
            mixer = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "scale": m.scale, "rot": {"dims": m.rot_dims, "base": m.rot_base}}
            mlp = None
            if lc.mlp is not None and lc.mlp.kind == "dense":
                mlp = {"kind": "dense", "ff": lc.mlp.ff}
            elif lc.mlp is not None:
                mlp = {"kind": "moe", "expert": {"ff": lc.mlp.ff}, "router": {"experts": lc.mlp.experts, "top": lc.mlp.top}}
                if lc.mlp.shared_ff is not None:
                    mlp["shared"] = {"ff": lc.mlp.shared_ff}
            layers.append({"type": lc.type, "mixer": mixer, "mlp": mlp})
        out = {
            "architecture": ARCHITECTURE, "vocab": self.vocab_size, "width": self.hidden_size, "norm": {"eps": self.eps},
            "logit_scale": self.logit_scale, "logit_softcap": self.logit_softcap, "layers": layers,
        }  # fmt: skip
        if self.loop is not None:
            out["loop"] = {"start": self.loop.start, "stop": self.loop.stop, "times": self.loop.times}
        return out


def uniform(
    *, vocab: int, width: int, num_layers: int, heads: int, kv_heads: int, dim: int, rot_dims: int, dense_ff: int, dense_layers: int,
    experts: int, top: int, ff: int, shared_ff: int | None, loop: LoopConfig | None = None, eps: float = 1e-5, base: float = 10000.0,
    logit_scale: float = 1.0, logit_softcap: float = 30.0,
) -> GukiraxConfig:  # fmt: skip
    """A configuration whose layers all have the same attention, whose first ``dense_layers`` layers have a dense
    feed-forward and whose other layers have routed experts: what the named shapes below are made with."""
    attn = TalkingAttentionConfig(heads, kv_heads, dim, dim, dim**-0.5, rot_dims, base)
    layers = [
        LayerConfig("attention", attn, FeedForwardConfig("dense", dense_ff) if i < dense_layers else FeedForwardConfig("moe", ff, experts, top, shared_ff))
        for i in range(num_layers)
    ]
    return GukiraxConfig(vocab, width, eps, logit_scale, logit_softcap, layers, loop)


# Named shapes with random weights: a small one for demonstrations, and one with the width, depth, heads and
# vocabulary of the 1B Llama shape this engine is measured on (a token's feed-forward flops are that shape's:
# 4 of 32 experts of 1,536 and a shared expert of 2,048; the first layer is dense), and one with those of the 3B
# Llama shape, heads of 128, and a stretch of four layers that runs twice.
GUKIRAX_PRESETS: dict[str, GukiraxConfig] = {
    "gukirax-tiny": uniform(
        vocab=256, width=96, num_layers=3, heads=4, kv_heads=2, dim=32, rot_dims=16, dense_ff=160, dense_layers=1, experts=8, top=2, ff=48,
        shared_ff=64, loop=LoopConfig(1, 3, 2), logit_scale=0.5,
    ),
    "gukirax-1b": uniform(
        vocab=128256, width=2048, num_layers=16, heads=32, kv_heads=8, dim=64, rot_dims=32, dense_ff=8192, dense_layers=1, experts=32, top=4,
        ff=1536, shared_ff=2048, base=500000.0, logit_scale=0.125,
    ),
    "gukirax-3b": uniform(
        vocab=128256, width=3072, num_layers=24, heads=24, kv_heads=8, dim=128, rot_dims=64, dense_ff=8192, dense_layers=2, experts=32, top=4,
        ff=1536, shared_ff=2048, loop=LoopConfig(10, 14, 2), base=500000.0, logit_scale=0.125,
    ),
}  # fmt: skip
