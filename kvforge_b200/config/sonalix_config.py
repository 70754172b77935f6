"""Typed configuration of the Sonalix decoder, read from its ``config.json``.

The file gives every size and every constant that differs between models of the design::

    {"architecture": "Sonalix", "vocab": V, "width": W, "norm": {"eps": e}, "embedding": {"scale": s},
     "residual_mult": m,
     "layers": [{"type": "attention" | "retention" | "latent_attention", "mixer": {...}, "mlp": {...} | null}, ...]}

An ``attention`` mixer: ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``softcap``, ``mask.size``,
``rot.{dims, base}``, ``v_mix``.  A ``retention`` mixer: ``heads``, ``dim``, ``vdim``, ``decay`` (one number a head),
``rot.{dims, base}``.  A ``latent_attention`` mixer: ``heads``, ``dim``, ``rot_dim``, ``vdim``, ``kv_rank``, ``q_rank``,
``scale``, ``rot.{dims, base}``.  A feed-forward: ``kind`` ``"dense"`` with ``ff``, or ``"moe"`` with ``expert.{ff, limit}``
and ``router.{experts, top}``.  Nothing here has a default that stands for a size.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

from .model_config import ConfigError

ARCHITECTURE = "Sonalix"


def _need(d, key: str, where: str):
    if not isinstance(d, dict) or key not in d:
        raise ConfigError(f"config.json lacks {where}{key}")
    return d[key]


@dataclass(frozen=True)
class Rotation:
    dims: int
    base: float

    @classmethod
    def from_dict(cls, d: dict | None, where: str, most: int) -> Rotation | None:
        if not d:
            return None
        out = cls(int(_need(d, "dims", where)), float(_need(d, "base", where)))
        if out.dims % 2 or not 0 < out.dims <= most:
            raise ConfigError(f"{where}dims must be even and at most {most}")
        return out

    def to_dict(self) -> dict:
        return {"dims": self.dims, "base": self.base}


@dataclass(frozen=True)
class WindowedAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: float | None
    window: int | None
    rot: Rotation | None
    v_mix: bool

    @classmethod
    def from_dict(cls, d: dict, where: str) -> WindowedAttentionConfig:
        mask = d.get("mask")
        dim = int(_need(d, "dim", where))
        cap = d.get("softcap")
        out = cls(
            heads=int(_need(d, "heads", where)), kv_heads=int(_need(d, "kv_heads", where)), dim=dim, vdim=int(_need(d, "vdim", where)),
            scale=float(_need(d, "scale", where)), softcap=float(cap) if cap else None,
            window=int(_need(mask, "size", where + "mask.")) if mask else None, rot=Rotation.from_dict(d.get("rot"), where + "rot.", dim),
            v_mix=bool(d.get("v_mix", False)),
        )  # fmt: skip
        if out.kv_heads <= 0 or out.heads % out.kv_heads:
            raise ConfigError(f"{where}heads must be a multiple of kv_heads")
        if out.window is not None and out.window <= 0:
            raise ConfigError(f"{where}mask.size must be positive")
        if out.softcap is not None and out.softcap <= 0:
            raise ConfigError(f"{where}softcap must be positive")
        return out

    def to_dict(self) -> dict:
        out = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale, "v_mix": self.v_mix}
        if self.softcap is not None:
            out["softcap"] = self.softcap
        if self.window is not None:
            out["mask"] = {"size": self.window}
        if self.rot is not None:
            out["rot"] = self.rot.to_dict()
        return out


@dataclass(frozen=True)
class RetentionConfig:
    heads: int
    dim: int
    vdim: int
    decay: tuple[float, ...]
    rot: Rotation | None

    @classmethod
    def from_dict(cls, d: dict, where: str) -> RetentionConfig:
        dim = int(_need(d, "dim", where))
        out = cls(
            heads=int(_need(d, "heads", where)), dim=dim, vdim=int(_need(d, "vdim", where)),
            decay=tuple(float(a) for a in _need(d, "decay", where)), rot=Rotation.from_dict(d.get("rot"), where + "rot.", dim),
        )  # fmt: skip
        if len(out.decay) != out.heads:
            raise ConfigError(f"{where}decay must hold one number per head")
        return out

    def to_dict(self) -> dict:
        out = {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "decay": list(self.decay)}
        if self.rot is not None:
            out["rot"] = self.rot.to_dict()
        return out


@dataclass(frozen=True)
class LatentAttentionConfig:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    q_rank: int
    scale: float
    rot: Rotation | None

    @classmethod
    def from_dict(cls, d: dict, where: str) -> LatentAttentionConfig:
        rot_dim = int(_need(d, "rot_dim", where))
        out = cls(
            heads=int(_need(d, "heads", where)), dim=int(_need(d, "dim", where)), rot_dim=rot_dim, vdim=int(_need(d, "vdim", where)),
            kv_rank=int(_need(d, "kv_rank", where)), q_rank=int(_need(d, "q_rank", where)), scale=float(_need(d, "scale", where)),
            rot=Rotation.from_dict(d.get("rot"), where + "rot.", rot_dim),
        )  # fmt: skip
        return out

    def to_dict(self) -> dict:
        out = {"heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim, "vdim": self.vdim, "kv_rank": self.kv_rank, "q_rank": self.q_rank, "scale": self.scale}
        if self.rot is not None:
            out["rot"] = self.rot.to_dict()
        return out


@dataclass(frozen=True)
class DenseConfig:
    ff: int

    def to_dict(self) -> dict:
        return {"kind": "dense", "ff": self.ff}


@dataclass(frozen=True)
class ExpertsConfig:
    experts: int
    top: int
    ff: int
    limit: float

    def to_dict(self) -> dict:
        return {"kind": "moe", "expert": {"ff": self.ff, "limit": self.limit}, "router": {"experts": self.experts, "top": self.top}}


def _mlp(d: dict | None, where: str):
    if d is None:
        return None
    kind = _need(d, "kind", where)
    if kind == "dense":
        return DenseConfig(int(_need(d, "ff", where)))
    if kind == "moe":
        r, e = _need(d, "router", where), _need(d, "expert", where)
        out = ExpertsConfig(
            experts=int(_need(r, "experts", where + "router.")), top=int(_need(r, "top", where + "router.")),
            ff=int(_need(e, "ff", where + "expert.")), limit=float(_need(e, "limit", where + "expert.")),
        )  # fmt: skip
        if not 0 < out.top <= out.experts:
            raise ConfigError(f"{where}router.top must be between 1 and the number of experts")
        return out
    raise ConfigError(f"{where}kind {kind!r} is not a feed-forward of this design ('dense', 'moe')")


MIXERS = {"attention": WindowedAttentionConfig, "retention": RetentionConfig, "latent_attention": LatentAttentionConfig}


@dataclass(frozen=True)
class LayerConfig:
    type: str
    mixer: WindowedAttentionConfig | RetentionConfig | LatentAttentionConfig
    mlp: DenseConfig | ExpertsConfig | None


@dataclass
class SonalixConfig:
    vocab_size: int
    hidden_size: int
    eps: float
    embedding_scale: float
    residual_mult: float
    layers: list[LayerConfig]
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

    def __post_init__(self) -> None:
        # the layers that mix values share the first one's values: they must be of one shape
        shapes = {(lc.mixer.kv_heads, lc.mixer.vdim) for lc in self.layers if lc.type == "attention" and lc.mixer.v_mix}
        if len(shapes) > 1:
            raise ConfigError("the attention layers that mix values must have the same kv_heads and vdim")

    @classmethod
    def from_dict(cls, d: dict[str, Any]) -> SonalixConfig:
        layers = []
        for i, ld in enumerate(_need(d, "layers", "")):
            where = f"layers[{i}]."
            kind = _need(ld, "type", where)
            if kind not in MIXERS:
                raise ConfigError(f"{where}type {kind!r} is not a mixer of this design ({sorted(MIXERS)})")
            layers.append(LayerConfig(kind, MIXERS[kind].from_dict(_need(ld, "mixer", where), where + "mixer."), _mlp(ld.get("mlp"), where + "mlp.")))
        emb = d.get("embedding") or {}
        return cls(
            vocab_size=int(_need(d, "vocab", "")), hidden_size=int(_need(d, "width", "")), eps=float(_need(_need(d, "norm", ""), "eps", "norm.")),
            embedding_scale=float(emb.get("scale", 1.0)), residual_mult=float(d.get("residual_mult", 1.0)), layers=layers, raw=dict(d),
        )  # fmt: skip

    def to_hf_dict(self) -> dict[str, Any]:
        return {
            "architecture": ARCHITECTURE, "vocab": self.vocab_size, "width": self.hidden_size, "norm": {"eps": self.eps},
            "embedding": {"scale": self.embedding_scale}, "residual_mult": self.residual_mult,
            "layers": [{"type": lc.type, "mixer": lc.mixer.to_dict(), "mlp": lc.mlp.to_dict() if lc.mlp is not None else None} for lc in self.layers],
        }  # fmt: skip


def patterned(
    *, vocab: int, width: int, pattern: str, repeats: int, heads: int, kv_heads: int, dim: int, window: int, softcap: float, ret_heads: int,
    ret_dim: int, latent_heads: int, latent_dim: int, rot_dim: int, kv_rank: int, q_rank: int, dense_ff: int, experts: int, top: int, ff: int,
    limit: float = 7.0, eps: float = 1e-6, residual_mult: float = 1.0, base: float = 10000.0,
) -> SonalixConfig:  # fmt: skip
    """A configuration whose layers follow ``pattern`` (a letter a layer: ``a`` attention, ``r`` retention, ``l`` latent
    attention) ``repeats`` times; the first layer has a dense feed-forward, the others routed experts: what the named
    shapes below are made with.  Retention heads decay by ``1 - 2^-(5 + h)``."""
    attn = WindowedAttentionConfig(heads, kv_heads, dim, dim, dim**-0.5, softcap, window, Rotation(dim, base), True)
    ret = RetentionConfig(ret_heads, ret_dim, ret_dim, tuple(1.0 - 2.0 ** -(5 + h % 8) for h in range(ret_heads)), Rotation(ret_dim, base))
    lat = LatentAttentionConfig(latent_heads, latent_dim, rot_dim, latent_dim, kv_rank, q_rank, (latent_dim + rot_dim) ** -0.5, Rotation(rot_dim, base))
    mixers = {"a": ("attention", attn), "r": ("retention", ret), "l": ("latent_attention", lat)}
    layers = []
    for i, letter in enumerate(pattern * repeats):
        kind, mixer = mixers[letter]
        layers.append(LayerConfig(kind, mixer, DenseConfig(dense_ff) if i == 0 else ExpertsConfig(experts, top, ff, limit)))
    return SonalixConfig(vocab, width, eps, float(width) ** 0.5, residual_mult, layers)


# Named shapes with random weights: a small one for demonstrations, and one with the width, depth and vocabulary of the
# 1B Llama shape this engine is measured on (a token's feed-forward has that shape's flops: 4 of 32 experts of three
# matrices of 1,408 where the Setenex shape of that size has two of 2,048).
SONALIX_PRESETS: dict[str, SonalixConfig] = {
    "sonalix-tiny": patterned(
        vocab=256, width=96, pattern="arl", repeats=1, heads=4, kv_heads=2, dim=32, window=24, softcap=15.0, ret_heads=2, ret_dim=16,
        latent_heads=3, latent_dim=16, rot_dim=8, kv_rank=32, q_rank=24, dense_ff=128, experts=8, top=2, ff=48, residual_mult=0.8,
    ),
    "sonalix-1b": patterned(
        vocab=128256, width=2048, pattern="aral", repeats=4, heads=32, kv_heads=8, dim=64, window=1024, softcap=30.0, ret_heads=16,
        ret_dim=128, latent_heads=16, latent_dim=128, rot_dim=64, kv_rank=512, q_rank=768, dense_ff=8192, experts=32, top=4, ff=1408,
        residual_mult=0.5, base=500000.0,
    ),
}  # fmt: skip
