"""The Sonalix decoder as a ``ModelSpec``: which parts, with which constants, under which tensor names.

Every layer is the pre-norm arrangement with a constant on what joins the stream
(``x += m * mixer(norm1(x))``, ``x += m * ffn(norm2(x))``) and a norm without statistics
(``tanh(alpha x) w + b``).  Its mixer is grouped-query attention under a sliding window (heads normed and turned in
split pairs, softly capped scores, a sink a head, values mixed with those of the first such layer), retention (a
matrix state a head with a fixed decay), or attention over a latent shared by keys and values whose queries come
through a latent of their own (a gate a channel).  Its feed-forward is the dense gated one or routed experts
(a router with a bias, softmax over the chosen logits, gated experts with clamped inputs), or absent.
Tensors of layer ``i`` start with ``l<i>.``."""

from __future__ import annotations

from ..config.sonalix_config import DenseConfig, ExpertsConfig, LatentAttentionConfig, RetentionConfig, SonalixConfig, WindowedAttentionConfig
from ..parts.base import PartSpec
from ..parts.model import LayerSpec, ModelSpec

# constants that the design fixes
EXPERT_GATE_SLOPE = 1.702  # the gate of an expert is g * sigmoid(1.702 g)
EXPERT_UP_SHIFT = 1.0  # and multiplies (u + 1)


def _rotary(head_dim: int, rot) -> PartSpec | None:
    if rot is None:
        return None
    return PartSpec("rotary", {"head_dim": head_dim, "rotary_dim": rot.dims, "theta": rot.base, "interleaved": False, "scaling": None})


def _attention(cfg: SonalixConfig, a: WindowedAttentionConfig, value_mix: str | None) -> PartSpec:
    return PartSpec(
        "paged_attention",
        {
            "hidden_size": cfg.hidden_size, "num_heads": a.heads, "num_kv_heads": a.kv_heads, "head_dim": a.dim, "v_head_dim": a.vdim,
            "scale": a.scale, "window": a.window, "position": _rotary(a.dim, a.rot), "qk_norm": {"eps": cfg.eps}, "softcap": a.softcap,
            "sink": True, "value_mix": value_mix,
            "names": {
                "q_proj.weight": "q", "k_proj.weight": "k", "v_proj.weight": "v", "o_proj.weight": "o",
                "q_norm.weight": "q.norm", "k_norm.weight": "k.norm",
            },
        },
    )  # fmt: skip


def _retention(cfg: SonalixConfig, r: RetentionConfig) -> PartSpec:
    return PartSpec(
        "retention",
        {
            "hidden_size": cfg.hidden_size, "num_heads": r.heads, "head_dim": r.dim, "v_head_dim": r.vdim, "decay": list(r.decay),
            "eps": cfg.eps, "position": _rotary(r.dim, r.rot), "gate": "silu",
        },
    )  # fmt: skip


def _latent(cfg: SonalixConfig, a: LatentAttentionConfig) -> PartSpec:
    return PartSpec(
        "latent_attention",
        {
            "hidden_size": cfg.hidden_size, "num_heads": a.heads, "head_dim": a.dim, "rot_dim": a.rot_dim, "v_head_dim": a.vdim,
            "kv_rank": a.kv_rank, "q_rank": a.q_rank, "eps": cfg.eps, "scale": a.scale, "window": None,
            "position": _rotary(a.rot_dim, a.rot), "gate": "sigmoid_channel",
        },
    )  # fmt: skip


def _feed_forward(cfg: SonalixConfig, m) -> PartSpec | None:
    if m is None:
        return None
    if isinstance(m, DenseConfig):
        return PartSpec(
            "gated_mlp",
            {
                "hidden_size": cfg.hidden_size, "intermediate_size": m.ff, "activation": "silu",
                "names": {"gate_proj.weight": "gate", "up_proj.weight": "up", "down_proj.weight": "down"},
            },
        )  # fmt: skip
    assert isinstance(m, ExpertsConfig)
    return PartSpec(
        "routed_experts",
        {
            "hidden_size": cfg.hidden_size, "experts": m.experts, "top": m.top, "intermediate_size": m.ff, "correction": False,
            "score": "chosen_softmax", "router_bias": True, "activation": "gated",
            "gated": {"limit": m.limit, "alpha": EXPERT_GATE_SLOPE, "shift": EXPERT_UP_SHIFT},
        },
    )  # fmt: skip


def sonalix_spec(cfg: SonalixConfig) -> ModelSpec:
    def norm(name: str) -> PartSpec:
        return PartSpec("tanh_norm", {"dim": cfg.hidden_size, "names": {"weight": name, "alpha": f"{name}.alpha", "bias": f"{name}.b"}})

    layers = []
    mixes_values = False  # the first layer that mixes values is the source of the others
    for i, lc in enumerate(cfg.layers):
        if lc.type == "attention":
            role = None
            if lc.mixer.v_mix:
                role = "mix" if mixes_values else "source"
                mixes_values = True
            mixer = _attention(cfg, lc.mixer, role)
        elif lc.type == "retention":
            mixer = _retention(cfg, lc.mixer)
        else:
            mixer = _latent(cfg, lc.mixer)
        ffn = _feed_forward(cfg, lc.mlp)
        block = PartSpec(
            "prenorm",
            {
                "norm1": norm("norm1"), "mixer": mixer, "norm2": norm("norm2") if ffn is not None else None, "ffn": ffn,
                "norm1_name": "", "norm2_name": "", "mixer_name": "mix", "ffn_name": "mlp", "residual_mult": cfg.residual_mult,
            },
        )  # fmt: skip
        layers.append(LayerSpec(block=block, prefix=f"l{i}."))
    return ModelSpec(
        architecture=cfg.architecture,
        hidden_size=cfg.hidden_size,
        vocab_size=cfg.vocab_size,
        layers=layers,
        final_norm=norm("norm"),
        final_norm_prefix="final.",
        embedding_name="embed",
        lm_head_name="head",
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size, "scale": cfg.embedding_scale}),
        ignore_suffixes=(),
        max_position_embeddings=cfg.max_position_embeddings,
    )
