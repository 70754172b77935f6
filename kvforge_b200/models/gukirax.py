"""The Gukirax decoder as a ``ModelSpec``: which parts, with which constants, under which tensor names.

The embedding's output is normed (layer norm with a weight, no bias) before anything reads it.  Every layer is
the sandwich arrangement: a norm before and after each sublayer, and a logistic gate, computed from the
sublayer's input, on its result.  The mixer is grouped-query attention whose values are the keys as projected,
whose queries and keys are rotated (split pairs, the first dims only) and then RMS-normed without a weight,
whose heads' scores are mixed before the softmax, and whose softmax has a sink per head.  The feed-forward is a
plain layer with the xIELU activation, or routed experts (softmax scores, weights not renormalised, squared
ReLU) beside a shared expert, or absent.  A stretch of layers may run several times with the same weights;
every pass has cache entries of its own and starts from ``W_in [x; x0]`` with ``x0`` the embedding's output.
The output head is the embedding's table; the logits are scaled and capped softly.  Tensors of layer ``i``
start with ``l<i>.``."""

from __future__ import annotations

from ..config.gukirax_config import FeedForwardConfig, GukiraxConfig, TalkingAttentionConfig
from ..parts.base import PartSpec
from ..parts.model import LayerCall, LayerSpec, ModelSpec


def _attention(cfg: GukiraxConfig, a: TalkingAttentionConfig) -> PartSpec:
    position = None
    if a.rot_dims:
        position = PartSpec("rotary", {"head_dim": a.dim, "rotary_dim": a.rot_dims, "theta": a.rot_base, "scaling": None})
    return PartSpec(
        "talking_attention",
        {
            "hidden_size": cfg.hidden_size, "num_heads": a.heads, "num_kv_heads": a.kv_heads, "head_dim": a.dim, "v_head_dim": a.vdim,
            "scale": a.scale, "position": position, "qk_norm": {"eps": cfg.eps}, "values": "keys", "talk": True, "sink": True,
            "names": {"q_proj.weight": "q", "k_proj.weight": "k", "o_proj.weight": "o"},
        },
    )  # fmt: skip


def _feed_forward(cfg: GukiraxConfig, f: FeedForwardConfig) -> PartSpec:
    if f.kind == "dense":
        return PartSpec("plain_mlp", {"hidden_size": cfg.hidden_size, "intermediate_size": f.ff, "activation": "xielu"})
    shared = None
    if f.shared_ff is not None:
        shared = PartSpec("plain_mlp", {"hidden_size": cfg.hidden_size, "intermediate_size": f.shared_ff, "activation": "relu2"})
    return PartSpec(
        "routed_experts",
        {
            "hidden_size": cfg.hidden_size, "experts": f.experts, "top": f.top, "intermediate_size": f.ff, "activation": "relu2",
            "score": "softmax", "normalize": False, "correction": False, "shared": shared,
        },
    )  # fmt: skip


def gukirax_spec(cfg: GukiraxConfig) -> ModelSpec:
    norm = PartSpec("layernorm", {"dim": cfg.hidden_size, "eps": cfg.eps})
    named = lambda name: PartSpec("layernorm", {"dim": cfg.hidden_size, "eps": cfg.eps, "names": {"weight": name}})  # noqa: E731
    layers = []
    for i, lc in enumerate(cfg.layers):
        block = PartSpec(
            "sandwich",
            {"hidden_size": cfg.hidden_size, "norm": norm, "mixer": _attention(cfg, lc.mixer), "ffn": _feed_forward(cfg, lc.mlp) if lc.mlp is not None else None},
        )
        layers.append(LayerSpec(block=block, prefix=f"l{i}."))
    n = len(cfg.layers)
    if cfg.loop is None:
        execution = [LayerCall(i) for i in range(n)]
    else:
        lp = cfg.loop
        execution = [LayerCall(i) for i in range(lp.start)]
        for _ in range(lp.times):
            execution += [LayerCall(i, mix_input=(i == lp.start)) for i in range(lp.start, lp.stop)]
        execution += [LayerCall(i) for i in range(lp.stop, n)]
    return ModelSpec(
        architecture=cfg.architecture,
        hidden_size=cfg.hidden_size,
        vocab_size=cfg.vocab_size,
        layers=layers,
        execution=execution,
        final_norm=named("norm"),
        final_norm_prefix="final.",
        embedding_name="embed",
        lm_head_name="head",
        tie_word_embeddings=True,
        head=PartSpec("linear_head", {"vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size, "scale": cfg.logit_scale, "softcap": cfg.logit_softcap}),
        ignore_suffixes=(),
        max_position_embeddings=cfg.max_position_embeddings,
        embedding_norm=named("norm"),
        embedding_norm_prefix="embed.",
        pass_mix_name="loop.in" if cfg.loop is not None else None,
    )
