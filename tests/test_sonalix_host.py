"""What of the Sonalix decoder needs no GPU: the configuration and its names, which layer is the source of
the mixed values, the state and cache that the model asks for, and the plain implementation's own pieces."""

from __future__ import annotations

import copy
import math

import pytest
import torch

import plain_sonalix as plain
from sonalix_cases import CASES, random_config, random_tensors, tensor_shapes


def parsed(config):
    from kvforge_b200.config.registry import architecture_of
    from kvforge_b200.parts.model import DecoderModel

    arch = architecture_of(config)
    cfg = arch.parse_config(config)
    return arch, cfg, DecoderModel(arch.build_spec(cfg))


@pytest.mark.parametrize("name", sorted(CASES) + ["drawn-5", "drawn-6", "drawn-7"])
def test_names_and_shapes_follow_the_configuration(name):
    config = CASES[name]["config"] if name in CASES else random_config(int(name.split("-")[1]))
    arch, cfg, model = parsed(config)
    got = {k: tuple(d.shape) for k, d in model.expected_weights().items()}
    assert got == tensor_shapes(config)
    # what the file says comes back when it is written again
    again = arch.parse_config(cfg.to_hf_dict())
    assert again.layers == cfg.layers and again.embedding_scale == cfg.embedding_scale and again.residual_mult == cfg.residual_mult
    # retention layers keep a state and no pages; the others pages and no state
    for ly, shape, owner in zip(config["layers"], model.state_shapes, model.call_group):
        if ly["type"] == "retention":
            m = ly["mixer"]
            assert shape == (m["heads"] * m["dim"] * m["vdim"],) and owner is None
        else:
            assert shape is None and owner is not None


def test_the_first_layer_that_mixes_values_is_the_source():
    _, _, model = parsed(CASES["b"]["config"])
    roles = [b.mixer.value_mix for b in model.blocks if b.mixer.kind == "paged_attention"]
    assert roles == ["source", None, "mix"]
    _, _, model = parsed(CASES["c"]["config"])
    assert [b.mixer.value_mix for b in model.blocks if b.mixer.kind == "paged_attention"] == [None, "source"]
    # windows of 37 and of 5 keys are cache groups of their own, the latent rows a third
    _, _, model = parsed(CASES["b"]["config"])
    assert sorted((g.need.kind, g.need.window, len(g.calls)) for g in model.groups) == [("full", None, 1), ("full", None, 1), ("window", 5, 1), ("window", 37, 2)]


def test_what_the_file_lacks_or_gets_wrong_is_named():
    from kvforge_b200.config.model_config import ConfigError
    from kvforge_b200.config.sonalix_config import SonalixConfig

    base = CASES["a"]["config"]
    for path, value in (
        (("layers", 0, "type"), "mamba"),
        (("layers", 0, "mixer", "decay"), [0.9]),
        (("layers", 1, "mixer", "kv_heads"), 3),
        (("layers", 1, "mixer", "rot", "dims"), 18),
        (("layers", 2, "mixer", "rot", "dims"), 7),
        (("layers", 0, "mlp", "kind"), "sparse"),
        (("layers", 0, "mlp", "router", "top"), 7),
        (("layers", 3, "mixer", "vdim"), 16),  # two layers that mix values of different shapes
    ):
        config = copy.deepcopy(base)
        d = config
        for k in path[:-1]:
            d = d[k]
        d[path[-1]] = value
        with pytest.raises(ConfigError):
            SonalixConfig.from_dict(config)
    for key in ("vocab", "width", "norm", "layers"):
        with pytest.raises(ConfigError):
            SonalixConfig.from_dict({k: v for k, v in base.items() if k != key})
    cfg = SonalixConfig.from_dict({k: v for k, v in base.items() if k not in ("embedding", "residual_mult")})
    assert cfg.embedding_scale == 1.0 and cfg.residual_mult == 1.0


def test_named_shapes():
    from kvforge_b200 import PRESETS

    for name in ("sonalix-tiny", "sonalix-1b"):
        _, cfg, model = parsed(PRESETS[name].to_hf_dict())
        assert cfg.layers == PRESETS[name].layers
        assert {ly.type for ly in cfg.layers} == {"attention", "retention", "latent_attention"}
        assert model.expected_weights()


def test_plain_pieces():
    """The plain implementation on hand-made cases."""
    # rotation of split pairs: dim i with dim i + dims/2; the rest stays
    x = torch.tensor([[[1.0, 2.0, 3.0, 4.0, 5.0, 6.0]]], dtype=torch.float64)
    y = plain.turn_halves(x, torch.tensor([3]), 4, 100.0)
    a0, a1 = 3.0, 3.0 / 10.0
    want = [1 * math.cos(a0) - 3 * math.sin(a0), 2 * math.cos(a1) - 4 * math.sin(a1), 3 * math.cos(a0) + 1 * math.sin(a0), 4 * math.cos(a1) + 2 * math.sin(a1), 5.0, 6.0]
    assert torch.allclose(y[0, 0], torch.tensor(want, dtype=torch.float64))
    # the router: the largest logits with their bias, softmax over them alone
    w = {"m.router": torch.eye(4, dtype=torch.float64), "m.router.b": torch.tensor([0.0, 0.0, 2.5, 0.0], dtype=torch.float64)}
    chosen, weights = plain.route(torch.tensor([[1.0, 3.0, 0.0, -1.0]], dtype=torch.float64), w, "m.", {"experts": 4, "top": 2})
    assert chosen[0].tolist() == [1, 2]
    assert torch.allclose(weights[0], torch.softmax(torch.tensor([3.0, 2.5], dtype=torch.float64), 0))
    # an expert: the gate cut from above, the up from both sides, one added to the up
    w = {"e.gate": torch.tensor([[1.0], [1.0]], dtype=torch.float64), "e.up": torch.tensor([[1.0], [-1.0]], dtype=torch.float64), "e.down": torch.eye(2, dtype=torch.float64)}
    out = plain.expert(torch.tensor([5.0], dtype=torch.float64), w, "e.", 2.0)
    g = 2.0 / (1.0 + math.exp(-1.702 * 2.0))
    assert torch.allclose(out, torch.tensor([g * 3.0, g * -1.0], dtype=torch.float64))
    out = plain.expert(torch.tensor([-5.0], dtype=torch.float64), w, "e.", 2.0)
    g = -5.0 / (1.0 + math.exp(1.702 * 5.0))
    assert torch.allclose(out, torch.tensor([g * -1.0, g * 3.0], dtype=torch.float64))


def test_plain_retention_is_a_decaying_sum():
    """``o_t = sum_(s <= t) a^(t-s) (q_t . k_s) v_s`` before the norm: the recurrence against the sum written out."""
    m = {"heads": 1, "dim": 4, "vdim": 3, "decay": [0.8]}
    g = torch.Generator().manual_seed(1)
    w = {"m." + k: torch.randn(s, generator=g, dtype=torch.float64) for k, s in {"q": (4, 6), "k": (4, 6), "v": (3, 6), "g": (3, 6), "o": (6, 3)}.items()}
    x = torch.randn(7, 6, generator=g, dtype=torch.float64)
    q, k, v = x @ w["m.q"].T, (x @ w["m.k"].T) * 0.5, x @ w["m.v"].T
    o = torch.stack([sum(0.8 ** (t - s) * (q[t] @ k[s]) * v[s] for s in range(t + 1)) for t in range(7)])
    want = (plain.unit_rms(o, 1e-6) * plain.silu(x @ w["m.g"].T)) @ w["m.o"].T
    assert torch.allclose(plain.retention(x, w, "m.", m, 1e-6, {}), want)


def test_plain_model_sees_the_window_and_carries_the_state():
    """In the plain model a change of a token shows in a later position's logits when the token lies inside the window
    (attention alone), and at any distance once a retention layer carries it."""
    attn = {"heads": 2, "kv_heads": 1, "dim": 8, "vdim": 8, "scale": 0.35, "softcap": 10.0, "mask": {"size": 4}, "rot": {"dims": 8, "base": 100.0}, "v_mix": True}
    config = {"architecture": "Sonalix", "vocab": 50, "width": 32, "norm": {"eps": 1e-5}, "residual_mult": 0.9, "layers": [{"type": "attention", "mlp": None, "mixer": attn}]}
    w = {k: v.double() for k, v in random_tensors(config, 3).items()}
    base = list(range(10, 30))
    ref = plain.logits(config, w, base)
    for j in (1, 15, 16, 19):
        toks = list(base)
        toks[j] += 1
        moved = float((plain.logits(config, w, toks)[19] - ref[19]).abs().max())
        assert (moved > 1e-9) == (19 - j < 4), (j, moved)
    config["layers"].append({"type": "retention", "mlp": None, "mixer": {"heads": 2, "dim": 8, "vdim": 4, "decay": [0.9, 0.99], "rot": {"dims": 8, "base": 100.0}}})
    w = {k: v.double() for k, v in random_tensors(config, 4).items()}
    ref = plain.logits(config, w, base)
    toks = list(base)
    toks[1] += 1
    assert float((plain.logits(config, w, toks)[19] - ref[19]).abs().max()) > 1e-9
