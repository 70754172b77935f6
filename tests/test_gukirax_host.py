"""The Gukirax decoder's configuration, naming and assembly, on the host (no GPU)."""

from __future__ import annotations

import json

import pytest
import torch

import plain_gukirax as plain
from gukirax_cases import CASES, random_config, random_tensors, tensor_shapes
from kvforge_b200.config.gukirax_config import GUKIRAX_PRESETS, GukiraxConfig
from kvforge_b200.config.model_config import ConfigError
from kvforge_b200.config.registry import PRESETS, architecture_of
from kvforge_b200.parts.model import DecoderModel


def build(config):
    arch = architecture_of(config)
    cfg = arch.parse_config(config)
    return cfg, arch.build_spec(cfg)


@pytest.mark.parametrize("name", sorted(CASES))
def test_names_and_shapes_follow_the_naming(name):
    config = CASES[name]["config"]
    cfg, spec = build(config)
    assert isinstance(cfg, GukiraxConfig)
    want = {k: v for k, v in DecoderModel(spec).expected_weights().items() if not v.optional}
    assert {k: tuple(v.shape) for k, v in want.items()} == tensor_shapes(config)
    kinds = {k.rsplit(".", 1)[-1]: v.kind for k, v in want.items()}
    assert kinds["talk"] == kinds["sink"] == kinds["b"] == kinds["norm1b"] == "vector"
    assert kinds["q"] == kinds["o"] == kinds["rg1"] == "matrix"


@pytest.mark.parametrize("seed", range(12))
def test_drawn_configurations_build_and_round_trip(seed):
    config = random_config(seed)
    cfg, spec = build(config)
    assert {k: tuple(v.shape) for k, v in DecoderModel(spec).expected_weights().items() if not v.optional} == tensor_shapes(config)
    again = GukiraxConfig.from_dict(json.loads(json.dumps(cfg.to_hf_dict())))
    assert again.layers == cfg.layers and again.loop == cfg.loop and again.logit_softcap == cfg.logit_softcap


def test_the_loop_becomes_the_run_order_with_a_cache_entry_per_run():
    config = CASES["a"]["config"]
    _, spec = build(config)
    assert [(c.layer, c.mix_input) for c in spec.execution] == plain.run_order(config)
    model = DecoderModel(spec)
    assert sum(len(g.calls) for g in model.groups) == len(spec.execution)
    # values narrower than keys are a group of their own
    assert len(model.groups) == 3
    _, flat = build(CASES["c"]["config"])
    assert not any(c.mix_input for c in flat.execution) and "loop.in" not in DecoderModel(flat).expected_weights()


def test_what_the_file_must_say():
    good = CASES["a"]["config"]
    for path, value in ((("layers", 0, "type"), "window"), (("layers", 1, "mlp", "kind"), "glu"), (("layers", 0, "mixer", "kv_heads"), 3),
                        (("layers", 0, "mixer", "rot", "dims"), 7), (("layers", 0, "mixer", "vdim"), 24), (("loop", "stop"), 9),
                        (("layers", 1, "mlp", "router", "top"), 7)):  # fmt: skip
        bad = json.loads(json.dumps(good))
        at = bad
        for key in path[:-1]:
            at = at[key]
        at[path[-1]] = value
        with pytest.raises(ConfigError):
            build(bad)
    for key in ("vocab", "width", "norm", "layers"):
        bad = {k: v for k, v in good.items() if k != key}
        with pytest.raises(ConfigError):
            build(bad)


def test_named_shapes():
    for name in GUKIRAX_PRESETS:
        cfg = PRESETS[name]
        spec = architecture_of({"architecture": "Gukirax"}).build_spec(cfg)
        model = DecoderModel(spec)
        assert model.expected_weights()
    assert PRESETS["gukirax-1b"].hidden_size == PRESETS["llama-3.2-1b"].hidden_size


def test_the_plain_model_feels_every_mechanism():
    """Leaving out the sink, the mixing of the heads, the gate, the second norm or the loop's input moves the plain
    logits by far more than any tolerance of the GPU tests."""
    config = CASES["a"]["config"]
    w = {k: v.double() for k, v in random_tensors(config, 5).items()}
    toks = [int(t) for t in torch.randint(0, config["vocab"], (40,), generator=torch.Generator().manual_seed(1))]
    ref = plain.logits(config, w, toks)
    scale = float(ref.pow(2).mean().sqrt())

    def moved(change):
        w2 = dict(w)
        change(w2)
        d = plain.logits(config, w2, toks) - ref
        return float(d.pow(2).mean().sqrt()) / scale

    def no_sink(w2):
        for k in w2:
            if k.endswith("sink"):
                w2[k] = torch.full_like(w2[k], -60.0)

    def no_talk(w2):
        for k in w2:
            if k.endswith("talk"):
                w2[k] = torch.eye(w2[k].shape[0], dtype=torch.float64)

    def no_gate(w2):
        for k in list(w2):
            if k.endswith(("rg1", "rg2")):
                w2[k] = torch.zeros_like(w2[k])
                w2[k + ".b"] = torch.full_like(w2[k + ".b"], 40.0)

    def no_x0(w2):
        width = config["width"]
        w2["loop.in"] = torch.cat([w2["loop.in"][:, :width], torch.zeros(width, width, dtype=torch.float64)], dim=1)

    for change in (no_sink, no_talk, no_gate, no_x0):
        assert moved(change) > 0.02, change.__name__
