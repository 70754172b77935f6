"""The Gukirax decoder on the GPU against the plain implementation (``plain_gukirax``): each mechanism
alone, then whole models with random weights made here, replayed whole, token by token, in portions down to
two tokens and mixed with other requests on few pages and slots; in 32-bit and in bfloat16, eager and as
captured graphs; and greedy generation through the engine's entry point."""

from __future__ import annotations

import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import plain_gukirax as plain
import traces
from gukirax_cases import CASES, attention, plain_logits, random_config, random_tensors, row_error, write_folder
from test_gpu_mopilorn import check, run_trace, tokens
from test_gpu_parts import context, runtime

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent
TOL = {"float32": 1e-4, "bfloat16": 0.25}
SHARP_TOL = 1e-3
LENGTHS = {"a": [70, 3, 41, 1, 26, 97], "b": [9, 120, 33, 2, 64, 50], "c": [45, 17, 5, 80, 30], "d": [130, 20, 75, 49, 9], "e": [66, 2, 31, 90]}
# the router's logits are spread wide where activations are rounded to bfloat16: a token's last chosen expert then
# carries little weight, and a choice that rounding turns moves the logits by little
SPREAD = {"float32": 1.5, "bfloat16": 5.0}


def build(tmp, name, config, w, lengths, seed=40):
    folder = write_folder(tmp / name, config, w)
    reqs = {f"{name}{i}": tokens(config["vocab"], n, seed + i) for i, n in enumerate(lengths)}
    ref = {rid: plain_logits(config, w, t) for rid, t in reqs.items()}
    scale = float(torch.cat(list(ref.values())).pow(2).mean().sqrt())
    return folder, reqs, ref, scale, w


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    """Per case and storage type: folder, requests, plain logits of every request whole, the logits' scale."""
    tmp = tmp_path_factory.mktemp("gukirax")
    out = {}
    for k, (name, case) in enumerate(sorted(CASES.items())):
        for dtype in ("float32", "bfloat16"):
            w = random_tensors(case["config"], 17 + k, router_spread=SPREAD[dtype])
            out[name, dtype] = build(tmp, f"{name}-{dtype}", case["config"], w, LENGTHS[name])
    return out


def regime_steps(reqs, regime):
    if regime == "whole":
        return traces.whole(reqs)
    if regime == "tail":
        return traces.tail_one_by_one(reqs, 40)
    if regime == "portions":
        return traces.portions(reqs)
    prompt_lens = {rid: max(1, len(t) - 14) for rid, t in reqs.items()}
    steps = traces.mixed(reqs, prompt_lens, max_live=4, seed=5)
    assert max(len(s["entries"]) for s in steps) >= 3
    return steps


# ------------------------------------------------------------------ whole models


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CASES))
@pytest.mark.parametrize("regime", ["whole", "tail", "portions", "mixed"])
def test_replay_regimes(models, name, dtype, regime):
    """Whole prompts; the last 40 tokens one by one; portions of 1 to 33 tokens; up to four live requests on as
    few pages as they need (pages and slots are used again).  Every pass of a looped layer has pages of its own."""
    folder, reqs, ref, scale, _ = models[name, dtype]
    steps = regime_steps(reqs, regime)
    outs, runner = run_trace(folder, dtype, steps, CASES[name]["block_size"])
    check(steps, outs, ref, scale, TOL[dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CASES))
@pytest.mark.parametrize("regime", ["tail", "mixed"])
def test_replay_as_captured_graphs(models, name, dtype, regime):
    """The way generation runs by default: single-token steps and steps of more than 16 tokens as CUDA graphs
    made for padded shapes.  Padding sequences and rows must leave every cache alone."""
    folder, reqs, ref, scale, _ = models[name, dtype]
    steps = traces.last_only(regime_steps(reqs, regime))
    outs, runner = run_trace(folder, dtype, steps, CASES[name]["block_size"], cuda_graphs=True)
    check(steps, outs, ref, scale, TOL[dtype])
    assert runner.core.runner.num_graph_kernels > 0


def test_batch_and_cutting_change_float32_logits_by_rounding_only(models):
    folder, reqs, ref, scale, _ = models["a", "float32"]
    whole, _ = run_trace(folder, "float32", traces.whole(reqs), 16)
    by_place = {}
    for rows, got in zip(traces.wanted_places(traces.whole(reqs)), whole):
        for i, place in enumerate(rows):
            by_place[place] = got[i]
    for regime in ("portions", "mixed"):
        steps = regime_steps(reqs, regime)
        outs, _ = run_trace(folder, "float32", steps, 16)
        worst = 0.0
        for rows, got in zip(traces.wanted_places(steps), outs):
            for i, place in enumerate(rows):
                worst = max(worst, float((got[i] - by_place[place]).abs().max()))
        assert worst <= 2e-5 * scale, (regime, worst)


@pytest.mark.parametrize("seed", [3, 12, 29, 41, 57, 68, 75, 86])
def test_configurations_drawn_at_random(tmp_path, seed):
    """Sizes that no hand-made case has (widths that are no multiple of 16, one head, twenty heads, one expert a
    token, nine experts, a single pass of a loop, a loop over everything, ...), each replayed whole, in portions
    and mixed, in both storage types."""
    config = random_config(seed)
    block_size = [4, 8, 16, 32][seed % 4]
    for dtype in ("float32", "bfloat16"):
        w = random_tensors(config, 100 + seed, router_spread=SPREAD[dtype])
        folder, reqs, ref, scale, _ = build(tmp_path, f"drawn-{dtype}", config, w, [90, 1, 37, 140], seed=seed)
        for regime in ("whole", "portions", "mixed"):
            steps = regime_steps(reqs, regime) if regime != "mixed" else traces.mixed(reqs, {r: max(1, len(t) - 10) for r, t in reqs.items()}, max_live=4, seed=seed)
            outs, _ = run_trace(folder, dtype, steps, block_size)
            check(steps, outs, ref, scale, TOL[dtype])


def sharpened(config):
    """Scores five times as large: a few keys take nearly all the weight, and the sink a good part of the rest."""
    cfg = json.loads(json.dumps(config))
    for ly in cfg["layers"]:
        ly["mixer"]["scale"] *= 5.0
    return cfg


def test_sharp_attention_far_keys_and_the_sink(tmp_path):
    """With sharp scores over sequences of several hundred tokens a far key among hundreds decides a row.  The
    plain model without the sinks, or with the heads' scores left unmixed, is far outside the tolerance."""
    for name in ("a", "c"):
        case = CASES[name]
        cfg = sharpened(case["config"])
        w = random_tensors(cfg, seed=91)
        folder, reqs, ref, scale, _ = build(tmp_path, f"sharp-{name}", cfg, w, [310, 150], seed=70)
        rid = f"sharp-{name}1"
        for leaf, value in (("sink", lambda t: torch.full_like(t, -80.0)), ("talk", lambda t: torch.eye(t.shape[0]))):
            w2 = {k: (value(v) if k.endswith(leaf) else v) for k, v in w.items()}
            off = plain_logits(cfg, w2, reqs[rid])
            errs = sorted(row_error(off[i], ref[rid][i], scale) for i in range(len(reqs[rid])))
            assert errs[int(len(errs) * 0.8)] > 20 * SHARP_TOL, (name, leaf)  # a fifth of the rows at least is far off
        for regime in ("whole", "tail", "portions"):
            steps = regime_steps(reqs, regime)
            outs, _ = run_trace(folder, "float32", steps, case["block_size"])
            check(steps, outs, ref, scale, SHARP_TOL, SHARP_TOL)


def test_long_decoding(models):
    """Three hundred tokens one by one after a prompt of five, eager in 32-bit and as graphs in bfloat16: the
    key ranges of the decode form grow from one to several, and pages are taken one after another."""
    for name in ("a", "b"):
        case = CASES[name]
        for dtype, graphs in (("float32", False), ("bfloat16", True)):
            folder, _, _, _, w = models[name, dtype]
            reqs = {"long": tokens(case["config"]["vocab"], 305, 7)}
            ref = {"long": plain_logits(case["config"], w, reqs["long"])}
            scale = float(ref["long"].pow(2).mean().sqrt())
            steps = traces.tail_one_by_one(reqs, 300)
            outs, _ = run_trace(folder, dtype, steps, case["block_size"], cuda_graphs=graphs)
            check(steps, outs, ref, scale, TOL[dtype])


def test_the_trace_program_reads_a_folder_and_writes_logits(models, tmp_path):
    folder, reqs, ref, scale, _ = models["b", "float32"]
    steps = traces.portions(dict(list(reqs.items())[:3]))
    lines = "\n".join(json.dumps(s) for s in steps) + "\n"
    out = tmp_path / "out"
    res = subprocess.run(
        [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", "float32", "--out", str(out), "--max-tokens", "256", "--max-live", "4"],
        input=lines, capture_output=True, text=True, timeout=600,
    )  # fmt: skip
    assert res.returncode == 0, res.stderr[-2000:]
    assert [ln for ln in res.stdout.splitlines() if ln.startswith("done")] == [f"done {s['step']}" for s in steps]
    vocab = CASES["b"]["config"]["vocab"]
    outs = [torch.from_numpy(np.fromfile(out / f"{s['step']}.f32", dtype="<f4").reshape(-1, vocab).copy()) for s in steps]
    check(steps, outs, ref, scale, TOL["float32"])


# ------------------------------------------------------------------ generation through the entry point


@pytest.mark.parametrize("name", ["a", "b", "d"])
def test_greedy_generation_through_the_engine(models, name):
    """``InferenceEngine.generate`` with its scheduler: more requests than slots, prompts cut into portions,
    decode steps as graphs, tokens read a step late."""
    from kvforge_b200 import CacheConfig, EngineConfig, InferenceEngine, SamplingParams, SchedulerConfig

    folder, _, _, _, w = models[name, "float32"]
    case = CASES[name]
    prompts = [tokens(case["config"]["vocab"], n, 300 + i) for i, n in enumerate([3, 40, 11, 1, 25, 18])]
    cfg = EngineConfig(
        cache=CacheConfig(block_size=case["block_size"], num_blocks=128),
        scheduler=SchedulerConfig(max_num_seqs=3, max_num_batched_tokens=32, max_model_len=128),
        dtype="float32",
    )
    engine = InferenceEngine(cfg, model=folder)
    outs = engine.generate(prompts, SamplingParams(max_tokens=12, temperature=0.0, ignore_eos=True))
    wd = {k: v.double() for k, v in w.items()}
    for p, o in zip(prompts, outs):
        assert o.output_token_ids == plain.greedy(case["config"], wd, p, 12)
    assert engine.core.state_slots.num_free == 3


def test_generation_from_a_named_shape_with_random_weights():
    from kvforge_b200 import PRESETS, EngineConfig, InferenceEngine, SamplingParams, SchedulerConfig

    cfg = EngineConfig(model=PRESETS["gukirax-tiny"], scheduler=SchedulerConfig(max_num_seqs=4, max_num_batched_tokens=64, max_model_len=96), dtype="bfloat16")
    engine = InferenceEngine(cfg)
    outs = engine.generate([[1, 2, 3], list(range(40))], SamplingParams(max_tokens=8, temperature=0.0, ignore_eos=True))
    assert all(len(o.output_token_ids) == 8 for o in outs)


# ------------------------------------------------------------------ mechanisms alone


def as_float(y, n):
    from kvforge_b200 import ops

    return y.t[:, :n].sum(0) if isinstance(y, ops.Partials) else y[:n].float()


def part_tol(dtype):
    return 2e-5 if dtype == torch.float32 else 3e-2


def rel_rows(got, want):
    return float((got.double() - want.double()).abs().max() / want.double().abs().max())


def bind(part, w, dtype):
    kinds = type(part).weight_decls(part.params)
    names = part.params.get("names", {})
    return {local: (w[names.get(local, local)].cuda() if decl.kind == "vector" else w[names.get(local, local)].to(dtype).cuda()) for local, decl in kinds.items()}


def talking_part(width, m, eps):
    from kvforge_b200.parts.base import PartSpec, build_part

    pos = PartSpec("rotary", {"head_dim": m["dim"], "rotary_dim": m["rot"]["dims"], "theta": m["rot"]["base"], "scaling": None}) if m["rot"]["dims"] else None
    return build_part("mixer", PartSpec("talking_attention", {
        "hidden_size": width, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"], "v_head_dim": m["vdim"], "scale": m["scale"],
        "position": pos, "qk_norm": {"eps": eps}, "values": "keys", "talk": True, "sink": True,
        "names": {"q_proj.weight": "q", "k_proj.weight": "k", "o_proj.weight": "o"}}), "m.")  # fmt: skip


def step_mixer(part, rt, x, bs, table, cuts, cache):
    """Run a mixer over a sequence cut into steps on pages of a shuffled table."""
    t = x.shape[0]
    slots = [table[p // bs] * bs + p % bs for p in range(t)]
    got = []
    for a, b in cuts:
        ctx = context(rt, [b - a], [a], bs, [table], slots[a:b])
        got.append(as_float(part.forward(ctx, x[a:b].cuda(), cache), b - a).cpu().clone())
    return torch.cat(got)


def mixer_weights(g, width, m, dtype):
    nh, nkv, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    w = {
        "q": torch.randn(nh * d, width, generator=g) / width**0.5, "k": torch.randn(nkv * d, width, generator=g) / width**0.5,
        "o": torch.randn(width, nh * dv, generator=g) / (nh * dv) ** 0.5, "talk": torch.eye(nh) * 0.8 + 0.5 * torch.randn(nh, nh, generator=g),
        "sink": 1.0 + torch.randn(nh, generator=g),
    }  # fmt: skip
    return {k: v.to(dtype).float() for k, v in w.items()}


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize(
    "nh,nkv,d,dv,rot,t,bs",
    [(6, 3, 24, 24, 8, 45, 4), (4, 4, 64, 64, 64, 200, 16), (8, 2, 128, 128, 32, 150, 8), (1, 1, 16, 8, 0, 70, 4), (20, 4, 8, 8, 8, 90, 32), (3, 1, 96, 96, 24, 300, 64),
     (32, 8, 64, 64, 32, 330, 16), (24, 8, 128, 128, 64, 210, 16), (12, 4, 64, 64, 16, 140, 8), (16, 1, 64, 64, 0, 97, 4), (64, 8, 64, 64, 64, 80, 32),
     (1, 1, 128, 128, 128, 170, 16), (40, 8, 64, 64, 32, 75, 16), (2, 2, 64, 32, 32, 60, 8), (16, 16, 64, 64, 32, 100, 16),
     (5, 5, 12, 12, 6, 60, 4), (3, 1, 20, 20, 10, 90, 8), (2, 2, 36, 36, 36, 70, 16), (4, 2, 100, 100, 50, 50, 4), (2, 1, 6, 6, 2, 40, 4)],
)  # fmt: skip
def test_attention_whose_heads_talk(dtype, nh, nkv, d, dv, rot, t, bs):
    """The whole sequence in one step, then portions and single tokens on top of the cache (the decode form: key
    ranges in parallel, then a merge), on pages in a shuffled order, against the plain mixer.  In bfloat16 heads of
    64 and of 128 whose values are as wide go to the tensor-core form: one, three, four and sixteen heads a key
    head (rows of a key head that fill an m-tile, fall short of one, or make several), one or two m-tiles a warp."""
    from kvforge_b200.parts.base import LayerCache

    rt = runtime(dtype, max_tokens=512)
    width, eps = 80, 1e-5
    m = attention(nh, nkv, d, rot, dv, base=300.0, scale=2.0 / d**0.5)
    part = talking_part(width, m, eps)
    g = torch.Generator().manual_seed(3)
    w = mixer_weights(g, width, m, dtype)
    part.bind(bind(part, w, dtype), rt)
    x = torch.randn(t, width, generator=g).to(dtype)
    ref = plain.talking_attention(x.double(), {"m." + k: v.double() for k, v in w.items()}, "m.", m, eps)
    nb = -(-t // bs) + 5
    table = [int(i) for i in torch.randperm(nb, generator=g)]
    need = part.cache_need()
    assert need.kind == "full" and need.kv_heads == nkv and need.head_dim == d
    cache = LayerCache(torch.zeros(nb, nkv, bs, d, device="cuda", dtype=dtype), torch.zeros(nb, nkv, bs, dv, device="cuda", dtype=dtype), 0)
    for cuts in ([(0, t)], [(0, 17), (17, 19), (19, 20), (20, 21), (21, 34), (34, 35), (35, 36), (36, t - 3), (t - 3, t - 2), (t - 2, t)]):
        got = step_mixer(part, rt, x, bs, table, cuts, cache)
        assert rel_rows(got, ref) < part_tol(dtype), cuts


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("far", [0, 1, 15, 16, 31, 32, 63, 64, 127, 128, 129, 255, 256, 511, 512, 640])
def test_one_far_key_takes_the_weight(far, dtype):
    """A sequence of 700 tokens whose last tokens ask for one key far back: that key's input is a multiple of
    theirs, queries and keys share their matrix and few dims turn, so its score stands far above the others'
    and the sink's is set beside it.  The key sits at the sequence's first places, around the borders of pages
    (16 tokens) and of the decode form's key ranges (128).  Prompts' rows and single decoded tokens must find it;
    the plain mixer without that key, or without the sink, gives another result by far.  In bfloat16 this is the
    tensor-core form, whose key tiles are 64 keys in prompts and 32 in the decode form."""
    from kvforge_b200.parts.base import LayerCache

    rt = runtime(dtype, max_tokens=1024)
    width, eps, t, bs, nh, d = 64, 1e-5, 700, 16, 4, 64
    m = attention(nh, nh, d, 4, d, base=10000.0, scale=0.5)
    part = talking_part(width, m, eps)
    g = torch.Generator().manual_seed(far)
    w = mixer_weights(g, width, m, dtype)
    w["k"] = w["q"].clone()
    w["talk"] = torch.eye(nh) + 0.1 * torch.randn(nh, nh, generator=g)
    w["sink"] = torch.full((nh,), 0.5 * d - 2.0)  # a score of (nearly) d * scale stands beside it
    x = torch.randn(t, width, generator=g)
    ask = list(range(t - 6, t))
    for i in ask:
        x[i] = x[far] * (0.5 + 0.1 * (i - t + 7))
    x = x.to(dtype).float()
    w = {k: v.to(dtype).float() for k, v in w.items()}
    tol = 1e-4 if dtype == torch.float32 else 2e-2
    part.bind(bind(part, w, dtype), rt)
    wd = {"m." + k: v.double() for k, v in w.items()}
    ref = plain.talking_attention(x.double(), wd, "m.", m, eps)
    x2 = x.clone()
    x2[far] = torch.randn(width, generator=g)
    without_key = plain.talking_attention(x2.double(), wd, "m.", m, eps)
    without_sink = plain.talking_attention(x.double(), {**wd, "m.sink": torch.full((nh,), -80.0, dtype=torch.float64)}, "m.", m, eps)
    if far < t - 6:
        assert rel_rows(without_key[ask], ref[ask]) > 0.05 and rel_rows(without_sink[ask], ref[ask]) > 0.05
    nb = t // bs + 3
    table = [int(i) for i in torch.randperm(nb, generator=g)]
    cache = LayerCache(torch.zeros(nb, nh, bs, d, device="cuda", dtype=dtype), torch.zeros(nb, nh, bs, d, device="cuda", dtype=dtype), 0)
    singles = [(i, i + 1) for i in range(t - 4, t)]
    for cuts in ([(0, t)], [(0, 300), (300, t - 4)] + singles, [(0, 2), (2, 130), (130, 132), (132, t - 5), (t - 5, t - 3), (t - 3, t - 2), (t - 2, t)]):
        got = step_mixer(part, rt, x.to(dtype), bs, table, cuts, cache)
        assert rel_rows(got[ask], ref[ask]) < tol, cuts
        assert rel_rows(got, ref) < tol, cuts


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n,width,ff", [(1, 48, 40), (7, 80, 136), (150, 64, 256)])
def test_plain_feed_forward_with_xielu(dtype, n, width, ff):
    from kvforge_b200.parts.base import PartSpec, build_part

    rt = runtime(dtype)
    part = build_part("ffn", PartSpec("plain_mlp", {"hidden_size": width, "intermediate_size": ff, "activation": "xielu"}), "m.")
    g = torch.Generator().manual_seed(n)
    w = {"up": (torch.randn(ff, width, generator=g) * 2.0 / width**0.5).to(dtype).float(), "down": (torch.randn(width, ff, generator=g) / ff**0.5).to(dtype).float(),
         "act": torch.tensor([0.7, -0.4])}  # fmt: skip
    part.bind(bind(part, w, dtype), rt)
    x = torch.randn(n, width, generator=g).to(dtype)
    ref = plain.dense_ff(x.double(), {"m." + k: v.double() for k, v in w.items()}, "m.")
    ctx = context(rt, [n], [0], 4, [[0]], [0] * n)
    assert rel_rows(as_float(part.forward(ctx, x.cuda()), n).cpu(), ref) < part_tol(dtype)


def test_activations_alone():
    """Both branches of xIELU around zero and far from it, the square of relu and the tanh form of GELU."""
    import math

    from kvforge_b200 import ops

    z = torch.cat([torch.linspace(-30, 30, 4001), torch.tensor([0.0, -0.0, 1e-6, -1e-6])]).view(1, -1)
    out = torch.empty_like(z, device="cuda")
    for p, q in ((0.7, -0.4), (-3.0, 2.5), (0.0, 0.0)):
        ops.unary_act(z.cuda(), out, "xielu", torch.tensor([p, q], device="cuda"))
        assert torch.allclose(out.cpu().double(), plain.xielu(z.double(), p, q), rtol=2e-6, atol=1e-6)
    ops.unary_act(z.cuda(), out, "relu2")
    assert torch.equal(out.cpu(), torch.relu(z).pow(2))
    ops.unary_act(z.cuda(), out, "gelu_tanh")
    zd = z.double()
    want = 0.5 * zd * (1 + torch.tanh(math.sqrt(2 / math.pi) * (zd + 0.044715 * zd**3)))
    assert torch.allclose(out.cpu().double(), want, rtol=2e-6, atol=1e-6)


@pytest.mark.parametrize("experts,top", [(6, 2), (8, 4), (4, 1), (9, 9), (40, 6), (2, 1)])
def test_softmax_router_alone(experts, top):
    """Chosen experts and their weights (the scores as they are: they do not sum to one) against the plain router."""
    from kvforge_b200 import ops

    g = torch.Generator().manual_seed(experts)
    width, n = 72, 200
    x = torch.randn(n, width, generator=g)
    w = {"m.router": torch.randn(experts, width, generator=g) * 0.3}
    chosen, weights = plain.route(x.double(), {k: v.double() for k, v in w.items()}, "m.", top)
    ids = torch.zeros(n, top, dtype=torch.int32, device="cuda")
    wts = torch.zeros(n, top, dtype=torch.float32, device="cuda")
    ops.moe_route(x.cuda(), w["m.router"].cuda(), None, top, 1, 1, 1e-20, ids, wts, True, False)
    same = 0
    for i in range(n):
        if sorted(ids[i].tolist()) == sorted(chosen[i].tolist()):
            same += 1
            order = {e: k for k, e in enumerate(ids[i].tolist())}
            got = torch.stack([wts[i, order[e]] for e in chosen[i].tolist()]).cpu()
            assert torch.allclose(got.double(), weights[i], atol=1e-6)
    assert same >= n - 2  # a near tie may fall the other way in 32-bit
    if top < experts:
        assert float(wts.sum(-1).max()) < 1.0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n", [1, 7, 30, 150, 400])
@pytest.mark.parametrize("shared", [None, 24])
def test_routed_experts_with_a_shared_expert(dtype, n, shared):
    from kvforge_b200.parts.base import PartSpec, build_part

    rt = runtime(dtype, max_tokens=512)
    width, experts, top, ff = 48, 6, 2, 40
    sp = PartSpec("plain_mlp", {"hidden_size": width, "intermediate_size": shared, "activation": "relu2"}) if shared else None
    part = build_part("ffn", PartSpec("routed_experts", {
        "hidden_size": width, "experts": experts, "top": top, "intermediate_size": ff, "activation": "relu2", "score": "softmax", "normalize": False,
        "correction": False, "shared": sp}), "m.")  # fmt: skip
    g = torch.Generator().manual_seed(11)
    w = {"router": torch.randn(experts, width, generator=g) * 0.8}
    for e in [f"e{i}" for i in range(experts)] + (["shared"] if shared else []):
        f = shared if e == "shared" else ff
        w[f"{e}.up"] = (torch.randn(f, width, generator=g) * 0.2).to(dtype).float()
        w[f"{e}.down"] = (torch.randn(width, f, generator=g) * 0.2).to(dtype).float()
    own = {k: v for k, v in w.items() if not k.startswith("shared.")}
    part.bind(bind(part, own, dtype), rt)
    if shared:
        part.shared.bind({"up": w["shared.up"].to(dtype).cuda(), "down": w["shared.down"].to(dtype).cuda()}, rt)
    x = torch.randn(n, width, generator=g).to(dtype)
    mlp = {"kind": "moe", "router": {"experts": experts, "top": top}, "shared": {"ff": shared} if shared else None}
    ref = plain.experts_ff(x.double(), {"m." + k: v.double() for k, v in w.items()}, "m.", mlp)
    ctx = context(rt, [n], [0], 4, [[0]], [0] * n)
    got = as_float(part.forward(ctx, x.cuda()), n).cpu()
    assert rel_rows(got, ref) < part_tol(dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width", [40, 96, 136, 1024])
def test_gated_normed_result_joins_the_stream(dtype, width):
    """``resid += norm(y * sigmoid(z + b)) * w_post`` and the next sublayer's input ``norm(resid) * w_next`` in one
    pass, against the plain formulas; the gate's logits are a view into a wider buffer."""
    from kvforge_b200 import ops

    g = torch.Generator().manual_seed(width)
    n, eps = 23, 1e-5
    resid = torch.randn(n, width, generator=g) * 3.0 + 0.5
    y = (torch.randn(n, width, generator=g) * 2.0).to(dtype)
    wide = torch.randn(n, width + 16, generator=g).to(dtype)
    b, w_post, w_next = (torch.randn(width, generator=g) * 0.5 for _ in range(3))
    want_resid = resid.double() + plain.layer_norm(y.double() * torch.sigmoid(wide[:, 8 : 8 + width].double() + b.double()), 1.0 + w_post.double(), eps)
    want_out = plain.layer_norm(want_resid, 1.0 + w_next.double(), eps)
    r = resid.cuda()
    out = torch.empty(n, width, device="cuda", dtype=dtype)
    ops.norm_step(r, ops.GatedWrite(y.cuda(), wide.cuda()[:, 8 : 8 + width], b.cuda(), (1.0 + w_post).cuda()), (1.0 + w_next).cuda(), out, eps, True)
    assert rel_rows(r.cpu(), want_resid) < 1e-5
    assert rel_rows(out.float().cpu(), want_out) < (1e-5 if dtype == torch.float32 else 1e-2)
    # the RMS norm through the same kernel, nothing pending
    ops.norm_step(r, None, w_next.cuda(), out, eps, False)
    want = want_resid / torch.sqrt(want_resid.pow(2).mean(-1, keepdim=True) + eps) * w_next.double()
    assert rel_rows(out.float().cpu(), want) < (1e-5 if dtype == torch.float32 else 1e-2)


def test_scaled_capped_logits():
    from kvforge_b200 import ops

    z = torch.randn(5, 333) * 40.0
    for scale, cap in ((0.25, 30.0), (2.0, 0.0), (1.0, 7.5)):
        got = z.clone().cuda()
        ops.scale_softcap(got, scale, cap)
        want = z.double() * scale
        want = cap * torch.tanh(want / cap) if cap else want
        assert torch.allclose(got.cpu().double(), want, rtol=2e-6, atol=1e-6)
