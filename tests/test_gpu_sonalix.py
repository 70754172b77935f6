"""The Sonalix decoder on the GPU against the plain implementation (``plain_sonalix``): each new
mechanism alone, then whole models with random weights made here, replayed whole, token by token, in
portions down to two tokens and mixed with other requests on few pages and slots; in 32-bit and in
bfloat16, eager and as captured graphs; and greedy generation through the engine's entry point."""

from __future__ import annotations

import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import plain_sonalix as plain
import traces
from sonalix_cases import CASES, attention, latent, plain_logits, random_config, random_tensors, retention, row_error, write_folder
from test_gpu_mopilorn import check, run_trace, tokens
from test_gpu_parts import context, runtime

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent
TOL = {"float32": 1e-4, "bfloat16": 0.25}
SHARP_TOL = 1e-3
LENGTHS = {"a": [70, 3, 41, 1, 26, 97], "b": [9, 120, 33, 2, 64, 50], "c": [45, 17, 5, 80, 30], "d": [130, 20, 75, 49, 9]}


def build(tmp, name, config, w, lengths, seed=40):
    folder = write_folder(tmp / name, config, w)
    reqs = {f"{name}{i}": tokens(config["vocab"], n, seed + i) for i, n in enumerate(lengths)}
    ref = {rid: plain_logits(config, w, t) for rid, t in reqs.items()}
    scale = float(torch.cat(list(ref.values())).pow(2).mean().sqrt())
    return folder, reqs, ref, scale, w


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    """Per case and storage type: folder, requests, plain logits of every request whole, the logits' scale.
    32-bit runs on weights whose router follows the token; bfloat16 on weights whose router biases decide the
    choice of experts, so that rounding cannot move a token to other experts than the plain model's."""
    tmp = tmp_path_factory.mktemp("sonalix")
    out = {}
    for k, (name, case) in enumerate(sorted(CASES.items())):
        out[name, "float32"] = build(tmp, name, case["config"], random_tensors(case["config"], 17 + k), LENGTHS[name])
        out[name, "bfloat16"] = build(tmp, name + "-fixed", case["config"], random_tensors(case["config"], 27 + k, fixed_choice=True), LENGTHS[name])
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
    """Whole prompts; the last 40 tokens one by one (every window passes over decoded tokens); portions of
    1 to 33 tokens; up to four live requests on as few pages as they need (pages and state slots are used again)."""
    folder, reqs, ref, scale, _ = models[name, dtype]
    steps = regime_steps(reqs, regime)
    outs, runner = run_trace(folder, dtype, steps, CASES[name]["block_size"])
    check(steps, outs, ref, scale, TOL[dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CASES))
@pytest.mark.parametrize("regime", ["tail", "mixed"])
def test_replay_as_captured_graphs(models, name, dtype, regime):
    """The way generation runs by default: single-token steps and steps of more than 16 tokens as CUDA
    graphs made for padded shapes.  Padding sequences and rows must leave every cache and every state alone."""
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
    steps = regime_steps(reqs, "mixed")
    outs, _ = run_trace(folder, "float32", steps, 16)
    worst = 0.0
    for rows, got in zip(traces.wanted_places(steps), outs):
        for i, place in enumerate(rows):
            worst = max(worst, float((got[i] - by_place[place]).abs().max()))
    assert worst <= 2e-5 * scale, worst


@pytest.mark.parametrize("seed", [3, 12, 29, 41, 57, 68, 75, 90])
def test_configurations_drawn_at_random(tmp_path, seed):
    """Sizes that no hand-made case has (widths and inner sizes that are no multiple of 8 or of 16, one head, twelve
    heads, heads of which only some dims turn, one expert a token, ...), each replayed whole, in portions and
    mixed, in both storage types."""
    config = random_config(seed)
    block_size = [4, 8, 16, 32][seed % 4]
    for dtype, fixed in (("float32", False), ("bfloat16", True)):
        folder, reqs, ref, scale, _ = build(tmp_path, f"drawn-{dtype}", config, random_tensors(config, 100 + seed, fixed_choice=fixed), [90, 1, 37, 140], seed=seed)
        for regime in ("whole", "portions", "mixed"):
            steps = regime_steps(reqs, regime) if regime != "mixed" else traces.mixed(reqs, {r: max(1, len(t) - 10) for r, t in reqs.items()}, max_live=4, seed=seed)
            outs, _ = run_trace(folder, dtype, steps, block_size)
            check(steps, outs, ref, scale, TOL[dtype])


def sharpened(w):
    """Queries and keys scaled up until a few keys take nearly all the weight."""
    w = dict(w)
    for k in list(w):
        if k.endswith(("mix.q.norm", "mix.k.norm")):
            w[k] = (w[k] * 2.5).to(torch.bfloat16).float()
        if k.endswith(("mix.uk",)):
            w[k] = (w[k] * 5.0).to(torch.bfloat16).float()
    return w


def test_sharp_attention_far_keys_window_edges_sinks_and_caps(tmp_path):
    """With sharp scores over sequences of several hundred tokens, a far key among hundreds (case c: no mask), the key at
    a window's edge, the sink, the cap and the mixed values decide the logits: the plain model with a window one off,
    without its sinks, without its cap or without the mixing of values is far outside the tolerance."""
    for name in ("c", "a", "b"):
        case = CASES[name]
        w = sharpened(random_tensors(case["config"], seed=91))
        folder, reqs, ref, scale, _ = build(tmp_path, f"sharp-{name}", case["config"], w, [310, 150], seed=70)
        rid = f"sharp-{name}1"

        def worst_miss(cfg2, w2):
            off = plain_logits(cfg2, w2, reqs[rid])
            return max(row_error(off[i], ref[rid][i], scale) for i in range(60, 150))

        attn = [i for i, ly in enumerate(case["config"]["layers"]) if ly["type"] == "attention"]
        if any("mask" in case["config"]["layers"][i]["mixer"] for i in attn):
            for d in (-1, 1):
                cfg2 = json.loads(json.dumps(case["config"]))
                for i in attn:
                    if "mask" in cfg2["layers"][i]["mixer"]:
                        cfg2["layers"][i]["mixer"]["mask"]["size"] += d
                assert worst_miss(cfg2, w) > 10 * SHARP_TOL, (name, "window", d)
        assert worst_miss(case["config"], {k: v for k, v in w.items() if not k.endswith("mix.sink")}) > 10 * SHARP_TOL, (name, "sink")
        if any("softcap" in case["config"]["layers"][i]["mixer"] for i in attn):
            cfg2 = json.loads(json.dumps(case["config"]))
            for i in attn:
                cfg2["layers"][i]["mixer"].pop("softcap", None)
            assert worst_miss(cfg2, w) > 10 * SHARP_TOL, (name, "softcap")
        if sum(bool(case["config"]["layers"][i]["mixer"].get("v_mix")) for i in attn) > 1:
            cfg2 = json.loads(json.dumps(case["config"]))
            for i in attn:
                cfg2["layers"][i]["mixer"]["v_mix"] = False
            assert worst_miss(cfg2, w) > 10 * SHARP_TOL, (name, "v_mix")
        for regime in ("whole", "tail", "portions"):
            steps = regime_steps(reqs, regime)
            outs, _ = run_trace(folder, "float32", steps, case["block_size"])
            check(steps, outs, ref, scale, SHARP_TOL, SHARP_TOL)


def test_long_decoding(models):
    """Three hundred tokens one by one after a prompt of five: windows pass over decoded tokens many times, pages of the
    windows are given back and taken again, and the retention state is carried through three hundred steps."""
    for name in ("a", "b"):
        case = CASES[name]
        for dtype, graphs in (("float32", False), ("bfloat16", True)):
            w = models[name, dtype][4]
            folder = models[name, dtype][0]
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


@pytest.mark.parametrize("kind", ["retention", "attention", "latent_attention"])
def test_models_of_one_kind_of_mixer(tmp_path, kind):
    """A model may have layers of one kind only: retention alone keeps no pages at all (state slots only), attention
    alone no state."""
    from sonalix_cases import dense, layer, model, moe

    mixer = {"retention": retention(2, 24, 16, [0.9, 0.97], rot=12), "attention": attention(4, 2, 16, 8, window=9, softcap=12.0),
             "latent_attention": latent(2, 16, 8, 16, 24, 32)}[kind]  # fmt: skip
    config = model(77, 56, [layer(kind, mixer, dense(40)), layer(kind, mixer, moe(5, 2, 24))], mult=0.9)
    for dtype, fixed in (("float32", False), ("bfloat16", True)):
        folder, reqs, ref, scale, w = build(tmp_path, f"{kind}-{dtype}", config, random_tensors(config, 7, fixed_choice=fixed), [60, 2, 31, 85], seed=3)
        for regime in ("whole", "portions", "mixed"):
            steps = regime_steps(reqs, regime)
            outs, _ = run_trace(folder, dtype, steps, 8)
            check(steps, outs, ref, scale, TOL[dtype])
    if kind == "retention":
        from kvforge_b200 import EngineConfig, InferenceEngine, SamplingParams, SchedulerConfig

        engine = InferenceEngine(EngineConfig(scheduler=SchedulerConfig(max_num_seqs=2, max_num_batched_tokens=16, max_model_len=64), dtype="float32"), model=folder)
        prompts = [tokens(77, n, 9 + n) for n in (5, 20, 1)]
        outs = engine.generate(prompts, SamplingParams(max_tokens=6, temperature=0.0, ignore_eos=True))
        wd = {k: v.double() for k, v in w.items()}
        # the folder of the last storage type holds the weights whose router biases decide the choice
        for p, o in zip(prompts, outs):
            assert o.output_token_ids == plain.greedy(config, wd, p, 6)


# ------------------------------------------------------------------ generation through the entry point


@pytest.mark.parametrize("name", ["a", "b", "d"])
def test_greedy_generation_through_the_engine(models, name):
    """``InferenceEngine.generate`` with its scheduler: more requests than state slots, prompts cut into portions,
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

    cfg = EngineConfig(model=PRESETS["sonalix-tiny"], scheduler=SchedulerConfig(max_num_seqs=4, max_num_batched_tokens=64, max_model_len=96), dtype="bfloat16")
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


def bind(part, w, dtype, rt):
    kinds = type(part).weight_decls(part.params)
    names = part.params.get("names") or {}
    bound = {}
    for local, decl in kinds.items():
        t = w[names.get(local, local)]
        bound[local] = t.cuda() if decl.kind == "vector" else t.to(dtype).cuda()
    part.bind(bound, rt)


def step_mixer(part, rt, x, bs, table, cuts, cache, slot=0):
    """Run a mixer over a sequence cut into steps on pages of a shuffled table and in a given state slot."""
    t = x.shape[0]
    slots = [table[p // bs] * bs + p % bs for p in range(t)]
    got = []
    for a, b in cuts:
        ctx = context(rt, [b - a], [a], bs, [table], slots[a:b])
        ctx.state_slots = torch.tensor([slot], dtype=torch.int32, device="cuda")
        got.append(as_float(part.forward(ctx, x[a:b].cuda(), cache), b - a).cpu().clone())
    return torch.cat(got)


CUTS = lambda t: ([(0, t)], [(0, 17), (17, 19), (19, 20), (20, 21), (21, 34), (34, 35), (35, 36), (36, t - 3), (t - 3, t - 2), (t - 2, t)])  # noqa: E731


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_without_statistics(dtype):
    """``tanh(alpha x) w + b`` on the stream plus what is pending, times a constant: a tensor, slices of a split product,
    nothing; rows gathered before the head; widths that do and do not take four numbers a thread."""
    from kvforge_b200 import ops
    from kvforge_b200.parts.base import PartSpec, build_part

    rt = runtime(dtype)
    g = torch.Generator().manual_seed(2)
    for width in (64, 100, 37):
        part = build_part("norm", PartSpec("tanh_norm", {"dim": width, "names": {"weight": "n", "alpha": "n.alpha", "bias": "n.b"}}), "x.")
        w = {"x.n": torch.randn(width, generator=g), "x.n.alpha": torch.tensor(0.37), "x.n.b": torch.randn(width, generator=g)}
        assert sorted(part.tensor_name(k) for k in type(part).weight_decls(part.params)) == sorted(w)
        part.bind({"weight": w["x.n"].cuda(), "alpha": w["x.n.alpha"].cuda(), "bias": w["x.n.b"].cuda()}, rt)
        resid = torch.randn(9, width, generator=g)
        delta = torch.randn(9, width, generator=g).to(dtype)
        slices = torch.randn(3, 9, width, generator=g)
        for pending, add in (
            (None, 0.0),
            (delta.cuda(), delta.double()),
            (ops.Scaled(delta.cuda(), 0.7), 0.7 * delta.double()),
            (ops.Scaled(ops.Partials(slices.cuda()), 1.3), 1.3 * slices.double().sum(0)),
            (ops.Scaled(None, 0.5), 0.0),
        ):
            r = resid.cuda().clone()
            out = part.forward(None, r, pending)
            want_sum = resid.double() + add
            assert torch.allclose(r.cpu().double(), want_sum, atol=1e-5)
            want = plain.tanh_norm(want_sum, {k: v.double() for k, v in w.items()}, "x.n")
            assert torch.allclose(out.float().cpu().double(), want, atol=part_tol(dtype), rtol=part_tol(dtype))
        rows = torch.tensor([7, 2, 2], dtype=torch.int32, device="cuda")
        r = resid.cuda().clone()
        out = part.forward(None, r, ops.Scaled(delta.cuda(), 0.7), rows=rows, num_rows=3)
        want = plain.tanh_norm((resid.double() + 0.7 * delta.double())[[7, 2, 2]], {k: v.double() for k, v in w.items()}, "x.n")
        assert torch.allclose(out.float().cpu().double(), want, atol=part_tol(dtype), rtol=part_tol(dtype))
        assert torch.equal(r.cpu(), resid)


def attention_part(width, m, eps, role):
    from kvforge_b200.parts.base import PartSpec, build_part

    rot = m.get("rot")
    pos = PartSpec("rotary", {"head_dim": m["dim"], "rotary_dim": rot["dims"], "theta": rot["base"], "interleaved": False}) if rot else None
    names = {"q_proj.weight": "q", "k_proj.weight": "k", "v_proj.weight": "v", "o_proj.weight": "o", "q_norm.weight": "q.norm", "k_norm.weight": "k.norm"}
    return build_part("mixer", PartSpec("paged_attention", {
        "hidden_size": width, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"], "v_head_dim": m["vdim"], "scale": m["scale"],
        "window": (m.get("mask") or {}).get("size"), "position": pos, "qk_norm": {"eps": eps}, "softcap": m.get("softcap"), "sink": True,
        "value_mix": role, "names": names}), "m.")  # fmt: skip


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window,cap", [(None, None), (7, 4.0), (33, 50.0), (1, 9.0), (70, None)])
@pytest.mark.parametrize("dk,dv,rot,t", [(24, 16, 8, 45), (64, 64, 64, 200), (128, 48, 2, 150), (128, 128, 64, 150)])
def test_attention_with_caps_sinks_and_mixed_values(dtype, window, cap, dk, dv, rot, t):
    """Two layers in one step: the first keeps its values for the second, which mixes them into its own before it caches
    them.  The whole sequence in one step, then portions and single tokens on top of the cache (the decode form: key
    ranges in parallel, the sink counted once), against the plain mixer.  Heads of 64 and of 128 with values as wide go
    to the tensor-core kernels in bfloat16 (tiles of 64 keys for prompts and portions, key ranges for single tokens)."""
    from kvforge_b200.parts.base import LayerCache

    rt = runtime(dtype)
    width, nh, nkv, bs, eps = 80, 6, 3, 4, 1e-5
    m = attention(nh, nkv, dk, dv, window=window, softcap=cap, rot=rot, base=500.0)
    g = torch.Generator().manual_seed(3)
    shapes = {"q": (nh * dk, width), "k": (nkv * dk, width), "v": (nkv * dv, width), "o": (width, nh * dv), "q.norm": (dk,), "k.norm": (dk,), "sink": (nh,), "vmix": ()}
    parts, ws = [], []
    for role in ("source", "mix"):
        w = {k: (torch.randn(s, generator=g) * 0.2 + (1.5 if "norm" in k else 0.0)).to(dtype).float() for k, s in shapes.items()}
        w["sink"] = (torch.randn(nh, generator=g) + 1.0).to(dtype).float()
        w["vmix"] = torch.tensor(0.35).to(dtype).float()
        part = attention_part(width, m, eps, role)
        bind(part, w, dtype, rt)
        parts.append(part)
        ws.append(w)
    x = [torch.randn(t, width, generator=g).to(dtype) for _ in range(2)]
    carried: dict = {}
    ref = [plain.windowed_attention(x[i].double(), {"m." + k: v.double() for k, v in ws[i].items()}, "m.", m, eps, carried) for i in range(2)]
    nb = 64
    table = [int(i) for i in torch.randperm(nb, generator=g)]
    need = parts[0].cache_need()
    assert need.kind == ("window" if window else "full") and need.value_dim == dv
    for cuts in CUTS(t):
        caches = [LayerCache(torch.zeros(nb, nkv, bs, dk, device="cuda", dtype=dtype), torch.zeros(nb, nkv, bs, dv, device="cuda", dtype=dtype), 0) for _ in range(2)]
        slots = [table[p // bs] * bs + p % bs for p in range(t)]
        got = [[], []]
        for a, b in cuts:
            ctx = context(rt, [b - a], [a], bs, [table], slots[a:b])
            for i in range(2):  # both layers inside one step, as a model runs them
                got[i].append(as_float(parts[i].forward(ctx, x[i][a:b].cuda(), caches[i]), b - a).cpu().clone())
        for i in range(2):
            assert rel_rows(torch.cat(got[i]), ref[i]) < part_tol(dtype), (cuts, i)


def test_one_far_key_and_the_sink_share_the_weight():
    """A query that matches one key far back and nothing else: the key's capped score and the sink stand beside each other
    in the denominator.  At the sequence's first places, around borders of pages, of key tiles and of the decode form's key
    ranges, in a prompt and decoded."""
    from kvforge_b200.parts.base import LayerCache

    dtype = torch.float32
    rt = runtime(dtype, max_tokens=512)
    width, nh, nkv, dk, dv, bs, eps, cap = 32, 2, 1, 16, 8, 16, 1e-6, 6.0
    m = attention(nh, nkv, dk, dv, window=None, softcap=cap, rot=0, scale=1.0)
    part = attention_part(width, m, eps, None)
    t = 300
    for far in (0, 1, 15, 16, 31, 32, 63, 64, 127, 128, 255, 256):
        g = torch.Generator().manual_seed(far)
        w = {"q": torch.zeros(nh * dk, width), "k": torch.zeros(nkv * dk, width), "v": torch.randn(nkv * dv, width, generator=g), "o": torch.randn(width, nh * dv, generator=g),
             "q.norm": torch.ones(dk), "k.norm": torch.ones(dk), "sink": torch.tensor([5.0, 6.5])}  # fmt: skip
        # queries and keys read the first dims of the input: token `far` carries a key, the last token the matching query
        for h in range(nh):
            w["q"][h * dk, 0] = 1.0
        w["k"][0, 1] = 1.0
        x = 0.01 * torch.randn(t, width, generator=g)
        x[:, 0] = 0.0
        x[:, 1] = -3.0
        x[far, 1] = 3.0
        x[t - 1, 0] = 4.0
        bind(part, w, dtype, rt)
        ref = plain.windowed_attention(x.double(), {"m." + k: v.double() for k, v in w.items()}, "m.", m, eps, {})
        table = [int(i) for i in torch.randperm(32, generator=g)]
        for cuts in ([(0, t)], [(0, t - 1), (t - 1, t)]):
            cache = LayerCache(torch.zeros(32, nkv, bs, dk, device="cuda"), torch.zeros(32, nkv, bs, dv, device="cuda"), 0)
            got = step_mixer(part, rt, x, bs, table, cuts, cache)
            assert rel_rows(got[-1:], ref[-1:]) < 1e-4, (far, cuts)
        w2 = dict(w, sink=torch.tensor([-30.0, -30.0]))
        off = plain.windowed_attention(x.double(), {"m." + k: v.double() for k, v in w2.items()}, "m.", m, eps, {})
        assert rel_rows(off[-1:], ref[-1:]) > 0.05  # without the sinks the row is another


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,dk,dv,rot,t", [(2, 16, 24, 16, 45), (3, 8, 8, 4, 60), (1, 32, 12, 0, 50), (2, 128, 64, 128, 150), (4, 64, 128, 32, 90), (2, 20, 100, 6, 40), (1, 256, 40, 256, 70), (2, 9, 5, 4, 40), (1, 512, 8, 0, 40)])
def test_retention_through_the_state(dtype, heads, dk, dv, rot, t):
    """Whole, in portions and token by token; in a slot that another request has used; beside another request."""
    from kvforge_b200.parts.base import LayerCache, PartSpec, build_part

    rt = runtime(dtype)
    width, eps = 72, 1e-6
    decay = [[0.9, 0.99, 0.9375, 1.0][h % 4] for h in range(heads)]
    m = retention(heads, dk, dv, decay, rot=rot, base=1000.0)
    pos = PartSpec("rotary", {"head_dim": dk, "rotary_dim": rot, "theta": 1000.0, "interleaved": False}) if rot else None
    part = build_part("mixer", PartSpec("retention", {"hidden_size": width, "num_heads": heads, "head_dim": dk, "v_head_dim": dv, "decay": decay, "eps": eps, "position": pos}), "m.")
    g = torch.Generator().manual_seed(7)
    shapes = {"q": (heads * dk, width), "k": (heads * dk, width), "v": (heads * dv, width), "g": (heads * dv, width), "o": (width, heads * dv)}
    w = {k: (torch.randn(s, generator=g) * (1.5 / s[-1] ** 0.5)).to(dtype).float() for k, s in shapes.items()}
    bind(part, w, dtype, rt)
    assert part.cache_need().kind == "none" and part.state_shape() == (heads * dk * dv,)
    x = torch.randn(t, width, generator=g).to(dtype)
    ref = plain.retention(x.double(), {"m." + k: v.double() for k, v in w.items()}, "m.", m, eps, {})
    state = torch.zeros(4, heads * dk * dv, device="cuda")
    cache = LayerCache(None, None, -1, True, state)
    for k, cuts in enumerate(([(0, t)], [(0, 17), (17, 19), (19, 20), (20, 21), (21, 34), (34, 35), (35, 36), (36, t - 3), (t - 3, t - 2), (t - 2, t)])):
        state[2] = 0  # the slot was used by the run before: a new request starts from zero
        got = step_mixer(part, rt, x, 1024, [0], cuts, cache, slot=2)
        assert rel_rows(got, ref) < part_tol(dtype), cuts
    # two requests in one step, the second half of one beside the whole of another
    x2 = torch.randn(23, width, generator=g).to(dtype)
    ref2 = plain.retention(x2.double(), {"m." + k: v.double() for k, v in w.items()}, "m.", m, eps, {})
    state.zero_()
    half = t // 2
    ctx = context(rt, [half], [0], 4, [[0]], [0] * half)
    ctx.state_slots = torch.tensor([3], dtype=torch.int32, device="cuda")
    part.forward(ctx, x[:half].cuda(), cache)
    ctx = context(rt, [23, t - half], [0, half], 4, [[0], [0]], [0] * (23 + t - half))
    ctx.state_slots = torch.tensor([1, 3], dtype=torch.int32, device="cuda")
    got = as_float(part.forward(ctx, torch.cat([x2, x[half:]]).cuda(), cache), 23 + t - half).cpu()
    assert rel_rows(got[:23], ref2) < part_tol(dtype)
    assert rel_rows(got[23:], ref[half:]) < part_tol(dtype)
    assert float(state[0].abs().max()) == 0.0 and float(state[2].abs().max()) == 0.0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,dk,dr,dv,rank,qr,rot", [(3, 16, 8, 24, 24, 40, 8), (5, 8, 16, 8, 40, 8, 6), (2, 32, 32, 16, 264, 100, 32), (16, 16, 32, 8, 64, 24, 32), (5, 8, 16, 8, 96, 56, 16), (2, 32, 64, 16, 512, 128, 64)])
def test_latent_attention_with_a_latent_of_the_queries(dtype, heads, dk, dr, dv, rank, qr, rot):
    """The queries come through a normed latent of their own, the pairs that turn are split, every earlier key is seen, and
    the gate has a number for every channel; whole, in portions and token by token."""
    from kvforge_b200.parts.base import LayerCache, PartSpec, build_part

    rt = runtime(dtype)
    width, bs, eps = 64, 8, 1e-6
    m = latent(heads, dk, dr, dv, rank, qr, base=300.0, rot=rot)
    pos = PartSpec("rotary", {"head_dim": dr, "rotary_dim": rot, "theta": 300.0, "interleaved": False})
    part = build_part("mixer", PartSpec("latent_attention", {
        "hidden_size": width, "num_heads": heads, "head_dim": dk, "rot_dim": dr, "v_head_dim": dv, "kv_rank": rank, "q_rank": qr, "eps": eps,
        "scale": m["scale"], "window": None, "position": pos, "gate": "sigmoid_channel"}), "m.")  # fmt: skip
    g = torch.Generator().manual_seed(5)
    shapes = {"dq": (qr, width), "dq.norm": (qr,), "uq": (heads * (dk + dr), qr), "dkv": (rank + dr, width), "dkv.norm": (rank,), "uk": (heads * dk, rank),
              "uv": (heads * dv, rank), "g": (heads * dv, width), "o": (width, heads * dv)}  # fmt: skip
    w = {k: (torch.randn(s, generator=g) * (2.0 / s[-1] ** 0.5) + (1.0 if "norm" in k else 0.0)).to(dtype).float() for k, s in shapes.items()}
    bind(part, w, dtype, rt)
    t = 50 if rank < 64 else 150
    x = torch.randn(t, width, generator=g).to(dtype)
    ref = plain.latent_attention(x.double(), {"m." + k: v.double() for k, v in w.items()}, "m.", m, eps, {})
    table = [int(i) for i in torch.randperm(24, generator=g)]
    k = torch.zeros(24, 1, bs, rank + dr, device="cuda", dtype=dtype)
    cache = LayerCache(k, k, 0)
    for cuts in ([(0, t)], [(0, 21), (21, 23), (23, 24), (24, 25), (25, 41), (41, 42), (42, t - 2), (t - 2, t - 1), (t - 1, t)]):
        got = step_mixer(part, rt, x, bs, table, cuts, cache)
        assert rel_rows(got, ref) < part_tol(dtype), cuts


@pytest.mark.parametrize("experts,top", [(6, 2), (8, 3), (4, 1), (12, 4), (40, 6), (5, 5)])
def test_router_with_a_bias_alone(experts, top):
    """Chosen experts and weights against the plain router, on tokens whose choice does not hang on the last bits."""
    from kvforge_b200 import ops

    g = torch.Generator().manual_seed(experts)
    width, n = 72, 200
    x = torch.randn(n, width, generator=g)
    w = {"m.router": torch.randn(experts, width, generator=g) * 0.3, "m.router.b": torch.randn(experts, generator=g)}
    chosen, weights = plain.route(x.double(), {k: v.double() for k, v in w.items()}, "m.", {"experts": experts, "top": top})
    ids = torch.zeros(n, top, dtype=torch.int32, device="cuda")
    wts = torch.zeros(n, top, dtype=torch.float32, device="cuda")
    ops.moe_route(x.cuda(), w["m.router"].cuda(), None, top, 1, 1, 0.0, ids, wts, bias=w["m.router.b"].cuda(), chosen_softmax=True)
    same = 0
    for i in range(n):
        if ids[i].tolist() == chosen[i].tolist():
            same += 1
            assert torch.allclose(wts[i].cpu().double(), weights[i], atol=1e-6)
            assert abs(float(wts[i].sum()) - 1.0) < 1e-6
    assert same >= n - 2  # a near tie may fall the other way in 32-bit


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("ff,limit", [(40, 2.5), (20, 0.7)])
@pytest.mark.parametrize("n", [1, 7, 30, 150, 400])
def test_gated_experts(dtype, n, ff, limit):
    """The feed-forward part against the plain one, for one token, a few and many (several tiles an expert; from 64 rows an
    expert on average the products run on the tcgen05 tensor cores); an inner size that is no multiple of 8; inputs large
    enough that the limit cuts gates and ups."""
    from kvforge_b200 import ops
    from kvforge_b200.parts.base import PartSpec, build_part

    rt = runtime(dtype, max_tokens=512)
    width, experts, top = 48, 6, 2
    part = build_part("ffn", PartSpec("routed_experts", {
        "hidden_size": width, "experts": experts, "top": top, "intermediate_size": ff, "correction": False, "score": "chosen_softmax",
        "router_bias": True, "activation": "gated", "gated": {"limit": limit, "alpha": 1.702, "shift": 1.0}}), "m.")  # fmt: skip
    g = torch.Generator().manual_seed(11)
    w = {"router": torch.randn(experts, width, generator=g) * 0.05, "router.b": 0.9 * torch.randperm(experts, generator=g).float()}
    for e in range(experts):
        w[f"e{e}.gate"] = (torch.randn(ff, width, generator=g) * 0.3).to(dtype).float()
        w[f"e{e}.up"] = (torch.randn(ff, width, generator=g) * 0.3).to(dtype).float()
        w[f"e{e}.down"] = (torch.randn(width, ff, generator=g) * 0.2).to(dtype).float()
    bind(part, w, dtype, rt)
    x = torch.randn(n, width, generator=g).to(dtype)
    mlp = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff, "limit": limit}}
    wd = {"m." + k: v.double() for k, v in w.items()}
    ref = plain.mixture_of_experts(x.double(), wd, "m.", mlp)
    unlimited = plain.mixture_of_experts(x.double(), wd, "m.", dict(mlp, expert={"ff": ff, "limit": 1e9}))
    assert rel_rows(unlimited, ref) > 0.05  # the limit matters on these inputs
    ctx = context(rt, [n], [0], 4, [[0]], [0] * n)
    got = as_float(part.forward(ctx, x.cuda()), n).cpu()
    assert rel_rows(got, ref) < part_tol(dtype)
    resid = torch.ones(n, width, device="cuda")
    ctx.residual = resid
    assert part.forward(ctx, x.cuda()) is ops.ADDED
    assert rel_rows(resid.cpu() - 1.0, ref) < part_tol(dtype) + 1e-6
