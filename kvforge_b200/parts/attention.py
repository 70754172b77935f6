"""Grouped-query attention over the paged cache (the mixer of the Llama decoder).

What it computes is umarhassan-cloud/kvforge's ``Attention.forward``
(src/tokenvault/model.py:77-92): bias-free q/k/v projections, rotation of q and k, the step's
k and v written to their slots *before* attention reads the cache, causal attention over
the block table (src/tokenvault/cache/paged_attention.py:66-91), output projection.
The three input projections are one product here (their weights are stacked at load).
"""

from __future__ import annotations

import math

import torch

from .. import ops
from .base import CacheNeed, Mixer, PartSpec, WeightDecl, build_part, register_mixer
from .projection import PART_ROWS, project


# Decode attention merges its key ranges through a thread-block cluster's shared memory only with
# this few (sequence, kv head) pairs: measured inside the decode step it gains 2 % at one sequence
# and loses at 8 and 64, where the ranges past the context (a captured graph's grid covers twice
# the context at most) hold their places until their cluster is done.
CLUSTER_MERGE_MAX_PAIRS = 16


def distance_buckets(rows: int, far: int) -> torch.Tensor:
    """Row of a distance-bias table of ``rows`` rows for every distance ``0 .. far`` (int32): the first
    half of the rows is one distance each, ``n -> n`` for ``n < rows // 2``; the second half divides the
    distances from ``rows // 2`` to ``far`` into steps of equal ratio,
    ``n -> half + floor(log(n / half) / log(far / half) * (rows - half))``, at most the last row, which also
    takes every distance beyond ``far``."""
    half = rows // 2
    if rows < 2 or far <= half:
        raise ValueError("a distance-bias table needs at least two rows and a farthest distance beyond half its rows")
    out = []
    for n in range(far + 1):
        out.append(n if n < half else min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half)))))
    return torch.tensor(out, dtype=torch.int32)


# keys per range of the decode form on the FP32 pipes when the scores take a bias, the window keeps first keys or the
# values lie inside wide keys: such a CTA is bound by its arithmetic, not by the bytes it pulls, so ranges are short
# and many (8 requests of 16 heads over a latent of 576 numbers: 231 us with ranges of 256 keys)
FP32_PIPE_RANGE = 64


def decode_scratch(rt, ctx, nh: int, nkv: int, d: int, dv: int, tickets: torch.Tensor | None, split: int | None = None):
    """What the decode form of attention (key ranges in parallel, then a merge) needs for this step:
    ((partial results, their maxima and sums, tickets), the longest context the grid reaches, keys per
    range).  Buffers are made for the longest context the engine takes; the grid follows the longest
    context of this step (of this graph, when the step is captured)."""
    bound = max(ctx.context_bound, ctx.max_context_len, rt.max_model_len, 1)
    reach = max(ctx.context_bound if ctx.context_bound > 0 else ctx.max_context_len, 1)
    # 32-bit: one range size whatever the batch, so a request's sums come in the same order beside
    # any number of others; bfloat16: longer ranges for many sequences (fewer CTAs, same bytes)
    if split is not None:  # one size whatever the batch (grown only where the longest context would make too many ranges)
        while -(-bound // split) > ops.MAX_ATTN_SPLITS:
            split *= 2
        smallest = split
    else:
        split = ops.attention_split_size(ctx.num_seqs if rt.dtype == torch.bfloat16 else 1, nkv, bound, reach, d)
        # made for the smallest range size, so that one buffer serves every batch size
        smallest = min(ops.attention_split_size(1, 1, bound), ops.attention_split_size(ops.ATTN_SHORT_RANGE_PAIRS[0], 1, bound))
    sa, sm = ops.attention_scratch_shapes(max(rt.max_seqs, ctx.num_seqs), nh, dv, bound, smallest)
    # a buffer per number of heads (and, by the buffers' key, per value size): layers of other shapes have their own
    acc = rt.buf(f"attn.part_acc.{nh}", sa[0] * sa[1] * sa[2], sa[3], torch.float32, cap=0).view(sa)
    ml = rt.buf(f"attn.part_ml.{nh}", sm[0] * sm[1] * sm[2], sm[3], torch.float32, cap=0).view(sm)
    return (acc, ml, tickets), reach, split


@register_mixer("paged_attention")
class PagedAttention(Mixer):
    """params: ``hidden_size``, ``num_heads``, ``num_kv_heads``, ``head_dim``; optional
    ``position`` (a position-encoding ``PartSpec`` or ``None``), ``window`` (keys a query
    sees, itself included; ``None`` = all), ``scale`` (default ``1/sqrt(head_dim)``),
    ``v_head_dim`` (size of a value head, default ``head_dim``) and ``conv`` (taps of a short causal
    convolution over time on every channel of q, k and v, between the projection and the rotation;
    its last ``conv - 1`` inputs are the mixer's state per request; tensors ``q_proj.conv`` ...),
    ``qk_norm`` (``{"eps": e}``: every query and key head is RMS-normed over its dims, with the tensors
    ``q_norm.weight`` / ``k_norm.weight`` of ``head_dim`` entries shared by the heads, before any rotation),
    ``distance_bias`` (``{"rows": B, "far": D}``: the tensor ``rel [B, num_heads]`` is added to the scaled
    scores by ``distance_buckets`` of the distance between query and key), ``keep_first`` (with a
    window: the first keys of a sequence that every later query sees, at their true positions),
    ``softcap`` (``c``: a scaled score ``s`` becomes ``c * tanh(s / c)``), ``sink`` (true: the tensor ``sink [num_heads]``;
    ``exp(sink_h)`` joins the softmax's denominator of head ``h`` without a key or a value) and ``value_mix``
    (``"source"``: the values as projected are also kept for the later layers of the step; ``"mix"``: the values become
    ``(1 - lambda) v + lambda v_source`` with the source layer's values of the same token, before they are cached;
    both declare the scalar tensor ``vmix``, which only ``"mix"`` uses; source and mixing layers have values of one shape).

    Rotation of split pairs with equal key and value sizes and no convolution takes the kernels
    of the Llama decoder; anything else (interleaved pairs, a value size of its own, a convolution,
    normed heads, a bias, kept first keys) goes through ``forward_general``: one product, the
    convolution, the rotary kernel (or the one that also norms the heads), and the attention kernel
    that takes the shape."""

    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        self.hidden = int(params["hidden_size"])
        self.nh = int(params["num_heads"])
        self.nkv = int(params["num_kv_heads"])
        self.d = int(params["head_dim"])
        if self.nkv <= 0 or self.nh % self.nkv:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        ops.check_head_dim(self.d)
        self.window = params.get("window")
        if self.window is not None and int(self.window) <= 0:
            raise ValueError("window must be positive")
        self.scale = float(params.get("scale") or 1.0 / math.sqrt(self.d))  # model.py:74
        pos = params.get("position")
        if isinstance(pos, dict):
            pos = PartSpec(pos["kind"], pos.get("params", {}))
        self.position_spec: PartSpec | None = pos
        self.position = None  # shared instance, set by the model before bind
        self.dv = int(params.get("v_head_dim") or self.d)
        ops.check_head_dim(self.dv)
        self.taps = int(params.get("conv") or 0)
        if self.taps < 0:
            raise ValueError("conv must be a number of taps")
        qk = params.get("qk_norm")
        self.qk_eps = float(qk["eps"]) if qk else None
        bias = params.get("distance_bias")
        self.bias_shape = (int(bias["rows"]), int(bias["far"])) if bias else None
        self.keep_first = int(params.get("keep_first") or 0)
        if self.keep_first < 0 or (self.keep_first and self.window is None):
            raise ValueError("keep_first is a count of keys and needs a window")
        self.softcap = float(params.get("softcap") or 0.0)
        if self.softcap < 0:
            raise ValueError("softcap must be positive")
        self.has_sink = bool(params.get("sink", False))
        self.value_mix = params.get("value_mix")
        if self.value_mix not in (None, "source", "mix"):
            raise ValueError("value_mix is 'source', 'mix' or None")
        self.q_dim = self.nh * self.d
        self.o_dim = self.nh * self.dv
        self.qkv_dim = (self.nh + self.nkv) * self.d + self.nkv * self.dv

    @classmethod
    def weight_decls(cls, params):
        h, nh, nkv, d = (int(params[k]) for k in ("hidden_size", "num_heads", "num_kv_heads", "head_dim"))
        dv = int(params.get("v_head_dim") or d)
        taps = int(params.get("conv") or 0)
        out = {
            "q_proj.weight": WeightDecl((nh * d, h)),
            "k_proj.weight": WeightDecl((nkv * d, h)),
            "v_proj.weight": WeightDecl((nkv * dv, h)),
            "o_proj.weight": WeightDecl((h, nh * dv)),
        }
        if taps:
            out["q_proj.conv"] = WeightDecl((nh * d, taps), kind="vector", init="conv")
            out["k_proj.conv"] = WeightDecl((nkv * d, taps), kind="vector", init="conv")
            out["v_proj.conv"] = WeightDecl((nkv * dv, taps), kind="vector", init="conv")
        if params.get("qk_norm"):
            out["q_norm.weight"] = WeightDecl((d,), kind="vector", init="ones")
            out["k_norm.weight"] = WeightDecl((d,), kind="vector", init="ones")
        if params.get("distance_bias"):
            out["rel"] = WeightDecl((int(params["distance_bias"]["rows"]), nh), kind="vector", init="small")
        if params.get("sink"):
            out["sink"] = WeightDecl((nh,), kind="vector", init="small")
        if params.get("value_mix"):
            out["vmix"] = WeightDecl((), kind="vector", init="unit")
        return out

    def cache_need(self) -> CacheNeed:
        v = None if self.dv == self.d else self.dv
        if self.window is None:
            return CacheNeed("full", self.nkv, self.d, None, v)
        return CacheNeed("window", self.nkv, self.d, int(self.window), v, keep_first=self.keep_first)

    def state_shape(self):
        return ((self.taps - 1) * self.qkv_dim,) if self.taps > 1 else None

    def bind(self, weights, rt):
        super().bind(weights, rt)
        self.w_qkv = torch.cat([weights["q_proj.weight"], weights["k_proj.weight"], weights["v_proj.weight"]], dim=0).contiguous()
        self.w_o = weights["o_proj.weight"].contiguous()
        # counters of finished key ranges per (sequence, kv head) for the decode form: zero between launches
        self._tickets = torch.zeros(max(1, rt.max_seqs) * self.nkv, dtype=torch.int32, device=rt.device)
        # the kernel of prompts and mixed batches takes its tiles of queries from a list made with the step
        self._query_tile = None
        self.w_conv = None
        if self.taps:
            self.w_conv = torch.cat([weights["q_proj.conv"], weights["k_proj.conv"], weights["v_proj.conv"]], dim=0).contiguous()
        self.q_norm_w = weights.get("q_norm.weight") if self.qk_eps is not None else None
        self.k_norm_w = weights.get("k_norm.weight") if self.qk_eps is not None else None
        self.bias = None
        if self.bias_shape is not None:
            self.bias = ops.DistanceBias(weights["rel"].contiguous(), distance_buckets(*self.bias_shape).to(rt.device))
        self.sinks = weights["sink"].contiguous() if self.has_sink else None
        self.v_lambda = weights["vmix"].reshape(1).contiguous() if self.value_mix == "mix" else None
        # kept first keys, a bias on the scores, capped scores and sinks are not the tcgen05 kernel's
        plain_scores = self.bias is None and not self.keep_first and not self.softcap and self.sinks is None
        if plain_scores and self.dv == self.d and ops.tcgen05_attention_supported(rt.dtype, self.nh, self.nkv, self.d, False):
            self._query_tile = ops.tcgen05_query_tile(self.nh, self.nkv)
            rt.query_tile_sizes.add(self._query_tile)
        if self.position_spec is not None and self.position is None:
            self.position = build_part("position", self.position_spec)
            self.position.bind({}, rt)
        table = self.position.table() if self.position is not None else None
        # no table: q and k are stored and used as the projections leave them
        self.inv_freq = table if table is not None else torch.empty(0, dtype=torch.float32, device=rt.device)
        self.interleaved = bool(getattr(self.position, "pairs_interleaved", False))
        self.general = bool(self.taps) or self.dv != self.d or self.interleaved or self.qk_eps is not None or not plain_scores or self.value_mix is not None

    def _scratch(self, ctx):
        rt = self.rt
        seqs = max(rt.max_seqs, ctx.num_seqs)
        if self._tickets.numel() < seqs * self.nkv:
            if rt.capturing or rt.graphs_captured:
                raise RuntimeError("the attention tickets would have to grow after or during graph capture")
            self._tickets = torch.zeros(seqs * self.nkv, dtype=torch.int32, device=rt.device)
        # a bias or kept first keys: the tensor-core kernel takes them with heads of 64 or 128 (and the ranges of any
        # other decode step); elsewhere the FP32 pipes, with short ranges
        special = self.bias is not None or self.keep_first > 0 or bool(self.softcap) or self.sinks is not None
        on_pipes = special and not (self.dv == self.d and ops.mma_attention_supported(rt.dtype, self.nh, self.nkv, self.d, True))
        return decode_scratch(rt, ctx, self.nh, self.nkv, self.d, self.dv, self._tickets, FP32_PIPE_RANGE if on_pipes else None)

    def forward(self, ctx, x: torch.Tensor, cache) -> torch.Tensor:
        rt = self.rt
        n = x.shape[0]
        if cache is None:
            raise RuntimeError("paged_attention needs a cache")
        if self.general:
            return self.forward_general(ctx, x, cache)
        skinny = ops.skinny_ok(x, self.w_qkv)
        if cache.writable:
            slots = ctx.slot_mappings[cache.group]
            splits = ops.skinny_splits(self.qkv_dim, self.hidden, n) if skinny else 1
            if splits > 1:
                # decode: slices of K in parallel; the rotation kernel sums them
                part = ops.Partials(rt.buf("attn.qkv_part", splits * n, self.qkv_dim, torch.float32, cap=PART_ROWS).view(splits, n, self.qkv_dim))
                ops.gemm_skinny(x, self.w_qkv, part)
                q = rt.buf("attn.q", n, self.q_dim)
                ops.rope_cache_write(part, ctx.positions, self.inv_freq, slots, cache.k, cache.v, self.nh, self.nkv, self.d, ctx.block_size, rt.err, q_out=q)
                q_stride = self.q_dim
            else:
                qkv = rt.buf("attn.qkv", n, self.qkv_dim)
                if skinny:
                    ops.gemm_skinny(x, self.w_qkv, qkv)
                else:
                    ops.linear(x, self.w_qkv, qkv)
                ops.rope_cache_write(qkv, ctx.positions, self.inv_freq, slots, cache.k, cache.v, self.nh, self.nkv, self.d, ctx.block_size, rt.err)
                q, q_stride = qkv, self.qkv_dim
        else:
            # reads another call's keys and values: only the queries are needed
            q = rt.buf("attn.q", n, self.q_dim)
            ops.linear(x, self.w_qkv[: self.q_dim], q)
            ops.rope_cache_write(q, ctx.positions, self.inv_freq, None, None, None, self.nh, 0, self.d, ctx.block_size)
            q_stride = self.q_dim
        out = rt.buf("attn.out", n, self.q_dim)
        self.attend(ctx, q, q_stride, out, cache)
        return project(rt, "attn.proj", out, self.w_o, ctx)

    def forward_general(self, ctx, x: torch.Tensor, cache):
        rt = self.rt
        n = x.shape[0]
        if not cache.writable:
            raise RuntimeError("a mixer in the general form keeps its own keys and values")
        qkv = rt.buf("attn.qkv", n, self.qkv_dim)
        if ops.skinny_ok(x, self.w_qkv):
            ops.gemm_skinny(x, self.w_qkv, qkv)
        else:
            ops.linear(x, self.w_qkv, qkv)
        if self.taps:
            mixed = rt.buf("attn.qkv_conv", n, self.qkv_dim)
            ops.causal_conv(qkv, self.w_conv, cache.state, ctx.query_start_loc, ctx.state_slots, ctx.num_seqs, mixed, max_query_len=ctx.max_query_len)
            qkv = mixed
        if self.qk_eps is not None or self.value_mix is not None:
            # the values of the step's source layer stay in a buffer of their own until the step is over
            carried = rt.buf("attn.v_source", n, self.nkv * self.dv) if self.value_mix else None
            ops.head_norm_cache(
                qkv, ctx.positions, self.q_norm_w, self.k_norm_w, self.qk_eps or 0.0, self.inv_freq, ctx.slot_mappings[cache.group], cache.k, cache.v,
                self.nh, self.nkv, self.d, self.dv, ctx.block_size, rt.err, interleaved=self.interleaved,
                v_keep=carried if self.value_mix == "source" else None, v_first=carried if self.value_mix == "mix" else None, v_lambda=self.v_lambda,
            )  # fmt: skip
        else:
            ops.rope_cache_general(
                qkv, ctx.positions, self.inv_freq, self.interleaved, ctx.slot_mappings[cache.group], cache.k, cache.v,
                self.nh, self.nkv, self.d, self.dv, ctx.block_size, rt.err,
            )  # fmt: skip
        out = rt.buf("attn.out", n, self.o_dim)
        self.attend(ctx, qkv, self.qkv_dim, out, cache)
        return project(rt, "attn.proj", out, self.w_o, ctx)

    def attend(self, ctx, q, q_stride, out, cache) -> None:
        scratch, bound, split = None, None, 256
        common = dict(
            window=int(self.window or 0), q_stride=q_stride, err=self.rt.err, dv=self.dv, keep_first=self.keep_first, bias=self.bias,
            softcap=self.softcap, sinks=self.sinks,
        )  # fmt: skip
        args = (q, out, cache.k, cache.v, ctx.block_tables[cache.group], ctx.query_start_loc, ctx.context_lens, ctx.num_seqs)
        shape = (self.nh, self.nkv, self.d, self.scale)
        # bfloat16: the decode kernel may lengthen its key ranges from the step's longest context (the merge
        # order then follows the batch, within rounding); 32-bit keeps one order whatever the batch
        wave = ops.attention_wave_target(ctx.num_seqs, self.nkv, self.d) if q.dtype == torch.bfloat16 else 0
        if ctx.all_single_query:
            scratch, bound, split = self._scratch(ctx)
        tiles = ctx.query_tiles.get(self._query_tile)
        if tiles is not None and tiles.num_single > 0 and self.dv == self.d and ops.tma_decode_supported(q.dtype, self.nh, self.nkv, self.d, ctx.block_size, cache.k.shape[0]):
            # a mixed batch: the sequences that bring one token go to the decode kernel (key ranges in
            # parallel), the portions of prompts to the kernel of prompts; each leaves the other's rows alone
            scratch, bound, split = self._scratch(ctx)
            side = self.rt.side_stream() if (self.rt.capturing and tiles.multi_count > 0) else None
            if side is not None:
                # the two kernels write other rows, and one is bound by the tensor cores, the other by memory: in
                # a captured step they are two branches that run side by side (32 decoding requests beside a
                # 1,024-token portion: 2.98 -> 2.86 ms at the 1B shape, 7.86 -> 7.58 ms at the 3B shape)
                main = torch.cuda.current_stream()
                side.wait_stream(main)
                with torch.cuda.stream(side):
                    ops.paged_attention(*args, ctx.max_query_len, *shape, query_tiles=(tiles.multi, tiles.multi_count), **common)
            ops.paged_attention(*args, 1, *shape, scratch=scratch, max_context=bound, split_size=split, kernel="tma", cluster=False, single_only=True, wave_target=wave, **common)
            if side is not None:
                torch.cuda.current_stream().wait_stream(side)
            elif tiles.multi_count > 0:
                ops.paged_attention(*args, ctx.max_query_len, *shape, query_tiles=(tiles.multi, tiles.multi_count), **common)
            return
        ops.paged_attention(
            *args, ctx.max_query_len, *shape, scratch=scratch, max_context=bound, split_size=split,
            cluster=ctx.num_seqs * self.nkv <= CLUSTER_MERGE_MAX_PAIRS, wave_target=wave if scratch is not None else 0,
            query_tiles=(tiles.tiles, tiles.count) if tiles is not None else None, **common,
        )  # fmt: skip
