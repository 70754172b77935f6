"""Grouped-query attention whose heads talk to one another before the softmax.

Per layer: ``q = W_q x``, ``k = W_k x``; the values are either a projection of their own or the keys as
projected (before rotation and norm), in which case the layer has no value matrix.  The first ``rotary_dim``
dims of every query and key head turn in split pairs ``(i, i + rot/2)`` with the position; after the rotation
every head may be divided by its root mean square (an RMS norm without a weight).  The scaled scores of all
heads at a (query, key) pair are mixed, ``s'_h = sum_g talk[h, g] s_g``, before the causal softmax, whose
denominator may also hold ``exp(sink_h)``, a learned number per head that has no key and no value.
"""

from __future__ import annotations

import math

import torch

from .. import ops
from .attention import decode_scratch
from .base import CacheNeed, Mixer, PartSpec, WeightDecl, build_part, register_mixer
from .projection import project

# keys per range of the decode form: a CTA holds every head's rows, so ranges are short and many
TALKING_RANGE = 128


@register_mixer("talking_attention")
class TalkingAttention(Mixer):
    """params: ``hidden_size``, ``num_heads``, ``num_kv_heads``, ``head_dim``; optional ``v_head_dim`` (default
    ``head_dim``), ``scale`` (default ``1/sqrt(head_dim)``), ``position`` (a rotary ``PartSpec`` of split pairs,
    or ``None``), ``qk_norm`` (``{"eps": e}``: q and k heads are RMS-normed without a weight after the rotation),
    ``values`` (``"keys"``: the value of a token is the first ``v_head_dim`` numbers of its key as projected;
    ``"projection"``: a matrix ``v_proj.weight`` of its own), ``talk`` (the tensor ``talk [H, H]``, target head
    first, mixes the heads' scores) and ``sink`` (the tensor ``sink [H]`` joins the softmax's denominator).

    A block may hand it further rows for its input product (``stack_input``): their result for the step is
    ``self.extra_out`` after ``forward``."""

    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        self.hidden = int(params["hidden_size"])
        self.nh = int(params["num_heads"])
        self.nkv = int(params["num_kv_heads"])
        self.d = int(params["head_dim"])
        self.dv = int(params.get("v_head_dim") or self.d)
        if self.nkv <= 0 or self.nh % self.nkv:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        if self.nh > ops.TALKING_MAX_HEADS:
            raise ValueError(f"attention whose heads talk takes at most {ops.TALKING_MAX_HEADS} heads")
        if not 0 < self.dv <= ops.TALKING_MAX_HEAD_DIM or not 0 < self.d <= ops.TALKING_MAX_HEAD_DIM:
            raise ValueError(f"attention whose heads talk takes heads of 1 to {ops.TALKING_MAX_HEAD_DIM} numbers")
        self.values = params.get("values", "projection")
        if self.values not in ("keys", "projection"):
            raise ValueError("values must be 'keys' or 'projection'")
        if self.values == "keys" and self.dv > self.d:
            raise ValueError("values taken from the keys cannot be wider than a key")
        self.scale = float(params.get("scale") or 1.0 / math.sqrt(self.d))
        pos = params.get("position")
        if isinstance(pos, dict):
            pos = PartSpec(pos["kind"], pos.get("params", {}))
        self.position_spec: PartSpec | None = pos
        self.position = None
        qk = params.get("qk_norm")
        self.qk_eps = float(qk["eps"]) if qk else None
        self.talks = bool(params.get("talk", True))
        self.has_sink = bool(params.get("sink", True))
        self.q_dim, self.k_dim = self.nh * self.d, self.nkv * self.d
        self.v_dim = self.nkv * self.dv if self.values == "projection" else 0
        self.o_dim = self.nh * self.dv
        self.extra_w = None
        self.extra_out = None

    @classmethod
    def weight_decls(cls, params):
        h, nh, nkv, d = (int(params[k]) for k in ("hidden_size", "num_heads", "num_kv_heads", "head_dim"))
        dv = int(params.get("v_head_dim") or d)
        out = {"q_proj.weight": WeightDecl((nh * d, h)), "k_proj.weight": WeightDecl((nkv * d, h)), "o_proj.weight": WeightDecl((h, nh * dv))}
        if params.get("values", "projection") == "projection":
            out["v_proj.weight"] = WeightDecl((nkv * dv, h))
        if params.get("talk", True):
            out["talk"] = WeightDecl((nh, nh), kind="vector", init="eye")
        if params.get("sink", True):
            out["sink"] = WeightDecl((nh,), kind="vector", init="small")
        return out

    def cache_need(self) -> CacheNeed:
        return CacheNeed("full", self.nkv, self.d, None, None if self.dv == self.d else self.dv)

    def stack_input(self, w: torch.Tensor) -> bool:
        """Further rows ``w [M, hidden]`` for the product that reads this mixer's input."""
        self.extra_w = w
        self._stack()
        return True

    def _stack(self) -> None:
        mats = list(self._own)
        rows = sum(t.shape[0] for t in mats)
        self.extra_off = -(-rows // 8) * 8  # the further rows start at a multiple of 8 columns
        if self.extra_w is not None:
            if self.extra_off > rows:
                mats.append(torch.zeros((self.extra_off - rows, self.hidden), dtype=mats[0].dtype, device=mats[0].device))
            mats.append(self.extra_w)
        total = sum(t.shape[0] for t in mats)
        if total % 8:
            mats.append(torch.zeros((8 - total % 8, self.hidden), dtype=mats[0].dtype, device=mats[0].device))
        self.w_in = torch.cat(mats, dim=0).contiguous()
        self.in_dim = self.w_in.shape[0]

    def bind(self, weights, rt):
        super().bind(weights, rt)
        self._own = [weights["q_proj.weight"], weights["k_proj.weight"]] + ([weights["v_proj.weight"]] if self.values == "projection" else [])
        self._stack()
        self.w_o = weights["o_proj.weight"].contiguous()
        self.talk = weights["talk"].contiguous() if self.talks else None
        self.sink = weights["sink"].contiguous() if self.has_sink else None
        if self.position_spec is not None and self.position is None:
            self.position = build_part("position", self.position_spec)
            self.position.bind({}, rt)
        table = self.position.table() if self.position is not None else None
        if table is not None and getattr(self.position, "pairs_interleaved", False):
            raise ValueError("attention whose heads talk turns split pairs")
        self.inv_freq = table if table is not None else torch.empty(0, dtype=torch.float32, device=rt.device)

    def forward(self, ctx, x: torch.Tensor, cache):
        rt = self.rt
        n = x.shape[0]
        if cache is None or not cache.writable:
            raise RuntimeError("attention whose heads talk keeps a cache of its own")
        y = rt.buf("talk.in", n, self.in_dim)
        if ops.skinny_ok(x, self.w_in):
            ops.gemm_skinny(x, self.w_in, y)
        else:
            ops.linear(x, self.w_in, y)
        self.extra_out = y[:, self.extra_off : self.extra_off + self.extra_w.shape[0]] if self.extra_w is not None else None
        from_keys = self.values == "keys"
        ops.qk_prepare(
            y, ctx.positions, self.inv_freq, self.qk_eps, ctx.slot_mappings[cache.group], cache.k, cache.v, self.nh, self.nkv, self.d, self.dv,
            k_off=self.q_dim, v_off=self.q_dim if from_keys else self.q_dim + self.k_dim, v_step=self.d if from_keys else self.dv,
            block_size=ctx.block_size, err=rt.err,
        )  # fmt: skip
        out = rt.buf("talk.out", n, self.o_dim)
        scratch, bound, split = None, None, TALKING_RANGE
        if ctx.all_single_query:
            (acc, ml, _), bound, split = decode_scratch(rt, ctx, self.nh, self.nkv, self.d, self.dv, None, TALKING_RANGE)
            scratch = (acc, ml)
        ops.talking_attention(
            y, out, cache.k, cache.v, ctx.block_tables[cache.group], ctx.query_start_loc, ctx.context_lens, ctx.num_seqs, ctx.max_query_len,
            self.nh, self.nkv, self.d, self.dv, self.scale, self.talk, self.sink, q_stride=self.in_dim, scratch=scratch, max_context=bound,
            split_size=split,
        )  # fmt: skip
        return project(rt, "attn.proj", out, self.w_o, ctx)
