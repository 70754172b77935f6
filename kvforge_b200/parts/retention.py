"""Retention: linear attention with one fixed decay a head, no softmax and no denominator.

Per layer ``q = W_q x``, ``k = W_k x`` (``H`` heads of ``head_dim``), ``v = W_v x`` (``H`` heads of ``v_head_dim``),
``g = W_g x``.  The first ``rotary_dim`` dims of every query and key head turn with the position; the keys are then
multiplied by ``head_dim^(-1/2)``.  Per head a matrix state ``S [head_dim, v_head_dim]`` is carried from token to
token, ``S_t = a_h S_(t-1) + k_t v_t^T``, and read out as ``o_t = S_t^T q_t``.  Every head's ``o`` is divided by its
root mean square, the heads are multiplied by ``silu(g)`` and projected back.  The state is the mixer's state slot
per request: 32-bit floats, zero for a new request; the mixer keeps no pages.
"""

from __future__ import annotations

import torch

from .. import ops
from .base import CacheNeed, Mixer, PartSpec, WeightDecl, build_part, register_mixer
from .projection import project


@register_mixer("retention")
class Retention(Mixer):
    """params: ``hidden_size``, ``num_heads``, ``head_dim``, ``v_head_dim``, ``decay`` (a list of ``num_heads`` numbers),
    ``eps`` (of the heads' norm); optional ``position`` (a rotary ``PartSpec`` or ``None``), ``key_scale`` (default
    ``head_dim^(-1/2)``) and ``gate`` (``"silu"``, ``"sigmoid"`` or ``None``; default ``"silu"``).

    Tensors: ``q [H*head_dim, W]``, ``k [H*head_dim, W]``, ``v [H*v_head_dim, W]``, ``g [H*v_head_dim, W]`` (with a gate),
    ``o [W, H*v_head_dim]``."""

    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        p = params
        self.hidden, self.nh = int(p["hidden_size"]), int(p["num_heads"])
        self.dk, self.dv = int(p["head_dim"]), int(p["v_head_dim"])
        self.decay_values = [float(a) for a in p["decay"]]
        if len(self.decay_values) != self.nh:
            raise ValueError("retention needs one decay per head")
        if not 0 < self.dk <= ops.RETENTION_MAX_KEY_DIM or self.dv <= 0:
            raise ValueError(f"retention takes key heads of at most {ops.RETENTION_MAX_KEY_DIM} numbers")
        self.eps = float(p["eps"])
        self.key_scale = float(p.get("key_scale") or self.dk**-0.5)
        self.gate = p.get("gate", "silu")
        if self.gate not in ("silu", "sigmoid", None):
            raise ValueError("the gate of retention is 'silu', 'sigmoid' or None")
        pos = p.get("position")
        if isinstance(pos, dict):
            pos = PartSpec(pos["kind"], pos.get("params", {}))
        self.position_spec: PartSpec | None = pos
        self.position = None
        self.k_off = self.nh * self.dk
        self.v_off = 2 * self.nh * self.dk
        self.g_off = self.v_off + self.nh * self.dv
        self.in_dim = -(-(self.g_off + (self.nh * self.dv if self.gate else 0)) // 8) * 8

    @classmethod
    def weight_decls(cls, params):
        w, h, dk, dv = (int(params[k]) for k in ("hidden_size", "num_heads", "head_dim", "v_head_dim"))
        out = {"q": WeightDecl((h * dk, w)), "k": WeightDecl((h * dk, w)), "v": WeightDecl((h * dv, w)), "o": WeightDecl((w, h * dv))}
        if params.get("gate", "silu") is not None:
            out["g"] = WeightDecl((h * dv, w))
        return out

    def cache_need(self) -> CacheNeed:
        return CacheNeed("none")

    def state_shape(self):
        return (self.nh * self.dk * self.dv,)

    def bind(self, weights, rt):
        super().bind(weights, rt)
        mats = [weights["q"], weights["k"], weights["v"]] + ([weights["g"]] if self.gate else [])
        rows = sum(t.shape[0] for t in mats)
        if rows < self.in_dim:  # rows of zeros up to a multiple of 8: the products want aligned widths
            mats.append(torch.zeros((self.in_dim - rows, self.hidden), dtype=mats[0].dtype, device=mats[0].device))
        self.w_in = torch.cat(mats, dim=0).contiguous()
        self.w_o = weights["o"].contiguous()
        self.decay = torch.tensor(self.decay_values, dtype=torch.float32, device=rt.device)
        if self.position_spec is not None and self.position is None:
            self.position = build_part("position", self.position_spec)
            self.position.bind({}, rt)
        self.inv_freq = self.position.table() if self.position is not None else None
        self.interleaved = bool(getattr(self.position, "pairs_interleaved", False))

    def forward(self, ctx, x: torch.Tensor, cache):
        rt = self.rt
        n = x.shape[0]
        if cache is None or cache.state is None:
            raise RuntimeError("retention needs its state slots")
        h, dk, dv = self.nh, self.dk, self.dv
        y = rt.buf("retention.in", n, self.in_dim)
        if ops.skinny_ok(x, self.w_in):
            ops.gemm_skinny(x, self.w_in, y)
        else:
            ops.linear(x, self.w_in, y)
        o = rt.buf("retention.o", n, h * dv, torch.float32)
        scratch = (
            rt.buf("retention.qn", n, h * dk, torch.float32),
            rt.buf("retention.kn", n, h * dk, torch.float32),
            rt.buf("retention.vn", n, h * dv, torch.float32),
        )
        ops.retention(
            y, 0, self.k_off, self.v_off, ctx.positions, self.inv_freq, self.interleaved, self.key_scale, self.decay, cache.state, o,
            ctx.query_start_loc, ctx.state_slots, ctx.num_seqs, h, dk, dv, scratch, max_query_len=ctx.max_query_len,
        )  # fmt: skip
        out = rt.buf("retention.out", n, h * dv)
        gate = y[:, self.g_off : self.g_off + h * dv] if self.gate else None
        ops.retention_gate(o, gate, self.eps, out, h, dv, self.gate)
        return project(rt, "retention.proj", out, self.w_o, ctx)
