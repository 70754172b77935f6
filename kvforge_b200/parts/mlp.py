"""Gated feed-forward (SwiGLU): ``down(silu(gate(x)) * up(x))``, bias-free
(umarhassan-cloud/kvforge ``MLP``, src/tokenvault/model.py:118-132).  The gate and up
projections are one product (weights stacked at load); the gate is applied in 32-bit."""

from __future__ import annotations

import torch

from .. import ops
from .base import FeedForward, WeightDecl, register_feed_forward
from .projection import project


@register_feed_forward("gated_mlp")
class GatedMLP(FeedForward):
    """params: ``hidden_size``, ``intermediate_size``, ``activation`` (only ``"silu"``)."""

    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        self.hidden = int(params["hidden_size"])
        self.inter = int(params["intermediate_size"])
        act = params.get("activation", "silu")
        if act != "silu":
            raise ValueError(f"activation {act!r} is not supported (only 'silu')")

    @classmethod
    def weight_decls(cls, params):
        h, i = int(params["hidden_size"]), int(params["intermediate_size"])
        return {
            "gate_proj.weight": WeightDecl((i, h)),
            "up_proj.weight": WeightDecl((i, h)),
            "down_proj.weight": WeightDecl((h, i)),
        }

    def bind(self, weights, rt):
        super().bind(weights, rt)
        gate, up = weights["gate_proj.weight"], weights["up_proj.weight"]
        # bfloat16: gate and up rows alternate in blocks of 8, the order in which the decode
        # product finds gate_i and up_i in one thread; float32: all gates, then all ups
        self.interleaved = gate.dtype == torch.bfloat16 and self.inter % ops.GATE_UP_BLOCK == 0 and self.inter % 8 == 0
        if self.interleaved:
            self.w_gate_up = ops.interleave_gate_up(gate, up)
        else:
            self.w_gate_up = torch.cat([gate, up], dim=0).contiguous()
        self.w_down = weights["down_proj.weight"].contiguous()

    def forward(self, ctx, x: torch.Tensor):
        rt = self.rt
        n = x.shape[0]
        act = rt.buf("mlp.act", n, self.inter)
        if self.interleaved and ops.skinny_ok(x, self.w_gate_up):
            ops.gemm_skinny(x, self.w_gate_up, act, mode="silu")  # a few tokens: stream the weights once
        elif self.interleaved and ops.tcgen05_ok(x, self.w_gate_up):
            # many tokens: tcgen05 tensor cores, the gate applied as the accumulator leaves tensor memory
            ops.gemm_tcgen05(x, self.w_gate_up, act, mode="silu", err=rt.err)
        else:
            gu = rt.buf("mlp.gate_up", n, 2 * self.inter)
            ops.linear(x, self.w_gate_up, gu)
            ops.silu_mul(gu, act, interleaved=self.interleaved)
        return project(rt, "mlp.out", act, self.w_down, ctx)


@register_feed_forward("plain_mlp")
class PlainMLP(FeedForward):
    """``down(act(up(x)))`` without biases and without a gate.  params: ``hidden_size``, ``intermediate_size``,
    ``activation``: ``"xielu"`` (with the tensor ``act [2]`` = (p, q): ``z > 0: softplus(p) z^2 + z/2``,
    ``z <= 0: (1/2 + softplus(q)) (exp(z) - 1 - z) + z/2``), ``"relu2"`` (the square of relu) or ``"gelu_tanh"``.
    The activation is computed in 32-bit and rounded once.  A block may hand it further rows for its first
    product (``stack_input``): their result for the step is ``self.extra_out`` after ``forward``."""

    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        self.hidden = int(params["hidden_size"])
        self.inter = int(params["intermediate_size"])
        self.activation = params.get("activation", "relu2")
        if self.activation not in ops.UNARY_ACTIVATIONS:
            raise ValueError(f"activation {self.activation!r} is not one of {sorted(ops.UNARY_ACTIVATIONS)}")
        self.extra_w = None
        self.extra_out = None

    @classmethod
    def weight_decls(cls, params):
        h, i = int(params["hidden_size"]), int(params["intermediate_size"])
        out = {"up": WeightDecl((i, h)), "down": WeightDecl((h, i))}
        if params.get("activation", "relu2") == "xielu":
            out["act"] = WeightDecl((2,), kind="vector", init="small")
        return out

    def stack_input(self, w: torch.Tensor) -> bool:
        self.extra_w = w
        self._stack()
        return True

    def _stack(self) -> None:
        mats = [self._up]
        self.extra_off = -(-self.inter // 8) * 8
        if self.extra_w is not None:
            if self.extra_off > self.inter:
                mats.append(torch.zeros((self.extra_off - self.inter, self.hidden), dtype=self._up.dtype, device=self._up.device))
            mats.append(self.extra_w)
        self.w_up = torch.cat(mats, dim=0).contiguous() if len(mats) > 1 else self._up.contiguous()

    def bind(self, weights, rt):
        super().bind(weights, rt)
        self._up = weights["up"]
        self._stack()
        self.w_down = weights["down"].contiguous()
        self.ab = weights["act"].contiguous() if self.activation == "xielu" else None

    def forward(self, ctx, x: torch.Tensor):
        rt = self.rt
        n = x.shape[0]
        u = rt.buf("pmlp.up", n, self.w_up.shape[0])
        if ops.skinny_ok(x, self.w_up):
            ops.gemm_skinny(x, self.w_up, u)
        else:
            ops.linear(x, self.w_up, u)
        self.extra_out = u[:, self.extra_off : self.extra_off + self.extra_w.shape[0]] if self.extra_w is not None else None
        act = rt.buf("pmlp.act", n, self.inter)
        ops.unary_act(u[:, : self.inter], act, self.activation, self.ab)
        return project(rt, "pmlp.out", act, self.w_down, ctx)
