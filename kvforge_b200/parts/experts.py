"""A feed-forward of many small experts of which every token uses a few.

Expert ``e`` is ``W_down[e] act(W_up[e] x)`` without biases.  The router's logits ``z = W_router x``
and everything made of them are 32-bit: scores ``s = sigmoid(z)`` (or ``softmax(z)`` over all experts); the
choice is made on ``s + correction`` (a tensor that shifts the choice, not the weights), among the experts of
the best groups only when the experts form groups; the chosen experts' results are summed with weights
``s / (sum of the chosen s + 1e-20)`` (or with the chosen ``s`` as they are).  A shared expert, a feed-forward
of its own that every token passes, may be added to the sum.

A router may add a bias to its logits (``z = W_router x + b``), and its weights may be a softmax over the chosen
logits alone (the logits then rank the experts).  A gated expert is ``W_down[e] join(W_gate[e] x, W_up[e] x)`` with
``join(g, u) = g' sigmoid(alpha g') (u' + shift)``, ``g' = min(g, limit)``, ``u' = clamp(u, -limit, limit)``.
"""

from __future__ import annotations

import torch

from .. import ops
from .base import FeedForward, PartSpec, WeightDecl, build_part, register_feed_forward

WEIGHT_SUM_EPS = 1e-20  # added to the sum of the chosen scores before the division


@register_feed_forward("routed_experts")
class RoutedExperts(FeedForward):
    """params: ``hidden_size``, ``experts``, ``top``, ``intermediate_size`` (of one expert), ``activation``
    (only ``"gelu"``, the exact one); optional ``groups`` and ``keep`` (the experts form ``groups`` equal
    groups of neighbours; a group is ranked by the sum of the top two shifted scores among its members, and
    only members of the ``keep`` best-ranked groups are eligible) and ``correction`` (default true: the tensor
    ``correction [experts]`` is added to the scores for the choice), ``activation`` (``"gelu"``, the exact one, or
    ``"relu2"``, the square of relu), ``score`` (``"sigmoid"`` or ``"softmax"``), ``normalize`` (default true; false:
    the weights are the chosen scores, not divided by their sum) and ``shared`` (the ``PartSpec`` of a feed-forward
    that runs for every token and is added; its tensors lie under ``shared.``); ``score: "chosen_softmax"`` (the
    logits rank the experts, the weights are a softmax over the chosen logits alone); ``router_bias`` (true: the
    tensor ``router.b [E]`` is added to the logits); ``activation: "gated"`` with ``gated: {"limit": l, "alpha": a,
    "shift": s}`` (each optional; the defaults make SwiGLU): an expert then also has ``e<i>.gate [ff, W]``.

    Tensors: ``router [E, W]``, ``correction [E]``, ``e<i>.up [ff, W]``, ``e<i>.down [W, ff]``."""

    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        p = params
        self.hidden, self.experts, self.top, self.ff = int(p["hidden_size"]), int(p["experts"]), int(p["top"]), int(p["intermediate_size"])
        self.groups = int(p.get("groups") or 1)
        self.keep = int(p.get("keep") or self.groups)
        self.corrected = bool(p.get("correction", True))
        self.activation = p.get("activation", "gelu")
        if self.activation not in ops.EXPERT_ACTIVATIONS:
            raise ValueError(f"the experts' activation is one of {sorted(ops.EXPERT_ACTIVATIONS)}")
        self.score = p.get("score", "sigmoid")
        if self.score not in ("sigmoid", "softmax", "chosen_softmax"):
            raise ValueError("score must be 'sigmoid', 'softmax' or 'chosen_softmax'")
        self.router_bias = bool(p.get("router_bias", False))
        self.gated = None
        if self.activation == "gated":
            g = p.get("gated") or {}
            self.gated = ops.GatedActivation(float(g.get("limit", float("inf"))), float(g.get("alpha", 1.0)), float(g.get("shift", 0.0)))
        # the inner size the kernels see: gate and up rows alternate in blocks of 8, so a gated expert is padded with rows of zeros
        self.ff_pad = -(-self.ff // ops.GATE_UP_BLOCK) * ops.GATE_UP_BLOCK if self.gated else self.ff
        self.normalize = bool(p.get("normalize", True))
        shared = p.get("shared")
        if isinstance(shared, dict):
            shared = PartSpec(shared["kind"], shared.get("params", {}))
        self.shared = build_part("ffn", shared, prefix + "shared.") if shared is not None else None
        if not 0 < self.top <= self.experts or self.experts % self.groups or not 0 < self.keep <= self.groups:
            raise ValueError("experts must divide into the groups, and top and keep must be within their counts")
        if self.top > self.keep * (self.experts // self.groups):
            raise ValueError("the groups that stay hold fewer experts than a token uses")

    @classmethod
    def weight_decls(cls, params):
        w, e, ff = int(params["hidden_size"]), int(params["experts"]), int(params["intermediate_size"])
        out = {"router": WeightDecl((e, w), kind="vector", init="normal")}
        if params.get("correction", True):
            out["correction"] = WeightDecl((e,), kind="vector", init="zeros")
        if params.get("router_bias"):
            out["router.b"] = WeightDecl((e,), kind="vector", init="zeros")
        for i in range(e):
            if params.get("activation") == "gated":
                out[f"e{i}.gate"] = WeightDecl((ff, w))
            out[f"e{i}.up"] = WeightDecl((ff, w))
            out[f"e{i}.down"] = WeightDecl((w, ff))
        return out

    def sub_parts(self):
        return [self.shared] if self.shared is not None else []

    def stack_input(self, w: torch.Tensor) -> bool:
        """Further rows for a product that reads this part's input: the shared expert's first product takes them."""
        if self.shared is None or not getattr(self.shared, "stack_input", None):
            return False
        return bool(self.shared.stack_input(w))

    @property
    def extra_out(self):
        return self.shared.extra_out

    def bind(self, weights, rt):
        super().bind(weights, rt)
        self.router = weights["router"].contiguous()
        self.correction = weights["correction"].contiguous() if self.corrected else None
        self.bias = weights["router.b"].contiguous() if self.router_bias else None
        if self.gated is None:
            self.w_up = torch.stack([weights[f"e{i}.up"] for i in range(self.experts)]).contiguous()
            self.w_down = torch.stack([weights[f"e{i}.down"] for i in range(self.experts)]).contiguous()
        else:
            # rows of zeros up to a multiple of 8 (a gate of zero gives zero whatever its up row holds), then gate and
            # up rows in alternating blocks of 8: the products' threads find a gate and its up side by side
            pad = self.ff_pad - self.ff

            def rows(t):
                return torch.cat([t, t.new_zeros((pad, t.shape[1]))]) if pad else t

            self.w_up = torch.stack([ops.interleave_gate_up(rows(weights[f"e{i}.gate"]), rows(weights[f"e{i}.up"])) for i in range(self.experts)]).contiguous()
            self.w_down = torch.stack([torch.cat([weights[f"e{i}.down"], weights[f"e{i}.down"].new_zeros((self.hidden, pad))], dim=1) if pad else weights[f"e{i}.down"] for i in range(self.experts)]).contiguous()
        self._meta = torch.zeros(4, dtype=torch.int32, device=rt.device)

    def forward(self, ctx, x: torch.Tensor):
        rt = self.rt
        n, top, e = x.shape[0], self.top, self.experts
        pairs_cap = rt.max_tokens * top
        ids = rt.buf("experts.ids", n, top, torch.int32)
        wts = rt.buf("experts.weights", n, top, torch.float32)
        ops.moe_route(
            x, self.router, self.correction, top, self.groups, self.keep, WEIGHT_SUM_EPS, ids, wts, self.score == "softmax", self.normalize,
            bias=self.bias, chosen_softmax=self.score == "chosen_softmax",
        )  # fmt: skip
        scratch = {
            "order": rt.buf("experts.order", n * top, 1, torch.int32, cap=pairs_cap),
            "tiles": rt.buf("experts.tiles", ops.moe_max_tiles(n * top, e), 3, torch.int32, cap=ops.moe_max_tiles(pairs_cap, e)),
            "meta": self._meta,
            "act": rt.buf("experts.act", n * top, self.ff_pad, cap=pairs_cap),
            "y": rt.buf("experts.y", n * top, self.hidden, torch.float32, cap=pairs_cap),
        }
        if x.dtype == torch.bfloat16 and n * top >= ops.GROUPED_TCGEN05_MIN_ROWS * e:
            scratch["xs"] = rt.buf("experts.xs", n * top, self.hidden, cap=pairs_cap)
        resid = getattr(ctx, "residual", None)
        if resid is not None and resid.shape[0] >= n and resid.shape[1] == self.hidden:
            ops.moe_experts(x, self.w_up, self.w_down, ids, wts, scratch, resid[:n], rt.err, self.activation, self.gated)
            return self.shared.forward(ctx, x) if self.shared is not None else ops.ADDED
        if self.shared is not None:
            # the shared expert first: when its result comes as the float slices of a split product, the routed sum is
            # added into the first slice and the slices are handed on as they are (whoever reads them adds them in order)
            y = self.shared.forward(ctx, x)
            if isinstance(y, ops.Partials) and y.t.dtype == torch.float32 and y.t.shape[1] >= n and y.t.shape[2] == self.hidden:
                ops.moe_experts(x, self.w_up, self.w_down, ids, wts, scratch, y.t[0, :n], rt.err, self.activation, self.gated)
                return y
            out = rt.buf("experts.out", n, self.hidden, torch.float32)
            out.zero_()
            ops.moe_experts(x, self.w_up, self.w_down, ids, wts, scratch, out, rt.err, self.activation, self.gated)
            if y is not None and y is not ops.ADDED:
                ops.add_residual(out, y[:n])
            return ops.Partials(out.view(1, n, self.hidden))
        out = rt.buf("experts.out", n, self.hidden, torch.float32)
        out.zero_()
        ops.moe_experts(x, self.w_up, self.w_down, ids, wts, scratch, out, rt.err, self.activation, self.gated)
        return ops.Partials(out.view(1, n, self.hidden))
