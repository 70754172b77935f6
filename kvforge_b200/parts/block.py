"""Arrangements of parts in a layer.

``prenorm`` is the Llama arrangement (umarhassan-cloud/kvforge, src/tokenvault/model.py:185-187):
``h = h + mixer(norm1(h)); h = h + ffn(norm2(h))``.  Each sum is folded into the norm that
follows it, so a block takes the sum still pending from the block before (``delta``) and
hands back its own.
"""

from __future__ import annotations

from .. import ops
from .base import Block, PartSpec, WeightDecl, build_part, register_block


def _spec(v) -> PartSpec:
    if isinstance(v, PartSpec):
        return v
    return PartSpec(v["kind"], v.get("params", {}))


def _stem(prefix: str, name: str) -> str:
    """Prefix of a sub-part's tensors: ``<layer prefix><name>.``, or the layer's own prefix for an
    empty name (the part's ``names`` then give its tensors' whole names under the layer)."""
    return f"{prefix}{name}." if name else prefix


@register_block("prenorm")
class PreNormBlock(Block):
    """params: ``norm1``, ``mixer``, ``norm2``, ``ffn`` (``PartSpec`` each; ``ffn`` and ``norm2`` may be ``None``: a
    layer without a feed-forward) and the weight-name stems ``norm1_name``, ``mixer_name``, ``norm2_name``,
    ``ffn_name`` under the layer's prefix; optional ``residual_mult`` (``m``: ``h = h + m * mixer(norm1(h))`` and the
    same for the feed-forward; the results are then handed on as ``ops.Scaled``, which the norms must take, and no
    part adds into the stream by itself)."""

    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        names = {
            "norm1": params.get("norm1_name", "input_layernorm"),
            "mixer": params.get("mixer_name", "self_attn"),
            "norm2": params.get("norm2_name", "post_attention_layernorm"),
            "ffn": params.get("ffn_name", "mlp"),
        }
        self.norm1 = build_part("norm", _spec(params["norm1"]), _stem(prefix, names["norm1"]))
        self.mixer = build_part("mixer", _spec(params["mixer"]), _stem(prefix, names["mixer"]))
        self.norm2 = self.ffn = None
        if params.get("ffn") is not None:
            self.norm2 = build_part("norm", _spec(params["norm2"]), _stem(prefix, names["norm2"]))
            self.ffn = build_part("ffn", _spec(params["ffn"]), _stem(prefix, names["ffn"]))
        mult = params.get("residual_mult")
        self.mult = None if mult is None or float(mult) == 1.0 else float(mult)

    def sub_parts(self):
        return [p for p in (self.norm1, self.mixer, self.norm2, self.ffn) if p is not None]

    def mixer_part(self):
        return self.mixer

    def forward(self, ctx, resid, delta, cache):
        if self.mult is None:
            x = self.norm1.forward(ctx, resid, delta)
            a = self.mixer.forward(ctx, x, cache)
            if self.ffn is None:
                return a
            x = self.norm2.forward(ctx, resid, a)
            return self.ffn.forward(ctx, x)
        keep, ctx.residual = ctx.residual, None  # a result is scaled before it joins the stream
        try:
            x = self.norm1.forward(ctx, resid, delta)
            a = ops.Scaled(self.mixer.forward(ctx, x, cache), self.mult)
            if self.ffn is None:
                return a
            x = self.norm2.forward(ctx, resid, a)
            return ops.Scaled(self.ffn.forward(ctx, x), self.mult)
        finally:
            ctx.residual = keep


@register_block("parallel")
class ParallelBlock(Block):
    """One norm a layer; the mixer and the feed-forward both read its output and both add to the
    stream: ``h = h + mixer(n(h)) + ffn(n(h))``.  params: ``norm``, ``mixer``, ``ffn`` (``PartSpec``
    each; ``ffn`` may be ``None``: a layer without a feed-forward) and the stems ``norm_name``,
    ``mixer_name``, ``ffn_name`` under the layer's prefix.

    Nothing reads the residual stream between the norm and the next layer's norm, so either part may
    add its result straight into the stream (``ops.ADDED``); of two results that are still pending
    one is added here and the other is handed to the next norm."""

    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        self.norm = build_part("norm", _spec(params["norm"]), _stem(prefix, params.get("norm_name", "norm1")))
        self.mixer = build_part("mixer", _spec(params["mixer"]), _stem(prefix, params.get("mixer_name", "mix")))
        self.ffn = None
        if params.get("ffn") is not None:
            self.ffn = build_part("ffn", _spec(params["ffn"]), _stem(prefix, params.get("ffn_name", "mlp")))

    def sub_parts(self):
        return [p for p in (self.norm, self.mixer, self.ffn) if p is not None]

    def mixer_part(self):
        return self.mixer

    def forward(self, ctx, resid, delta, cache):
        x = self.norm.forward(ctx, resid, delta)
        a = self.mixer.forward(ctx, x, cache)
        if self.ffn is None:
            return a
        f = self.ffn.forward(ctx, x)
        if a is ops.ADDED or a is None:
            return f
        if f is ops.ADDED or f is None:
            return a
        n = resid.shape[0]
        if isinstance(f, ops.Partials):
            for s in range(f.nsplit):
                ops.add_residual(resid, f.t[s, :n])
        else:
            ops.add_residual(resid, f[:n])
        return a


@register_block("stream_prenorm")
class StreamPreNormBlock(Block):
    """The pre-norm arrangement over several residual streams (hyper-connections).  A token has
    ``S`` streams ``x_1 .. x_S``; sublayer ``q`` (1: the mixer, 2: the feed-forward) reads
    ``u = sum_s in_q[s] x_s``, computes ``y = f(norm_q(u))`` and writes, for all ``t`` from the old
    streams, ``x_t <- sum_s mix_q[s, t] x_s + out_q[t] y``.  A write is folded into the read that
    follows it (one kernel), so the block takes the write still pending from the block before and
    hands back its own.

    params: ``streams``, ``norm1``, ``mixer``, ``norm2``, ``ffn`` (``PartSpec`` each; ``ffn`` and
    ``norm2`` may be ``None``: a layer without a feed-forward), the stems ``norm1_name``,
    ``mixer_name``, ``norm2_name``, ``ffn_name``, and ``hc1_name`` / ``hc2_name`` under which the
    float tensors ``in [S]``, ``out [S]`` and ``mix [S, S]`` (from, to) of each sublayer lie."""

    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        self.streams = int(params["streams"])
        if not 0 < self.streams <= ops.MAX_STREAMS:
            raise ValueError(f"between 1 and {ops.MAX_STREAMS} residual streams")
        self.norm1 = build_part("norm", _spec(params["norm1"]), _stem(prefix, params.get("norm1_name", "norm1")))
        self.mixer = build_part("mixer", _spec(params["mixer"]), _stem(prefix, params.get("mixer_name", "mix")))
        self.ffn = self.norm2 = None
        if params.get("ffn") is not None:
            self.norm2 = build_part("norm", _spec(params["norm2"]), _stem(prefix, params.get("norm2_name", "norm2")))
            self.ffn = build_part("ffn", _spec(params["ffn"]), _stem(prefix, params.get("ffn_name", "mlp")))

    @classmethod
    def weight_decls(cls, params):
        s = int(params["streams"])
        out = {}
        for key, default in (("hc1_name", "hc1"), ("hc2_name", "hc2")):
            if default == "hc2" and params.get("ffn") is None:
                continue
            stem = params.get(key, default)
            out[f"{stem}.in"] = WeightDecl((s,), kind="vector", init="ones")
            out[f"{stem}.out"] = WeightDecl((s,), kind="vector", init="ones")
            out[f"{stem}.mix"] = WeightDecl((s, s), kind="vector", init="eye")
        return out

    def bind(self, weights, rt):
        super().bind(weights, rt)
        p = self.params
        self.hc = []
        for key, default in (("hc1_name", "hc1"), ("hc2_name", "hc2")):
            stem = p.get(key, default)
            if f"{stem}.in" in weights:
                self.hc.append(tuple(weights[f"{stem}.{k}"].contiguous() for k in ("in", "mix", "out")))

    def sub_parts(self):
        return [p for p in (self.norm1, self.mixer, self.norm2, self.ffn) if p is not None]

    def mixer_part(self):
        return self.mixer

    def forward(self, ctx, resid, delta, cache):
        keep, ctx.residual = ctx.residual, None  # no part may add into one of several streams by itself
        try:
            read, mix, out = self.hc[0]
            x = self.norm1.forward(ctx, resid, delta, read=read)
            pending = ops.StreamWrite(self.mixer.forward(ctx, x, cache), mix, out)
            if self.ffn is not None:
                read, mix, out = self.hc[1]
                x = self.norm2.forward(ctx, resid, pending, read=read)
                pending = ops.StreamWrite(self.ffn.forward(ctx, x), mix, out)
        finally:
            ctx.residual = keep
        return pending


@register_block("sandwich")
class SandwichBlock(Block):
    """A norm before and after each sublayer, and a gate on the sublayer's result:
    ``h = norm1(x); x = x + norm1b(mixer(h) * sigmoid(W_g1 h + b_g1))`` and the same with the feed-forward
    (``norm2``, ``norm2b``, ``W_g2``, ``b_g2``).  The gate, the norm after the sublayer and the residual sum are
    folded into the kernel of the norm that follows (an ``ops.GatedWrite`` is what the block hands on).

    params: ``hidden_size``, ``norm`` (the ``PartSpec`` of all four norms, e.g. ``layernorm``), ``mixer``, ``ffn``
    (``PartSpec``; ``ffn`` may be ``None``), ``gate`` (default true: the tensors ``<gate1_name> [W, W]`` and
    ``<gate1_name>.b [W]``, and the same for the feed-forward), and the names ``norm1_name``, ``norm1_post_name``,
    ``norm2_name``, ``norm2_post_name``, ``mixer_name``, ``ffn_name``, ``gate1_name``, ``gate2_name`` under the
    layer's prefix.  A sublayer that can take further rows into its input product (``stack_input``) computes the
    gate's logits there; otherwise the block runs the product itself."""

    DEFAULT_NAMES = {
        "norm1_name": "norm1", "norm1_post_name": "norm1b", "norm2_name": "norm2", "norm2_post_name": "norm2b",
        "mixer_name": "mix", "ffn_name": "mlp", "gate1_name": "rg1", "gate2_name": "rg2",
    }  # fmt: skip

    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        self.hidden = int(params["hidden_size"])
        nm = {k: params.get(k, v) for k, v in self.DEFAULT_NAMES.items()}
        self.names = nm
        self.gated = bool(params.get("gate", True))
        self.gates = [None, None]
        norm = _spec(params["norm"])

        def named_norm(name):
            return build_part("norm", PartSpec(norm.kind, {**norm.params, "names": {"weight": name}}), prefix)

        self.norm1, self.norm1_post = named_norm(nm["norm1_name"]), named_norm(nm["norm1_post_name"])
        self.mixer = build_part("mixer", _spec(params["mixer"]), _stem(prefix, nm["mixer_name"]))
        self.ffn = self.norm2 = self.norm2_post = None
        if params.get("ffn") is not None:
            self.norm2, self.norm2_post = named_norm(nm["norm2_name"]), named_norm(nm["norm2_post_name"])
            self.ffn = build_part("ffn", _spec(params["ffn"]), _stem(prefix, nm["ffn_name"]))

    @classmethod
    def weight_decls(cls, params):
        if not params.get("gate", True):
            return {}
        w = int(params["hidden_size"])
        out = {}
        for key in ("gate1_name", "gate2_name"):
            if key == "gate2_name" and params.get("ffn") is None:
                continue
            stem = params.get(key, cls.DEFAULT_NAMES[key])
            out[stem] = WeightDecl((w, w))
            out[f"{stem}.b"] = WeightDecl((w,), kind="vector", init="zeros")
        return out

    def sub_parts(self):
        return [p for p in (self.norm1, self.norm1_post, self.mixer, self.norm2, self.norm2_post, self.ffn) if p is not None]

    def mixer_part(self):
        return self.mixer

    def bind(self, weights, rt):
        super().bind(weights, rt)
        self.gates = []  # per sublayer: (matrix or None when the sublayer computes the logits, bias)
        for key, part in (("gate1_name", self.mixer), ("gate2_name", self.ffn)):
            if part is None or not self.gated:
                self.gates.append(None)
                continue
            stem = self.names[key]
            w, b = weights[stem].contiguous(), weights[f"{stem}.b"].contiguous()
            stacked = bool(getattr(part, "stack_input", None)) and part.stack_input(w)
            self.gates.append((None if stacked else w, b))

    def _gate(self, ctx, which: int, part, x):
        g = self.gates[which]
        if g is None:
            return None, None
        w, b = g
        if w is None:
            return part.extra_out, b
        z = self.rt.buf(f"block.gate{which}", x.shape[0], self.hidden)
        if ops.skinny_ok(x, w):
            ops.gemm_skinny(x, w, z)
        else:
            ops.linear(x, w, z)
        return z, b

    def forward(self, ctx, resid, delta, cache):
        keep, ctx.residual = ctx.residual, None  # a result is gated and normed before it joins the stream
        try:
            x = self.norm1.forward(ctx, resid, delta)
            y = self.mixer.forward(ctx, x, cache)
            z, b = self._gate(ctx, 0, self.mixer, x)
            pending = ops.GatedWrite(y, z, b, self.norm1_post.weight)
            if self.ffn is not None:
                x = self.norm2.forward(ctx, resid, pending)
                y = self.ffn.forward(ctx, x)
                z, b = self._gate(ctx, 1, self.ffn, x)
                pending = ops.GatedWrite(y, z, b, self.norm2_post.weight)
        finally:
            ctx.residual = keep
        return pending
