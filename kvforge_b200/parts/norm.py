"""RMSNorm fused with the residual sum.

Formula of umarhassan-cloud/kvforge's ``RMSNorm`` (src/tokenvault/model.py:35-38):
``y = (x * rsqrt(mean(x^2) + eps)) * w`` in 32-bit, rounded once.  The residual stream
itself is float here, so ``resid + delta`` is a 32-bit sum as well.
"""

from __future__ import annotations

import torch

from .. import ops
from .base import Norm, WeightDecl, register_norm


@register_norm("rmsnorm")
class RMSNorm(Norm):
    """params: ``dim``, ``eps``; optional ``one_plus`` (the tensor holds the weight's offset from one and the rows
    are multiplied by ``1 + w``; the sum is made once, in 32-bit, when the tensor is bound)."""

    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        self.dim = int(params["dim"])
        self.eps = float(params["eps"])
        self.one_plus = bool(params.get("one_plus", False))

    @classmethod
    def weight_decls(cls, params):
        return {"weight": WeightDecl((int(params["dim"]),), kind="vector", init="zeros" if params.get("one_plus") else "ones")}

    def bind(self, weights, rt):
        super().bind(weights, rt)
        self.weight = weights["weight"] + 1.0 if self.one_plus else weights["weight"]

    def forward(self, ctx, resid: torch.Tensor, delta, rows: torch.Tensor | None = None, num_rows: int | None = None):
        """``delta``: ``None``, a tensor in the storage type, or ``ops.Partials``."""
        n = num_rows if rows is not None else resid.shape[0]
        out = self.rt.buf("norm.out" if rows is None else "norm.rows", n, self.dim)
        ops.add_rmsnorm(resid, delta, self.weight, out, self.eps, rows)
        return out


@register_norm("stream_rmsnorm")
class StreamRMSNorm(Norm):
    """RMSNorm of a read-out of several residual streams ``[N, S*dim]``.  params: ``dim``, ``eps``,
    ``streams``.  ``forward`` takes the write that the sublayer before left pending (an
    ``ops.StreamWrite`` or ``None``), moves the streams on, and norms ``sum_t read[t] x_t``
    (``read=None``: the plain sum, what a model's final norm reads)."""

    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        self.dim = int(params["dim"])
        self.eps = float(params["eps"])
        self.streams = int(params["streams"])

    @classmethod
    def weight_decls(cls, params):
        return {"weight": WeightDecl((int(params["dim"]),), kind="vector", init="ones")}

    def bind(self, weights, rt):
        super().bind(weights, rt)
        self.weight = weights["weight"]

    def forward(self, ctx, resid: torch.Tensor, delta, rows: torch.Tensor | None = None, num_rows: int | None = None, read: torch.Tensor | None = None):
        if delta is ops.ADDED:
            raise RuntimeError("a part added into the residual stream of a model that has several")
        n = num_rows if rows is not None else resid.shape[0]
        out = self.rt.buf("norm.out" if rows is None else "norm.rows", n, self.dim)
        ops.stream_step(resid, delta, read, self.weight, out, self.eps, self.streams, rows)
        return out


@register_norm("layernorm")
class LayerNorm(Norm):
    """Layer norm with a weight and no bias, ``(x - mean) / sqrt(var + eps) * w`` with the variance of the
    deviations, in 32-bit.  params: ``dim``, ``eps``; optional ``centred`` (default true; false: the RMS norm
    through the same kernel).  What the sublayer before left pending may be an ``ops.GatedWrite``: a result that
    is gated, normed in the same way with a weight of its own and only then added to the stream."""

    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        self.dim = int(params["dim"])
        self.eps = float(params["eps"])
        self.centred = bool(params.get("centred", True))

    @classmethod
    def weight_decls(cls, params):
        return {"weight": WeightDecl((int(params["dim"]),), kind="vector", init="ones")}

    def bind(self, weights, rt):
        super().bind(weights, rt)
        self.weight = weights["weight"]

    def forward(self, ctx, resid: torch.Tensor, delta, rows: torch.Tensor | None = None, num_rows: int | None = None):
        n = num_rows if rows is not None else resid.shape[0]
        out = self.rt.buf("norm.out" if rows is None else "norm.rows", n, self.dim)
        ops.norm_step(resid, delta, self.weight, out, self.eps, self.centred, rows)
        return out

    def settle(self, ctx, resid: torch.Tensor, delta, out: torch.Tensor | None = None) -> None:
        """Adds what is pending into the stream without norming it; ``out`` (storage type) gets the stream's rows."""
        ops.norm_step(resid, delta, None, out, self.eps, self.centred)

    def replace(self, ctx, resid: torch.Tensor, out: torch.Tensor | None = None) -> None:
        """The stream itself becomes its normed rows (float); ``out`` gets them in the storage type."""
        ops.norm_step(resid, None, self.weight, out, self.eps, self.centred, store_normed=True)


@register_norm("tanh_norm")
class TanhNorm(Norm):
    """A norm that computes no mean and no variance: ``tanh(alpha * x) * w + b`` per number, with a learned scalar
    ``alpha``, in 32-bit.  params: ``dim``.  Tensors: ``weight [dim]``, ``alpha []``, ``bias [dim]``.  What the
    sublayer before left pending may be an ``ops.Scaled``: it joins the stream multiplied by a constant."""

    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        self.dim = int(params["dim"])

    @classmethod
    def weight_decls(cls, params):
        d = int(params["dim"])
        return {
            "weight": WeightDecl((d,), kind="vector", init="ones"),
            "alpha": WeightDecl((), kind="vector", init="half"),
            "bias": WeightDecl((d,), kind="vector", init="zeros"),
        }

    def bind(self, weights, rt):
        super().bind(weights, rt)
        self.weight, self.bias = weights["weight"], weights["bias"]
        self.alpha = weights["alpha"].reshape(1).contiguous()

    def forward(self, ctx, resid: torch.Tensor, delta, rows: torch.Tensor | None = None, num_rows: int | None = None):
        n = num_rows if rows is not None else resid.shape[0]
        out = self.rt.buf("norm.out" if rows is None else "norm.rows", n, self.dim)
        ops.tanh_norm(resid, delta, self.alpha, self.weight, self.bias, out, rows)
        return out
