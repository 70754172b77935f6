"""Attention whose keys and values are made from one small latent per token.

Per token the layer projects its input to ``rank`` latent numbers (RMS-normed) and to ``rot_dim``
numbers of a key part that turns with the position and is shared by all heads; these ``rank +
rot_dim`` numbers are all the cache holds.  Head ``h`` has the key ``[W_uk[h] c, k_rot]`` and the
value ``W_uv[h] c``.  Since ``q . (W_uk[h] c) = (W_uk[h]^T q) . c``, the key up-projection is folded
into the queries and the value up-projection is applied to the attention's result: attention itself
runs over the cache as it is, every head reading the one row per token (keys ``[c, k_rot]``,
values ``c``, the row's first ``rank`` numbers), so a decode step reads ``rank + rot_dim`` numbers per
cached token instead of ``heads * (dim + vdim)``.
"""

from __future__ import annotations

import torch

from .. import ops
from .attention import FP32_PIPE_RANGE, decode_scratch
from .base import CacheNeed, Mixer, PartSpec, WeightDecl, build_part, register_mixer
from .projection import project


# keys per range of the decode form on the tensor cores: a CTA brings its 16 query rows in once per range, so ranges
# are longer than on the FP32 pipes; still short enough that a few sequences make a few hundred CTAs
TENSOR_CORE_RANGE = 128


@register_mixer("latent_attention")
class LatentAttention(Mixer):
    """params: ``hidden_size``, ``num_heads``, ``head_dim`` (a query's and key's part that does not turn),
    ``rot_dim`` (the part that does), ``v_head_dim``, ``kv_rank``, ``eps`` (of the latent's norm), ``scale``;
    optional ``window`` (keys a query sees, itself included), ``position`` (a rotary ``PartSpec`` over at most
    ``rot_dim`` dims, interleaved or split pairs, or ``None``), ``gate`` (``"sigmoid"``: every head's result is
    multiplied by the logistic function of one more projection of the input, one number a head; ``"sigmoid_channel"``:
    one number for every channel of every head; or ``None``) and ``q_rank`` (the queries come through a latent of
    their own: ``c_q = rmsnorm(W_dq x)`` with the weight ``dq.norm`` and ``eps``, ``q = W_uq c_q``).

    Tensors: ``q [H*(head_dim+rot_dim), W]`` (one head after the other, in each the part that does not turn first), or
    with ``q_rank`` ``dq [q_rank, W]``, ``dq.norm [q_rank]`` and ``uq [H*(head_dim+rot_dim), q_rank]``;
    ``dkv [kv_rank+rot_dim, W]``, ``dkv.norm [kv_rank]``, ``uk [H*head_dim, kv_rank]``,
    ``uv [H*v_head_dim, kv_rank]``, ``g [H, W]`` or ``[H*v_head_dim, W]`` (with a gate), ``o [W, H*v_head_dim]``."""

    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        p = params
        self.hidden, self.nh = int(p["hidden_size"]), int(p["num_heads"])
        self.dk, self.dr, self.dv, self.rank = int(p["head_dim"]), int(p["rot_dim"]), int(p["v_head_dim"]), int(p["kv_rank"])
        self.eps, self.scale = float(p["eps"]), float(p["scale"])
        self.window = p.get("window")
        if self.window is not None and int(self.window) <= 0:
            raise ValueError("window must be positive")
        self.gated = p.get("gate") is not None
        if self.gated and p["gate"] not in ("sigmoid", "sigmoid_channel"):
            raise ValueError("the gate of latent attention is 'sigmoid', 'sigmoid_channel' or None")
        self.gate_cols = 0 if not self.gated else self.nh * (self.dv if p["gate"] == "sigmoid_channel" else 1)
        self.q_rank = int(p.get("q_rank") or 0)
        if self.dr % 2 or self.rank % 8 or (self.rank + self.dr) % 8 or self.dk % 8 or self.dv % 8:
            raise ValueError("latent attention needs an even rot_dim and sizes that are multiples of 8")
        ops.check_head_dim(self.rank + self.dr, ops.MAX_KEY_DIM)
        ops.check_head_dim(self.rank, ops.MAX_VALUE_DIM)
        pos = p.get("position")
        if isinstance(pos, dict):
            pos = PartSpec(pos["kind"], pos.get("params", {}))
        self.position_spec: PartSpec | None = pos
        self.position = None
        self.q_cols = self.nh * (self.dk + self.dr)
        # the first product's rows: the queries (or their latent), the keys' and values' latent with the shared key part, the gate
        self.c_off = self.q_rank or self.q_cols
        self.g_off = self.c_off + self.rank + self.dr
        self.in_dim = -(-(self.g_off + self.gate_cols) // 8) * 8
        self.d = self.rank + self.dr

    @classmethod
    def weight_decls(cls, params):
        w, h = int(params["hidden_size"]), int(params["num_heads"])
        dk, dr, dv, r = (int(params[k]) for k in ("head_dim", "rot_dim", "v_head_dim", "kv_rank"))
        qr = int(params.get("q_rank") or 0)
        queries = {"q": WeightDecl((h * (dk + dr), w))}
        if qr:
            queries = {"dq": WeightDecl((qr, w)), "dq.norm": WeightDecl((qr,), kind="vector", init="ones"), "uq": WeightDecl((h * (dk + dr), qr), init="wide")}
        out = {
            **queries,
            "dkv": WeightDecl((r + dr, w)),
            "dkv.norm": WeightDecl((r,), kind="vector", init="ones"),
            "uk": WeightDecl((h * dk, r), init="wide"),
            "uv": WeightDecl((h * dv, r), init="wide"),
            "o": WeightDecl((w, h * dv)),
        }
        if params.get("gate") is not None:
            out["g"] = WeightDecl((h * dv if params["gate"] == "sigmoid_channel" else h, w))
        return out

    def cache_need(self) -> CacheNeed:
        if self.window is None:
            return CacheNeed("full", 1, self.d, None, self.rank, v_in_k=True)
        return CacheNeed("window", 1, self.d, int(self.window), self.rank, v_in_k=True)

    def bind(self, weights, rt):
        super().bind(weights, rt)
        parts = [weights["dq"] if self.q_rank else weights["q"], weights["dkv"]] + ([weights["g"]] if self.gated else [])
        self.w_uq = weights["uq"].contiguous() if self.q_rank else None
        self.cq_weight = weights["dq.norm"] if self.q_rank else None
        rows = sum(t.shape[0] for t in parts)
        if rows < self.in_dim:  # rows of zeros up to a multiple of 8: the products want aligned widths
            parts.append(torch.zeros((self.in_dim - rows, self.hidden), dtype=parts[0].dtype, device=parts[0].device))
        self.w_in = torch.cat(parts, dim=0).contiguous()
        self.c_weight = weights["dkv.norm"]
        h, dk, dv, r = self.nh, self.dk, self.dv, self.rank
        uk, uv = weights["uk"].view(h, dk, r), weights["uv"].view(h, dv, r)
        if rt.dtype == torch.float32:
            self.w_uk = uk.transpose(1, 2).contiguous()  # [H, r, dk]: rows are the outputs of the folded product
            self.w_uv = uv.contiguous()  # [H, dv, r]
        else:
            self.w_uk = uk.contiguous()  # [H, dk, r] as the batched library product reads it
            self.w_uv = uv.transpose(1, 2).contiguous()  # [H, r, dv]
        self.w_o = weights["o"].contiguous()
        if self.position_spec is not None and self.position is None:
            self.position = build_part("position", self.position_spec)
            self.position.bind({}, rt)
        table = self.position.table() if self.position is not None else None
        self.interleaved = bool(getattr(self.position, "pairs_interleaved", False))
        self.inv_freq = table

    def _per_head(self, a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
        """``out[:, h] = a[:, h] @ W[h]`` for every head: ``a [N, H, K]`` and ``out [N, H, M]`` are views
        whose rows may be wider than they are.  bfloat16: one batched library product; 32-bit: the
        engine's own product, one launch a head."""
        if a.dtype == torch.float32:
            for h in range(self.nh):
                ops.gemm_nt_f32(a[:, h], w[h], out[:, h])
        else:
            torch.bmm(a.permute(1, 0, 2), w, out=out.permute(1, 0, 2))

    def forward(self, ctx, x: torch.Tensor, cache):
        rt = self.rt
        n = x.shape[0]
        if cache is None or not cache.writable:
            raise RuntimeError("latent attention keeps a cache of its own")
        h, dk, dr, dv, r, d = self.nh, self.dk, self.dr, self.dv, self.rank, self.d
        y = rt.buf("latent.in", n, self.in_dim)
        if ops.skinny_ok(x, self.w_in):
            ops.gemm_skinny(x, self.w_in, y)
        else:
            ops.linear(x, self.w_in, y)
        qa = rt.buf("latent.qa", n, h * d)
        q = None
        if self.q_rank:
            # the queries' latent, normed, and the queries made from it
            cq = rt.buf("latent.cq", n, self.q_rank)
            ops.row_rmsnorm(y[:, : self.q_rank], self.cq_weight, self.eps, cq)
            q = rt.buf("latent.q", n, self.q_cols)
            if ops.skinny_ok(cq, self.w_uq):
                ops.gemm_skinny(cq, self.w_uq, q)
            else:
                ops.linear(cq, self.w_uq, q)
        ops.latent_prepare(
            y, 0, self.c_off, ctx.positions, self.c_weight, self.eps, self.inv_freq, ctx.slot_mappings[cache.group], cache.k, qa,
            h, dk, dr, r, ctx.block_size, rt.err, interleaved=self.interleaved, q=q,
        )  # fmt: skip
        # the key up-projection folded into the queries
        q_heads = (q if q is not None else y[:, : self.q_cols]).view(n, h, dk + dr)
        self._per_head(q_heads[:, :, :dk], self.w_uk, qa.view(n, h, d)[:, :, :r])
        o_lat = rt.buf("latent.o", n, h * r)
        tensor_cores = ops.latent_attention_supported(qa.dtype, d, r)
        scratch, bound, split = None, None, 256
        if ctx.all_single_query:
            (acc, ml, _), bound, split = decode_scratch(rt, ctx, h, 1, d, r, None, TENSOR_CORE_RANGE if tensor_cores else FP32_PIPE_RANGE)
            scratch = (acc, ml)
        if tensor_cores:
            ops.latent_attention(
                qa, o_lat, cache.k, ctx.block_tables[cache.group], ctx.query_start_loc, ctx.context_lens, ctx.num_seqs, ctx.max_query_len,
                h, d, r, self.scale, window=int(self.window or 0), scratch=scratch, max_context=bound, split_size=split,
            )  # fmt: skip
        else:
            # 32-bit, or a latent whose size the tensor-core kernel does not take: the FP32 pipes
            ops.paged_attention(
                qa, o_lat, cache.k, cache.k, ctx.block_tables[cache.group], ctx.query_start_loc, ctx.context_lens, ctx.num_seqs,
                ctx.max_query_len, h, 1, d, self.scale, window=int(self.window or 0), scratch=scratch, max_context=bound,
                split_size=split, err=rt.err, dv=r,
            )  # fmt: skip
        out = rt.buf("latent.out", n, h * dv)
        self._per_head(o_lat.view(n, h, r), self.w_uv, out.view(n, h, dv))
        if self.gated:
            # one number a head, or one a channel (the same kernel over "heads" of one channel)
            per = dv if self.gate_cols == h else 1
            ops.head_gate(out, y[:, self.g_off : self.g_off + self.gate_cols], self.gate_cols, per)
        return project(rt, "attn.proj", out, self.w_o, ctx)
