"""Python faces of the CUDA launchers in ``csrc/`` (loaded through ``native``).

Every function checks device, dtype, layout and size, then launches on torch's current
stream.  A launcher's non-zero return raises with the kernel's name.  Nothing here has a
CPU path: a tensor that is not on a CUDA device is an error.
"""

from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch

from . import native

_SUF = {torch.float32: "f32", torch.bfloat16: "bf16"}

# p = pointer, i = int, l = long long, f = float
_SIGNATURES = {
    "kvf_embed_{s}": "pppppiiifpp",
    "kvf_add_rmsnorm_{s}": "pppilpppiifp",
    "kvf_add_residual_{s}": "pplp",
    "kvf_rope_cache_{s}": "ppilppppppiiiiiilpp",
    "kvf_silu_mul_{s}": "ppliip",
    "kvf_cast_from_float_{s}": "pplp",
    "kvf_paged_attention_generic_{s}": "pppppppiiiiiiiiiifiiiippiipifpp",
    "kvf_paged_attention_mma_bf16": "pppppppiiiiiiiiifiiiippp",
    "kvf_paged_attention_mma_biased_bf16": "pppppppiiiiiiiiifiipifpp",
    "kvf_latent_attention_bf16": "ppppppiiiiiiiiifiiiippp",
    "kvf_paged_attention_decode_biased_bf16": "pppppppiiiiiiiifiiiipppipifpp",
    "kvf_paged_attention_tcgen05_bf16": "pppppppiiiiiiiiilfipipp",
    "kvf_paged_attention_decode_fused_bf16": "pppppppiiiiiiiifiiiipppp",
    "kvf_paged_attention_decode_tma_bf16": "pppppppiiiiiiiilfiiiippppiip",
    "kvf_gemm_nt_f32": "pppiiiiiip",
    "kvf_gemm_skinny_bf16": "pppiiiiiiiilp",
    "kvf_set_pdl": "i",
    "kvf_gemm_tcgen05_bf16": "pppiiiiiiipp",
    "kvf_sample_f32": "pliippppppp",
    "kvf_argmax_f32": "pliipipp",
    "kvf_scale_softcap_f32": "plffp",
    # library "mixers"
    "kvf_causal_conv_{s}": "pipplppiiiiipiip",
    "kvf_gated_delta_{s}": "pppipipippiplpippiiiiiffiippppilp",
    "kvf_gated_head_norm_{s}": "pipipfiliipip",
    "kvf_hc_step_{s}": "pppilppppppiiifp",
    "kvf_branch_norm_mean_{s}": "pppppilifpp",
    "kvf_rope_cache_general_{s}": "pipppppiiiiiiiilpp",
    "kvf_replicate_streams": "ppliip",
    "kvf_softcap_f32": "plfp",
    "kvf_mixers_set_pdl": "i",
    # library "routed"
    "kvf_head_norm_cache_{s}": "plpppfpipppiiiiiilpipppp",
    "kvf_latent_prepare_{s}": "pliippfpipppiiiiiilpiplp",
    "kvf_row_rmsnorm_{s}": "plpfliplp",
    "kvf_head_gate_{s}": "pplliip",
    "kvf_add_row_f32": "pplip",
    "kvf_moe_route_{s}": "plppiiiiiifipppp",
    "kvf_moe_experts_{s}": "plppppiiiiippppppifffp",
    "kvf_moe_max_tiles": "ii",
    "kvf_moe_sort": "piiipppp",
    "kvf_moe_gather_bf16": "plpiiipp",
    "kvf_moe_combine": "pppiiip",
    "kvf_gemm_grouped_tcgen05_bf16": "pppiiiiiiipppipfffp",
    "kvf_routed_set_pdl": "i",
    # library "gated"
    "kvf_norm_step_{s}": "pppplliplppppliiiifp",
    "kvf_qk_prepare_{s}": "pliiippiifpppiiiiiilpp",
    "kvf_unary_act_{s}": "plplliipp",
    "kvf_talking_attention_{s}": "pppppppppiiiiiiiiiifiiiippp",
    "kvf_talking_attention_mma_bf16": "pppppppppiiiiiiiiiifiiiippp",
    "kvf_talking_mma_ok": "iiiiii",
    "kvf_gated_set_pdl": "i",
    # library "decay"
    "kvf_retention_{s}": "pliiippiifpplplppiliiipppip",
    "kvf_retention_gate_{s}": "plplfiliiplp",
    "kvf_tanh_norm_{s}": "pppilfppppplip",
    "kvf_decay_set_pdl": "i",
}
_CTYPES = {"p": ctypes.c_void_p, "i": ctypes.c_int, "l": ctypes.c_longlong, "f": ctypes.c_float}

_bound: dict[tuple[str, str], object] = {}


def _fn(name: str, lib: str = "core", signature: str | None = None):
    key = (lib, name)
    f = _bound.get(key)
    if f is None:
        cdll = native.load(lib)
        try:
            f = getattr(cdll, name)
        except AttributeError as e:  # pragma: no cover - a build that lacks a symbol
            raise RuntimeError(f"native library '{lib}' lacks {name}") from e
        sig = signature
        if sig is None:
            for pat, s in _SIGNATURES.items():
                if pat.format(s="f32") == name or pat.format(s="bf16") == name:
                    sig = s
                    break
        if sig is None:
            raise RuntimeError(f"no signature known for {name}")
        f.argtypes = [_CTYPES[c] for c in sig]
        f.restype = ctypes.c_int
        _bound[key] = f
        if lib in _PDL_SETTERS and name != _PDL_SETTERS[lib]:
            _sync_library_pdl()
    return f


@dataclass
class Partials:
    """The float slices ``[S, M, N]`` that a split-K product leaves; whoever consumes them
    sums them in slice order."""

    t: torch.Tensor

    @property
    def nsplit(self) -> int:
        return self.t.shape[0]

    @property
    def split_stride(self) -> int:
        return self.t.stride(0)


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The current stream's handle.  ``torch.cuda.current_stream()`` builds a Python object on every
    call (some 15 us); a step of many tokens launches about 130 kernels from Python, so the raw
    handle is asked for directly where torch offers it."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


_pdl_state = None


def set_pdl(enabled: bool) -> None:
    """Ask for programmatic dependent launch on every later launch of this library: a kernel
    may then be scheduled, and prefetch weights, while the kernel ahead of it in the stream is
    still running; it waits before it touches that kernel's results."""
    global _pdl_state
    enabled = bool(enabled)
    if _pdl_state is not enabled:
        _fn("kvf_set_pdl")(1 if enabled else 0)
        _pdl_state = enabled
    _sync_library_pdl()


# every shared library has a flag of its own; it follows the core's once the library is loaded
_PDL_SETTERS = {"mixers": "kvf_mixers_set_pdl", "routed": "kvf_routed_set_pdl", "gated": "kvf_gated_set_pdl", "decay": "kvf_decay_set_pdl"}
_library_pdl: dict[str, bool] = {}


def _sync_library_pdl() -> None:
    for lib, setter in _PDL_SETTERS.items():
        if lib in native._loaded and _pdl_state is not None and _library_pdl.get(lib) is not _pdl_state:
            _fn(setter, lib)(1 if _pdl_state else 0)
            _library_pdl[lib] = _pdl_state


def _sync_mixers_pdl() -> None:
    _sync_library_pdl()


# Kernels of this library launched so far (library matrix products are not counted).
launch_count = 0


def _check(rc: int, name: str, kernels: int = 1) -> None:
    global launch_count
    if rc != 0:
        raise RuntimeError(f"CUDA launcher {name} failed with cudaError {rc}")
    launch_count += kernels


def _need(t: torch.Tensor, dtype: torch.dtype | None, what: str, contiguous: bool = True) -> None:
    if not t.is_cuda:
        raise RuntimeError(f"{what} must be a CUDA tensor (this engine has no CPU path)")
    if dtype is not None and t.dtype != dtype:
        raise TypeError(f"{what} must be {dtype}, got {t.dtype}")
    if contiguous and not t.is_contiguous():
        raise ValueError(f"{what} must be contiguous")


def _suffix(dtype: torch.dtype) -> str:
    try:
        return _SUF[dtype]
    except KeyError:
        raise TypeError(f"storage type {dtype} is not supported (float32 or bfloat16)") from None


# ------------------------------------------------------------------ elementwise


def embed(
    table: torch.Tensor,
    ids: torch.Tensor,
    resid: torch.Tensor,
    err: torch.Tensor | None = None,
    feedback_rows: torch.Tensor | None = None,
    feedback: torch.Tensor | None = None,
    scale: float = 1.0,
) -> None:
    """``resid[n, :] = float(table[id, :]) * scale``; ``ids`` int32 ``[N]``, ``resid`` float ``[N, H]``.
    Where ``feedback_rows[n] >= 0`` the id is ``feedback[feedback_rows[n]]`` (a token sampled on
    the device in the step before) instead of ``ids[n]``."""
    s = _suffix(table.dtype)
    _need(table, None, "table")
    _need(ids, torch.int32, "ids")
    _need(resid, torch.float32, "resid")
    n, h = resid.shape
    if table.shape[1] != h or ids.numel() < n:
        raise ValueError("embed: shapes do not agree")
    if feedback_rows is not None:
        _need(feedback_rows, torch.int32, "feedback_rows")
        _need(feedback, torch.int32, "feedback")
        if feedback_rows.numel() < n:
            raise ValueError("embed: feedback_rows is too short")
    name = f"kvf_embed_{s}"
    _check(_fn(name)(_ptr(table), _ptr(ids), _ptr(feedback_rows), _ptr(feedback), _ptr(resid), n, h, table.shape[0], float(scale), _ptr(err), _stream()), name)


def add_rmsnorm(
    resid: torch.Tensor,
    delta: torch.Tensor | Partials | None,
    weight: torch.Tensor,
    out: torch.Tensor,
    eps: float,
    rows: torch.Tensor | None = None,
) -> None:
    """``v = resid (+ delta)``; ``out = T(v * rsqrt(mean(v^2) + eps) * weight)``.

    ``delta`` is a tensor in the storage type or the ``Partials`` of a split-K product.
    Without ``rows`` the sum is written back into ``resid``.  With ``rows`` (int32 ``[R]``)
    row ``r`` of ``out`` comes from row ``rows[r]`` and ``resid`` is left as it is.
    """
    s = _suffix(out.dtype)
    _need(resid, torch.float32, "resid")
    _need(weight, torch.float32, "norm weight")
    _need(out, None, "out")
    h = resid.shape[-1]
    n_rows = out.shape[0]
    if out.shape[-1] != h or weight.numel() != h:
        raise ValueError("add_rmsnorm: widths do not agree")
    dptr, pptr, nsplit, stride = None, None, 0, 0
    if delta is ADDED:
        delta = None
    if isinstance(delta, Partials):
        _need(delta.t, torch.float32, "partials", contiguous=False)
        if delta.t.shape[-1] != h or delta.t.stride(1) != h or delta.t.stride(2) != 1:
            raise ValueError("add_rmsnorm: partials must be [S, M, H] with dense rows")
        pptr, nsplit, stride = _ptr(delta.t), delta.nsplit, delta.split_stride
    elif delta is not None:
        _need(delta, out.dtype, "delta")
        if delta.shape[-1] != h:
            raise ValueError("add_rmsnorm: delta width")
        dptr = _ptr(delta)
    if rows is not None:
        _need(rows, torch.int32, "rows")
        if rows.numel() < n_rows:
            raise ValueError("add_rmsnorm: fewer row indices than output rows")
    elif resid.shape[0] < n_rows:
        raise ValueError("add_rmsnorm: fewer residual rows than output rows")
    name = f"kvf_add_rmsnorm_{s}"
    _check(
        _fn(name)(_ptr(resid), dptr, pptr, nsplit, stride, _ptr(weight), _ptr(out), _ptr(rows), n_rows, h, float(eps), _stream()),
        name,
    )


def add_residual(resid: torch.Tensor, delta: torch.Tensor) -> None:
    """``resid += float(delta)`` over the first ``delta.numel()`` elements."""
    s = _suffix(delta.dtype)
    _need(resid, torch.float32, "resid")
    _need(delta, None, "delta")
    if delta.numel() > resid.numel():
        raise ValueError("add_residual: delta is larger than resid")
    name = f"kvf_add_residual_{s}"
    _check(_fn(name)(_ptr(resid), _ptr(delta), delta.numel(), _stream()), name)


def rope_cache_write(
    qkv: torch.Tensor | Partials,
    positions: torch.Tensor,
    inv_freq: torch.Tensor,
    slots: torch.Tensor | None,
    kcache: torch.Tensor | None,
    vcache: torch.Tensor | None,
    nh: int,
    nkv: int,
    d: int,
    block_size: int,
    err: torch.Tensor | None = None,
    q_out: torch.Tensor | None = None,
) -> None:
    """Rotate q and k of ``qkv [N, (nh+2nkv)*d]``; write k and v to their slots.

    ``qkv`` in the storage type: q is rotated in place.  ``qkv`` as ``Partials`` of a split-K
    product: the slices are summed in float and q goes to ``q_out [N, nh*d]``.
    ``inv_freq`` float ``[rot/2]`` fixes how many leading dims turn (``rot <= d``).
    ``kcache/vcache``: ``[num_blocks, nkv, block_size, d]``.  ``slots=None`` rotates q only.
    """
    width = (nh + 2 * nkv) * d
    qptr, pptr, nsplit, stride, qo = None, None, 0, 0, None
    if isinstance(qkv, Partials):
        if q_out is None:
            raise ValueError("rope_cache_write: partials need q_out")
        _need(qkv.t, torch.float32, "partials", contiguous=False)
        if qkv.t.shape[-1] != width or qkv.t.stride(1) != width or qkv.t.stride(2) != 1:
            raise ValueError("rope_cache_write: partials must be [S, N, width] with dense rows")
        n = qkv.t.shape[1]
        dtype = q_out.dtype
        _need(q_out, None, "q_out")
        if tuple(q_out.shape) != (n, nh * d):
            raise ValueError("rope_cache_write: q_out shape")
        pptr, nsplit, stride, qo = _ptr(qkv.t), qkv.nsplit, qkv.split_stride, _ptr(q_out)
    else:
        _need(qkv, None, "qkv")
        n = qkv.shape[0]
        dtype = qkv.dtype
        if qkv.shape[1] != width:
            raise ValueError("rope_cache_write: qkv width")
        qptr = _ptr(qkv)
        if q_out is not None:
            _need(q_out, dtype, "q_out")
            qo = _ptr(q_out)
    s = _suffix(dtype)
    _need(positions, torch.int32, "positions")
    _need(inv_freq, torch.float32, "inv_freq")
    rot = 2 * inv_freq.numel()
    if rot > d:
        raise ValueError("rope_cache_write: more frequencies than head_dim/2")
    num_slots = 0
    if slots is not None:
        _need(slots, torch.int32, "slots")
        _need(kcache, dtype, "kcache")
        _need(vcache, dtype, "vcache")
        if tuple(kcache.shape[1:]) != (nkv, block_size, d) or kcache.shape != vcache.shape:
            raise ValueError("rope_cache_write: cache shape must be [num_blocks, nkv, block_size, d]")
        num_slots = kcache.shape[0] * block_size
    name = f"kvf_rope_cache_{s}"
    _check(
        _fn(name)(
            qptr, pptr, nsplit, stride, qo, _ptr(positions), _ptr(inv_freq), _ptr(slots), _ptr(kcache), _ptr(vcache),
            n, nh, nkv, d, rot, block_size, num_slots, _ptr(err), _stream(),
        ),
        name,
    )  # fmt: skip


GATE_UP_BLOCK = 8  # gate and up rows alternate in blocks of this many in the interleaved layout


def interleave_gate_up(w_gate: torch.Tensor, w_up: torch.Tensor) -> torch.Tensor:
    """``[g0..7, u0..7, g8..15, u8..15, ...]``: the row order in which the skinny product finds
    ``gate_i`` and ``up_i`` in one thread's accumulators."""
    i, h = w_gate.shape
    if i % GATE_UP_BLOCK:
        raise ValueError("interleave_gate_up: the intermediate size must be a multiple of 8")
    b = GATE_UP_BLOCK
    return torch.stack([w_gate.view(i // b, b, h), w_up.view(i // b, b, h)], dim=1).reshape(2 * i, h).contiguous()


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor, interleaved: bool = False) -> None:
    """``out[n, i] = silu(gate_i) * up_i`` computed in float.  Columns of ``gate_up [N, 2I]``:
    all gates then all ups, or (``interleaved``) alternating in blocks of 8."""
    s = _suffix(gate_up.dtype)
    _need(gate_up, None, "gate_up")
    _need(out, gate_up.dtype, "out")
    n, i2 = gate_up.shape
    if out.shape[0] != n or out.shape[1] * 2 != i2:
        raise ValueError("silu_mul: shapes do not agree")
    if interleaved and out.shape[1] % GATE_UP_BLOCK:
        raise ValueError("silu_mul: interleaved layout needs a multiple of 8")
    name = f"kvf_silu_mul_{s}"
    _check(_fn(name)(_ptr(gate_up), _ptr(out), n, out.shape[1], GATE_UP_BLOCK if interleaved else 0, _stream()), name)


def cast_from_float(src: torch.Tensor, out: torch.Tensor) -> None:
    s = _suffix(out.dtype)
    _need(src, torch.float32, "src")
    _need(out, None, "out")
    if src.numel() != out.numel():
        raise ValueError("cast_from_float: sizes differ")
    name = f"kvf_cast_from_float_{s}"
    _check(_fn(name)(_ptr(src), _ptr(out), src.numel(), _stream()), name)


# ------------------------------------------------------------------ attention

MAX_ATTN_SPLITS = 1024  # ranges per (sequence, head) the merge kernel takes


ATTN_ONE_WAVE = 888  # CTAs of the decode attention that run as one wave (six fit an SM, 148 SMs)
ATTN_ONE_WAVE_FEW_PAIRS = 640  # the same with fewer than 32 (sequence, kv head) pairs, whose merges are long: room to spare


ATTN_MIN_SPLIT = 128  # the shortest range any batch gets: scratch is made for it
# With this many (sequence, kv head) pairs (4 to 8 sequences of 8 kv heads) ranges of 128 keys: the
# ranges of 256 keys are too few CTAs to pull the bandwidth, and the last CTA of a pair still merges
# few (decode steps of the 1B shape at 2,088 keys: 4 sequences 0.796 -> 0.773 ms, 6 0.797 -> 0.785,
# 8 0.803 -> 0.789 ms; at 3,040 to 5,040 keys 1.5 to 3 %).  With up to 16 pairs the ranges of a pair
# are a thread-block cluster of at most 16 CTAs, which ranges of 256 keys keep to longer contexts
# (one sequence 0.704 against 0.738 ms); from 96 pairs on shorter ranges lose (12 sequences 0.876
# against 0.928 ms).
ATTN_SHORT_RANGE_PAIRS = (17, 64)
# with heads wider than 64 only up to this many pairs (8 sequences of the 3B shape at 2,074 keys: 1.925 ms a step
# with a grid for ranges of 128 keys, 1.847 ms with one for 256; 4 sequences 1.695 against 1.730 ms)
ATTN_SHORT_RANGE_PAIRS_WIDE_HEADS = 32
# ... and only while the step's reach (the longest context, or what a captured graph was made for) is at most
# this: a grid made for ranges of 128 keys over a long reach is mostly CTAs that leave at once, and they
# cost (8 sequences at 8,030 keys 1.100 against 1.042 ms, at 32,798 keys 2.385 against 2.178 ms)
ATTN_SHORT_RANGE_REACH = 4096


def attention_split_size(num_seqs: int, nkv: int, max_context: int = 0, reach: int = 0, head_dim: int = 64) -> int:
    """Keys per range of the decode form, as the launch fixes it.  A range is a CTA, and a CTA has
    a fixed cost of a few microseconds (its chain of dependent reads, its share of the merge), so
    ranges are not short: 256 keys, 128 with 17 to 64 (sequence, kv head) pairs and a ``reach`` of at most 4,096 keys, 512 with 256 or more
    (measured inside the decode step at 1 to 64 sequences), and more when the context is so long that there would
    be more than ``MAX_ATTN_SPLITS`` of them.  Ranges start at multiples of the size.  (The TMA
    kernel may double the size further at run time, see ``attention_wave_target``.)  Since the
    size follows the number of sequences, so does the order in which a context's keys are merged:
    a caller that wants sums that do not depend on the batch at all (the 32-bit path) passes
    ``num_seqs=1``."""
    pairs = num_seqs * nkv
    if pairs >= 256:
        split = 512 if head_dim <= 64 else 1024  # (64 sequences of the 3B and 8B shapes: 1 % faster than with 512)
    elif ATTN_SHORT_RANGE_PAIRS[0] <= pairs <= (ATTN_SHORT_RANGE_PAIRS[1] if head_dim <= 64 else ATTN_SHORT_RANGE_PAIRS_WIDE_HEADS) and reach <= ATTN_SHORT_RANGE_REACH:
        split = ATTN_MIN_SPLIT
    else:
        split = 256
    while -(-max_context // split) > MAX_ATTN_SPLITS:
        split *= 2
    return split


def attention_wave_target(num_seqs: int, nkv: int, head_dim: int = 64) -> int:
    """How many live CTAs the TMA decode kernel aims at: it doubles the range size, on the
    device, from the step's longest context, until the ranges of all (sequence, kv head) pairs
    are at most this many: one wave of CTAs for few pairs (8 sequences at 4,096 keys: ranges of
    256 make 1,024 CTAs, a wave and a small second one, 21.7 us; ranges of 512 one wave, 15.3 us;
    at 3,026 keys 768 CTAs of 256 keys are still one wave and beat 384 of 512: the batch-8 step
    takes 0.846 instead of 0.871 ms; with 2 sequences at 12,000 keys it is the other way round,
    0.911 against 0.890 ms, since the last CTA of a pair then merges 47 ranges: hence the lower
    number for few pairs), at most six ranges a pair for many (64 sequences at 8,192 keys: ranges
    of 512 take 196 us, ranges of 2,048 take 162 us; four a pair made ranges so long that their
    CTAs no longer ran as even waves).  The launch's grid is made for the smallest size; CTAs of
    ranges that a larger size leaves without keys exit at once."""
    pairs = num_seqs * nkv
    one_wave = ATTN_ONE_WAVE if pairs >= 32 else ATTN_ONE_WAVE_FEW_PAIRS
    if head_dim > 64:
        # a CTA's ring is twice the size and three fit an SM: half the CTAs are a wave (8 sequences of the
        # 3B shape at 4,026 keys: 2.255 -> 2.188 ms a step, of the 8B shape 4.113 -> 4.035 ms)
        one_wave //= 2
    return max(one_wave, 6 * pairs)


def attention_scratch_shapes(max_seqs: int, nh: int, d: int, max_context: int, split_size: int = 256) -> tuple[tuple[int, ...], tuple[int, ...]]:
    """Shapes of the float scratch the decode form needs for contexts up to ``max_context``."""
    splits = max(1, -(-max_context // split_size))
    return (max_seqs, nh, splits, d), (max_seqs, nh, splits, 2)


MAX_KEY_DIM = 1024  # what the FP32-pipe attention kernel takes (a latent shared by all heads is this wide)
MAX_VALUE_DIM = 512


def check_head_dim(d: int, most: int = 256) -> None:
    if d <= 0 or d % 8 != 0 or d > most:
        raise ValueError(f"head_dim {d} is not supported: it must be a multiple of 8, at most {most}")


@dataclass
class DistanceBias:
    """A learned bias on attention scores by distance: ``table`` float ``[rows, heads]`` and
    ``bucket`` int32 ``[far + 1]``, the row for every distance up to ``far`` (farther keys take the
    row of ``far``).  The kernels read ``by_distance`` float ``[heads, far + 1]``, the table spread out
    over the distances with a head's values side by side: one load a score, and neighbouring keys in
    neighbouring words."""

    table: torch.Tensor
    bucket: torch.Tensor
    by_distance: torch.Tensor | None = None

    def __post_init__(self) -> None:
        if self.by_distance is None:
            self.by_distance = self.table[self.bucket.long()].t().contiguous()


def mma_attention_supported(dtype: torch.dtype, nh: int, nkv: int, d: int, decode_form: bool) -> bool:
    """Whether the tensor-core kernel (``csrc/attention_mma.cu``) takes this shape."""
    g = nh // max(nkv, 1)
    return dtype == torch.bfloat16 and d in (64, 128) and g <= (16 if decode_form else 64)


TC_ATTN_ROWS = 128  # (token, head of a group) rows of a CTA of the tcgen05 attention kernel


def tcgen05_query_tile(nh: int, nkv: int) -> int:
    """Queries of one sequence that a CTA of the tcgen05 attention kernel takes."""
    return max(1, TC_ATTN_ROWS // max(1, nh // nkv))


def tcgen05_attention_supported(dtype: torch.dtype, nh: int, nkv: int, d: int, decode_form: bool) -> bool:
    """Whether the tcgen05 kernel (``csrc/attention_tcgen05.cu``) takes this shape: many queries
    (not the decode form), bfloat16, head size 64 or 128."""
    return dtype == torch.bfloat16 and d in (64, 128) and not decode_form and nh // max(nkv, 1) <= 128


def tma_decode_supported(dtype: torch.dtype, nh: int, nkv: int, d: int, block_size: int, num_blocks: int) -> bool:
    """Whether the TMA decode kernel (``csrc/attention_decode_tma.cu``) takes this shape."""
    return (
        dtype == torch.bfloat16 and d in (64, 128) and nh // max(nkv, 1) <= 8 and block_size % 16 == 0
        and num_blocks * nkv * block_size < 2**31 - 16
    )  # fmt: skip


def paged_attention(
    q: torch.Tensor,
    out: torch.Tensor,
    kcache: torch.Tensor,
    vcache: torch.Tensor,
    block_tables: torch.Tensor,
    qsl: torch.Tensor,
    ctx_lens: torch.Tensor,
    num_seqs: int,
    max_q_len: int,
    nh: int,
    nkv: int,
    d: int,
    scale: float,
    window: int = 0,
    q_stride: int | None = None,
    scratch: tuple[torch.Tensor, ...] | None = None,
    max_context: int | None = None,
    split_size: int = 256,
    kernel: str = "auto",
    err: torch.Tensor | None = None,
    cluster: bool = True,
    query_tiles: tuple[torch.Tensor, int] | None = None,
    single_only: bool = False,
    wave_target: int = 0,
    dv: int | None = None,
    keep_first: int = 0,
    bias: DistanceBias | None = None,
    softcap: float = 0.0,
    sinks: torch.Tensor | None = None,
) -> None:
    """Paged GQA attention of a flat batch (the contract is at the top of
    ``csrc/attention_generic.cu``).

    ``dv``: size of a value head when it differs from ``d`` (``vcache`` is then
    ``[num_blocks, nkv, block_size, dv]`` and ``out`` ``[N, nh*dv]``); only the FP32-pipe kernel
    takes such a shape.  So it is with ``vcache is kcache`` (a value is the first ``dv`` numbers of
    its key).  ``keep_first`` (under a window, the first keys of every sequence stay visible at any
    distance), ``bias`` (added to the scaled scores, by distance and head), ``softcap`` (``c > 0``: a scaled
    score ``s`` becomes ``c * tanh(s / c)``) and ``sinks`` (float ``[nh]``: ``exp(sinks[h])`` joins the softmax's
    denominator of head ``h``; it has no key and no value) are taken by the FP32-pipe kernel and, for bfloat16
    heads of 64 or 128 with values as wide, by the mma.sync kernels.

    ``q``: rows of ``q_stride`` elements whose first ``nh*d`` are the query heads; ``out``:
    ``[N, nh*d]``.  With ``scratch`` (and every sequence holding one query) the decode form
    runs: key ranges of ``split_size`` in parallel, then a merge; ``max_context`` bounds the
    contexts.  ``kernel``: ``"auto"`` takes, for bfloat16, the tcgen05 kernel (many queries, head
    size 64) or the mma.sync kernel (decode form; head size 128) and the FP32-pipe kernel
    elsewhere; ``"generic"``, ``"mma"``, ``"tma"`` and ``"tcgen05"`` force one (tests).  ``err``: the
    device error flag (a bounded wait inside a kernel raises it).  ``cluster``: the TMA decode kernel
    merges up to 16 key ranges through a thread-block cluster's shared memory (else through the
    scratch and the tickets).  ``query_tiles``: for the tcgen05 kernel, an int32 array of (sequence or
    -1, first query) pairs, one per tile of ``tcgen05_query_tile`` queries, and how many of them to
    launch; without it the grid spans every sequence times the tiles of the longest query run.
    ``single_only`` (TMA decode kernel): of a mixed batch only the sequences that bring exactly one
    query are computed; the rows of the others are left untouched.  ``wave_target`` (TMA decode
    kernel, 0 = off): the kernel doubles ``split_size`` until the ranges of the step's longest
    context, over all pairs, are at most this many (``attention_wave_target``).
    """
    s = _suffix(q.dtype)
    capped = float(softcap) > 0.0 or sinks is not None
    if float(softcap) < 0.0:
        raise ValueError("paged_attention: softcap must be positive (0: none)")
    special = vcache is kcache or keep_first > 0 or bias is not None or d > 256 or (dv or d) > 256 or capped
    # kept first keys and a bias alone, on heads of 64 or 128 in bfloat16 with many queries: the tile form of the mma.sync kernel
    biased_mma = (
        special and vcache is not kcache and (dv or d) == d and kernel == "auto"
        and mma_attention_supported(q.dtype, nh, nkv, d, scratch is not None) and (q_stride or q.shape[-1]) % 2 == 0 and out.shape[-1] % 2 == 0
        and (scratch is None or len(scratch) > 2)
    )  # fmt: skip
    if special and not biased_mma:
        if kernel not in ("auto", "generic"):
            raise ValueError("only the FP32-pipe attention kernel takes kept first keys, a distance bias, capped scores, sinks, values inside keys or heads wider than 256")
        kernel = "generic"
    check_head_dim(d, MAX_KEY_DIM if special and not biased_mma else 256)
    _need(q, None, "q")
    _need(out, q.dtype, "out")
    _need(kcache, q.dtype, "kcache")
    _need(vcache, q.dtype, "vcache")
    _need(block_tables, torch.int32, "block_tables")
    _need(qsl, torch.int32, "query_start_loc")
    _need(ctx_lens, torch.int32, "context_lens")
    dv = d if dv is None else int(dv)
    check_head_dim(dv, MAX_VALUE_DIM if special else 256)
    v_stride = dv
    if vcache is kcache:
        if dv > d:
            raise ValueError("paged_attention: values inside keys cannot be wider than the keys")
        v_stride = d
    if kcache.dim() != 4 or kcache.shape[1] != nkv or kcache.shape[3] != d or tuple(vcache.shape) != (*kcache.shape[:3], v_stride):
        raise ValueError("paged_attention: cache shapes must be [num_blocks, nkv, block_size, d] and [..., dv]")
    if special and 4 * (32 * (d + 4) + (0 if vcache is kcache else 32 * (dv + 4)) + 16 * d + 512) > 227 * 1024:
        raise ValueError(f"paged_attention: heads of {d} and {dv} do not fit the kernel's shared memory")
    bias_args = (None, 0)
    if bias is not None:
        _need(bias.table, torch.float32, "bias table")
        _need(bias.bucket, torch.int32, "bias buckets")
        if bias.table.dim() != 2 or bias.table.shape[1] != nh or bias.bucket.numel() < 1:
            raise ValueError("paged_attention: the bias table must be [rows, heads]")
        _need(bias.by_distance, torch.float32, "bias by distance")
        if tuple(bias.by_distance.shape) != (nh, bias.bucket.numel()):
            raise ValueError("paged_attention: the bias by distance must be [heads, far + 1]")
        bias_args = (_ptr(bias.by_distance), bias.bucket.numel() - 1)
    if keep_first < 0:
        raise ValueError("paged_attention: keep_first is a count of keys")
    if sinks is not None:
        _need(sinks, torch.float32, "sinks")
        if sinks.numel() != nh:
            raise ValueError("paged_attention: one sink per head")
    if dv != d:
        if kernel not in ("auto", "generic"):
            raise ValueError("only the FP32-pipe attention kernel takes a value size of its own")
        kernel = "generic"
    block_size = kcache.shape[2]
    if q_stride is None:
        q_stride = q.shape[-1]
    bt_stride = block_tables.shape[-1] if block_tables.dim() == 2 else block_tables.numel() // max(1, num_seqs)
    split, max_splits, grid_splits, pa, pm, tickets = 0, 0, 0, None, None, None
    if scratch is not None:
        pa, pm = scratch[:2]
        _need(pa, torch.float32, "scratch acc")
        _need(pm, torch.float32, "scratch ml")
        if len(scratch) > 2:
            tickets = scratch[2]
            _need(tickets, torch.int32, "scratch tickets")
            if tickets.numel() < num_seqs * nkv:
                raise ValueError("paged_attention: too few tickets (one per sequence and kv head)")
        if max_q_len != 1:
            raise ValueError("the decode form needs one query per sequence")
        if split_size <= 0 or split_size % 64:
            raise ValueError("split_size must be a positive multiple of 64")
        split = split_size
        max_splits = pa.shape[2]
        if pa.shape[0] < num_seqs or pa.shape[1] != nh or pa.shape[3] != dv:
            raise ValueError("paged_attention: scratch shape does not fit")
        if max_context is None or -(-max_context // split) > max_splits:
            raise ValueError("paged_attention: scratch is too small for the longest context")
        grid_splits = max(1, -(-max_context // split))
        if grid_splits > MAX_ATTN_SPLITS:
            raise ValueError("paged_attention: too many key ranges; use a larger split_size")
    decode_form = scratch is not None
    use_tc = tcgen05_attention_supported(q.dtype, nh, nkv, d, decode_form) and q_stride % 8 == 0 and out.shape[-1] % 8 == 0 and max_q_len > 1
    use_mma = mma_attention_supported(q.dtype, nh, nkv, d, decode_form)
    if biased_mma and scratch is not None:
        name = "kvf_paged_attention_decode_biased_bf16"
        _check(
            _fn(name)(
                _ptr(q), _ptr(out), _ptr(kcache), _ptr(vcache), _ptr(block_tables), _ptr(qsl), _ptr(ctx_lens),
                num_seqs, q_stride, out.shape[-1], bt_stride, nh, nkv, d, block_size, float(scale),
                int(window), split, max_splits, grid_splits, _ptr(pa), _ptr(pm), _ptr(tickets), int(keep_first), *bias_args, float(softcap), _ptr(sinks), _stream(),
            ),
            name,
        )  # fmt: skip
        return
    if biased_mma:
        name = "kvf_paged_attention_mma_biased_bf16"
        _check(
            _fn(name)(
                _ptr(q), _ptr(out), _ptr(kcache), _ptr(vcache), _ptr(block_tables), _ptr(qsl), _ptr(ctx_lens),
                num_seqs, max_q_len, q_stride, out.shape[-1], bt_stride, nh, nkv, d, block_size, float(scale), int(window),
                int(keep_first), *bias_args, float(softcap), _ptr(sinks), _stream(),
            ),
            name,
        )  # fmt: skip
        return
    if kernel == "generic":
        use_tc = use_mma = False
    elif kernel == "tma":
        pass
    elif kernel == "mma":
        if not use_mma:
            raise ValueError("the mma.sync attention kernel does not take this shape")
        use_tc = False
    elif kernel == "tcgen05":
        if not tcgen05_attention_supported(q.dtype, nh, nkv, d, decode_form):
            raise ValueError("the tcgen05 attention kernel does not take this shape")
        use_tc = True
    if use_tc:
        name = "kvf_paged_attention_tcgen05_bf16"
        tiles, n_tiles = None, 0
        if query_tiles is not None and 0 < query_tiles[1] <= 65535:
            tiles, n_tiles = query_tiles
            _need(tiles, torch.int32, "query_tiles")
            if tiles.numel() < 2 * n_tiles:
                raise ValueError("paged_attention: the list of query tiles is shorter than the launch")
        _check(
            _fn(name)(
                _ptr(q), _ptr(out), _ptr(kcache), _ptr(vcache), _ptr(block_tables), _ptr(qsl), _ptr(ctx_lens),
                num_seqs, max_q_len, q_stride, out.shape[-1], bt_stride, nh, nkv, d, block_size, int(kcache.shape[0]),
                float(scale), int(window), _ptr(tiles), n_tiles, _ptr(err), _stream(),
            ),
            name,
        )  # fmt: skip
        return
    use_tma = tickets is not None and tma_decode_supported(q.dtype, nh, nkv, d, block_size, kcache.shape[0])
    if (kernel == "tma" or single_only) and not use_tma:
        raise ValueError("the TMA decode kernel does not take this shape (or no tickets were given)")
    if use_tma and kernel in ("auto", "tma"):
        name = "kvf_paged_attention_decode_tma_bf16"
        _check(
            _fn(name)(
                _ptr(q), _ptr(out), _ptr(kcache), _ptr(vcache), _ptr(block_tables), _ptr(qsl), _ptr(ctx_lens),
                num_seqs, q_stride, out.shape[-1], bt_stride, nh, nkv, d, block_size, int(kcache.shape[0]), float(scale),
                int(window), split, max_splits, grid_splits, _ptr(pa), _ptr(pm), _ptr(tickets), _ptr(err), int(bool(cluster)) | (2 if single_only else 0), int(wave_target), _stream(),
            ),
            name,
        )  # fmt: skip
        return
    if use_mma and tickets is not None:
        name = "kvf_paged_attention_decode_fused_bf16"
        _check(
            _fn(name)(
                _ptr(q), _ptr(out), _ptr(kcache), _ptr(vcache), _ptr(block_tables), _ptr(qsl), _ptr(ctx_lens),
                num_seqs, q_stride, out.shape[-1], bt_stride, nh, nkv, d, block_size, float(scale),
                int(window), split, max_splits, grid_splits, _ptr(pa), _ptr(pm), _ptr(tickets), _stream(),
            ),
            name,
        )  # fmt: skip
        return
    name = "kvf_paged_attention_mma_bf16" if use_mma else f"kvf_paged_attention_generic_{s}"
    _check(
        _fn(name)(
            _ptr(q), _ptr(out), _ptr(kcache), _ptr(vcache), _ptr(block_tables), _ptr(qsl), _ptr(ctx_lens),
            num_seqs, max_q_len, q_stride, out.shape[-1], bt_stride, nh, nkv, d, *((dv,) if not use_mma else ()), block_size, float(scale),
            int(window), split, max_splits, grid_splits, _ptr(pa), _ptr(pm), *(() if use_mma else (int(keep_first), v_stride, *bias_args, float(softcap), _ptr(sinks))), _stream(),
        ),
        name,
        2 if scratch is not None else 1,
    )  # fmt: skip


def latent_attention_supported(dtype: torch.dtype, d: int, dv: int) -> bool:
    """Whether the tensor-core kernel for a cache of one row per token (``csrc/attention_latent.cu``) takes the shape."""
    return dtype == torch.bfloat16 and d % 16 == 0 and d <= MAX_KEY_DIM and dv % 32 == 0 and dv // 32 in (2, 3, 4, 8, 16) and dv <= d


def latent_attention(
    q: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, block_tables: torch.Tensor, qsl: torch.Tensor, ctx_lens: torch.Tensor,
    num_seqs: int, max_q_len: int, nh: int, d: int, dv: int, scale: float, window: int = 0,
    scratch: tuple[torch.Tensor, ...] | None = None, max_context: int | None = None, split_size: int = 128,
) -> None:  # fmt: skip
    """Attention of a flat batch over a paged cache of ONE row of ``d`` numbers per token (``cache [blocks, 1,
    block_size, d]``): the row is every head's key and its first ``dv`` numbers every head's value.  ``q [N, nh*d]``,
    ``out [N, nh*dv]``, bfloat16, on the tensor cores.  With ``scratch`` (partial results ``[B, nh, splits, dv]`` and
    their maxima and sums ``[B, nh, splits, 2]``, float) and one query a sequence the decode form runs: ranges of
    ``split_size`` keys in parallel, then a merge."""
    if not latent_attention_supported(q.dtype, d, dv):
        raise ValueError("latent_attention: the kernel does not take this shape")
    _need(q, torch.bfloat16, "q")
    _need(out, torch.bfloat16, "out")
    _need(cache, torch.bfloat16, "cache")
    _need(block_tables, torch.int32, "block_tables")
    _need(qsl, torch.int32, "query_start_loc")
    _need(ctx_lens, torch.int32, "context_lens")
    if cache.dim() != 4 or cache.shape[1] != 1 or cache.shape[3] != d or q.shape[-1] != nh * d or out.shape[-1] != nh * dv:
        raise ValueError("latent_attention: shapes do not agree")
    bt_stride = block_tables.shape[-1] if block_tables.dim() == 2 else block_tables.numel() // max(1, num_seqs)
    split, max_splits, grid_splits, pa, pm = 0, 0, 0, None, None
    if scratch is not None:
        pa, pm = scratch[:2]
        _need(pa, torch.float32, "scratch acc")
        _need(pm, torch.float32, "scratch ml")
        if max_q_len != 1 or split_size <= 0 or split_size % 32:
            raise ValueError("latent_attention: the decode form needs one query per sequence and ranges of a multiple of 32 keys")
        split, max_splits = split_size, pa.shape[2]
        if pa.shape[0] < num_seqs or pa.shape[1] != nh or pa.shape[3] != dv:
            raise ValueError("latent_attention: scratch shape does not fit")
        if max_context is None or -(-max_context // split) > max_splits:
            raise ValueError("latent_attention: scratch is too small for the longest context")
        grid_splits = max(1, -(-max_context // split))
    name = "kvf_latent_attention_bf16"
    _check(
        _fn(name)(
            _ptr(q), _ptr(out), _ptr(cache), _ptr(block_tables), _ptr(qsl), _ptr(ctx_lens), num_seqs, max_q_len, q.shape[-1], out.shape[-1],
            bt_stride, nh, d, dv, int(cache.shape[2]), float(scale), int(window), split, max_splits, grid_splits, _ptr(pa), _ptr(pm), _stream(),
        ),
        name,
        2 if scratch is not None else 1,
    )  # fmt: skip


def paged_attention_generic(*args, **kw) -> None:
    """``paged_attention`` on the FP32-pipe kernel whatever the shape."""
    kw["kernel"] = "generic"
    paged_attention(*args, **kw)


# ------------------------------------------------------------------ matrix products


def gemm_nt_f32(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """``out[M, N] = a[M, K] @ w[N, K]^T`` on the FP32 pipes (no tensor cores).  Row strides
    may exceed the widths (views of wider buffers)."""
    for t, what in ((a, "a"), (w, "w"), (out, "out")):
        _need(t, torch.float32, what, contiguous=False)
        if t.dim() != 2 or t.stride(1) != 1:
            raise ValueError(f"gemm_nt_f32: {what} must be 2-D with unit inner stride")
    m, k = a.shape
    n = w.shape[0]
    if w.shape[1] != k or tuple(out.shape) != (m, n):
        raise ValueError("gemm_nt_f32: shapes do not agree")
    name = "kvf_gemm_nt_f32"
    _check(
        _fn(name)(_ptr(a), _ptr(w), _ptr(out), m, n, k, a.stride(0), w.stride(0), out.stride(0), _stream()),
        name,
    )


SKINNY_MAX_M = 64  # what the kernel takes
SKINNY_USE_M = 16  # up to here it beats the library product (measured on B200); above, the library is used
SKINNY_MAX_SPLIT = 16


def skinny_ok(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether the decode product (``csrc/gemm_skinny_bf16.cu``) takes ``x @ w^T``."""
    return (
        x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and 0 < x.shape[0] <= SKINNY_USE_M
        and x.shape[1] % 8 == 0 and x.stride(1) == 1 and w.stride(1) == 1 and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
    )  # fmt: skip


def skinny_splits(n_out: int, k: int, m: int = 8) -> int:
    """Slices of K so that a product with few output rows still fills the SMs, each slice at least
    256 wide.  Up to 8 tokens three CTAs of 64 rows fit an SM, and about 384 CTAs (2.6 an SM) were
    best in whole decode steps of all three shapes, with at most 10 slices: the kernel that sums the
    slices is the longer for each one.  (1B shape, 8 sequences: qkv / output / down with 5 / 8 / 8
    slices 0.812 ms a step, with 8 / 8 / 10 slices 0.802 ms, with 8 / 8 / 16 slices 0.845 ms; one
    sequence 0.730 -> 0.703 ms; the 3B shape 2.018 -> 1.974 ms.)  From 9 tokens on a CTA's tiles are
    larger and two fit an SM: about 256 CTAs (with 384 the 16-sequence step took 1.036 instead of
    0.925 ms)."""
    ctas = -(-n_out // 64)
    few = m <= 8
    want = round((384 if few else 256) / ctas)
    while want > 1 and want * ctas > (444 if few else 296):  # more CTAs than are on the SMs at once
        want -= 1
    s = max(1, min(want, k // 256, 10 if few else SKINNY_MAX_SPLIT))
    k_iters = -(-k // 64)
    while s > 1 and (s - 1) * -(-k_iters // s) * 64 >= k:  # the last slice would be empty
        s -= 1
    return s


def gemm_skinny(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor | Partials, mode: str = "plain") -> None:
    """``x [M<=64, K] @ w [N, K]^T`` in bfloat16 with float accumulation.

    ``out``: a bfloat16 or float ``[M, N]`` tensor, ``Partials`` (``[S, M, N]`` float, one slice
    of K each), or with ``mode="silu"`` a bfloat16 ``[M, N/2]`` tensor that receives
    ``silu(gate) * up`` for ``w`` in the interleaved gate/up layout.
    """
    m, k = x.shape
    if not (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and 0 < m <= SKINNY_MAX_M and k % 8 == 0
            and x.stride(1) == 1 and w.stride(1) == 1 and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0):  # fmt: skip
        raise ValueError("gemm_skinny: needs bfloat16, M <= 64, K % 8 == 0, unit inner strides")
    n = w.shape[0]
    if w.shape[1] != k:
        raise ValueError("gemm_skinny: inner sizes differ")
    ksplit, stride = 1, 0
    if isinstance(out, Partials):
        t = out.t
        _need(t, torch.float32, "partials", contiguous=False)
        if tuple(t.shape[1:]) != (m, n) or t.stride(2) != 1:
            raise ValueError("gemm_skinny: partials must be [S, M, N]")
        code, ksplit, stride, ldo, optr = 2, t.shape[0], t.stride(0), t.stride(1), _ptr(t)
    else:
        _need(out, None, "out", contiguous=False)
        if out.stride(1) != 1:
            raise ValueError("gemm_skinny: out needs unit inner stride")
        if mode == "silu":
            if out.dtype != torch.bfloat16 or tuple(out.shape) != (m, n // 2):
                raise ValueError("gemm_skinny: silu output must be bfloat16 [M, N/2]")
            code = 3
        elif tuple(out.shape) != (m, n):
            raise ValueError("gemm_skinny: out shape")
        elif out.dtype == torch.bfloat16:
            code = 0
        elif out.dtype == torch.float32:
            code = 1
        else:
            raise TypeError("gemm_skinny: out must be bfloat16 or float32")
        ldo, optr = out.stride(0), _ptr(out)
    name = "kvf_gemm_skinny_bf16"
    _check(_fn(name)(_ptr(x), _ptr(w), optr, m, n, k, x.stride(0), w.stride(0), ldo, code, ksplit, stride, _stream()), name)


TCGEN05_MIN_TILES = 120  # below this many 128 x 256 output tiles the persistent grid leaves SMs idle


def tcgen05_ok(x: torch.Tensor, w: torch.Tensor, min_tiles: int = TCGEN05_MIN_TILES) -> bool:
    """Whether the tensor-memory product (``csrc/gemm_tcgen05_bf16.cu``) takes ``x @ w^T`` and
    has enough output tiles to fill the device."""
    tiles = -(-x.shape[0] // 128) * -(-w.shape[0] // 256)
    return tiles >= min_tiles and (
        x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[1] % 8 == 0 and x.stride(1) == 1
        and w.stride(1) == 1 and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
        and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
    )  # fmt: skip


def gemm_tcgen05(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, mode: str = "plain", err: torch.Tensor | None = None) -> None:
    """``x [M, K] @ w [N, K]^T`` in bfloat16 on the tcgen05 tensor cores (TMA loads, float
    accumulation in tensor memory).  ``out``: bfloat16 ``[M, N]``, or with ``mode="silu"``
    bfloat16 ``[M, N/2] = silu(gate) * up`` for ``w`` in the interleaved gate/up layout."""
    if not tcgen05_ok(x, w, min_tiles=0):
        raise ValueError("gemm_tcgen05: needs bfloat16, K % 8 == 0, unit inner strides, 16-byte aligned rows")
    m, k = x.shape
    n = w.shape[0]
    if w.shape[1] != k:
        raise ValueError("gemm_tcgen05: inner sizes differ")
    _need(out, torch.bfloat16, "out", contiguous=False)
    if out.stride(1) != 1 or out.stride(0) % 8 or out.data_ptr() % 16:
        raise ValueError("gemm_tcgen05: out needs unit inner stride and 16-byte aligned rows")
    if mode == "silu":
        if tuple(out.shape) != (m, n // 2) or n % 16:
            raise ValueError("gemm_tcgen05: silu output must be [M, N/2] with N % 16 == 0")
        code = 3
    else:
        if tuple(out.shape) != (m, n):
            raise ValueError("gemm_tcgen05: out shape")
        code = 0
    name = "kvf_gemm_tcgen05_bf16"
    _check(_fn(name)(_ptr(x), _ptr(w), _ptr(out), m, n, k, x.stride(0), w.stride(0), out.stride(0), code, _ptr(err), _stream()), name)


def linear(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """``out = x @ w^T`` for ``x [M, K]``, ``w [N, K]``.

    float32: the engine's own FFMA kernel (true 32-bit).  bfloat16 inputs: cuBLAS through
    ``torch.mm`` with 32-bit accumulation, the library product that umarhassan-cloud/kvforge
    itself uses (``nn.Linear``, src/tokenvault/model.py:70-73); ``out`` may be bfloat16 or
    float32.
    """
    if x.dtype == torch.float32:
        gemm_nt_f32(x, w, out)
        return
    _need(x, torch.bfloat16, "x", contiguous=False)
    _need(w, torch.bfloat16, "w", contiguous=False)
    if out.dtype == torch.bfloat16:
        torch.mm(x, w.t(), out=out)
    elif out.dtype == torch.float32:
        torch.mm(x, w.t(), out_dtype=torch.float32, out=out)
    else:
        raise TypeError("linear: out must be bfloat16 or float32")


class _Added:
    """What a mixer or a feed-forward returns when it has added its result into the step's float
    residual stream (``StepContext.residual``) itself: nothing is left for the norm to add."""

    def __repr__(self) -> str:
        return "ADDED"


ADDED = _Added()


def linear_add(x: torch.Tensor, w: torch.Tensor, acc: torch.Tensor) -> None:
    """``acc += x @ w^T`` for bfloat16 ``x [M, K]``, ``w [N, K]`` and float ``acc [M, N]``: the library
    product with 32-bit accumulation whose epilogue reads and writes ``acc`` in 32-bit, so the sum
    with the residual stream is never rounded to bfloat16 and costs no pass of its own."""
    _need(x, torch.bfloat16, "x", contiguous=False)
    _need(w, torch.bfloat16, "w", contiguous=False)
    _need(acc, torch.float32, "acc", contiguous=False)
    if tuple(acc.shape) != (x.shape[0], w.shape[0]) or w.shape[1] != x.shape[1]:
        raise ValueError("linear_add: shapes do not agree")
    torch.addmm(acc, x, w.t(), out_dtype=torch.float32, out=acc)


LIBRARY_SPLIT_MAX_M = 128  # up to here the library product of a narrow output gains from slices of K


def library_splits(m: int, n_out: int, k: int) -> int:
    """Slices of K for the library product ``[m, k] x [n_out, k]^T`` of a few dozen tokens.  With
    so few rows and an output no wider than K (the output and down projections) the library
    launches too few CTAs to pull the weights at the rate of HBM; as a batched product over
    slices of K it does (measured on B200 at 32 to 128 rows on the projections of three model
    shapes: 13.3 -> 8.6 us for [2048, 8192] at 64 rows).  1 = no gain expected."""
    if not (SKINNY_USE_M < m <= LIBRARY_SPLIT_MAX_M) or n_out > k or k < 2048:
        return 1
    s = 4 if m <= 64 else 2
    return s if k % (s * 64) == 0 else 1


def linear_split_k(x: torch.Tensor, w: torch.Tensor, part: Partials) -> None:
    """``part[s] = x[:, slice s of K] @ w[:, slice s of K]^T`` in float, one batched library
    product; whoever consumes the slices sums them in slice order."""
    _need(x, torch.bfloat16, "x")
    _need(w, torch.bfloat16, "w")
    m, k = x.shape
    n = w.shape[0]
    t = part.t
    s = t.shape[0]
    if t.dtype != torch.float32 or tuple(t.shape) != (s, m, n) or not t.is_contiguous() or w.shape[1] != k or k % s:
        raise ValueError("linear_split_k: the slices must be contiguous float [S, M, N] with S dividing K")
    ks = k // s
    torch.bmm(x.view(m, s, ks).permute(1, 0, 2), w.view(n, s, ks).permute(1, 2, 0), out_dtype=torch.float32, out=t)


# ------------------------------------------------------------------ sampling


def sample(
    logits: torch.Tensor,
    out_tokens: torch.Tensor,
    temps: torch.Tensor | None = None,
    top_ks: torch.Tensor | None = None,
    top_ps: torch.Tensor | None = None,
    rand_keys: torch.Tensor | None = None,
    probs_out: torch.Tensor | None = None,
) -> None:
    """One token per row of float ``logits [R, V]``.  ``temps=None`` is greedy for all rows.
    ``rand_keys`` int64 ``[R]``: the draw of a row depends on its key alone."""
    _need(logits, torch.float32, "logits", contiguous=False)
    if logits.dim() != 2 or logits.stride(1) != 1:
        raise ValueError("sample: logits must be [R, V] with unit inner stride")
    r, v = logits.shape
    _need(out_tokens, torch.int32, "out_tokens")
    if out_tokens.numel() < r:
        raise ValueError("sample: out_tokens is too short")
    for t, dt, what in (
        (temps, torch.float32, "temps"),
        (top_ks, torch.int32, "top_ks"),
        (top_ps, torch.float32, "top_ps"),
        (rand_keys, torch.int64, "rand_keys"),
    ):
        if t is not None:
            _need(t, dt, what)
            if t.numel() < r:
                raise ValueError(f"sample: {what} is too short")
    if probs_out is not None:
        _need(probs_out, torch.float32, "probs_out")
        if tuple(probs_out.shape) != (r, v):
            raise ValueError("sample: probs_out shape")
    name = "kvf_sample_f32"
    _check(
        _fn(name)(
            _ptr(logits), logits.stride(0), r, v, _ptr(temps), _ptr(top_ks), _ptr(top_ps), _ptr(rand_keys),
            _ptr(out_tokens), _ptr(probs_out), _stream(),
        ),
        name,
    )  # fmt: skip


# stretches of a row of logits that a CTA each looks through (8 rows of 128,256 in the decode step: 32 stretches
# 0.789 ms a step, 128 stretches 0.782 ms; 64 rows the same either way)
ARGMAX_CHUNKS = 128


def argmax(logits: torch.Tensor, out_tokens: torch.Tensor, partial: torch.Tensor) -> None:
    """Greedy tokens of float ``logits [R, V]`` (lowest index among equal maxima) in two short
    kernels; ``partial``: int64 scratch ``[R, ARGMAX_CHUNKS]``."""
    _need(logits, torch.float32, "logits", contiguous=False)
    if logits.dim() != 2 or logits.stride(1) != 1:
        raise ValueError("argmax: logits must be [R, V] with unit inner stride")
    r, v = logits.shape
    _need(out_tokens, torch.int32, "out_tokens")
    _need(partial, torch.int64, "partial")
    if out_tokens.numel() < r or partial.numel() < r * ARGMAX_CHUNKS:
        raise ValueError("argmax: an output or scratch buffer is too small")
    name = "kvf_argmax_f32"
    _check(_fn(name)(_ptr(logits), logits.stride(0), r, v, _ptr(partial), ARGMAX_CHUNKS, _ptr(out_tokens), _stream()), name, 2)


def splitmix64(z: int) -> int:
    """The host twin of the device generator (``csrc/sampling.cu``): the 64-bit value whose
    high-multiply with the total mass picks the token."""
    m = (1 << 64) - 1
    z = (z + 0x9E3779B97F4A7C15) & m
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & m
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & m
    return z ^ (z >> 31)


# ------------------------------------------------------------------ mixers with a running state (library "mixers")

MIXERS_LIB = "mixers"


def _rows2d(t: torch.Tensor, dtype: torch.dtype | None, what: str) -> None:
    """A 2-D tensor (or a column slice of one): unit inner stride, any row stride."""
    _need(t, dtype, what, contiguous=False)
    if t.dim() != 2 or t.stride(1) != 1:
        raise ValueError(f"{what} must be 2-D with unit inner stride")


def _state_view(state: torch.Tensor, width: int, what: str) -> tuple[int, int]:
    """Pointer to slot 0's part and the stride between slots of a float state ``[slots, width]``
    (a column slice of the pool's rows)."""
    _need(state, torch.float32, what, contiguous=False)
    if state.dim() != 2 or state.shape[1] != width or state.stride(1) != 1:
        raise ValueError(f"{what} must be float [slots, {width}] with unit inner stride")
    return state.data_ptr(), state.stride(0)


def causal_conv(
    x: torch.Tensor, weight: torch.Tensor, state: torch.Tensor, qsl: torch.Tensor, state_slots: torch.Tensor,
    num_seqs: int, out: torch.Tensor, activation: str | None = None, max_query_len: int = 0,
) -> None:  # fmt: skip
    """Short causal convolution over time per channel of a flat batch, and the state moved on.

    ``x [N, C]`` (rows may be a slice of a wider buffer), ``weight`` float ``[C, taps]`` whose last
    column multiplies the current token, ``state`` float ``[slots, (taps-1)*C]``: the last
    ``taps-1`` inputs of each sequence, oldest first, zeros before its start.  ``out [N, C]`` gets
    the sums (``activation``: ``None`` or ``"silu"``); afterwards the state holds this step's last
    inputs.  Sequences without rows and slots below zero are left alone.  ``max_query_len`` (0 =
    unknown): the most rows a sequence brings; up to 4 (with 2 to 4 taps) one kernel does both."""
    s = _suffix(x.dtype)
    _rows2d(x, None, "x")
    _rows2d(out, x.dtype, "out")
    _need(weight, torch.float32, "conv weight")
    n, c = x.shape
    taps = weight.shape[1]
    if tuple(weight.shape) != (c, taps) or tuple(out.shape) != (n, c):
        raise ValueError("causal_conv: shapes do not agree")
    if activation not in (None, "silu"):
        raise ValueError("causal_conv: activation must be None or 'silu'")
    sptr, sstride = (0, 0) if taps == 1 else _state_view(state, (taps - 1) * c, "conv state")
    _need(qsl, torch.int32, "query_start_loc")
    _need(state_slots, torch.int32, "state_slots")
    name = f"kvf_causal_conv_{s}"
    _check(
        _fn(name, MIXERS_LIB)(
            _ptr(x), x.stride(0), _ptr(weight), sptr, sstride, _ptr(qsl), _ptr(state_slots), n, num_seqs, c, taps,
            1 if activation == "silu" else 0, _ptr(out), out.stride(0), int(max_query_len), _stream(),
        ),
        name,
        1 if taps == 1 or (0 < max_query_len <= 4 and 2 <= taps <= 4) else 2,
    )  # fmt: skip


def gated_delta(
    q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, beta_logits: torch.Tensor, step_logits: torch.Tensor,
    a_log: torch.Tensor, dt_bias: torch.Tensor, state: torch.Tensor, out: torch.Tensor, qsl: torch.Tensor,
    state_slots: torch.Tensor, num_seqs: int, num_heads: int, num_kv_heads: int, dk: int, dv: int, q_scale: float,
    norm_eps: float = 1e-6, max_query_len: int = 0, scratch: tuple[torch.Tensor, ...] | None = None,
    logit_slices: int = 0, logit_slice_stride: int = 0,
) -> None:  # fmt: skip
    """The gated delta rule over a flat batch, token by token per sequence, on the state
    ``S [heads, dk, dv]`` of each sequence's slot (``csrc/sequence_mix.cuh`` has the equations).

    ``q, k [N, G*dk]`` and ``v [N, H*dv]`` are column slices of one buffer (same row stride);
    ``beta_logits`` float ``[N, H]``; ``step_logits`` float ``[N, H]`` (one decay a head) or
    ``[N, H*dk]`` (one a key channel), with ``dt_bias`` of the same width and ``a_log [H]``;
    ``out`` float ``[N, H*dv]`` gets the read-out.  ``max_query_len`` (0 = unknown): the most rows any
    sequence of the step brings; up to 4 the kernel takes the form made for steps of single tokens.
    ``scratch``: float buffers ``(kn [N, H*dk], qn [N, H*dk], gn [N, H*dk] or None, sc [N, H*4])`` for what
    a kernel of its own makes of every token before the walk (unit k and q, decays, beta, k.q); without it
    they are allocated here (tests; a step of the engine passes persistent buffers).  Two launches.
    ``logit_slices > 1``: ``beta_logits`` (and per-head ``step_logits``) are slice 0 of that many float
    slices of a split-K product, ``logit_slice_stride`` elements apart, summed in slice order."""
    s = _suffix(q.dtype)
    h, g = int(num_heads), int(num_kv_heads)
    for t, w, what in ((q, g * dk, "q"), (k, g * dk, "k"), (v, h * dv, "v")):
        _rows2d(t, q.dtype, what)
        if t.shape[1] != w or t.shape[0] != q.shape[0] or t.stride(0) != q.stride(0):
            raise ValueError(f"gated_delta: {what} must be [N, {w}] with the row stride of q")
    n = q.shape[0]
    _rows2d(beta_logits, torch.float32, "beta_logits")
    _rows2d(step_logits, torch.float32, "step_logits")
    _rows2d(out, torch.float32, "out")
    per_channel = step_logits.shape[1] != h
    if beta_logits.shape != (n, h) or step_logits.shape[1] not in (h, h * dk) or step_logits.shape[0] != n or tuple(out.shape) != (n, h * dv):
        raise ValueError("gated_delta: shapes do not agree")
    _need(a_log, torch.float32, "A_log")
    _need(dt_bias, torch.float32, "dt_bias")
    if a_log.numel() != h or dt_bias.numel() != step_logits.shape[1]:
        raise ValueError("gated_delta: A_log must be [H] and dt_bias as wide as the step logits")
    sptr, sstride = _state_view(state, h * dk * dv, "delta state")
    _need(qsl, torch.int32, "query_start_loc")
    _need(state_slots, torch.int32, "state_slots")
    if scratch is None:
        mk = lambda w: torch.empty((n, w), dtype=torch.float32, device=q.device)  # noqa: E731
        scratch = (mk(h * dk), mk(h * dk), mk(h * dk) if per_channel else None, mk(h * 4))
    kn, qn, gn, sc = scratch
    for t, w, what in ((kn, h * dk, "kn"), (qn, h * dk, "qn"), (gn, h * dk, "gn"), (sc, h * 4, "sc")):
        if t is None and what == "gn" and not per_channel:
            continue
        _need(t, torch.float32, f"scratch {what}")
        if tuple(t.shape) != (n, w):
            raise ValueError(f"gated_delta: scratch {what} must be float [{n}, {w}]")
    name = f"kvf_gated_delta_{s}"
    _check(
        _fn(name, MIXERS_LIB)(
            _ptr(q), _ptr(k), _ptr(v), q.stride(0), _ptr(beta_logits), beta_logits.stride(0), _ptr(step_logits),
            step_logits.stride(0), _ptr(a_log), _ptr(dt_bias), 1 if per_channel else 0, sptr, sstride, _ptr(out),
            out.stride(0), _ptr(qsl), _ptr(state_slots), num_seqs, h, g, dk, dv, float(q_scale), float(norm_eps), int(max_query_len),
            n, _ptr(kn), _ptr(qn), _ptr(gn) if per_channel else None, _ptr(sc), int(logit_slices), int(logit_slice_stride), _stream(),
        ),
        name,
        2,
    )  # fmt: skip


def gated_head_norm(
    o: torch.Tensor, gate: torch.Tensor | None, weight: torch.Tensor, eps: float, out: torch.Tensor, num_heads: int, dv: int,
    activation: str | None = "silu",
) -> None:  # fmt: skip
    """``out[n, h, :] = o / sqrt(mean(o^2) + eps) * weight * act(gate)`` per token and head; ``o``
    float ``[N, H*dv]``, ``gate`` and ``out`` in the storage type, ``activation``: ``"silu"``,
    ``"sigmoid"`` or ``None`` (no gate)."""
    s = _suffix(out.dtype)
    _rows2d(o, torch.float32, "o")
    _rows2d(out, None, "out")
    _need(weight, torch.float32, "head norm weight")
    n = o.shape[0]
    if o.shape[1] != num_heads * dv or tuple(out.shape) != (n, num_heads * dv) or weight.numel() != dv:
        raise ValueError("gated_head_norm: shapes do not agree")
    act = {None: 0, "silu": 1, "sigmoid": 2}.get(activation, -1)
    if act < 0:
        raise ValueError("gated_head_norm: activation must be 'silu', 'sigmoid' or None")
    gptr, gstride = None, 0
    if act:
        _rows2d(gate, out.dtype, "gate")
        if tuple(gate.shape) != (n, num_heads * dv):
            raise ValueError("gated_head_norm: gate shape")
        gptr, gstride = _ptr(gate), gate.stride(0)
    name = f"kvf_gated_head_norm_{s}"
    _check(
        _fn(name, MIXERS_LIB)(_ptr(o), o.stride(0), gptr, gstride, _ptr(weight), float(eps), act, n, num_heads, dv, _ptr(out), out.stride(0), _stream()),
        name,
    )


# ------------------------------------------------------------------ several residual streams (library "mixers")

MAX_STREAMS = 16
MAX_BRANCHES = 4


@dataclass
class StreamWrite:
    """What a sublayer of a block with several residual streams leaves for the next read: its
    result ``y`` (a tensor in the storage type or ``Partials``), and how it enters the streams:
    ``x_t <- sum_s mix[s, t] x_s + out[t] y``."""

    y: torch.Tensor | Partials
    mix: torch.Tensor  # float [S, S], (from, to)
    out: torch.Tensor  # float [S]


def stream_step(
    streams: torch.Tensor, pending: StreamWrite | None, read: torch.Tensor | None, norm_weight: torch.Tensor, out: torch.Tensor,
    eps: float, num_streams: int, rows: torch.Tensor | None = None,
) -> None:  # fmt: skip
    """One kernel between two sublayers of a model with ``S`` residual streams ``[N, S*W]`` (float):
    the pending write moves the streams on, then ``u = sum_t read[t] x_t`` (``read=None``: the plain
    sum of the streams) is normed: ``out = T(u * rsqrt(mean(u^2) + eps) * norm_weight)``.  With
    ``rows`` (int32) out row ``r`` comes from token ``rows[r]`` and the streams are not written."""
    s = _suffix(out.dtype)
    _need(streams, torch.float32, "streams")
    _need(out, None, "out")
    _need(norm_weight, torch.float32, "norm weight")
    w = out.shape[-1]
    n_rows = out.shape[0]
    if streams.shape[-1] != num_streams * w or norm_weight.numel() != w or not 0 < num_streams <= MAX_STREAMS:
        raise ValueError("stream_step: shapes do not agree")
    yptr, pptr, nsplit, stride, mix, ow = None, None, 0, 0, None, None
    if pending is not None:
        y = pending.y
        if isinstance(y, Partials):
            _need(y.t, torch.float32, "partials", contiguous=False)
            if y.t.shape[-1] != w or y.t.stride(1) != w or y.t.stride(2) != 1:
                raise ValueError("stream_step: partials must be [S, N, W] with dense rows")
            pptr, nsplit, stride = _ptr(y.t), y.nsplit, y.split_stride
        else:
            _need(y, out.dtype, "pending result")
            if y.shape[-1] != w:
                raise ValueError("stream_step: pending result width")
            yptr = _ptr(y)
        _need(pending.mix, torch.float32, "mix")
        _need(pending.out, torch.float32, "out weights")
        if pending.mix.numel() != num_streams * num_streams or pending.out.numel() != num_streams:
            raise ValueError("stream_step: mix must be [S, S] and out [S]")
        mix, ow = pending.mix, pending.out
    if read is not None:
        _need(read, torch.float32, "read weights")
        if read.numel() != num_streams:
            raise ValueError("stream_step: read must be [S]")
    if rows is not None:
        _need(rows, torch.int32, "rows")
        if rows.numel() < n_rows:
            raise ValueError("stream_step: fewer row indices than output rows")
    elif streams.shape[0] < n_rows:
        raise ValueError("stream_step: fewer stream rows than output rows")
    name = f"kvf_hc_step_{s}"
    _check(
        _fn(name, MIXERS_LIB)(
            _ptr(streams), yptr, pptr, nsplit, stride, _ptr(mix), _ptr(ow), _ptr(read), _ptr(norm_weight), _ptr(out), _ptr(rows),
            n_rows, num_streams, w, float(eps), _stream(),
        ),
        name,
    )  # fmt: skip


def replicate_streams(src: torch.Tensor, streams: torch.Tensor, num_streams: int) -> None:
    """``streams[n, s, :] = src[n, :]`` for every stream (float)."""
    _need(src, torch.float32, "src")
    _need(streams, torch.float32, "streams")
    n, w = src.shape
    if tuple(streams.shape) != (n, num_streams * w):
        raise ValueError("replicate_streams: shapes do not agree")
    name = "kvf_replicate_streams"
    _check(_fn(name, MIXERS_LIB)(_ptr(src), _ptr(streams), n, num_streams, w, _stream()), name)


def branch_norm_mean(results: list, weights: list[torch.Tensor], eps: float, out: torch.Tensor) -> None:
    """``out = T(mean_b rmsnorm(results[b]) * weights[b])`` over the model width: the results of
    mixers that ran side by side on the same input (tensors in the storage type or ``Partials``)."""
    s = _suffix(out.dtype)
    _need(out, None, "out")
    n, w = out.shape
    nb = len(results)
    if not 0 < nb <= MAX_BRANCHES or len(weights) != nb:
        raise ValueError(f"branch_norm_mean: between 1 and {MAX_BRANCHES} branches, a weight each")
    P, L, I = ctypes.c_void_p * nb, ctypes.c_longlong * nb, ctypes.c_int * nb
    ys, ps, ns, ss, ws = P(), P(), I(), L(), P()
    for b, (y, wt) in enumerate(zip(results, weights)):
        _need(wt, torch.float32, "branch norm weight")
        if wt.numel() != w:
            raise ValueError("branch_norm_mean: weight width")
        ws[b] = wt.data_ptr()
        if isinstance(y, Partials):
            _need(y.t, torch.float32, "partials", contiguous=False)
            if tuple(y.t.shape[1:]) != (n, w) or y.t.stride(1) != w or y.t.stride(2) != 1:
                raise ValueError("branch_norm_mean: partials must be [S, N, W] with dense rows")
            ys[b], ps[b], ns[b], ss[b] = None, y.t.data_ptr(), y.nsplit, y.split_stride
        else:
            _need(y, out.dtype, "branch result")
            if tuple(y.shape) != (n, w):
                raise ValueError("branch_norm_mean: result shape")
            ys[b], ps[b], ns[b], ss[b] = y.data_ptr(), None, 0, 0
    name = f"kvf_branch_norm_mean_{s}"
    _check(_fn(name, MIXERS_LIB)(ys, ps, ns, ss, ws, nb, n, w, float(eps), _ptr(out), _stream()), name)


def softcap(logits: torch.Tensor, cap: float) -> None:
    """``logits <- cap * tanh(logits / cap)`` in place (float)."""
    _need(logits, torch.float32, "logits")
    name = "kvf_softcap_f32"
    _check(_fn(name, MIXERS_LIB)(_ptr(logits), logits.numel(), float(cap), _stream()), name)


def rope_cache_general(
    qkv: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor, interleaved: bool, slots: torch.Tensor | None,
    kcache: torch.Tensor | None, vcache: torch.Tensor | None, nh: int, nkv: int, dk: int, dv: int, block_size: int,
    err: torch.Tensor | None = None,
) -> None:  # fmt: skip
    """Rotary encoding and cache write in the general form: rows of ``qkv`` hold ``nh`` query heads
    and ``nkv`` key heads of ``dk`` and ``nkv`` value heads of ``dv``; the first ``2*len(inv_freq)``
    dims of q and k turn, pairs ``(2i, 2i+1)`` when ``interleaved`` else ``(i, i + rot/2)``; q in
    place, k and v to ``slots`` of ``kcache [blocks, nkv, block_size, dk]`` / ``vcache [..., dv]``."""
    s = _suffix(qkv.dtype)
    _rows2d(qkv, None, "qkv")
    n = qkv.shape[0]
    if qkv.shape[1] != (nh + nkv) * dk + nkv * dv:
        raise ValueError("rope_cache_general: qkv width")
    _need(positions, torch.int32, "positions")
    _need(inv_freq, torch.float32, "inv_freq")
    rot = 2 * inv_freq.numel()
    if rot > dk:
        raise ValueError("rope_cache_general: more frequencies than dk/2")
    num_slots = 0
    if slots is not None:
        _need(slots, torch.int32, "slots")
        _need(kcache, qkv.dtype, "kcache")
        _need(vcache, qkv.dtype, "vcache")
        if tuple(kcache.shape[1:]) != (nkv, block_size, dk) or tuple(vcache.shape) != (*kcache.shape[:3], dv):
            raise ValueError("rope_cache_general: cache shapes must be [num_blocks, nkv, block_size, dk] and [..., dv]")
        num_slots = kcache.shape[0] * block_size
    name = f"kvf_rope_cache_general_{s}"
    _check(
        _fn(name, MIXERS_LIB)(
            _ptr(qkv), qkv.stride(0), _ptr(positions), _ptr(inv_freq), _ptr(slots), _ptr(kcache), _ptr(vcache), n, nh, nkv,
            dk, dv, rot, 1 if interleaved else 0, block_size, num_slots, _ptr(err), _stream(),
        ),
        name,
    )  # fmt: skip


# ------------------------------------------------------------------ normed heads, latent keys, routed experts (library "routed")

ROUTED_LIB = "routed"


def add_row(resid: torch.Tensor, row: torch.Tensor) -> None:
    """``resid[n, :] += row`` for every row of the float residual stream."""
    _need(resid, torch.float32, "resid")
    _need(row, torch.float32, "row")
    if resid.dim() != 2 or row.numel() != resid.shape[1]:
        raise ValueError("add_row: the row must be as wide as the stream")
    name = "kvf_add_row_f32"
    _check(_fn(name, ROUTED_LIB)(_ptr(resid), _ptr(row), resid.shape[0], resid.shape[1], _stream()), name)


def head_norm_cache(
    qkv: torch.Tensor, positions: torch.Tensor, q_weight: torch.Tensor | None, k_weight: torch.Tensor | None, eps: float,
    inv_freq: torch.Tensor | None, slots: torch.Tensor | None, kcache: torch.Tensor | None, vcache: torch.Tensor | None,
    nh: int, nkv: int, dk: int, dv: int, block_size: int, err: torch.Tensor | None = None, interleaved: bool = True,
    v_keep: torch.Tensor | None = None, v_first: torch.Tensor | None = None, v_lambda: torch.Tensor | None = None,
) -> None:  # fmt: skip
    """What follows the q/k/v product of an attention layer whose queries and keys are normed per
    head: rows of ``qkv`` hold ``nh`` query heads and ``nkv`` key heads of ``dk`` and ``nkv`` value heads
    of ``dv``.  Query and key heads become ``x / sqrt(mean(x^2) + eps) * weight`` (``weight`` float
    ``[dk]``, shared by the heads; ``None``: left as they are), then their first ``2*len(inv_freq)``
    dims turn in interleaved pairs ``(2i, 2i+1)`` or, with ``interleaved=False``, in split pairs ``(i, i + rot/2)``
    (``None``: no rotation); queries in place, keys and values to ``slots`` of
    ``kcache [blocks, nkv, block_size, dk]`` / ``vcache [..., dv]``.  ``v_keep [N, nkv*dv]``: the values as projected
    are copied there as well (for later layers of the step).  ``v_first [N, nkv*dv]`` with ``v_lambda`` (a float
    scalar on the device): the cached value is ``(1 - lambda) v + lambda v_first``."""
    s = _suffix(qkv.dtype)
    _rows2d(qkv, None, "qkv")
    n = qkv.shape[0]
    if qkv.shape[1] != (nh + nkv) * dk + nkv * dv or dk % 2:
        raise ValueError("head_norm_cache: qkv width")
    _need(positions, torch.int32, "positions")
    for w, what in ((q_weight, "query norm weight"), (k_weight, "key norm weight")):
        if w is not None:
            _need(w, torch.float32, what)
            if w.numel() != dk:
                raise ValueError(f"head_norm_cache: the {what} must have {dk} entries")
    rot = 0
    if inv_freq is not None and inv_freq.numel():
        _need(inv_freq, torch.float32, "inv_freq")
        rot = 2 * inv_freq.numel()
        if rot > dk:
            raise ValueError("head_norm_cache: more frequencies than dk/2")
    num_slots = 0
    if slots is not None:
        _need(slots, torch.int32, "slots")
        _need(kcache, qkv.dtype, "kcache")
        _need(vcache, qkv.dtype, "vcache")
        if tuple(kcache.shape[1:]) != (nkv, block_size, dk) or tuple(vcache.shape) != (*kcache.shape[:3], dv):
            raise ValueError("head_norm_cache: cache shapes must be [num_blocks, nkv, block_size, dk] and [..., dv]")
        num_slots = kcache.shape[0] * block_size
    for t, what in ((v_keep, "v_keep"), (v_first, "v_first")):
        if t is not None:
            _need(t, qkv.dtype, what)
            if tuple(t.shape) != (n, nkv * dv):
                raise ValueError(f"head_norm_cache: {what} must be [N, nkv*dv]")
    if v_first is not None:
        _need(v_lambda, torch.float32, "v_lambda")
        if v_lambda.numel() != 1:
            raise ValueError("head_norm_cache: v_lambda is one number")
    name = f"kvf_head_norm_cache_{s}"
    _check(
        _fn(name, ROUTED_LIB)(
            _ptr(qkv), qkv.stride(0), _ptr(positions), _ptr(q_weight), _ptr(k_weight), float(eps), _ptr(inv_freq) if rot else None, rot,
            _ptr(slots), _ptr(kcache), _ptr(vcache), n, nh, nkv if slots is not None else 0, dk, dv, block_size, num_slots, _ptr(err),
            0 if interleaved else 1, _ptr(v_keep), _ptr(v_first), _ptr(v_lambda) if v_first is not None else None, _stream(),
        ),
        name,
    )  # fmt: skip


def latent_prepare(
    x: torch.Tensor, q_off: int, c_off: int, positions: torch.Tensor, c_weight: torch.Tensor, eps: float, inv_freq: torch.Tensor | None,
    slots: torch.Tensor, cache: torch.Tensor, qa: torch.Tensor, nh: int, dk: int, dr: int, rank: int, block_size: int,
    err: torch.Tensor | None = None, interleaved: bool = True, q: torch.Tensor | None = None,
) -> None:  # fmt: skip
    """For an attention layer whose keys and values come from one latent per token.  Rows of ``x`` hold,
    from column ``q_off``, ``nh`` query heads of ``dk + dr`` and, from ``c_off``, ``rank`` latent numbers and
    ``dr`` numbers of a key part shared by all heads.  The latent, RMS-normed with ``c_weight``, and the
    shared key part, turned with the position, go to ``slots`` of ``cache [blocks, 1, block_size, rank + dr]``;
    every query head's last ``dr`` numbers, turned, go to columns ``rank .. rank + dr`` of its head in
    ``qa [N, nh * (rank + dr)]``.  Pairs are interleaved ``(2i, 2i+1)`` or, with ``interleaved=False``, split
    ``(i, i + rot/2)``; ``inv_freq`` float ``[rot/2]``, ``rot <= dr``.  ``q [N, nh*(dk+dr)]``: the query heads lie in
    rows of their own (``q_off`` is then ignored)."""
    s = _suffix(x.dtype)
    _rows2d(x, None, "x")
    _need(qa, x.dtype, "qa")
    _need(cache, x.dtype, "cache")
    _need(positions, torch.int32, "positions")
    _need(slots, torch.int32, "slots")
    _need(c_weight, torch.float32, "latent norm weight")
    n = x.shape[0]
    if q is not None:
        _rows2d(q, x.dtype, "q")
        if tuple(q.shape) != (n, nh * (dk + dr)):
            raise ValueError("latent_prepare: q must be [N, nh*(dk+dr)]")
        q_off = 0
    if (q is None and q_off + nh * (dk + dr) > x.shape[1]) or c_off + rank + dr > x.shape[1] or c_weight.numel() != rank or dr % 2:
        raise ValueError("latent_prepare: the columns do not fit the rows")
    if tuple(qa.shape) != (n, nh * (rank + dr)) or tuple(cache.shape[1:]) != (1, block_size, rank + dr):
        raise ValueError("latent_prepare: qa must be [N, nh*(rank+dr)] and the cache [blocks, 1, block_size, rank+dr]")
    rot = 0
    if inv_freq is not None and inv_freq.numel():
        _need(inv_freq, torch.float32, "inv_freq")
        rot = 2 * inv_freq.numel()
        if rot > dr:
            raise ValueError("latent_prepare: more frequencies than dr/2")
    name = f"kvf_latent_prepare_{s}"
    _check(
        _fn(name, ROUTED_LIB)(
            _ptr(x), x.stride(0), int(q_off), int(c_off), _ptr(positions), _ptr(c_weight), float(eps), _ptr(inv_freq) if rot else None, rot,
            _ptr(slots), _ptr(cache), _ptr(qa), n, nh, dk, dr, rank, block_size, cache.shape[0] * block_size, _ptr(err),
            0 if interleaved else 1, _ptr(q), q.stride(0) if q is not None else 0, _stream(),
        ),
        name,
    )  # fmt: skip


def row_rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor) -> None:
    """``out[n] = x[n] / sqrt(mean(x[n]^2) + eps) * weight`` in float, rounded once; ``x [N, r]`` may be a column range of
    wider rows, ``out [N, r]`` likewise, ``weight`` float ``[r]``."""
    s = _suffix(x.dtype)
    _rows2d(x, None, "x")
    _rows2d(out, x.dtype, "out")
    _need(weight, torch.float32, "norm weight")
    if out.shape != x.shape or weight.numel() != x.shape[1]:
        raise ValueError("row_rmsnorm: shapes do not agree")
    name = f"kvf_row_rmsnorm_{s}"
    _check(_fn(name, ROUTED_LIB)(_ptr(x), x.stride(0), _ptr(weight), float(eps), x.shape[0], x.shape[1], _ptr(out), out.stride(0), _stream()), name)


def head_gate(y: torch.Tensor, gate: torch.Tensor, nh: int, dv: int) -> None:
    """``y[n, h, :] *= 1 / (1 + exp(-gate[n, h]))`` in place; ``y [N, nh*dv]`` contiguous, ``gate [N, nh]``
    a column range of a wider row."""
    s = _suffix(y.dtype)
    _need(y, None, "y")
    _rows2d(gate, y.dtype, "gate")
    n = y.shape[0]
    if y.shape[1] != nh * dv or tuple(gate.shape) != (n, nh):
        raise ValueError("head_gate: shapes do not agree")
    name = f"kvf_head_gate_{s}"
    _check(_fn(name, ROUTED_LIB)(_ptr(y), _ptr(gate), gate.stride(0), n, nh, dv, _stream()), name)


def moe_max_tiles(n_pairs: int, num_experts: int) -> int:
    return int(_fn("kvf_moe_max_tiles", ROUTED_LIB)(int(n_pairs), int(num_experts)))


def moe_route(
    x: torch.Tensor, router: torch.Tensor, correction: torch.Tensor | None, top: int, groups: int, keep: int, norm_eps: float,
    ids: torch.Tensor, weights: torch.Tensor, softmax: bool = False, normalize: bool = True, bias: torch.Tensor | None = None,
    chosen_softmax: bool = False,
) -> None:  # fmt: skip
    """Per token of ``x [N, W]``: logits ``router [E, W] x`` in float, scores ``s = sigmoid(z)``; the ``top``
    experts with the largest ``s + correction`` among the best ``keep`` of ``groups`` equal groups of
    neighbouring experts (a group's rank: the sum of the top two ``s + correction`` among its members) are chosen
    (``ids`` int32 ``[N, top]``); their weights are their ``s`` over the sum of those (+ ``norm_eps``)
    (``weights`` float ``[N, top]``).  ``softmax``: the scores are ``softmax(z)`` over all experts instead;
    ``normalize=False``: the weights are the chosen scores as they are.  ``bias`` (float ``[E]``) is added to the
    logits.  ``chosen_softmax``: the logits themselves rank the experts and the weights are a softmax over the chosen
    logits alone (``softmax``, ``normalize`` and ``norm_eps`` then play no part)."""
    s = _suffix(x.dtype)
    _rows2d(x, None, "x")
    _need(router, torch.float32, "router")
    n, w = x.shape
    e = router.shape[0]
    if router.dim() != 2 or router.shape[1] != w:
        raise ValueError("moe_route: router must be [E, W]")
    if correction is not None:
        _need(correction, torch.float32, "correction")
        if correction.numel() != e:
            raise ValueError("moe_route: one correction per expert")
    if bias is not None:
        _need(bias, torch.float32, "router bias")
        if bias.numel() != e:
            raise ValueError("moe_route: one bias per expert")
    _need(ids, torch.int32, "ids")
    _need(weights, torch.float32, "weights")
    if tuple(ids.shape) != (n, top) or tuple(weights.shape) != (n, top):
        raise ValueError("moe_route: ids and weights must be [N, top]")
    flags = 4 if chosen_softmax else (1 if softmax else 0) | (0 if normalize else 2)
    name = f"kvf_moe_route_{s}"
    _check(
        _fn(name, ROUTED_LIB)(_ptr(x), x.stride(0), _ptr(router), _ptr(correction), n, w, e, int(top), int(groups), int(keep), float(norm_eps), flags, _ptr(ids), _ptr(weights), _ptr(bias), _stream()),
        name,
    )


# what the experts' kernels apply between their two products; "gated": the first matrix holds gate and up rows in
# alternating blocks of GATE_UP_BLOCK (``interleave_gate_up``) and the two are joined (``GatedActivation``)
EXPERT_ACTIVATIONS = {"gelu": 0, "relu2": 1, "gated": 2}


@dataclass(frozen=True)
class GatedActivation:
    """``g' / (1 + exp(-alpha g')) * (u' + shift)`` with ``g' = min(g, limit)`` and ``u' = clamp(u, -limit, limit)``:
    the defaults are SwiGLU (``silu(g) * u``)."""

    limit: float = float("inf")
    alpha: float = 1.0
    shift: float = 0.0

GROUPED_TILE_ROWS = 128  # rows of a tile of the tensor-memory product
# from this many rows an expert (on average) the two products of routed experts run on the tcgen05 tensor cores
GROUPED_TCGEN05_MIN_ROWS = 64


def moe_experts(
    x: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, scratch: dict, resid: torch.Tensor,
    err: torch.Tensor | None = None, activation: str = "gelu", gated: GatedActivation | None = None,
) -> None:  # fmt: skip
    """``resid[n] += sum_k weights[n, k] * w_down[e] act(w_up[e] x[n])`` with ``e = ids[n, k]`` and ``act`` the exact
    GELU (``"gelu"``) or the square of relu (``"relu2"``): the pairs are
    ordered by expert, every expert's rows go through its two products in tiles, and the results are
    summed per token in the order of ``k``.  ``w_up [E, ff, W]``, ``w_down [E, W, ff]``; ``scratch``: ``order``
    int32 ``[N*top]``, ``tiles`` int32 ``[3*max_tiles]``, ``meta`` int32 ``[4]``, ``act [N*top, ff]``, ``y`` float
    ``[N*top, W]``, and for many bfloat16 rows ``xs [N*top, W]`` (the pairs' rows side by side by expert).  With
    ``activation="gated"`` ``w_up`` is ``[E, 2*ff, W]``, gate and up rows alternating in blocks of 8, and ``gated`` says how
    they are joined.  Four
    launches, five through the tensor-memory product (``err``: the device flag its bounded waits raise)."""
    s = _suffix(x.dtype)
    if activation not in EXPERT_ACTIVATIONS:
        raise ValueError(f"moe_experts: activation {activation!r} is not one of {sorted(EXPERT_ACTIVATIONS)}")
    act_kind = EXPERT_ACTIVATIONS[activation]
    _rows2d(x, None, "x")
    _need(w_up, x.dtype, "w_up")
    _need(w_down, x.dtype, "w_down")
    _need(resid, torch.float32, "resid")
    n, w = x.shape
    is_gated = activation == "gated"
    ga = gated or GatedActivation()
    e, ff = w_up.shape[0], w_up.shape[1] // (2 if is_gated else 1)
    top = ids.shape[1]
    if is_gated and ff % GATE_UP_BLOCK:
        raise ValueError("moe_experts: gated experts need an inner size that is a multiple of 8")
    if tuple(w_up.shape) != (e, ff * (2 if is_gated else 1), w) or tuple(w_down.shape) != (e, w, ff) or tuple(resid.shape) != (n, w):
        raise ValueError("moe_experts: shapes do not agree")
    _need(ids, torch.int32, "ids")
    _need(weights, torch.float32, "weights")
    order, tiles, meta, act, y = (scratch[k] for k in ("order", "tiles", "meta", "act", "y"))
    _need(order, torch.int32, "order")
    _need(tiles, torch.int32, "tiles")
    _need(meta, torch.int32, "meta")
    _need(act, x.dtype, "act")
    _need(y, torch.float32, "y")
    if order.numel() < n * top or tiles.numel() < 3 * moe_max_tiles(n * top, e) or act.numel() < n * top * ff or y.numel() < n * top * w:
        raise ValueError("moe_experts: a scratch buffer is too small")
    pairs = n * top
    xs = scratch.get("xs")
    if x.dtype == torch.bfloat16 and xs is not None and pairs >= GROUPED_TCGEN05_MIN_ROWS * e and w % 8 == 0 and ff % 8 == 0 and x.stride(0) % 8 == 0:
        # many rows an expert: both products on the tcgen05 tensor cores, over row tiles of 128 of one expert
        _need(xs, torch.bfloat16, "xs")
        if xs.numel() < pairs * w:
            raise ValueError("moe_experts: a scratch buffer is too small")
        row_tiles = pairs // GROUPED_TILE_ROWS + e
        st = _stream()
        _check(_fn("kvf_moe_sort", ROUTED_LIB)(_ptr(ids), pairs, e, GROUPED_TILE_ROWS, _ptr(order), _ptr(tiles), _ptr(meta), st), "kvf_moe_sort")
        _check(_fn("kvf_moe_gather_bf16", ROUTED_LIB)(_ptr(x), x.stride(0), _ptr(order), top, pairs, w, _ptr(xs), st), "kvf_moe_gather_bf16")
        g = _fn("kvf_gemm_grouped_tcgen05_bf16")
        fl = (float(ga.limit), float(ga.alpha), float(ga.shift))
        _check(g(_ptr(xs), _ptr(w_up), _ptr(act), pairs, ff * (2 if is_gated else 1), w, e, w, ff, 1 + act_kind, _ptr(tiles), _ptr(meta), None, row_tiles, _ptr(err), *fl, st), "kvf_gemm_grouped_tcgen05_bf16")
        _check(g(_ptr(act), _ptr(w_down), _ptr(y), pairs, w, ff, e, ff, w, 0, _ptr(tiles), _ptr(meta), _ptr(order), row_tiles, _ptr(err), *fl, st), "kvf_gemm_grouped_tcgen05_bf16")
        _check(_fn("kvf_moe_combine", ROUTED_LIB)(_ptr(resid), _ptr(y), _ptr(weights), n, w, top, st), "kvf_moe_combine")
        return
    name = f"kvf_moe_experts_{s}"
    _check(
        _fn(name, ROUTED_LIB)(
            _ptr(x), x.stride(0), _ptr(w_up), _ptr(w_down), _ptr(ids), _ptr(weights), n, w, ff, e, top, _ptr(order), _ptr(tiles), _ptr(meta),
            _ptr(act), _ptr(y), _ptr(resid), act_kind, float(ga.limit), float(ga.alpha), float(ga.shift), _stream(),
        ),
        name,
        4,
    )  # fmt: skip


# ------------------------------------------------------------------ library "gated"
# gated and normed sublayer results, rotation followed by a head norm, attention whose heads talk

GATED_LIB = "gated"


@dataclass
class GatedWrite:
    """A sublayer's result that is still to be gated, normed and added to the residual stream:
    ``resid += norm(y * sigmoid(z + z_bias)) * post_w``.  ``y``: a tensor in the storage type or the
    ``Partials`` of a split product; ``z``: gate logits in the storage type ``[N, W]`` (a view with a row
    stride of its own is fine) or ``None`` (no gate); ``post_w``: float ``[W]`` or ``None`` (added as it is).
    The norm that consumes it decides the norm's kind and eps: the same as its own."""

    y: "torch.Tensor | Partials"
    z: torch.Tensor | None = None
    z_bias: torch.Tensor | None = None
    post_w: torch.Tensor | None = None


def norm_step(
    resid: torch.Tensor,
    pending,
    next_w: torch.Tensor | None,
    out: torch.Tensor | None,
    eps: float,
    centred: bool = True,
    rows: torch.Tensor | None = None,
    store_normed: bool = False,
) -> None:
    """One pass over every row of the float residual stream ``resid [N, W]``:

    * ``pending`` (``None``, ``ADDED``, a tensor, ``Partials`` or a ``GatedWrite``) is gated, normed and added
      (the sum is written back unless ``rows`` picks rows);
    * ``out`` (storage type, rows may be a view of a wider buffer) gets the row normed with ``next_w``
      (``None``: the row itself); with ``store_normed`` the normed row also replaces the residual row.

    The norm is the layer norm ``(x - mean) / sqrt(var + eps) * w`` with the variance of the deviations
    (``centred``), or the RMS norm ``x / sqrt(mean(x^2) + eps) * w``."""
    _need(resid, torch.float32, "resid")
    w = resid.shape[-1]
    if pending is ADDED:
        pending = None
    gw = pending if isinstance(pending, GatedWrite) else GatedWrite(pending) if pending is not None else None
    if out is not None:
        s = _suffix(out.dtype)
        _need(out, None, "out", contiguous=False)
        if out.dim() != 2 or out.stride(1) != 1 or out.shape[1] != w:
            raise ValueError("norm_step: out must be [rows, W] with unit inner stride")
        n_rows, optr, ostride = out.shape[0], _ptr(out), out.stride(0)
    else:
        n_rows, optr, ostride = resid.shape[0], None, 0
        s = None
    yptr = pptr = zptr = None
    ystride = sstride = zstride = nsplit = 0
    if gw is not None:
        if isinstance(gw.y, Partials):
            _need(gw.y.t, torch.float32, "partials", contiguous=False)
            if gw.y.t.shape[-1] != w or gw.y.t.stride(1) != w or gw.y.t.stride(2) != 1:
                raise ValueError("norm_step: partials must be [S, M, W] with dense rows")
            pptr, nsplit, sstride = _ptr(gw.y.t), gw.y.nsplit, gw.y.split_stride
        else:
            _need(gw.y, None, "pending result", contiguous=False)
            if gw.y.dim() != 2 or gw.y.stride(1) != 1 or gw.y.shape[1] != w:
                raise ValueError("norm_step: the pending result must be [N, W] with unit inner stride")
            if s is not None and _suffix(gw.y.dtype) != s:
                raise TypeError("norm_step: the pending result and out must have the storage type")
            s = _suffix(gw.y.dtype)
            yptr, ystride = _ptr(gw.y), gw.y.stride(0)
        if gw.z is not None:
            _need(gw.z, None, "gate logits", contiguous=False)
            if gw.z.dim() != 2 or gw.z.stride(1) != 1 or gw.z.shape[1] != w:
                raise ValueError("norm_step: gate logits must be [N, W] with unit inner stride")
            if s is not None and _suffix(gw.z.dtype) != s:
                raise TypeError("norm_step: gate logits must have the storage type")
            s = _suffix(gw.z.dtype)
            zptr, zstride = _ptr(gw.z), gw.z.stride(0)
        for t, what in ((gw.z_bias, "gate bias"), (gw.post_w, "post-norm weight")):
            if t is not None:
                _need(t, torch.float32, what)
                if t.numel() != w:
                    raise ValueError(f"norm_step: {what} must have W entries")
    if next_w is not None:
        _need(next_w, torch.float32, "norm weight")
        if next_w.numel() != w:
            raise ValueError("norm_step: norm weight must have W entries")
    if rows is not None:
        _need(rows, torch.int32, "rows")
        if rows.numel() < n_rows:
            raise ValueError("norm_step: fewer row indices than output rows")
    elif resid.shape[0] < n_rows:
        raise ValueError("norm_step: fewer residual rows than output rows")
    name = f"kvf_norm_step_{s or 'f32'}"
    _check(
        _fn(name, GATED_LIB)(
            _ptr(resid), _ptr(rows), yptr, pptr, ystride, sstride, nsplit, zptr, zstride,
            _ptr(gw.z_bias) if gw else None, _ptr(gw.post_w) if gw else None, _ptr(next_w), optr, ostride,
            n_rows, w, 1 if centred else 0, 1 if store_normed else 0, float(eps), _stream(),
        ),
        name,
    )  # fmt: skip


def qk_prepare(
    x: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor, norm_eps: float | None, slots: torch.Tensor,
    kcache: torch.Tensor, vcache: torch.Tensor, nh: int, nkv: int, d: int, dv: int, k_off: int, v_off: int, v_step: int,
    block_size: int, err: torch.Tensor | None = None,
) -> None:  # fmt: skip
    """Rows of ``x`` hold ``nh`` query heads of ``d`` from column 0, ``nkv`` key heads from column ``k_off`` and
    the value heads' sources from column ``v_off`` (``v_step`` apart, the first ``dv`` numbers of each).  The
    values go to their slots as they are.  The first ``2 * len(inv_freq)`` dims of every query and key head turn
    in split pairs ``(i, i + rot/2)`` by ``pos * inv_freq[i]``; then, unless ``norm_eps`` is ``None``, the head is
    divided by ``sqrt(mean(x^2) + norm_eps)``.  Queries are written back in place, keys to their slots."""
    s = _suffix(x.dtype)
    _rows2d(x, None, "x")
    _need(positions, torch.int32, "positions")
    _need(inv_freq, torch.float32, "inv_freq")
    _need(slots, torch.int32, "slots")
    _need(kcache, x.dtype, "kcache")
    _need(vcache, x.dtype, "vcache")
    n = x.shape[0]
    rot = 2 * inv_freq.numel()
    if rot > d or tuple(kcache.shape[1:]) != (nkv, block_size, d) or tuple(vcache.shape[1:]) != (nkv, block_size, dv) or kcache.shape[0] != vcache.shape[0]:
        raise ValueError("qk_prepare: cache shapes must be [blocks, nkv, block_size, d] and [..., dv], and rot <= d")
    if k_off < nh * d or k_off + nkv * d > x.shape[1] or v_off + (nkv - 1) * v_step + dv > x.shape[1] or positions.numel() < n or slots.numel() < n:
        raise ValueError("qk_prepare: the rows do not hold what the offsets say")
    name = f"kvf_qk_prepare_{s}"
    _check(
        _fn(name, GATED_LIB)(
            _ptr(x), x.stride(0), int(k_off), int(v_off), int(v_step), _ptr(positions), _ptr(inv_freq), rot, 0 if norm_eps is None else 1,
            float(norm_eps or 0.0), _ptr(slots), _ptr(kcache), _ptr(vcache), n, nh, nkv, d, dv, block_size, kcache.shape[0] * block_size,
            _ptr(err), _stream(),
        ),
        name,
    )  # fmt: skip


UNARY_ACTIVATIONS = {"xielu": 0, "relu2": 1, "gelu_tanh": 2}


def unary_act(x: torch.Tensor, out: torch.Tensor, kind: str, ab: torch.Tensor | None = None) -> None:
    """``out = act(x)`` row by row in float, rounded once.  ``xielu`` with the two numbers ``ab = (p, q)``:
    ``z > 0: softplus(p) z^2 + z/2``, ``z <= 0: (1/2 + softplus(q)) (exp(z) - 1 - z) + z/2``; ``relu2``:
    ``relu(z)^2``; ``gelu_tanh``: ``0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)))``."""
    s = _suffix(x.dtype)
    _rows2d(x, None, "x")
    _rows2d(out, x.dtype, "out")
    if kind not in UNARY_ACTIVATIONS or out.shape != x.shape:
        raise ValueError("unary_act: unknown activation or shapes differ")
    if kind == "xielu":
        _need(ab, torch.float32, "xielu parameters")
        if ab.numel() != 2:
            raise ValueError("unary_act: xielu takes two numbers")
    name = f"kvf_unary_act_{s}"
    _check(_fn(name, GATED_LIB)(_ptr(x), x.stride(0), _ptr(out), out.stride(0), x.shape[0], x.shape[1], UNARY_ACTIVATIONS[kind], _ptr(ab), _stream()), name)


def scale_softcap(logits: torch.Tensor, scale: float, cap: float) -> None:
    """``logits <- cap * tanh(scale * logits / cap)`` in place (``cap == 0``: ``scale * logits``)."""
    _need(logits, torch.float32, "logits")
    name = "kvf_scale_softcap_f32"
    _check(_fn(name)(_ptr(logits), logits.numel(), float(scale), float(cap), _stream()), name)


TALKING_MAX_HEADS = 64  # what the kernel's CTA of eight warps holds: a row per (head, query), eight rows a warp
TALKING_MAX_HEAD_DIM = 256  # any size up to here: sizes that are no multiple of a 16-byte load go number by number
TALKING_MMA_RANGE_STEP = 32  # keys per tile of the tensor-core form's key ranges

_talking_mma_known: dict[tuple, bool] = {}


def talking_mma_supported(dtype: torch.dtype, nh: int, nkv: int, d: int, dv: int, decode_form: bool, talk: bool = True) -> bool:
    """Whether the tensor-core form of ``talking_attention`` takes this shape: bfloat16 storage, heads of 64 or 128
    with values as wide as keys, and head counts whose rows and tiles fit a CTA (the library decides)."""
    if dtype != torch.bfloat16 or d != dv or d not in (64, 128):
        return False
    key = (nh, nkv, d, bool(decode_form), bool(talk))
    if key not in _talking_mma_known:
        _talking_mma_known[key] = bool(_fn("kvf_talking_mma_ok", GATED_LIB)(nh, nkv, d, dv, 1 if decode_form else 0, 1 if talk else 0))
    return _talking_mma_known[key]


def talking_attention(
    q: torch.Tensor, out: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, block_tables: torch.Tensor,
    query_start_loc: torch.Tensor, context_lens: torch.Tensor, num_seqs: int, max_query_len: int, nh: int, nkv: int, d: int, dv: int,
    scale: float, talk: torch.Tensor | None, sink: torch.Tensor | None, q_stride: int | None = None, window: int = 0,
    scratch: tuple | None = None, max_context: int | None = None, split_size: int = 256,
) -> None:  # fmt: skip
    """Causal attention over the paged cache whose heads' scores are mixed before the softmax
    (``s'_h = sum_g talk[h, g] s_g``, ``talk`` float ``[nh, nh]`` or ``None``) and whose softmax may have a sink
    (``sink`` float ``[nh]``: ``exp(sink_h)`` joins the denominator, with no key and no value).  ``q`` rows hold
    ``nh`` heads of ``d`` (row stride ``q_stride``), ``out [N, nh * dv]``; ``scratch``: the decode form (every
    sequence one query; key ranges of ``split_size`` in parallel, then a merge) with ``(part_acc, part_ml, _)``
    as ``attention_scratch_shapes`` gives them."""
    s = _suffix(q.dtype)
    _need(q, None, "q", contiguous=False)
    _need(out, q.dtype, "out")
    _need(kcache, q.dtype, "kcache")
    _need(vcache, q.dtype, "vcache")
    for t, what in ((block_tables, "block_tables"), (query_start_loc, "query_start_loc"), (context_lens, "context_lens")):
        _need(t, torch.int32, what)
    block_size = kcache.shape[2]
    if tuple(kcache.shape[1:]) != (nkv, block_size, d) or tuple(vcache.shape[1:]) != (nkv, block_size, dv) or out.shape[1] != nh * dv:
        raise ValueError("talking_attention: cache or output shape")
    if nh > TALKING_MAX_HEADS:
        raise ValueError(f"talking_attention: at most {TALKING_MAX_HEADS} heads")
    for t, shape, what in ((talk, (nh, nh), "talk"), (sink, (nh,), "sink")):
        if t is not None:
            _need(t, torch.float32, what)
            if tuple(t.shape) != shape:
                raise ValueError(f"talking_attention: {what} must be {shape}")
    acc = ml = None
    split = max_splits = grid_splits = 0
    if scratch is not None:
        acc, ml = scratch[0], scratch[1]
        split = int(split_size)
        max_splits = acc.shape[2]
        bound = max(int(max_context or 0), 1)
        grid_splits = min(max_splits, -(-bound // split))
        if acc.shape[0] < num_seqs or acc.shape[1] != nh or acc.shape[3] != dv or -(-bound // split) > max_splits:
            raise ValueError("talking_attention: scratch too small for this step")
    name = f"kvf_talking_attention_{s}"
    if talking_mma_supported(q.dtype, nh, nkv, d, dv, scratch is not None, talk is not None) and (scratch is None or split % TALKING_MMA_RANGE_STEP == 0):
        name = "kvf_talking_attention_mma_bf16"  # the two products on the tensor cores; mixing, softmax and sink in float
    _check(
        _fn(name, GATED_LIB)(
            _ptr(q), _ptr(out), _ptr(kcache), _ptr(vcache), _ptr(block_tables), _ptr(query_start_loc), _ptr(context_lens), _ptr(talk), _ptr(sink),
            int(num_seqs), int(max_query_len), int(q_stride or q.stride(0)), out.stride(0), block_tables.stride(0), nh, nkv, d, dv, block_size,
            float(scale), int(window), split, max_splits, grid_splits, _ptr(acc), _ptr(ml), _stream(),
        ),
        name,
        2 if scratch is not None else 1,
    )  # fmt: skip


# ------------------------------------------------------------------ library "decay"
# a norm without statistics, and a recurrent mixer with one fixed decay a head

DECAY_LIB = "decay"


@dataclass
class Scaled:
    """A sublayer's result that joins the residual stream multiplied by ``mult``: ``what`` is a tensor in the
    storage type, ``Partials`` or ``None``; the norm that follows adds ``mult * what`` in 32-bit."""

    what: object
    mult: float


def tanh_norm(
    resid: torch.Tensor, delta: torch.Tensor | Partials | Scaled | None, alpha: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor,
    out: torch.Tensor | None, rows: torch.Tensor | None = None,
) -> None:  # fmt: skip
    """``v = resid + mult * delta`` (written back into ``resid`` unless ``rows`` is given), ``out = T(tanh(alpha * v) *
    weight + bias)``: a norm that computes no mean and no variance.  ``alpha`` is a float scalar on the device,
    ``weight`` and ``bias`` float ``[H]``.  ``delta``: a tensor in the storage type, the ``Partials`` of a split product, or
    either inside ``Scaled`` (``mult`` is 1 otherwise).  With ``rows`` (int32 ``[R]``) row ``r`` of ``out`` comes from row
    ``rows[r]``.  ``out=None``: only the sum is made."""
    _need(resid, torch.float32, "resid")
    for t, what in ((alpha, "alpha"), (weight, "norm weight"), (bias, "norm bias")):
        _need(t, torch.float32, what)
    h = resid.shape[-1]
    if alpha.numel() != 1 or weight.numel() != h or bias.numel() != h:
        raise ValueError("tanh_norm: alpha is one number, weight and bias are as wide as the stream")
    mult = 1.0
    if isinstance(delta, Scaled):
        delta, mult = delta.what, float(delta.mult)
    if delta is ADDED:
        delta = None
    dptr, pptr, nsplit, stride = None, None, 0, 0
    dtype = out.dtype if out is not None else None
    if isinstance(delta, Partials):
        _need(delta.t, torch.float32, "partials", contiguous=False)
        if delta.t.shape[-1] != h or delta.t.stride(1) != h or delta.t.stride(2) != 1:
            raise ValueError("tanh_norm: partials must be [S, M, H] with dense rows")
        pptr, nsplit, stride = _ptr(delta.t), delta.nsplit, delta.split_stride
    elif delta is not None:
        _need(delta, dtype, "delta")
        if delta.shape[-1] != h:
            raise ValueError("tanh_norm: delta width")
        dptr = _ptr(delta)
        dtype = delta.dtype
    if dtype is None:
        dtype = torch.float32  # nothing in the storage type is read or written
    s = _suffix(dtype)
    if out is not None:
        _need(out, None, "out")
        if out.shape[-1] != h:
            raise ValueError("tanh_norm: widths do not agree")
    n_rows = out.shape[0] if out is not None else (delta.t.shape[1] if isinstance(delta, Partials) else delta.shape[0] if delta is not None else 0)
    if rows is not None:
        _need(rows, torch.int32, "rows")
        if rows.numel() < n_rows:
            raise ValueError("tanh_norm: fewer row indices than output rows")
    elif resid.shape[0] < n_rows:
        raise ValueError("tanh_norm: fewer residual rows than output rows")
    name = f"kvf_tanh_norm_{s}"
    _check(
        _fn(name, DECAY_LIB)(_ptr(resid), dptr, pptr, nsplit, stride, mult, _ptr(alpha), _ptr(weight), _ptr(bias), _ptr(out), _ptr(rows), n_rows, h, _stream()),
        name,
    )


RETENTION_MAX_KEY_DIM = 512  # rows of a head's state that the walk holds in the registers of 32 lanes


def retention(
    x: torch.Tensor, q_off: int, k_off: int, v_off: int, positions: torch.Tensor, inv_freq: torch.Tensor | None, interleaved: bool,
    k_scale: float, decay: torch.Tensor, state: torch.Tensor, out: torch.Tensor, qsl: torch.Tensor, state_slots: torch.Tensor,
    num_seqs: int, num_heads: int, dk: int, dv: int, scratch: tuple[torch.Tensor, torch.Tensor, torch.Tensor] | None = None,
    max_query_len: int = 0,
) -> None:  # fmt: skip
    """Retention over a flat batch, token by token per sequence, on the float state ``S [heads, dk, dv]`` of each
    sequence's slot: ``S <- decay[h] S + k v^T``, ``out = S^T q`` (float ``[N, H*dv]``).  Rows of ``x`` hold the
    projections: ``H`` query heads of ``dk`` from column ``q_off``, key heads from ``k_off``, value heads of ``dv`` from
    ``v_off``.  The first ``2*len(inv_freq)`` dims of q and k turn with the position (split pairs ``(i, i + rot/2)``
    unless ``interleaved``), then k is multiplied by ``k_scale``; all of that in float.  ``scratch``: float buffers
    ``(qn [N, H*dk], kn [N, H*dk], vn [N, H*dv])``; without it they are allocated here.  ``max_query_len`` (0 = unknown):
    the most rows a sequence of the step brings (a step of single tokens stages less).  Two launches."""
    s = _suffix(x.dtype)
    _rows2d(x, None, "x")
    n = x.shape[0]
    h = int(num_heads)
    if not 0 < dk <= RETENTION_MAX_KEY_DIM or dv <= 0:
        raise ValueError(f"retention: key heads of 1 to {RETENTION_MAX_KEY_DIM} numbers")
    if max(q_off, k_off) + h * dk > x.shape[1] or v_off + h * dv > x.shape[1]:
        raise ValueError("retention: the columns do not fit the rows")
    _need(positions, torch.int32, "positions")
    _need(decay, torch.float32, "decay")
    if decay.numel() != h:
        raise ValueError("retention: one decay per head")
    rot = 0
    if inv_freq is not None and inv_freq.numel():
        _need(inv_freq, torch.float32, "inv_freq")
        rot = 2 * inv_freq.numel()
        if rot > dk:
            raise ValueError("retention: more frequencies than dk/2")
    _rows2d(out, torch.float32, "out")
    if tuple(out.shape) != (n, h * dv):
        raise ValueError("retention: out must be float [N, H*dv]")
    sptr, sstride = _state_view(state, h * dk * dv, "retention state")
    _need(qsl, torch.int32, "query_start_loc")
    _need(state_slots, torch.int32, "state_slots")
    if scratch is None:
        mk = lambda w: torch.empty((n, w), dtype=torch.float32, device=x.device)  # noqa: E731
        scratch = (mk(h * dk), mk(h * dk), mk(h * dv))
    qn, kn, vn = scratch
    for t, w, what in ((qn, h * dk, "qn"), (kn, h * dk, "kn"), (vn, h * dv, "vn")):
        _need(t, torch.float32, f"scratch {what}")
        if tuple(t.shape) != (n, w):
            raise ValueError(f"retention: scratch {what} must be float [{n}, {w}]")
    name = f"kvf_retention_{s}"
    _check(
        _fn(name, DECAY_LIB)(
            _ptr(x), x.stride(0), int(q_off), int(k_off), int(v_off), _ptr(positions), _ptr(inv_freq) if rot else None, rot,
            0 if interleaved else 1, float(k_scale), _ptr(decay), sptr, sstride, _ptr(out), out.stride(0), _ptr(qsl), _ptr(state_slots),
            int(num_seqs), n, h, int(dk), int(dv), _ptr(qn), _ptr(kn), _ptr(vn), int(max_query_len), _stream(),
        ),
        name,
        2,
    )  # fmt: skip


def retention_gate(o: torch.Tensor, gate: torch.Tensor | None, eps: float, out: torch.Tensor, num_heads: int, dv: int, activation: str | None = "silu") -> None:
    """``out[n, h, :] = o / sqrt(mean(o^2) + eps) * act(gate)`` per token and head (a unit norm without a weight); ``o``
    float ``[N, H*dv]``, ``gate`` and ``out`` in the storage type (column ranges of wider rows are fine), ``activation``:
    ``"silu"``, ``"sigmoid"`` or ``None`` (no gate)."""
    s = _suffix(out.dtype)
    _rows2d(o, torch.float32, "o")
    _rows2d(out, None, "out")
    n = o.shape[0]
    if o.shape[1] != num_heads * dv or tuple(out.shape) != (n, num_heads * dv):
        raise ValueError("retention_gate: shapes do not agree")
    act = {None: 0, "silu": 1, "sigmoid": 2}.get(activation, -1)
    if act < 0:
        raise ValueError("retention_gate: activation must be 'silu', 'sigmoid' or None")
    gptr, gstride = None, 0
    if act:
        _rows2d(gate, out.dtype, "gate")
        if tuple(gate.shape) != (n, num_heads * dv):
            raise ValueError("retention_gate: gate shape")
        gptr, gstride = _ptr(gate), gate.stride(0)
    name = f"kvf_retention_gate_{s}"
    _check(_fn(name, DECAY_LIB)(_ptr(o), o.stride(0), gptr, gstride, float(eps), act, n, num_heads, dv, _ptr(out), out.stride(0), _stream()), name)
