"""Tensor-level wrappers of the CUDA kernels.

Each function checks devices, dtypes, shapes and strides on the host, then launches on
the current CUDA stream.  Tensors that are not on a CUDA device are refused: there is no
CPU path.  Parts call these functions through the module (``ops.add_rmsnorm(...)``).
"""
from __future__ import annotations

import ctypes

import torch

from ..errors import KernelError
from . import attention_fast, gemm_skinny, gemm_tc
from . import library as _library

PAGE = 64                      # tokens per cache page (DL_PAGE in csrc/common.cuh)
_P, _I, _F = _library._P, _library._I, _library._F
_library.register_signatures({
    "dl_embed_positions": [_P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _P],
    "dl_branch_norm_add": [_P, _P, _I, _I, _P, _F, _P, _P, _P, _I, _I, _I, _F, _P],
    "dl_add_rows": [_P, _P, _I, _I, _P],
    "dl_gated_activation": [_P, _P, _I, _P, _I, _I, _I, _I, _F, _F, _P],
    "dl_gla_scan": [_P, _P, _P, _I, _P, _I, _P, _I, _P, _P, _P, _I, _P, _I, _I, _I, _I, _I, _I, _F, _F, _P],
    "dl_head_norm_gate": [_P, _I, _P, _I, _P, _P, _I, _I, _I, _I, _I, _F, _I, _P],
    "dl_route_topk": [_P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P, _I, _F, _P],
    "dl_head_rmsnorm": [_P, _I, _P, _I, _I, _P, _P, _I, _I, _I, _I, _F, _P],
    "dl_delta_rule": [_P, _I, _P, _I, _I, _P, _I, _P, _I, _P, _P, _P, _P, _P, _P, _P, ctypes.c_long, _I,
                      _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _F, _F, _I, _P],
    "dl_expert_gate_up": [_P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _F, _F, _P, _P],
    "dl_expert_down": [_P, _P, _P, _P, _P, _I, _P, _I, _I, _I, _I, _I, _I, _P, _I, _P, _I, _I, _P],
    "dl_expert_sort": [_P, _I, _I, _P, _P, _I, _P],
    "dl_expert_gather": [_P, _I, _P, _P, _I, _I, _I, _P, _P],
    "dl_expert_combine": [_P, _I, _P, _P, _P, _I, _P, _I, _I, _I, _P, _I, _P, _P, _I, _I, _I, _P],
    "dl_stream_norm": [_P, _P, _I, _I, _P, _P, _P, _P, _P, _P, _P, _I, _P, _I, _I, _I, _F, _I, _P],
    "dl_stream_copies": [_P, _P, _I, _I, _I, _F, _P],
    "dl_embed_copies": [_P, _I, _I, _P, _P, _I, _I, _I, _I, _F, _P],
    "dl_group_rmsnorm": [_P, _I, _P, _I, _I, _P, _I, _I, _I, _F, _P],
    "dl_pair_norm_sum": [_P, _P, _P, _P, _P, _I, _I, _F, _F, _F, _P],
    "dl_scale_values": [_P, ctypes.c_longlong, _F, _P],
    "dl_unary_activation": [_P, _I, _P, _I, _I, _I, _I, _P],
    "dl_softcap": [_P, ctypes.c_longlong, _F, _P],
    "dl_head_gate": [_P, _I, _P, _I, _I, _I, _I, _I, _P],
    "dl_gemm_tc_grouped_bf16": [_P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _P, _I, _I, _F, _F, _I, _P, _P],
})
_DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1}


def _code(dtype):
    try:
        return _DTYPE_CODE[dtype]
    except KeyError:
        raise KernelError(f"kernels take float32 or bfloat16, not {dtype}") from None


def _stream():
    return _library.current_stream()


def _need_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("kernels run on CUDA tensors only: there is no CPU fallback")
    _library.require_device()


def _ptr(t):
    return None if t is None else t.data_ptr()


def _rows_view(t, what):
    """A 2-D tensor whose rows are contiguous (a column slice of a wider matrix is fine)."""
    if t.dim() != 2 or (t.shape[1] > 1 and t.stride(1) != 1):
        raise KernelError(f"{what}: need a 2-D tensor with contiguous rows, got shape "
                          f"{tuple(t.shape)} strides {t.stride()}")
    return t.stride(0) if t.shape[0] > 1 else max(t.stride(0), t.shape[1])


def _int32(t, what):
    if t.dtype != torch.int32 or not t.is_contiguous():
        raise KernelError(f"{what}: need a contiguous int32 tensor")
    return t


# ------------------------------------------------------------------ embedding
def gather_rows(table, ids, out=None, out_dtype=torch.float32):
    """out[r] = table[ids[r]] as ``out_dtype``.  table [n, width] float32 or bfloat16 (rows contiguous,
    possibly with gaps between them); ids int32 [R]; float32 out, or bfloat16 from a bfloat16 table."""
    _need_cuda(table, ids, out)
    stride = _rows_view(table, "gather_rows table")
    _int32(ids, "gather_rows ids")
    n, width = table.shape
    rows = ids.numel()
    if out is None:
        out = torch.empty((rows, width), dtype=out_dtype, device=table.device)
    elif out.shape != (rows, width) or out.dtype != out_dtype or not out.is_contiguous():
        raise KernelError(f"gather_rows: out must be contiguous {out_dtype} [rows, width]")
    if out_dtype != torch.float32 and out_dtype != table.dtype:
        raise KernelError(f"gather_rows: rows of {table.dtype} are gathered as float32 or as they are, not as {out_dtype}")
    _library.call("dl_gather_rows", _ptr(table), _code(table.dtype), stride, _ptr(ids), _ptr(out), _code(out_dtype),
                  rows, width, n, _stream())
    return out


def embed_positions(table, pos_table, ids, positions):
    """out[r] = table[ids[r]] + pos_table[positions[r]] in float32.  Both tables [n, width] contiguous
    and of one dtype; ids, positions int32 [R]."""
    _need_cuda(table, pos_table, ids, positions)
    if table.dim() != 2 or pos_table.dim() != 2 or table.shape[1] != pos_table.shape[1] or table.dtype != pos_table.dtype \
            or not table.is_contiguous() or not pos_table.is_contiguous():
        raise KernelError("embed_positions: need two contiguous tables of one dtype and one width")
    _int32(ids, "embed_positions ids")
    _int32(positions, "embed_positions positions")
    rows = ids.numel()
    if positions.numel() != rows:
        raise KernelError("embed_positions: one position per id")
    out = torch.empty((rows, table.shape[1]), dtype=torch.float32, device=table.device)
    _library.call("dl_embed_positions", _ptr(table), _ptr(pos_table), _code(table.dtype), _ptr(ids), _ptr(positions),
                  _ptr(out), rows, table.shape[1], table.shape[0], pos_table.shape[0], _stream())
    return out


# ------------------------------------------------- products not yet launched
class PendingProduct:
    """x W^T (float32 result of bfloat16 operands) that ``linear(..., lazy=True)`` has not launched
    yet.  Given to ``add_rmsnorm`` as the delta, the product itself adds its result into the stream
    (the decode kernels in their epilogue, the library product as its accumulate operand); anyone
    else calls ``tensor()`` (or ``resolve``) and gets the plain float32 product."""

    def __init__(self, x, w, resident):
        self.x, self.w, self.resident = x, w, resident
        self.shape = (x.shape[0], w.shape[0])

    def tensor(self):
        return linear(self.x, self.w, out_dtype=torch.float32, resident=self.resident)

    def add_into(self, residual):
        """residual += x W^T by the library product with the stream as its accumulate operand (one
        rounding of accumulator + stream, as the separate addition has; no [T, N] product is
        written and read back).  False when the sizes belong to the decode kernels or the
        tensors do not fit; nothing has happened then."""
        x = self.x
        if isinstance(x, ScaledRows) or x.dtype != torch.bfloat16 or not x.is_cuda or x.dim() != 2 \
                or residual.dtype != torch.float32 or not residual.is_contiguous() \
                or tuple(residual.shape) != self.shape or gemm_skinny.takes(x, self.w):
            return False
        torch.addmm(residual, x, self.w.t(), out_dtype=torch.float32, out=residual)
        return True


class ScaledRows:
    """A normalised stream still lacking its factor per row: ``data`` = stream * gain (bfloat16) and the
    sums of squares per part of 16 (the mma.sync product's) or 128 columns (the tcgen05 product's), left by the product that added into the stream.  ``linear``
    and ``gated_linear`` take it as x and apply rsqrt(mean + eps) to their output rows - the product
    of the normalised rows, since the factor is one number per row.  ``tensor()`` gives the
    normalised rows themselves (valid until the stream is added to again)."""

    def __init__(self, data, sums, width, eps, stream, gain):
        self.data, self.sums, self.width, self.eps = data, sums, width, eps
        self.stream, self.gain = stream, gain
        self.shape, self.dtype = data.shape, data.dtype

    def row_sums(self):
        return self.sums, self.sums.numel() // gemm_skinny.sum_stride(self.data.shape[0]), self.width, self.eps

    def tensor(self):
        return add_rmsnorm(self.stream, None, self.gain, self.eps, self.data.dtype)


class NormedBranch:
    """A branch output that joins the stream only after a norm of its own: ``data`` [T, H] (float32 or
    bfloat16, or a product not yet launched) is divided by its rows' root mean square (``eps`` inside
    the root) and multiplied by ``gain`` before the addition.  ``extra`` (float32 [T, H] or None) is
    added to the stream as it is at the same time.  ``add_rmsnorm`` takes it as the delta and does
    norm, addition and the next norm in one kernel."""

    def __init__(self, data, gain, eps, extra=None):
        self.data, self.gain, self.eps, self.extra = data, gain, float(eps), extra
        self.shape = tuple(data.shape)

    def with_extra(self, extra):
        if self.extra is not None:
            raise KernelError("a normed branch takes one extra addend")
        return NormedBranch(self.data, self.gain, self.eps, extra)

    def tensor(self):
        """The normalised branch (and the extra addend) as one float32 tensor."""
        out = torch.zeros(self.shape, dtype=torch.float32, device=self.gain.device)
        add_normed_branch(out, self)
        return out


def resolve(value):
    """The tensor behind a PendingProduct, ScaledRows or NormedBranch; tensors and None pass through."""
    return value.tensor() if isinstance(value, (PendingProduct, ScaledRows, NormedBranch)) else value


def narrow_rows(value, ids):
    """The rows ``ids`` (int32 on the device) of a branch output, in its own dtype.  Of a product not
    yet launched only those rows of x are kept, so that the product is computed for them alone."""
    if value is None:
        return None
    if isinstance(value, PendingProduct):
        x = resolve(value.x)
        return PendingProduct(gather_rows(x, ids, out_dtype=x.dtype), value.w, value.resident)
    if isinstance(value, StreamWrite):
        return value.narrowed(ids)
    if isinstance(value, NormedBranch):
        return NormedBranch(narrow_rows(value.data, ids), value.gain, value.eps,
                            None if value.extra is None else gather_rows(value.extra, ids))
    value = resolve(value)
    return gather_rows(value, ids, out_dtype=value.dtype)


# ----------------------------------------------------------------------- norm
def add_rmsnorm(residual, delta, gain, eps, out_dtype, lazy=False):
    """residual += delta (when delta is given), then rmsnorm(residual) * gain in ``out_dtype``.

    residual: float32 [T, H] contiguous, updated in place.  delta: [T, H] float32/bfloat16, a
    PendingProduct, or None.  gain: float32 [H].  ``lazy``: the caller will hand the result straight
    to ``linear`` / ``gated_linear``, so it may be a ScaledRows: a pending product then does the
    addition itself and the next product the normalisation, with no kernel in between."""
    if isinstance(delta, NormedBranch):
        return add_normed_branch(residual, delta, gain, eps, out_dtype)
    if isinstance(delta, PendingProduct):
        fused = _add_product_scaled(residual, delta, gain, eps, out_dtype) if lazy else None
        if fused is not None:
            return fused
        delta = None if delta.add_into(residual) else delta.tensor()
    _need_cuda(residual, delta, gain)
    if residual.dtype != torch.float32 or residual.dim() != 2 or not residual.is_contiguous():
        raise KernelError("rmsnorm: the residual stream must be contiguous float32 [T, H]")
    rows, width = residual.shape
    if gain.dtype != torch.float32 or gain.shape != (width,) or not gain.is_contiguous():
        raise KernelError(f"rmsnorm: gain must be float32 [{width}]")
    if delta is not None and (delta.shape != residual.shape or not delta.is_contiguous()):
        raise KernelError("rmsnorm: delta must be contiguous with the residual's shape")
    out = torch.empty((rows, width), dtype=out_dtype, device=residual.device)
    _library.call("dl_add_rmsnorm", _ptr(residual), _ptr(delta),
                  _code(delta.dtype) if delta is not None else 0, _ptr(gain), _ptr(out),
                  _code(out_dtype), rows, width, float(eps), _stream())
    return out


def add_normed_branch(residual, branch, gain=None, eps=0.0, out_dtype=None):
    """residual += rmsnorm(branch.data) * branch.gain (+ branch.extra), in place; with ``gain`` also returns
    rmsnorm(residual) * gain in ``out_dtype`` (one kernel), else None."""
    data = resolve(branch.data)
    _need_cuda(residual, data, branch.gain, branch.extra, gain)
    if residual.dtype != torch.float32 or residual.dim() != 2 or not residual.is_contiguous():
        raise KernelError("normed branch: the residual stream must be contiguous float32 [T, H]")
    rows, width = residual.shape
    stride = _rows_view(data, "normed branch")
    if tuple(data.shape) != (rows, width):
        raise KernelError(f"normed branch: a branch of shape {tuple(data.shape)} does not fit a stream of {(rows, width)}")
    for g in (branch.gain, gain):
        if g is not None and (g.dtype != torch.float32 or g.shape != (width,) or not g.is_contiguous()):
            raise KernelError(f"normed branch: gains must be float32 [{width}]")
    extra = branch.extra
    if extra is not None and (extra.dtype != torch.float32 or tuple(extra.shape) != (rows, width) or not extra.is_contiguous()):
        raise KernelError("normed branch: the extra addend must be contiguous float32 with the stream's shape")
    out = torch.empty((rows, width), dtype=out_dtype, device=residual.device) if gain is not None else None
    _library.call("dl_branch_norm_add", _ptr(residual), _ptr(data), _code(data.dtype), stride, _ptr(branch.gain),
                  branch.eps, _ptr(extra), _ptr(gain), _ptr(out), _code(out_dtype) if out is not None else 0, rows, width,
                  float(eps), _stream())
    return out


def add_rows(residual, other):
    """residual += other, both contiguous float32 of one shape, in place."""
    _need_cuda(residual, other)
    if residual.dtype != torch.float32 or other.dtype != torch.float32 or residual.shape != other.shape \
            or residual.dim() != 2 or not residual.is_contiguous() or not other.is_contiguous():
        raise KernelError("add_rows: need two contiguous float32 tensors of one shape")
    _library.call("dl_add_rows", _ptr(residual), _ptr(other), residual.shape[0], residual.shape[1], _stream())
    return residual


STREAM_NORMS = {"layernorm": 0, "rmsnorm": 1}


class StreamWrite:
    """A sublayer's output that has not joined a stream of copies yet: ``data`` [T, H] (a tensor or a product not yet
    launched) is multiplied by ``scale`` (float32 [H] or None) and enters copy t with weight ``out[t]``, while the old
    copies are mixed by ``mix`` [copies, copies] (from, to).  ``stream_norm`` takes it as its delta."""

    def __init__(self, data, scale, mix, out):
        self.data, self.scale, self.mix, self.out = data, scale, mix, out
        self.shape = tuple(data.shape)

    def narrowed(self, ids):
        return StreamWrite(narrow_rows(self.data, ids), self.scale, self.mix, self.out)


def stream_norm(x, copies, write, read, gain, bias, eps, out_dtype, kind="layernorm", summed=False):
    """One pass over a stream of ``copies`` copies, x float32 [T, copies * H] (updated in place): the ``write`` of the sublayer
    that ran last (a ``StreamWrite`` or None), then u = sum_s read[s] x_s (``read`` float32 [copies], None: every copy
    once) and its norm (``kind`` "layernorm": (u - mean) / sqrt(var + eps) * gain + bias; "rmsnorm": u / sqrt(mean u^2 + eps)
    * gain) in ``out_dtype``.  ``gain`` None: no norm.  ``summed``: also return u itself in float32.  Returns the normed rows,
    or (normed, u) with ``summed``."""
    if kind not in STREAM_NORMS:
        raise KernelError(f"stream_norm: unknown norm {kind!r}; known: {sorted(STREAM_NORMS)}")
    y = scale = mix = outw = None
    if write is not None:
        y, scale, mix, outw = resolve(write.data), write.scale, write.mix, write.out
    _need_cuda(x, y, scale, mix, outw, read, gain, bias)
    S = int(copies)
    if x.dtype != torch.float32 or x.dim() != 2 or not x.is_contiguous() or x.shape[1] % S:
        raise KernelError("stream_norm: the stream must be contiguous float32 [T, copies * H]")
    T, H = x.shape[0], x.shape[1] // S
    for t, shape, what in ((scale, (H,), "scale"), (mix, (S, S), "mix"), (outw, (S,), "out"), (read, (S,), "read"), (gain, (H,), "gain"),
                           (bias, (H,), "bias")):
        if t is not None and (t.dtype != torch.float32 or tuple(t.shape) != shape or not t.is_contiguous()):
            raise KernelError(f"stream_norm: {what} must be contiguous float32 {list(shape)}")
    ys = 0
    if y is not None:
        ys = _rows_view(y, "stream_norm y")
        if tuple(y.shape) != (T, H):
            raise KernelError(f"stream_norm: a sublayer's output of shape {tuple(y.shape)} does not fit a stream of {(T, H)}")
    normed = torch.empty((T, H), dtype=out_dtype, device=x.device) if gain is not None else None
    u = torch.empty((T, H), dtype=torch.float32, device=x.device) if summed else None
    _library.call("dl_stream_norm", _ptr(x), _ptr(y), _code(y.dtype) if y is not None else 0, ys, _ptr(scale), _ptr(mix), _ptr(outw),
                  _ptr(read), _ptr(gain), _ptr(bias), _ptr(normed), _code(out_dtype) if normed is not None else 0, _ptr(u), T, S, H,
                  float(eps), STREAM_NORMS[kind], _stream())
    return (normed, u) if summed else normed


def stream_copies(x, copies, factor=1.0):
    """x float32 [T, H] -> float32 [T, copies * H]: every copy is x * factor."""
    _need_cuda(x)
    if x.dtype != torch.float32 or x.dim() != 2 or not x.is_contiguous():
        raise KernelError("stream_copies: need contiguous float32 [T, H]")
    out = torch.empty((x.shape[0], int(copies) * x.shape[1]), dtype=torch.float32, device=x.device)
    _library.call("dl_stream_copies", _ptr(x), _ptr(out), x.shape[0], int(copies), x.shape[1], float(factor), _stream())
    return out


def embed_copies(table, ids, copies, factor=1.0):
    """out[r, s] = table[ids[r]] * factor for each of ``copies`` copies s: float32 [R, copies * width], the embedding as the
    start of a stream of copies.  table [n, width] float32 or bfloat16 (rows contiguous); ids int32 [R]."""
    _need_cuda(table, ids)
    stride = _rows_view(table, "embed_copies table")
    _int32(ids, "embed_copies ids")
    n, width = table.shape
    out = torch.empty((ids.numel(), int(copies) * width), dtype=torch.float32, device=table.device)
    _library.call("dl_embed_copies", _ptr(table), _code(table.dtype), stride, _ptr(ids), _ptr(out), ids.numel(), int(copies), width, n,
                  float(factor), _stream())
    return out


def group_rmsnorm(x, gain, width_a, width_b, eps):
    """Columns [0, width_a) of every row divided by their root mean square (eps inside the root) and multiplied by their
    gains, and the same for columns [width_a, width_a + width_b) on their own: queries and keys of a stacked projection,
    each normalised over all its heads at once.  gain float32 [width_a + width_b]; x may be a column view.  Returns a new
    tensor of x's dtype."""
    _need_cuda(x, gain)
    width = int(width_a) + int(width_b)
    if x.dim() != 2 or x.shape[1] != width or gain.dtype != torch.float32 or gain.shape != (width,) or not gain.is_contiguous():
        raise KernelError(f"group_rmsnorm: x [T, {width}] and a float32 gain per column")
    out = torch.empty((x.shape[0], width), dtype=x.dtype, device=x.device)
    _library.call("dl_group_rmsnorm", _ptr(x), _rows_view(x, "group_rmsnorm x"), _ptr(out), out.stride(0), _code(x.dtype), _ptr(gain),
                  x.shape[0], int(width_a), int(width_b), float(eps), _stream())
    return out


def pair_norm_sum(a, b, gain_a, gain_b, eps, weight_a=0.5, weight_b=0.5):
    """weight_a * rms(a) * gain_a + weight_b * rms(b) * gain_b per row, float32; a, b contiguous float32 [T, H]."""
    _need_cuda(a, b, gain_a, gain_b)
    if a.dtype != torch.float32 or b.dtype != torch.float32 or a.shape != b.shape or a.dim() != 2 or not a.is_contiguous() \
            or not b.is_contiguous():
        raise KernelError("pair_norm_sum: two contiguous float32 tensors of one shape")
    for g in (gain_a, gain_b):
        if g.dtype != torch.float32 or g.shape != (a.shape[1],) or not g.is_contiguous():
            raise KernelError(f"pair_norm_sum: gains must be contiguous float32 [{a.shape[1]}]")
    out = torch.empty_like(a)
    _library.call("dl_pair_norm_sum", _ptr(a), _ptr(b), _ptr(gain_a), _ptr(gain_b), _ptr(out), a.shape[0], a.shape[1], float(eps),
                  float(weight_a), float(weight_b), _stream())
    return out


def scale_values(values, factor):
    """values *= factor in place (contiguous float32)."""
    _need_cuda(values)
    if values.dtype != torch.float32 or not values.is_contiguous():
        raise KernelError("scale_values: need a contiguous float32 tensor")
    _library.call("dl_scale_values", _ptr(values), values.numel(), float(factor), _stream())
    return values


def _add_product_scaled(residual, product, gain, eps, out_dtype):
    x = product.x
    rows = x.row_sums() if isinstance(x, ScaledRows) else None
    xt = x.data if rows is not None else x
    if out_dtype != torch.bfloat16 or residual.dtype != torch.float32 or residual.dim() != 2 \
            or residual.stride(1) != 1 or tuple(residual.shape) != product.shape \
            or gain.dtype != torch.float32 or gain.shape != (residual.shape[1],) or not gain.is_contiguous() \
            or not gemm_skinny.takes(xt, product.w):
        return None
    _need_cuda(residual, xt, product.w, gain)
    scaled, sums = gemm_skinny.run(xt, product.w, torch.float32, resident=product.resident, row_sums=rows,
                                   into=(residual, gain))
    return ScaledRows(scaled, sums, residual.shape[1], eps, residual, gain)


# --------------------------------------------------- position + cache write
def rope_cache_write(q, k, v, cos, sin, rotary_dim, token_seq, token_pos, block_table,
                     k_pool, v_pool, n_heads, n_kv_heads, head_dim, write_cache=True, value_dim=None, biases=None):
    """Rotate Q in place (and K on its way into the cache); store K and V at each token's page.

    q [T, nh*hd], k [T, nkv*hd], v [T, nkv*vd]: row-contiguous views of one dtype (vd = ``value_dim``, default hd).
    cos, sin: float32 [positions, rotary_dim/2] (None with rotary_dim 0: no rotation).  k_pool [pages, nkv, 64, hd],
    v_pool [pages, nkv, vd, 64].  block_table int32 [B, P]; token_seq/token_pos int32 [T].  ``biases``: (q, k, v)
    float32 vectors (each may be None) that the kernel adds to the projections before it rotates them."""
    vd = int(value_dim or head_dim)
    qb, kb, vb = biases if biases is not None else (None, None, None)
    _need_cuda(q, k, v, cos, sin, token_seq, token_pos, block_table, k_pool, v_pool, qb, kb, vb)
    for b, n, what in ((qb, n_heads * head_dim, "q"), (kb, n_kv_heads * head_dim, "k"), (vb, n_kv_heads * vd, "v")):
        if b is not None and (b.dtype != torch.float32 or b.shape != (n,) or not b.is_contiguous()):
            raise KernelError(f"rope: the {what} bias must be contiguous float32 [{n}]")
    T = q.shape[0]
    qs = _rows_view(q, "rope q")
    if q.shape[1] != n_heads * head_dim:
        raise KernelError("rope: q width is not n_heads * head_dim")
    ks = vs = 0
    n_pages = 0
    bt_stride = 0
    if write_cache:
        ks = _rows_view(k, "rope k")
        vs = _rows_view(v, "rope v")
        if k.shape != (T, n_kv_heads * head_dim) or v.shape != (T, n_kv_heads * vd):
            raise KernelError("rope: k must be [T, n_kv_heads * head_dim] and v [T, n_kv_heads * value_dim]")
        if k.dtype != q.dtype or v.dtype != q.dtype or k_pool.dtype != q.dtype or v_pool.dtype != q.dtype:
            raise KernelError("rope: q, k, v and the cache must share one dtype")
        n_pages = _check_pools(k_pool, v_pool, n_kv_heads, head_dim, vd)
        _int32(block_table, "block_table")
        bt_stride = block_table.shape[1]
        _int32(token_seq, "token_seq")
    _int32(token_pos, "token_pos")
    table_rows = 0
    if rotary_dim:
        if cos.dtype != torch.float32 or sin.dtype != torch.float32 or cos.shape != sin.shape \
                or cos.dim() != 2 or cos.shape[1] != rotary_dim // 2 or not cos.is_contiguous() \
                or not sin.is_contiguous():
            raise KernelError("rope: cos/sin must be contiguous float32 [positions, rotary_dim/2]")
        table_rows = cos.shape[0]
    _library.call("dl_rope_cache_write", _ptr(q), qs, _ptr(k) if write_cache else None, ks,
                  _ptr(v) if write_cache else None, vs, _code(q.dtype),
                  _ptr(cos) if rotary_dim else None, _ptr(sin) if rotary_dim else None,
                  int(rotary_dim), table_rows, _ptr(token_seq) if write_cache else None, _ptr(token_pos),
                  _ptr(block_table) if write_cache else None, bt_stride,
                  _ptr(k_pool) if write_cache else None, _ptr(v_pool) if write_cache else None, n_pages,
                  T, n_heads, n_kv_heads, head_dim, vd, _ptr(qb), _ptr(kb) if write_cache else None,
                  _ptr(vb) if write_cache else None, 1 if write_cache else 0, _stream())


def _check_pools(k_pool, v_pool, n_kv_heads, head_dim, value_dim=None):
    vd = value_dim or head_dim
    if k_pool.dim() != 4 or not k_pool.is_contiguous() or not v_pool.is_contiguous() \
            or tuple(k_pool.shape[1:]) != (n_kv_heads, PAGE, head_dim) \
            or tuple(v_pool.shape) != (k_pool.shape[0], n_kv_heads, vd, PAGE):
        raise KernelError(f"cache pools must be K [pages, {n_kv_heads}, {PAGE}, {head_dim}] and "
                          f"V [pages, {n_kv_heads}, {vd}, {PAGE}], got {tuple(k_pool.shape)} "
                          f"and {tuple(v_pool.shape)}")
    return k_pool.shape[0]


def head_gate(o, gate, n_heads, width):
    """o[t, h, :] *= sigmoid(gate[t, h]) in place, for o [T, n_heads*width] and gate [T, n_heads] (a column view is
    fine) of o's dtype.  Returns o."""
    _need_cuda(o, gate)
    if o.dim() != 2 or o.shape[1] != n_heads * width or gate.shape != (o.shape[0], n_heads) or gate.dtype != o.dtype:
        raise KernelError("head_gate: o [T, heads*width] and one gate logit per (row, head) of o's dtype")
    _library.call("dl_head_gate", _ptr(o), _rows_view(o, "head_gate o"), _ptr(gate), _rows_view(gate, "head_gate gate"),
                  _code(o.dtype), o.shape[0], n_heads, width, _stream())
    return o


# ------------------------------------------------------------------ attention
class ScoreHook:
    """A change of the attention scores before the softmax: ``softcap`` > 0 turns a score s into
    softcap * tanh(s / softcap); ``slopes`` (float32 [n_heads] on the device) then adds
    slope * (key position - query position).  Only the generic kernel honours a hook: the
    tensor-core kernels take none, so a mixer that sets one runs on the generic kernel."""

    def __init__(self, softcap=0.0, slopes=None):
        self.softcap = float(softcap)
        self.slopes = slopes
        if self.softcap < 0:
            raise KernelError("a score hook's softcap must be 0 (none) or positive")

    def __bool__(self):
        return self.softcap > 0 or self.slopes is not None


def attention(q, k_pool, v_pool, token_seq, token_pos, block_table, n_heads, n_kv_heads,
              head_dim, scale, window=0, plan=None, score_hook=None, value_dim=None, gate=None, keep_first=0, sinks=None):
    """Causal attention of the step's tokens over their sequences' cached keys and values.

    q [T, nh*hd] (row-contiguous view); returns [T, nh*vd] of q's dtype (vd = ``value_dim``, default hd).
    ``window`` 0 means every earlier key; w > 0 means the last w keys.  ``plan`` carries the per-step layout
    (sequence lengths, chunking) that the tensor-core kernels need; without one, for sizes
    they do not take (values of another width than the keys among them), or with a ``score_hook``, the generic
    kernel runs.  ``gate`` [T, nh] of q's dtype (a column view is fine): head h's output is multiplied by
    sigmoid(gate[t, h]) - in the generic kernel's last step, or by ``head_gate`` behind a tensor-core kernel.
    ``keep_first`` n > 0 (with a window): a sequence's first n keys stay visible when the window has passed them.
    ``sinks`` float32 [nh]: head h's softmax has one more term exp(sinks[h]) in its denominator, with no key and no value."""
    vd = int(value_dim or head_dim)
    _need_cuda(q, k_pool, v_pool, token_seq, token_pos, block_table, gate, sinks)
    if sinks is not None and (sinks.dtype != torch.float32 or sinks.shape != (n_heads,) or not sinks.is_contiguous()):
        raise KernelError(f"attention: the sinks must be contiguous float32 [{n_heads}]")
    if keep_first < 0 or (keep_first and not window):
        raise KernelError("attention: kept first tokens need a window (and cannot be negative)")
    T = q.shape[0]
    gs = 0
    if gate is not None:
        gs = _rows_view(gate, "attention gate")
        if gate.shape != (T, n_heads) or gate.dtype != q.dtype:
            raise KernelError("attention: the gate holds one logit per (token, head) in q's dtype")
    qs = _rows_view(q, "attention q")
    if q.shape[1] != n_heads * head_dim:
        raise KernelError("attention: q width is not n_heads * head_dim")
    if k_pool.dtype != q.dtype or v_pool.dtype != q.dtype:
        raise KernelError("attention: q and the cache must share one dtype")
    n_pages = _check_pools(k_pool, v_pool, n_kv_heads, head_dim, vd)
    _int32(token_seq, "token_seq")
    _int32(token_pos, "token_pos")
    _int32(block_table, "block_table")
    out = torch.empty((T, n_heads * vd), dtype=q.dtype, device=q.device)
    softcap, slopes = 0.0, None
    if score_hook:
        softcap, slopes = score_hook.softcap, score_hook.slopes
        if slopes is not None and (slopes.dtype != torch.float32 or slopes.shape != (n_heads,) or not slopes.is_contiguous()
                                   or not slopes.is_cuda):
            raise KernelError(f"attention: a score hook's slopes must be contiguous float32 [{n_heads}] on the device")
    if plan is not None and q.dtype == torch.bfloat16 and not score_hook and vd == head_dim:
        if attention_fast.run(q, qs, out, k_pool, v_pool, n_pages, token_seq, token_pos, block_table,
                              n_heads, n_kv_heads, head_dim, float(scale), int(window), plan,
                              keep_first=int(keep_first), sinks=sinks):
            return out if gate is None else head_gate(out, gate, n_heads, vd)
    _library.call("dl_attention_generic", _ptr(q), qs, _ptr(out), out.stride(0), _code(q.dtype),
                  _ptr(k_pool), _ptr(v_pool), n_pages, _ptr(token_seq), _ptr(token_pos),
                  _ptr(block_table), block_table.shape[1], T, n_heads, n_kv_heads, head_dim, vd,
                  float(scale), int(window), float(softcap), _ptr(slopes), _ptr(gate), gs, int(keep_first), _ptr(sinks), _stream())
    return out


def rope_cache_attention(q, k, v, cos, sin, rotary_dim, token_seq, token_pos, block_table, k_pool, v_pool,
                         n_heads, n_kv_heads, head_dim, scale, window=0, plan=None, score_hook=None,
                         value_dim=None, biases=None, gate=None, keep_first=0, sinks=None):
    """``rope_cache_write`` followed by ``attention`` (same arguments, same result).  A bfloat16
    decode step (one new token per sequence) with a full-width rotation of head size 64 or 128, or
    with no rotation, runs as one kernel that adds the biases, rotates q, puts the new keys and values into the
    cache, attends and gates the heads; everything else runs the kernels one after the other."""
    if plan is not None and q.is_cuda and q.dtype == torch.bfloat16 and not score_hook and (value_dim or head_dim) == head_dim \
            and (k is not None or biases is not None or gate is not None) and not keep_first and sinks is None:
        out = attention_fast.decode_fresh(q, k, v, cos, sin, rotary_dim, block_table, k_pool, v_pool, n_heads,
                                          n_kv_heads, head_dim, float(scale), int(window), plan, biases=biases, gate=gate)
        if out is not None:
            return out
    rope_cache_write(q, k, v, cos, sin, rotary_dim, token_seq, token_pos, block_table, k_pool, v_pool,
                     n_heads, n_kv_heads, head_dim, write_cache=k is not None, value_dim=value_dim, biases=biases)
    return attention(q, k_pool, v_pool, token_seq, token_pos, block_table, n_heads, n_kv_heads, head_dim,
                     scale, window, plan=plan, score_hook=score_hook, value_dim=value_dim, gate=gate,
                     keep_first=keep_first, sinks=sinks)


def qkv_rope_cache(x, w_qkv, cos, sin, rotary_dim, token_seq, token_pos, block_table, k_pool, v_pool,
                   n_heads, n_kv_heads, head_dim):
    """The Q/K/V product of a prompt step with the rotation and the cache write in its epilogue: returns
    the rotated queries [T, nh*hd] (the rotated keys and the values are in the cache), or None when the
    step is not one the tcgen05 product takes this way (few rows, other head sizes, a partial rotation,
    float32) - the caller then runs ``linear`` and ``rope_cache_attention``.  Same bits as those."""
    q_cols, kv_cols = n_heads * head_dim, n_kv_heads * head_dim
    if isinstance(x, ScaledRows) or not x.is_cuda \
            or not gemm_tc.takes_qkv(x, w_qkv, q_cols, kv_cols, head_dim, rotary_dim, cos, sin, k_pool, v_pool):
        return None
    _need_cuda(x, w_qkv, cos, sin, token_seq, token_pos, block_table, k_pool, v_pool)
    _check_pools(k_pool, v_pool, n_kv_heads, head_dim)
    _int32(token_seq, "token_seq")
    _int32(token_pos, "token_pos")
    _int32(block_table, "block_table")
    if token_pos.numel() != x.shape[0] or token_seq.numel() != x.shape[0] or cos.shape != sin.shape \
            or cos.shape[1] != head_dim // 2:
        raise KernelError("qkv_rope_cache: one position and sequence per row, tables [positions, head_dim/2]")
    return gemm_tc.run_qkv(x, w_qkv, q_cols, kv_cols, head_dim, n_kv_heads, cos, sin, token_pos, token_seq, block_table,
                           k_pool, v_pool)


# ---------------------------------------------------------------- feed-forward
def swiglu(gate_up):
    """silu(gate) * up for gate_up = [gate | up] of shape [T, 2I]; returns [T, I]."""
    _need_cuda(gate_up)
    if gate_up.dim() != 2 or gate_up.shape[1] % 2 or not gate_up.is_contiguous():
        raise KernelError("swiglu: need a contiguous [T, 2I] tensor")
    rows, two_i = gate_up.shape
    width = two_i // 2
    out = torch.empty((rows, width), dtype=gate_up.dtype, device=gate_up.device)
    esize = gate_up.element_size()
    _library.call("dl_swiglu", gate_up.data_ptr(), gate_up.data_ptr() + width * esize, two_i,
                  _ptr(out), _code(gate_up.dtype), rows, width, _stream())
    return out


GATINGS = {"silu": 0, "gelu_tanh": 1, "clamped_sigmoid": 2, "relu2": 3}
UNGATED = frozenset({"relu2"})      # activations of ONE product, act(u): no gate rows in the matrix (GATE_RELU2 in csrc/gating.cuh)


def gated_activation(gate_up, kind, limit=0.0, alpha=1.0):
    """act(gate, up) for gate_up = [gate | up] of shape [T, 2I]; returns [T, I].  ``kind``: "silu"
    (g sigmoid(g) u), "gelu_tanh" (tanh form of gelu(g), times u) or "clamped_sigmoid"
    (g' sigmoid(alpha g') (u' + 1) with g' = min(g, limit), u' = clamp(u, -limit, limit))."""
    _need_cuda(gate_up)
    if kind not in GATINGS or kind in UNGATED:
        raise KernelError(f"gated_activation: unknown gating {kind!r}; known: {sorted(set(GATINGS) - UNGATED)}")
    if gate_up.dim() != 2 or gate_up.shape[1] % 2 or not gate_up.is_contiguous():
        raise KernelError("gated_activation: need a contiguous [T, 2I] tensor")
    rows, two_i = gate_up.shape
    width = two_i // 2
    out = torch.empty((rows, width), dtype=gate_up.dtype, device=gate_up.device)
    _library.call("dl_gated_activation", gate_up.data_ptr(), gate_up.data_ptr() + width * gate_up.element_size(), two_i,
                  _ptr(out), _code(gate_up.dtype), rows, width, GATINGS[kind], float(limit), float(alpha), _stream())
    return out


# ------------------------------------------------------- gated linear attention
def gla_scan(q, k, v, z, z_bias, cu_new, slots, state, n_heads, dim, vdim, q_scale, tau=1.0):
    """The recurrence S_t = diag(alpha_t) S_(t-1) + k_t v_t^T, o_t = S_t^T (q_t q_scale) with
    alpha_t = sigmoid(z_t + z_bias)^(1/tau), over each sequence's new rows in order, from and into
    ``state`` float32 [slots, H, dim, vdim].  q, k [T, H*dim] and v [T, H*vdim] are column views of one
    matrix (a common row stride) and of one dtype, z float32 [T, H*dim].  With ``z`` None the decay is one constant
    per head, ``z_bias`` float32 [H] holding it, and q, k and v pass through silu on their way into the recurrence.
    Returns o float32 [T, H*vdim]."""
    _need_cuda(q, k, v, z, z_bias, cu_new, slots, state)
    T = q.shape[0]
    ld = _rows_view(q, "gla q")
    if _rows_view(k, "gla k") != ld or _rows_view(v, "gla v") != ld or k.shape != (T, n_heads * dim) \
            or q.shape != k.shape or v.shape != (T, n_heads * vdim) or (z is not None and z.shape != k.shape):
        raise KernelError("gla_scan: q, k, v must be column views of one matrix, z [T, H*dim]")
    if not (q.dtype == k.dtype == v.dtype) or (z is not None and z.dtype != torch.float32):
        raise KernelError("gla_scan: q, k and v must share one dtype and z be float32")
    zs = _rows_view(z, "gla z") if z is not None else 0
    n_bias = n_heads * dim if z is not None else n_heads
    if z_bias.dtype != torch.float32 or z_bias.shape != (n_bias,) or not z_bias.is_contiguous():
        raise KernelError(f"gla_scan: the decay bias (or, without logits, the heads' decays) must be float32 [{n_bias}]")
    if state.dtype != torch.float32 or not state.is_contiguous() or tuple(state.shape[1:]) != (n_heads, dim, vdim):
        raise KernelError("gla_scan: the state must be contiguous float32 [slots, H, dim, vdim]")
    _int32(cu_new, "gla cu_new")
    _int32(slots, "gla slots")
    out = torch.empty((T, n_heads * vdim), dtype=torch.float32, device=q.device)
    _library.call("dl_gla_scan", _ptr(q), _ptr(k), _ptr(v), ld, _ptr(z), zs, _ptr(z_bias), _code(q.dtype), _ptr(cu_new),
                  _ptr(slots), _ptr(state), state.shape[0], _ptr(out), out.stride(0), slots.numel(), T, n_heads, dim, vdim,
                  float(q_scale), float(tau), _stream())
    return out


HEAD_GATES = {"silu": 0, "sigmoid": 1}


def head_norm_gate(o, g, gain, n_heads, vdim, eps, out_dtype, gate="silu"):
    """Each head's rows of o (float32 [T, H*vdim]) divided by their root mean square, times ``gain``
    (float32 [vdim], shared by the heads), times silu(g) or (``gate`` "sigmoid") sigmoid(g) (g [T, H*vdim] of
    ``out_dtype``, a column view is fine)."""
    if gate not in HEAD_GATES:
        raise KernelError(f"head_norm_gate: unknown gate {gate!r}; known: {sorted(HEAD_GATES)}")
    _need_cuda(o, g, gain)
    T = o.shape[0]
    gs = _rows_view(g, "head_norm_gate g")
    if o.dtype != torch.float32 or not o.is_contiguous() or o.shape != (T, n_heads * vdim) or g.shape != o.shape \
            or g.dtype != out_dtype or gain.dtype != torch.float32 or gain.shape != (vdim,) or not gain.is_contiguous():
        raise KernelError("head_norm_gate: o float32 [T, H*vdim], g of the output's dtype and shape, gain float32 [vdim]")
    out = torch.empty((T, n_heads * vdim), dtype=out_dtype, device=o.device)
    _library.call("dl_head_norm_gate", _ptr(o), o.stride(0), _ptr(g), gs, _ptr(gain), _ptr(out), out.stride(0),
                  _code(out_dtype), T, n_heads, vdim, float(eps), HEAD_GATES[gate], _stream())
    return out


def head_rmsnorm(x, gain_a, heads_a, dim, eps, gain_b=None, heads_b=0):
    """Every head of a row normalised on its own: y[t, h, :] = x[t, h, :] / sqrt(mean(x[t, h, :]^2) + eps) * gain[:].  The
    row holds ``heads_a`` heads under ``gain_a`` and behind them ``heads_b`` heads under ``gain_b`` (queries and keys of
    one stacked projection), each ``dim`` wide; x may be a column view.  Returns a new tensor of x's dtype."""
    _need_cuda(x, gain_a, gain_b)
    T, width = x.shape[0], (heads_a + heads_b) * dim
    if x.dim() != 2 or x.shape[1] != width:
        raise KernelError(f"head_rmsnorm: x must be [T, {width}]")
    for g, n in ((gain_a, heads_a), (gain_b, heads_b)):
        if n and (g is None or g.dtype != torch.float32 or g.shape != (dim,) or not g.is_contiguous()):
            raise KernelError(f"head_rmsnorm: a gain must be contiguous float32 [{dim}]")
    out = torch.empty((T, width), dtype=x.dtype, device=x.device)
    _library.call("dl_head_rmsnorm", _ptr(x), _rows_view(x, "head_rmsnorm x"), _ptr(out), out.stride(0), _code(x.dtype),
                  _ptr(gain_a), _ptr(gain_b), T, int(heads_a), int(heads_b), int(dim), float(eps), _stream())
    return out


# ------------------------------------------------------------------ delta rule
def delta_rule(x, taps, b_logit, z, dt_bias, a_log, token_seq, cu_new, slots, memory, n_heads, n_kv_heads, dim, vdim,
               q_scale, unit_eps, head_decay=False):
    """The gated delta rule with a decay per key channel over each sequence's new rows in order.

    x [T, >= C]: the stacked projection, its first C = 2*G*dim + H*vdim columns the channels of q, k (G = ``n_kv_heads``
    heads of ``dim``) and v (H = ``n_heads`` heads of ``vdim``); ``taps`` [C, K] of x's dtype: a causal convolution over
    time per channel, then silu; q and k unit vectors per head (x / sqrt(sum x^2 + unit_eps)), q times ``q_scale``;
    beta = sigmoid(b_logit) [T, H]; g = exp(-exp(a_log[h]) softplus(z + dt_bias)) with z float32 [T, H*dim].  Per head
    (query/key head h // (H/G)): S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q.
    ``memory`` float32 [slots, H*dim*vdim + (K-1)*C]: per slot the states and behind them the convolution's last K - 1
    inputs; read and updated.  ``head_decay``: one decay for all key channels of a head, z float32 [T, H] and dt_bias [H].
    Returns o float32 [T, H*vdim]."""
    _need_cuda(x, taps, b_logit, z, dt_bias, a_log, token_seq, cu_new, slots, memory)
    T = x.shape[0]
    H, G = int(n_heads), int(n_kv_heads)
    C, K = 2 * G * dim + H * vdim, taps.shape[1]
    ld = _rows_view(x, "delta_rule x")
    if x.shape[1] < C or taps.shape != (C, K) or taps.dtype != x.dtype or not taps.is_contiguous():
        raise KernelError(f"delta_rule: x must hold {C} channels and the taps be [{C}, K] of its dtype")
    n_decays = H if head_decay else H * dim
    if b_logit.shape != (T, H) or b_logit.dtype != x.dtype or z.shape != (T, n_decays) or z.dtype != torch.float32:
        raise KernelError(f"delta_rule: b_logit [T, H] of x's dtype, z float32 [T, {n_decays}]")
    for t, n, what in ((dt_bias, n_decays, "dt_bias"), (a_log, H, "a_log")):
        if t.dtype != torch.float32 or t.shape != (n,) or not t.is_contiguous():
            raise KernelError(f"delta_rule: {what} must be contiguous float32 [{n}]")
    n_state = H * dim * vdim
    if memory.dtype != torch.float32 or memory.dim() != 2 or memory.shape[1] != n_state + (K - 1) * C or memory.stride(1) != 1:
        raise KernelError(f"delta_rule: a slot's memory must be float32 [{n_state + (K - 1) * C}]")
    _int32(token_seq, "delta_rule token_seq")
    _int32(cu_new, "delta_rule cu_new")
    _int32(slots, "delta_rule slots")
    f32 = dict(dtype=torch.float32, device=x.device)
    qo, ko = torch.empty((T, G * dim), **f32), torch.empty((T, G * dim), **f32)
    vo, go = torch.empty((T, H * vdim), **f32), torch.empty((T, H * dim), **f32)
    bo, out = torch.empty((T, H), **f32), torch.empty((T, H * vdim), **f32)
    _library.call("dl_delta_rule", _ptr(x), ld, _ptr(taps), K, _code(x.dtype), _ptr(b_logit), _rows_view(b_logit, "delta_rule b"),
                  _ptr(z), _rows_view(z, "delta_rule z"), _ptr(dt_bias), _ptr(a_log), _ptr(token_seq), _ptr(cu_new), _ptr(slots),
                  memory.data_ptr(), memory.data_ptr() + 4 * n_state, memory.stride(0), memory.shape[0],
                  _ptr(qo), _ptr(ko), _ptr(vo), _ptr(go), _ptr(bo), _ptr(out), slots.numel(), T, H, G, int(dim), int(vdim),
                  float(q_scale), float(unit_eps), 1 if head_decay else 0, _stream())
    return out


# ---------------------------------------------------------------------- experts
ROUTER_SCORINGS = {"softmax_chosen": 0, "sigmoid": 1, "softmax_all": 2}


def route_topk(x, w_router, bias, top, scoring="softmax_chosen", experts=None, with_logits=False, groups=None,
               correction=None, normalise=False, weight_scale=1.0):
    """The ``top`` experts with the largest float32 logits x R^T + bias per row (ties: the lower index) and their
    weights: the softmax over the chosen logits alone (``scoring`` "softmax_chosen"), or each chosen expert's own
    sigmoid(logit), not renormalised ("sigmoid"), or its share of the softmax over all experts, not renormalised
    ("softmax_all").  ``groups`` (count, keep): the experts lie in ``count`` equal runs of neighbours, a run scores its
    largest logit, and only the experts of the ``keep`` best runs can be chosen.  ``experts``: the first that many rows of ``w_router`` are the
    experts' (default all); rows behind them ride the same product (a per-token gate, say) and only show in the logits.
    With "softmax_all" and no groups: ``correction`` (float32 [E]) is added to the shares for the choice alone (the
    weights stay the shares), ``normalise`` divides the chosen weights by their sum + 1e-20, and ``weight_scale``
    multiplies them.
    Returns (ids int32 [T, top], weights float32 [T, top]), and the float32 logits [T, rows of w_router] behind them
    ``with_logits``."""
    _need_cuda(x, w_router, bias)
    if scoring not in ROUTER_SCORINGS:
        raise KernelError(f"route_topk: unknown scoring {scoring!r}; known: {sorted(ROUTER_SCORINGS)}")
    rows_w, K = w_router.shape
    E = int(experts) if experts is not None else rows_w
    if not 0 < E <= rows_w:
        raise KernelError(f"route_topk: {E} experts in a matrix of {rows_w} rows")
    if x.shape[1] != K or x.dtype != w_router.dtype or not w_router.is_contiguous():
        raise KernelError(f"route_topk: x {tuple(x.shape)} does not match the router {tuple(w_router.shape)}")
    if bias is not None and (bias.dtype != torch.float32 or bias.shape != (E,) or not bias.is_contiguous()):
        raise KernelError(f"route_topk: the bias must be float32 [{E}]")
    if not 0 < top <= E:
        raise KernelError(f"route_topk: cannot choose {top} of {E} experts")
    n_groups, keep_groups = (int(groups[0]), int(groups[1])) if groups else (0, 0)
    if groups and (n_groups <= 0 or E % n_groups or not 0 < keep_groups <= n_groups or top > keep_groups * (E // n_groups)):
        raise KernelError(f"route_topk: {E} experts in {n_groups} runs of which {keep_groups} stay cannot give {top} choices")
    if correction is not None and (correction.dtype != torch.float32 or correction.shape != (E,) or not correction.is_contiguous()):
        raise KernelError(f"route_topk: the correction must be float32 [{E}]")
    if (correction is not None or normalise or float(weight_scale) != 1.0) and (scoring != "softmax_all" or groups):
        raise KernelError("route_topk: a correction, normalised weights and a scale go with 'softmax_all' without groups")
    T = x.shape[0]
    z = linear(x, w_router, out_dtype=torch.float32, resident=True)         # float32 accumulation, float32 logits
    ids = torch.empty((T, top), dtype=torch.int32, device=x.device)
    weights = torch.empty((T, top), dtype=torch.float32, device=x.device)
    _library.call("dl_route_topk", _ptr(z), z.stride(0) if T > 1 else rows_w, _ptr(bias), _ptr(ids), _ptr(weights), T, E, top,
                  ROUTER_SCORINGS[scoring], n_groups, keep_groups, _ptr(correction), 1 if normalise else 0, float(weight_scale),
                  _stream())
    return (ids, weights, z) if with_logits else (ids, weights)


def _row_scale(row_scale, ids, what):
    if row_scale is not None and (row_scale.dtype != torch.float32 or row_scale.shape != ids.shape or not row_scale.is_contiguous()):
        raise KernelError(f"{what}: the row scale must be contiguous float32 [T, top]")
    return row_scale


def _addend(addend, addend_gate, T, N, what):
    """(row stride of the addend, row stride of its gate) after checking both."""
    astride = gstride = 0
    if addend is not None:
        astride = _rows_view(addend, what + " addend")
        if addend.dtype != torch.float32 or addend.shape != (T, N):
            raise KernelError(f"{what}: the addend must be float32 [T, N]")
    if addend_gate is not None:
        if addend is None or addend_gate.dtype != torch.float32 or addend_gate.dim() != 2 or addend_gate.shape[0] != T \
                or addend_gate.stride(1) != 1:
            raise KernelError(f"{what}: the addend's gate is one float32 logit per token (column 0 of a [T, n] view)")
        gstride = addend_gate.stride(0) if T > 1 else max(addend_gate.stride(0), 1)
    return astride, gstride


def expert_gate_up(x, ids, w_gate_up, kind, limit=0.0, alpha=1.0, row_scale=None):
    """Row (t, j) = act(G_e x_t, U_e x_t) for e = ids[t, j].  x [T, K]; w_gate_up [E, 2*ff, K] (an expert's gate
    rows, then its up rows); returns [T*top, ff] in x's dtype.  For an activation of one product (``UNGATED``) the
    matrices are [E, ff, K] and the row is act(U_e x_t).  ``row_scale`` float32 [T, top]: row (t, j) takes
    x_t * row_scale[t, j] as its input (an expert whose weight multiplies what goes in, not what comes out)."""
    _need_cuda(x, ids, w_gate_up, row_scale)
    xs = _rows_view(x, "expert x")
    _int32(ids, "expert ids")
    halves = 1 if kind in UNGATED else 2
    if w_gate_up.dim() != 3 or not w_gate_up.is_contiguous() or w_gate_up.shape[1] % halves or w_gate_up.shape[2] != x.shape[1] \
            or w_gate_up.dtype != x.dtype or ids.dim() != 2 or ids.shape[0] != x.shape[0]:
        raise KernelError("expert_gate_up: x [T, K], ids [T, top], weights [E, 2*ff, K] ([E, ff, K] without a gate) of x's dtype")
    E, rows_w, K = w_gate_up.shape
    ff = rows_w // halves
    T, top = ids.shape
    out = torch.empty((T * top, ff), dtype=x.dtype, device=x.device)
    _library.call("dl_expert_gate_up", _ptr(x), xs, _ptr(ids), _ptr(w_gate_up), _ptr(out), _code(x.dtype), T, top, K,
                  ff, E, GATINGS[kind], float(limit), float(alpha), _ptr(_row_scale(row_scale, ids, "expert_gate_up")), _stream())
    return out


def _identity(identity, T, N, dtype, what):
    """(rows, row stride, count) of the input that identity experts give back, after checking it."""
    if identity is None:
        return None, 0, 0
    rows, count = identity
    if count <= 0 or rows.dtype != dtype or rows.shape != (T, N):
        raise KernelError(f"{what}: identity experts give back rows [T, N] of the experts' dtype")
    return rows, _rows_view(rows, what + " identity"), int(count)


def expert_down(h, ids, weights, w_down, addend=None, addend_gate=None, identity=None):
    """out[t] = sum_j weights[t, j] * D_e(t,j) h[t*top + j]  (+ addend[t]), float32 [T, N].  h [T*top, ff];
    w_down [E, N, ff] of h's dtype; weights float32 [T, top] or None (all 1); addend float32 [T, N] (rows contiguous)
    or None; ``addend_gate`` float32, one logit per token (column 0 of a [T, n] view): the addend times its sigmoid.
    ``identity`` (x [T, N] of h's dtype, n): ids E .. E + n - 1 name experts without matrices that give back their input,
    weight * x[t]."""
    _need_cuda(h, ids, weights, w_down, addend, addend_gate)
    _int32(ids, "expert ids")
    T, top = ids.shape
    if w_down.dim() != 3 or not w_down.is_contiguous() or w_down.dtype != h.dtype or not h.is_contiguous() \
            or h.shape != (T * top, w_down.shape[2]) or (weights is not None and (
                weights.dtype != torch.float32 or weights.shape != ids.shape or not weights.is_contiguous())):
        raise KernelError("expert_down: h [T*top, ff], ids and float32 weights [T, top], matrices [E, N, ff] of h's dtype")
    E, N, ff = w_down.shape
    astride, gstride = _addend(addend, addend_gate, T, N, "expert_down")
    irows, istride, icount = _identity(identity, T, N, h.dtype, "expert_down")
    out = torch.empty((T, N), dtype=torch.float32, device=h.device)
    _library.call("dl_expert_down", _ptr(h), _ptr(ids), _ptr(weights), _ptr(w_down), _ptr(addend), astride, _ptr(out),
                  _code(h.dtype), T, top, ff, N, E, _ptr(addend_gate), gstride, _ptr(irows), istride, icount, _stream())
    return out


GROUPED_MIN_ROWS = 128         # (token, choice) rows from which the experts' products run as tensor-core tiles
EXPERT_TILE = 128              # rows of a tile (EX_TILE in csrc/experts.cu, GT_BM in csrc/gemm_tc.cu)


def experts_grouped_takes(x, ids, w_gate_up, w_down):
    """Do the sorted, tensor-core products take this step's experts?  bfloat16, enough rows to fill tiles, and
    widths and addresses that the copy engine takes (multiples of 8 values, 16-byte aligned)."""
    T, top = ids.shape
    K, ff = w_gate_up.shape[2], w_down.shape[2]
    return (x.dtype == torch.bfloat16 and T * top >= GROUPED_MIN_ROWS and K % 8 == 0 and ff % 8 == 0
            and x.stride(1) == 1 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0
            and w_gate_up.data_ptr() % 16 == 0 and w_down.data_ptr() % 16 == 0)


def experts_grouped(x, ids, weights, w_gate_up, w_down, kind, limit=0.0, alpha=1.0, addend=None, row_scale=None,
                    addend_gate=None, identity=None):
    """The same result as ``expert_gate_up`` followed by ``expert_down``, for many rows: the (token, choice) rows are
    sorted by expert on the device, each expert's run padded to whole tiles, and the two products run on the tensor
    cores (tcgen05) with the gating in the first one's epilogue; a last kernel sums every token's choices with
    their weights (and the addend).  Shapes depend only on the step's sizes, never on the choice.  ``weights`` None,
    ``row_scale``, ``addend_gate`` and activations of one product as in those two (the row scale is applied as the rows
    are gathered, the activation in the first product's epilogue); ``identity`` as in ``expert_down``."""
    _need_cuda(x, ids, weights, w_gate_up, w_down, addend, row_scale, addend_gate)
    _int32(ids, "expert ids")
    T, top = ids.shape
    gated = kind not in UNGATED
    E, rows_w, K = w_gate_up.shape
    ff, N = (rows_w // 2 if gated else rows_w), w_down.shape[1]
    rows = T * top
    tiles = (rows + EXPERT_TILE - 1) // EXPERT_TILE + E - 1          # every expert may end in a tile that is not full
    dev = x.device
    place = torch.empty(rows, dtype=torch.int32, device=dev)
    tile_expert = torch.empty(tiles, dtype=torch.int32, device=dev)
    _library.call("dl_expert_sort", _ptr(ids), rows, E, _ptr(place), _ptr(tile_expert), tiles, _stream())
    sorted_x = torch.empty((tiles * EXPERT_TILE, K), dtype=torch.bfloat16, device=dev)
    _library.call("dl_expert_gather", _ptr(x), x.stride(0) if T > 1 else K, _ptr(place), _ptr(sorted_x), rows, top, K,
                  _ptr(_row_scale(row_scale, ids, "experts_grouped")), _stream())
    status = _library.status_word(dev).data_ptr()
    h = torch.empty((tiles * EXPERT_TILE, ff), dtype=torch.bfloat16, device=dev)
    _library.call("dl_gemm_tc_grouped_bf16", _ptr(sorted_x), K, _ptr(w_gate_up), _ptr(h), 1, ff, tiles * EXPERT_TILE, ff, K, E,
                  _ptr(tile_expert), 1 if gated else 0, GATINGS[kind], float(limit), float(alpha), 0, status, _stream())
    y = torch.empty((tiles * EXPERT_TILE, N), dtype=torch.float32, device=dev)
    _library.call("dl_gemm_tc_grouped_bf16", _ptr(h), ff, _ptr(w_down), _ptr(y), 0, N, tiles * EXPERT_TILE, N, ff, E,
                  _ptr(tile_expert), 0, 0, 0.0, 0.0, 0, status, _stream())
    astride, gstride = _addend(addend, addend_gate, T, N, "experts_grouped")
    irows, istride, icount = _identity(identity, T, N, torch.bfloat16, "experts_grouped")
    out = torch.empty((T, N), dtype=torch.float32, device=dev)
    _library.call("dl_expert_combine", _ptr(y), N, _ptr(place), _ptr(weights), _ptr(addend), astride, _ptr(out), T, top, N,
                  _ptr(addend_gate), gstride, _ptr(ids), _ptr(irows), istride, E, icount, _stream())
    return out


# --------------------------------------------------------------------- linear
def linear_per_head(x, w):
    """y[t, h, :] = W[h] x[t, h, :] for x [T, H*a] (rows contiguous) and W [H, b, a]; returns [T, H*b] in x's dtype.
    bfloat16: one batched library product with float32 accumulation; float32: the FFMA product head by head."""
    _need_cuda(x, w)
    if w.dim() != 3 or not w.is_contiguous() or x.dim() != 2 or x.shape[1] != w.shape[0] * w.shape[2] or x.dtype != w.dtype:
        raise KernelError(f"linear_per_head: x {tuple(x.shape)} does not match W {tuple(w.shape)}")
    H, b, a = w.shape
    T = x.shape[0]
    xs = _rows_view(x, "linear_per_head x")
    y = torch.empty((T, H * b), dtype=x.dtype, device=x.device)
    if T == 0:
        return y
    if x.dtype == torch.float32:
        for h in range(H):
            _library.call("dl_gemm_f32", x.data_ptr() + 4 * h * a, xs, w[h].data_ptr(), y.data_ptr() + 4 * h * b, H * b,
                          T, b, a, _stream())
        return y
    xv = x.as_strided((H, T, a), (a, xs, 1))
    torch.bmm(xv, w.transpose(1, 2), out=y.view(T, H, b).transpose(0, 1))
    return y


def linear(x, w, out_dtype=None, resident=False, lazy=False):
    """y = x W^T for W [N, K].  ``resident``: the caller vouches that nothing still pending on the
    stream writes W (a model's weights), which lets the decode kernel start streaming W while
    the kernel before it finishes.  ``lazy`` (float32 results of bfloat16 rows): return a
    PendingProduct, for a caller whose result goes to ``add_rmsnorm`` as the delta.  x may be a
    ScaledRows.

    float32: the library's own FFMA kernel (true 32-bit, the same bits for any number of rows).
    bfloat16: cuBLAS through torch with float32 accumulation, the library product that the
    reference also uses for its projections (src/DotLLM.Cuda/CudaGemm.cs:29-40)."""
    given, rows = x, None
    if isinstance(x, ScaledRows):
        if gemm_skinny.takes(x.data, w):
            rows, x = x.row_sums(), x.data
        else:
            given = x = x.tensor()
    _need_cuda(x, w)
    if w.dim() != 2 or not w.is_contiguous() or x.dim() != 2 or x.shape[1] != w.shape[1]:
        raise KernelError(f"linear: x {tuple(x.shape)} does not match W {tuple(w.shape)}")
    if x.dtype != w.dtype:
        raise KernelError(f"linear: x is {x.dtype} but W is {w.dtype}")
    out_dtype = out_dtype or x.dtype
    M, K = x.shape
    N = w.shape[0]
    if lazy and out_dtype == torch.float32 and x.dtype == torch.bfloat16 and M > 0:
        return PendingProduct(given, w, resident)
    if rows is not None:
        return gemm_skinny.run(x, w, out_dtype, resident=resident, row_sums=rows)
    if x.dtype == torch.float32:
        if out_dtype != torch.float32:
            raise KernelError("linear: the float32 product writes float32")
        xs = _rows_view(x, "linear x")
        y = torch.empty((M, N), dtype=torch.float32, device=x.device)
        _library.call("dl_gemm_f32", _ptr(x), xs, _ptr(w), _ptr(y), N, M, N, K, _stream())
        return y
    if x.dtype != torch.bfloat16:
        raise KernelError(f"linear: unsupported dtype {x.dtype}")
    if M > 0:
        y = gemm_skinny.maybe_run(x, w, out_dtype, resident=resident)
        if y is not None:
            return y
    if out_dtype == torch.bfloat16:
        return torch.mm(x, w.t())
    return torch.mm(x, w.t(), out_dtype=out_dtype)


def unary_activation(x, kind):
    """act(x) for an activation of one product (``UNGATED``); x [T, N] (rows contiguous), returns a contiguous [T, N]."""
    _need_cuda(x)
    if kind not in UNGATED:
        raise KernelError(f"unary_activation: {kind!r} is no activation of one product; known: {sorted(UNGATED)}")
    out = torch.empty(x.shape, dtype=x.dtype, device=x.device)
    _library.call("dl_unary_activation", _ptr(x), _rows_view(x, "unary_activation x"), _ptr(out), _code(x.dtype), x.shape[0],
                  x.shape[1], GATINGS[kind], _stream())
    return out


ACTIVATED_TC_MIN_ROWS = 129     # fewer rows (a decode step) take the plain product's kernels and then the activation


def activated_linear(x, w, kind, resident=False):
    """act(x W^T) for W [N, K] and an activation of one product (``UNGATED``); returns [T, N] in x's dtype.  Many bfloat16
    rows (a prompt step): the tcgen05 product with the activation in its epilogue; a few rows (a decode step): the
    weight-streaming product with it in its epilogue; otherwise the product and then the activation."""
    x = resolve(x) if isinstance(x, ScaledRows) else x
    _need_cuda(x, w)
    if kind not in UNGATED:
        raise KernelError(f"activated_linear: {kind!r} is no activation of one product; known: {sorted(UNGATED)}")
    if x.dtype == torch.bfloat16 and w.dim() == 2 and x.dim() == 2 and x.shape[1] == w.shape[1] and gemm_tc.takes(x, w) \
            and x.shape[0] >= ACTIVATED_TC_MIN_ROWS:
        return gemm_tc.run_activated(x, w, GATINGS[kind])
    if x.dtype == torch.bfloat16 and w.dim() == 2 and x.dim() == 2 and x.shape[1] == w.shape[1] and 0 < x.shape[0] <= gemm_skinny.SKINNY_ROWS \
            and gemm_skinny.takes(x, w):
        return gemm_skinny.run_activated(x, w, GATINGS[kind], resident=resident)
    return unary_activation(linear(x, w, resident=resident), kind)


def softcap(values, cap):
    """values = cap * tanh(values / cap) in place (float32, contiguous); returns values."""
    _need_cuda(values)
    if values.dtype != torch.float32 or not values.is_contiguous() or not cap > 0:
        raise KernelError("softcap: contiguous float32 values and a positive cap")
    _library.call("dl_softcap", _ptr(values), values.numel(), float(cap), _stream())
    return values


def gated_linear(x, w_gate_up, resident=False, kind="silu", limit=0.0, alpha=1.0):
    """silu(x Wg^T) * (x Wu^T) for W = [Wg; Wu] of shape [2I, K]; returns [T, I] in x's dtype.
    In bfloat16 one kernel does the product and the gating in float32: the weight-streaming
    kernel for a few rows, the tcgen05 kernel for many.  In float32 the product is followed by
    the gating kernel.  ``kind``: another gating of ``GATINGS`` instead of silu; the weight-streaming
    product (up to 10 rows) and the tcgen05 product (17 rows and more) have it in their epilogues too; the rows
    between, and float32, run the product and then ``gated_activation``."""
    if kind != "silu":
        x = resolve(x) if isinstance(x, ScaledRows) else x
        _need_cuda(x, w_gate_up)
        if x.dtype == torch.bfloat16 and w_gate_up.dim() == 2 and x.dim() == 2 and x.shape[1] == w_gate_up.shape[1] \
                and w_gate_up.is_contiguous() and w_gate_up.shape[0] % 2 == 0 and x.shape[0] > 0:
            if gemm_skinny.takes_gating(x, w_gate_up):
                return gemm_skinny.run_gating(x, w_gate_up, GATINGS[kind], limit, alpha, resident=resident)
            if gemm_tc.takes(x, w_gate_up, fuse_swiglu=True):
                return gemm_tc.run_gated(x, w_gate_up, GATINGS[kind], limit, alpha)
        return gated_activation(linear(x, w_gate_up, resident=resident), kind, limit, alpha)
    if isinstance(x, ScaledRows):
        if w_gate_up.dim() == 2 and x.shape[1] == w_gate_up.shape[1] and gemm_skinny.takes(x.data, w_gate_up, True):
            _need_cuda(x.data, w_gate_up)
            return gemm_skinny.run(x.data, w_gate_up, x.dtype, fuse_swiglu=True, resident=resident, row_sums=x.row_sums())
        x = x.tensor()
    _need_cuda(x, w_gate_up)
    if w_gate_up.dim() != 2 or w_gate_up.shape[0] % 2 or not w_gate_up.is_contiguous() or x.dim() != 2 \
            or x.shape[1] != w_gate_up.shape[1]:
        raise KernelError(f"gated_linear: x {tuple(x.shape)} does not match W {tuple(w_gate_up.shape)}")
    if x.dtype == torch.bfloat16 and x.shape[0] > 0:
        y = gemm_skinny.maybe_run(x, w_gate_up, x.dtype, fuse_swiglu=True, resident=resident)
        if y is not None:
            return y
        if gemm_tc.takes(x, w_gate_up, fuse_swiglu=True):
            return gemm_tc.run(x, w_gate_up, x.dtype, fuse_swiglu=True)
    return swiglu(linear(x, w_gate_up))


# ------------------------------------------------------------------- sampling
def sample(logits, temperature=None, top_k=None, top_p=None, min_p=None, uniform=None, out=None, split=None):
    """One token per row of float32 logits [R, V].  With ``temperature`` None every row is
    greedy (first index of the maximum).  Otherwise per-row float32/int32 tensors [R] give the
    chain temperature -> top-k -> top-p -> min-p and ``uniform`` the draw in [0, 1);
    a row with temperature <= 0 is greedy.  ``split``: None lets the library choose between one
    block per row and a cluster of blocks per row (long rows, few of them); False / True force
    one or the other - they give the same tokens."""
    _need_cuda(logits, temperature, top_k, top_p, min_p, uniform)
    if logits.dtype != torch.float32 or logits.dim() != 2 or logits.stride(1) != 1:
        raise KernelError("sample: logits must be float32 [rows, vocab] with contiguous rows")
    rows, vocab = logits.shape
    for name, t, dt in (("temperature", temperature, torch.float32), ("top_k", top_k, torch.int32),
                        ("top_p", top_p, torch.float32), ("min_p", min_p, torch.float32),
                        ("uniform", uniform, torch.float32)):
        if t is not None and (t.dtype != dt or t.shape != (rows,) or not t.is_contiguous()):
            raise KernelError(f"sample: {name} must be a contiguous {dt} tensor of {rows} values")
    if out is None:
        out = torch.empty((rows,), dtype=torch.int32, device=logits.device)
    elif out.dtype != torch.int32 or out.shape != (rows,) or not out.is_contiguous() or not out.is_cuda:
        raise KernelError("sample: out must be a contiguous int32 CUDA tensor of one id per row")
    _library.call("dl_sample", _ptr(logits), logits.stride(0) if rows > 1 else vocab, rows, vocab,
                  _ptr(temperature), _ptr(top_k), _ptr(top_p), _ptr(min_p), _ptr(uniform), _ptr(out),
                  0 if split is None else (2 if split else 1), _stream())
    return out


def repetition_penalty(logits, prev, prev_len, penalty, window, row_map=None, append=None):
    """In place: each distinct id among the last ``window[r]`` (0 = all) of row r's
    ``prev[r, :prev_len[r]]`` has its logit divided (if positive) or multiplied by ``penalty[r]``.
    ``row_map`` (int32 [rows]): row r's ids are in ``prev[row_map[r]]`` instead.  ``append`` =
    (positions, ids), int32 [rows] each: before anything else id r is written at ``prev[row, positions[r]]``
    (a position < 0: nothing), for callers that keep the histories on the device and send one id a step."""
    _need_cuda(logits, prev, prev_len, penalty, window, row_map)
    if logits.dtype != torch.float32 or logits.dim() != 2 or logits.stride(1) != 1:
        raise KernelError("repetition_penalty: logits must be float32 [rows, vocab]")
    rows, vocab = logits.shape
    if prev.dtype != torch.int32 or prev.dim() != 2 or not prev.is_contiguous() or (row_map is None and prev.shape[0] < rows):
        raise KernelError("repetition_penalty: prev must be contiguous int32 [rows, n]")
    _int32(prev_len, "prev_len")
    _int32(window, "window")
    if row_map is not None:
        _int32(row_map, "row_map")
    pos = tok = None
    if append is not None:
        pos, tok = append
        _need_cuda(pos, tok)
        _int32(pos, "append positions")
        _int32(tok, "append ids")
    if penalty.dtype != torch.float32 or not penalty.is_contiguous():
        raise KernelError("repetition_penalty: penalty must be float32 [rows]")
    for name, t in (("prev_len", prev_len), ("window", window), ("penalty", penalty), ("row_map", row_map), ("append positions", pos),
                    ("append ids", tok)):
        if t is not None and t.numel() != rows:
            raise KernelError(f"repetition_penalty: {name} must hold one value per row ({rows}), got {t.numel()}")
    _library.call("dl_repetition_penalty", _ptr(logits), logits.stride(0) if rows > 1 else vocab, rows,
                  vocab, _ptr(prev), prev.shape[1], prev.shape[0], _ptr(row_map), _ptr(pos), _ptr(tok), _ptr(prev_len),
                  _ptr(penalty), _ptr(window), _stream())
    return logits
