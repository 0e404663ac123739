"""`rms_norm`, `fused_add_rms_norm` and their `_fp8_quant` forms as PyTorch custom ops over libzck_b200.

Same schemas, aliasing rules and rounding points as the reference's src/zig_cu_kernels/torch/rms_norm.py (`rms_norm`
:486-488, `fused_add_rms_norm` :428-429, :491-496, `run` :328-370): `h = x + residual` rounded once to the dtype of `x`
and returned as `residual_out`; `y = weight * dtype_of_x(h * rsqrt(mean(h^2) + eps))` (LlamaRMSNorm) for a BF16
weight, `weight * (h * r)` for an FP32 weight, `(h * r) * (1 + weight)` when zero-centered. Outputs may be the exact
views `x` or `residual`; any other overlap goes through a temporary. The launch shape depends on the row width only,
so results do not depend on the batch.

`rms_norm_fp8_quant` / `fused_add_rms_norm_fp8_quant` (reference :499-518, ops :432-434): the BF16 result is quantized
in the same pass. `fp8_scaling="tensorwise"` takes the caller's one-element `fp8_scale`; `"block128"` computes one
scale per row and 128 values and returns `(q, scales[, residual_out])` with the bits of `quantize_fp8_rows(norm)`;
`"rowwise"` computes one FP32 scale per row, `scales (rows, 1)`.
"""

import math

import torch

from .. import _lib
from .common import GROUP, KINDS, block_scales_like, need_choice, need_dtype, raw_stream, row_matrix, writes_in_place
from .ops import Out, Param, define

__all__ = ["rms_norm", "fused_add_rms_norm", "rms_norm_fp8_quant", "fused_add_rms_norm_fp8_quant", "rms_norm_op",
           "rms_norm_out_op", "fused_add_rms_norm_op", "fused_add_rms_norm_out_op", "rms_norm_fp8_quant_op",
           "rms_norm_fp8_quant_out_op", "fused_add_rms_norm_fp8_quant_op", "fused_add_rms_norm_fp8_quant_out_op"]

BF16, F32, FP8, E8M0 = torch.bfloat16, torch.float32, torch.float8_e4m3fn, torch.float8_e8m0fnu
COMPUTED_SCALINGS = ("rowwise", "block128")
X_DTYPES = (BF16, F32)
MAX_ROW_BYTES = 131072
LIMIT_32 = (1 << 32) - 1


def check_common(x, residual, weight, fp8_scale, zero_centered, out_dtype):
    need_dtype("x", x, X_DTYPES)
    if x.dim() < 1:
        raise ValueError("x needs at least one dimension")
    need_dtype("residual", residual, (x.dtype,))
    need_dtype("weight", weight, X_DTYPES)
    if weight is None and zero_centered:
        raise ValueError("zero_centered needs a weight")
    if fp8_scale is not None:
        need_dtype("fp8_scale", fp8_scale, (F32,))
        if out_dtype not in (None, FP8):
            raise ValueError(f"with fp8_scale the output dtype must be {FP8}, got {out_dtype}")
    elif out_dtype is not None:
        need_choice("out_dtype", out_dtype, X_DTYPES)


def check_common_sizes(x, residual, weight, fp8_scale):
    width = x.shape[-1]
    if residual is not None and residual.shape != x.shape:
        raise ValueError(f"residual must have the shape {tuple(x.shape)}, got {tuple(residual.shape)}")
    if weight is not None and tuple(weight.shape) != (width,):
        raise ValueError(f"weight must have the shape {(width,)}, got {tuple(weight.shape)}")
    if width % 8:
        raise ValueError(f"the row length must be a multiple of 8, got {width}")
    if width * x.element_size() > MAX_ROW_BYTES:
        raise ValueError(f"rows of {width} {x.dtype} values are too wide: at most {MAX_ROW_BYTES} bytes")
    if math.prod(x.shape[:-1]) > LIMIT_32:
        raise ValueError(f"x has {math.prod(x.shape[:-1])} rows, more than 2^32 - 1")
    if fp8_scale is not None and fp8_scale.numel() != 1:
        raise ValueError(f"fp8_scale must hold one element, got the shape {tuple(fp8_scale.shape)}")


def y_like(x, fp8_scale, out_dtype):
    if out_dtype is not None:
        return x.new_empty(x.shape, dtype=out_dtype)
    return x.new_empty(x.shape, dtype=FP8 if fp8_scale is not None else BF16)


def rows_for_kernel(tensor, align, output=False):
    """Row stride the kernel takes for `tensor`, or None when it needs a copy or a temporary."""
    rows = row_matrix(tensor, align)
    if rows is None:
        return None
    count, step = rows
    if output and count > 1 and step < tensor.shape[-1]:
        return None
    return step


def vector_ready(tensor):
    return (tensor.shape[-1] <= 1 or tensor.stride(-1) == 1) and tensor.data_ptr() % 16 == 0


def y_alignment(x, out):
    """Bytes one thread stores per 16-byte chunk of x: the alignment the kernel needs for rows of `out`."""
    values = 16 // x.element_size()
    return min(16, values * out.element_size())


def run_norm(x, residual, weight, fp8_scale, eps, zero_centered, out, residual_out, scales_out=None, rowwise=False):
    """Queues one launch. With `scales_out` (block128 scales `(rows, width/128)`, or rowwise scales `(rows, 1)`) `out`
    holds E4M3 codes."""
    if tuple(out.shape) != tuple(x.shape):
        raise ValueError(f"out must have the shape {tuple(x.shape)}, got {tuple(out.shape)}")
    if residual_out is not None and tuple(residual_out.shape) != tuple(x.shape):
        raise ValueError(f"residual_out must have the shape {tuple(x.shape)}, got {tuple(residual_out.shape)}")
    rows, width = math.prod(x.shape[:-1]), x.shape[-1]
    scales_shape = (rows, 1) if rowwise else (rows, width // GROUP)
    if scales_out is not None and tuple(scales_out.shape) != scales_shape:
        raise ValueError(f"scales_out must have the shape {scales_shape}, got {tuple(scales_out.shape)}")
    if rows == 0 or width == 0:
        return
    # Inputs the kernel cannot address in place are copied once.
    x_in = x if rows_for_kernel(x, 16) is not None else x.clone(memory_format=torch.contiguous_format)
    r_in = residual
    if residual is not None and rows_for_kernel(residual, 16) is None:
        r_in = residual.clone(memory_format=torch.contiguous_format)
    w_in = weight if weight is None or vector_ready(weight) else weight.clone(memory_format=torch.contiguous_format)
    s_in = fp8_scale
    row_inputs = [t for t in (x, residual) if t is not None]
    others = [t for t in (weight, fp8_scale) if t is not None]
    # Outputs: in place when the layout fits and the only overlap is with a row input as the very same view.
    y_aliases = [t for t in row_inputs if t.dtype == out.dtype]
    y_inputs = others + [t for t in row_inputs if t.dtype != out.dtype]
    y_fits = rows_for_kernel(out, y_alignment(x, out), output=True) is not None
    y_target = out if y_fits and writes_in_place(out, y_inputs, y_aliases) else torch.empty(
        out.shape, dtype=out.dtype, device=out.device)
    h_target = None
    if residual_out is not None:
        h_fits = rows_for_kernel(residual_out, 16, output=True) is not None
        h_target = residual_out if h_fits and writes_in_place(residual_out, others, row_inputs) else torch.empty(
            residual_out.shape, dtype=residual_out.dtype, device=residual_out.device)
        # The two outputs of one launch must not be the same input view in different roles when a copy was made.
    weight_kind = _lib.WEIGHT_NONE
    if weight is not None:
        weight_kind = (_lib.WEIGHT_BF16 if weight.dtype == BF16 else _lib.WEIGHT_F32) | (
            _lib.WEIGHT_ZERO_CENTERED if zero_centered else 0)
    device = x.get_device()
    leading = (x_in.data_ptr(), KINDS[x.dtype], rows_for_kernel(x_in, 16),
               None if r_in is None else r_in.data_ptr(), 0 if r_in is None else rows_for_kernel(r_in, 16),
               None if h_target is None else h_target.data_ptr(),
               0 if h_target is None else rows_for_kernel(h_target, 16, output=True),
               None if w_in is None else w_in.data_ptr(), weight_kind)
    y_stride = rows_for_kernel(y_target, y_alignment(x, out), output=True)
    if scales_out is None:
        _lib.check(_lib.library().zck_fused_add_rms_norm(
            *leading, None if s_in is None else s_in.data_ptr(), y_target.data_ptr(), KINDS[out.dtype], y_stride,
            rows, width, float(eps), device, raw_stream(device)))
    elif rowwise:
        direct = (writes_in_place(scales_out, [*others, *row_inputs]) and scales_out.data_ptr() % 4 == 0 and
                  (rows <= 1 or scales_out.stride(0) >= 1))
        scales_target = scales_out if direct else torch.empty((rows, 1), dtype=F32, device=x.device)
        _lib.check(_lib.library().zck_fused_add_rms_norm_quant(
            *leading, y_target.data_ptr(), y_stride, scales_target.data_ptr(),
            scales_target.stride(0) if rows > 1 else 1, _lib.SCALES_ROW_F32, rows, width, float(eps), device,
            raw_stream(device)))
        if scales_target is not scales_out:
            scales_out.copy_(scales_target)
    else:
        # Scales in place when they have the quantizer's layout (rows contiguous, one column per group) and overlap
        # nothing that is read; otherwise through a temporary of that layout.
        groups = width // GROUP
        direct = ((rows <= 1 or scales_out.stride(0) == 1) and (groups <= 1 or scales_out.stride(1) >= rows) and
                  writes_in_place(scales_out, [*others, *row_inputs]) and
                  (scales_out.dtype == E8M0 or scales_out.data_ptr() % 4 == 0))
        scales_target = scales_out if direct else block_scales_like(x, scales_out.dtype)
        _lib.check(_lib.library().zck_fused_add_rms_norm_quant(
            *leading, y_target.data_ptr(), y_stride, scales_target.data_ptr(),
            scales_target.stride(1) if groups > 1 else rows,
            _lib.SCALES_BLOCK_E8M0 if scales_out.dtype == E8M0 else _lib.SCALES_BLOCK_F32, rows, width, float(eps),
            device, raw_stream(device)))
        if scales_target is not scales_out:
            scales_out.copy_(scales_target)
    if y_target is not out:
        out.copy_(y_target)
    if h_target is not residual_out:
        residual_out.copy_(h_target)


# ---- rms_norm ------------------------------------------------------------------------------------------------------

def check_plain(x, weight, fp8_scale, eps, zero_centered, out_dtype):
    check_common(x, None, weight, fp8_scale, zero_centered, out_dtype)


def check_plain_sizes(x, weight, fp8_scale, eps, zero_centered, out_dtype):
    check_common_sizes(x, None, weight, fp8_scale)


def plain_y(x, weight, fp8_scale, eps, zero_centered, out_dtype):
    return y_like(x, fp8_scale, out_dtype)


def plain_into(x, weight, fp8_scale, eps, zero_centered, out):
    run_norm(x, None, weight, fp8_scale, eps, zero_centered, out, None)


RMS_NORM = define(
    "rms_norm",
    params=[Param("Tensor", "x"), Param("Tensor?", "weight"), Param("Tensor?", "fp8_scale"), Param("float", "eps"),
            Param("bool", "zero_centered"), Param("ScalarType", "out_dtype")],
    outs=[Out("out", "out", plain_y, "out_dtype")], check=check_plain, check_sizes=check_plain_sizes, run=plain_into)
rms_norm_op, rms_norm_out_op = RMS_NORM.functional, RMS_NORM.out


# ---- fused_add_rms_norm --------------------------------------------------------------------------------------------

def check_fused(x, residual, weight, fp8_scale, eps, zero_centered, out_dtype):
    check_common(x, residual, weight, fp8_scale, zero_centered, out_dtype)


def check_fused_sizes(x, residual, weight, fp8_scale, eps, zero_centered, out_dtype):
    check_common_sizes(x, residual, weight, fp8_scale)


def fused_y(x, residual, weight, fp8_scale, eps, zero_centered, out_dtype):
    return y_like(x, fp8_scale, out_dtype)


def fused_h(x, residual, weight, fp8_scale, eps, zero_centered, out_dtype):
    return x.new_empty(x.shape)


def fused_into(x, residual, weight, fp8_scale, eps, zero_centered, out, residual_out):
    run_norm(x, residual, weight, fp8_scale, eps, zero_centered, out, residual_out)


FUSED_ADD = define(
    "fused_add_rms_norm",
    params=[Param("Tensor", "x"), Param("Tensor", "residual"), Param("Tensor?", "weight"),
            Param("Tensor?", "fp8_scale"), Param("float", "eps"), Param("bool", "zero_centered"),
            Param("ScalarType", "out_dtype")],
    outs=[Out("out", "out", fused_y, "out_dtype"), Out("residual_out", "residual_out", fused_h, "x")],
    check=check_fused, check_sizes=check_fused_sizes, run=fused_into)
fused_add_rms_norm_op, fused_add_rms_norm_out_op = FUSED_ADD.functional, FUSED_ADD.out


# ---- rms_norm_fp8_quant, fused_add_rms_norm_fp8_quant (computed scales) --------------------------------------------

def check_quant(x, residual, weight, zero_centered, fp8_scaling, fp8_scale_dtype):
    check_common(x, residual, weight, None, zero_centered, None)
    need_choice("fp8_scaling", fp8_scaling, COMPUTED_SCALINGS)
    need_choice("fp8_scale_dtype", fp8_scale_dtype, (F32, E8M0) if fp8_scaling == "block128" else (F32,))


def check_quant_sizes(x, residual, weight, fp8_scaling):
    check_common_sizes(x, residual, weight, None)
    if fp8_scaling == "block128" and x.shape[-1] % GROUP:
        raise ValueError(f"fp8_scaling='block128' needs a row length that is a multiple of {GROUP}")


def codes_like(x):
    return x.new_empty(x.shape, dtype=FP8)


def computed_scales_like(x, fp8_scaling, fp8_scale_dtype):
    if fp8_scaling == "rowwise":
        return x.new_empty((math.prod(x.shape[:-1]), 1), dtype=F32)
    return block_scales_like(x, fp8_scale_dtype)


PLAIN_QUANT = define(
    "rms_norm_fp8_quant",
    params=[Param("Tensor", "x"), Param("Tensor?", "weight"), Param("float", "eps"), Param("bool", "zero_centered"),
            Param("str", "fp8_scaling"), Param("ScalarType", "fp8_scale_dtype")],
    outs=[Out("out", "out", lambda x, weight, eps, zero_centered, fp8_scaling, fp8_scale_dtype: codes_like(x), FP8),
          Out("scales_out", "scales_out",
              lambda x, weight, eps, zero_centered, fp8_scaling, fp8_scale_dtype: computed_scales_like(
                  x, fp8_scaling, fp8_scale_dtype),
              "fp8_scale_dtype")],
    check=lambda x, weight, eps, zero_centered, fp8_scaling, fp8_scale_dtype: check_quant(
        x, None, weight, zero_centered, fp8_scaling, fp8_scale_dtype),
    check_sizes=lambda x, weight, eps, zero_centered, fp8_scaling, fp8_scale_dtype: check_quant_sizes(
        x, None, weight, fp8_scaling),
    run=lambda x, weight, eps, zero_centered, fp8_scaling, out, scales_out: run_norm(
        x, None, weight, None, eps, zero_centered, out, None, scales_out, fp8_scaling == "rowwise"))
rms_norm_fp8_quant_op, rms_norm_fp8_quant_out_op = PLAIN_QUANT.functional, PLAIN_QUANT.out

FUSED_QUANT = define(
    "fused_add_rms_norm_fp8_quant",
    params=[Param("Tensor", "x"), Param("Tensor", "residual"), Param("Tensor?", "weight"), Param("float", "eps"),
            Param("bool", "zero_centered"), Param("str", "fp8_scaling"), Param("ScalarType", "fp8_scale_dtype")],
    outs=[Out("out", "out",
              lambda x, residual, weight, eps, zero_centered, fp8_scaling, fp8_scale_dtype: codes_like(x), FP8),
          Out("scales_out", "scales_out",
              lambda x, residual, weight, eps, zero_centered, fp8_scaling, fp8_scale_dtype: computed_scales_like(
                  x, fp8_scaling, fp8_scale_dtype), "fp8_scale_dtype"),
          Out("residual_out", "residual_out",
              lambda x, residual, weight, eps, zero_centered, fp8_scaling, fp8_scale_dtype: x.new_empty(x.shape), "x")],
    check=lambda x, residual, weight, eps, zero_centered, fp8_scaling, fp8_scale_dtype: check_quant(
        x, residual, weight, zero_centered, fp8_scaling, fp8_scale_dtype),
    check_sizes=lambda x, residual, weight, eps, zero_centered, fp8_scaling, fp8_scale_dtype: check_quant_sizes(
        x, residual, weight, fp8_scaling),
    run=lambda x, residual, weight, eps, zero_centered, fp8_scaling, out, scales_out, residual_out: run_norm(
        x, residual, weight, None, eps, zero_centered, out, residual_out, scales_out, fp8_scaling == "rowwise"))
fused_add_rms_norm_fp8_quant_op, fused_add_rms_norm_fp8_quant_out_op = FUSED_QUANT.functional, FUSED_QUANT.out


def given_scale(fp8_scaling, fp8_scale, fp8_scale_dtype, scales_out):
    """Checks the scale arguments of a `_fp8_quant` function; True when the call takes the caller's scale."""
    if fp8_scaling != "tensorwise":
        if fp8_scale is not None:
            raise ValueError(f"fp8_scaling={fp8_scaling!r} computes the scales and takes no fp8_scale")
        return False
    if fp8_scale is None:
        raise ValueError("fp8_scaling='tensorwise' needs fp8_scale")
    if fp8_scale.numel() != 1:
        raise ValueError(f"fp8_scale must hold one element, got the shape {tuple(fp8_scale.shape)}")
    if fp8_scale_dtype != F32:
        raise ValueError(f"fp8_scaling='tensorwise' takes FP32 scales, got fp8_scale_dtype={fp8_scale_dtype}")
    if scales_out is not None:
        raise ValueError("fp8_scaling='tensorwise' returns fp8_scale and takes no scales_out")
    return True


def _resolved(x, out_dtype):
    return getattr(x, "dtype", None) if out_dtype is None else out_dtype


def rms_norm(x, weight, eps, *, zero_centered=False, out_dtype=None, out=None):
    """RMS norm of the rows of `x`, times `weight` unless it is None."""
    return RMS_NORM(x, weight, None, eps, zero_centered, _resolved(x, out_dtype), outputs={"out": out})


def fused_add_rms_norm(x, residual, weight, eps, *, zero_centered=False, out_dtype=None, out=None, residual_out=None):
    """`(y, residual_out)`: the residual stream `x + residual` and its RMS norm, in one pass over the rows."""
    return FUSED_ADD(x, residual, weight, None, eps, zero_centered, _resolved(x, out_dtype),
                     outputs={"out": out, "residual_out": residual_out})


def rms_norm_fp8_quant(x, weight, eps, *, fp8_scaling, fp8_scale=None, fp8_scale_dtype=torch.float32, zero_centered=False,
                       out=None, scales_out=None):
    """`(q, scales)`: E4M3 codes of the BF16 RMS norm of `x` and their scales for the scaling type `fp8_scaling`."""
    if given_scale(fp8_scaling, fp8_scale, fp8_scale_dtype, scales_out):
        return RMS_NORM(x, weight, fp8_scale, eps, zero_centered, FP8, outputs={"out": out}), fp8_scale.reshape(())
    return PLAIN_QUANT(x, weight, eps, zero_centered, fp8_scaling, fp8_scale_dtype,
                       outputs={"out": out, "scales_out": scales_out})


def fused_add_rms_norm_fp8_quant(x, residual, weight, eps, *, fp8_scaling, fp8_scale=None, fp8_scale_dtype=torch.float32,
                                 zero_centered=False, out=None, scales_out=None, residual_out=None):
    """`(q, scales, residual_out)`: the results of `fused_add_rms_norm`, quantized as in `rms_norm_fp8_quant`."""
    if given_scale(fp8_scaling, fp8_scale, fp8_scale_dtype, scales_out):
        q, h = FUSED_ADD(x, residual, weight, fp8_scale, eps, zero_centered, FP8,
                         outputs={"out": out, "residual_out": residual_out})
        return q, fp8_scale.reshape(()), h
    return FUSED_QUANT(x, residual, weight, eps, zero_centered, fp8_scaling, fp8_scale_dtype,
                       outputs={"out": out, "scales_out": scales_out, "residual_out": residual_out})
