"""Op layer without a GPU: the registered schemas are the reference's (src/zig_cu_kernels/torch/*.py builds the same
strings from its `define` calls) and the fake kernels give the shapes, dtypes and strides of the real ones."""

import pytest
import torch
from torch._subclasses.fake_tensor import FakeTensorMode

import zig_cu_kernels.torch as ops  # noqa: F401  (registers the ops)

FP8, E8M0, BF16, F32 = torch.float8_e4m3fn, torch.float8_e8m0fnu, torch.bfloat16, torch.float32

SCHEMAS = """
fp8_gemm(Tensor a, Tensor b, Tensor scale_a, Tensor scale_b, Tensor? bias, Tensor? residual, str activation, bool use_fast_accum) -> Tensor
fp8_gemm_out(Tensor a, Tensor b, Tensor scale_a, Tensor scale_b, Tensor? bias, Tensor? residual, str activation, bool use_fast_accum, Tensor(a8!) out) -> ()
fp8_gated_gemm(Tensor a, Tensor w_gate, Tensor w_up, Tensor scale_a, Tensor scale_gate, Tensor scale_up, Tensor? bias_gate, Tensor? bias_up, Tensor? residual, str activation, bool use_fast_accum) -> Tensor
fp8_gated_gemm_out(Tensor a, Tensor w_gate, Tensor w_up, Tensor scale_a, Tensor scale_gate, Tensor scale_up, Tensor? bias_gate, Tensor? bias_up, Tensor? residual, str activation, bool use_fast_accum, Tensor(a11!) out) -> ()
gated_gemm(Tensor a, Tensor w_gate, Tensor w_up, Tensor? bias_gate, Tensor? bias_up, Tensor? residual, str activation) -> Tensor
gated_gemm_out(Tensor a, Tensor w_gate, Tensor w_up, Tensor? bias_gate, Tensor? bias_up, Tensor? residual, str activation, Tensor(a7!) out) -> ()
quantize_fp8_rows(Tensor x, ScalarType scale_dtype) -> (Tensor, Tensor)
quantize_fp8_rows_out(Tensor x, Tensor(a1!) q, Tensor(a2!) scales) -> ()
quantize_fp8_tiles(Tensor w, ScalarType scale_dtype) -> (Tensor, Tensor)
quantize_fp8_tiles_out(Tensor w, Tensor(a1!) q, Tensor(a2!) scales) -> ()
quantize_fp8_tensorwise(Tensor x) -> (Tensor, Tensor)
quantize_fp8_tensorwise_out(Tensor x, Tensor(a1!) q, Tensor(a2!) scale) -> ()
quantize_fp8_static(Tensor x, Tensor scale) -> Tensor
quantize_fp8_static_out(Tensor x, Tensor scale, Tensor(a2!) q) -> ()
rms_norm(Tensor x, Tensor? weight, Tensor? fp8_scale, float eps, bool zero_centered, ScalarType out_dtype) -> Tensor
rms_norm_out(Tensor x, Tensor? weight, Tensor? fp8_scale, float eps, bool zero_centered, Tensor(a5!) out) -> ()
fused_add_rms_norm(Tensor x, Tensor residual, Tensor? weight, Tensor? fp8_scale, float eps, bool zero_centered, ScalarType out_dtype) -> (Tensor, Tensor)
fused_add_rms_norm_out(Tensor x, Tensor residual, Tensor? weight, Tensor? fp8_scale, float eps, bool zero_centered, Tensor(a6!) out, Tensor(a7!) residual_out) -> ()
rms_norm_fp8_quant(Tensor x, Tensor? weight, float eps, bool zero_centered, str fp8_scaling, ScalarType fp8_scale_dtype) -> (Tensor, Tensor)
rms_norm_fp8_quant_out(Tensor x, Tensor? weight, float eps, bool zero_centered, str fp8_scaling, Tensor(a5!) out, Tensor(a6!) scales_out) -> ()
fused_add_rms_norm_fp8_quant(Tensor x, Tensor residual, Tensor? weight, float eps, bool zero_centered, str fp8_scaling, ScalarType fp8_scale_dtype) -> (Tensor, Tensor, Tensor)
fused_add_rms_norm_fp8_quant_out(Tensor x, Tensor residual, Tensor? weight, float eps, bool zero_centered, str fp8_scaling, Tensor(a6!) out, Tensor(a7!) scales_out, Tensor(a8!) residual_out) -> ()
"""


def test_schemas_are_the_reference_ones():
    for line in SCHEMAS.strip().splitlines():
        name = line.split("(", 1)[0]
        schema = str(getattr(torch.ops.zig_cu_kernels, name).default._schema)
        assert schema == "zig_cu_kernels::" + line, name


def test_fake_kernels_give_the_layouts_of_the_real_ones():
    with FakeTensorMode():
        x = torch.empty(4, 9, 512, device="cuda", dtype=BF16)
        w = torch.empty(384, 512, device="cuda", dtype=BF16)
        weight = torch.empty(512, device="cuda", dtype=BF16)
        a, scale_a = ops.quantize_fp8_rows(x)
        assert a.shape == x.shape and a.dtype == FP8 and scale_a.shape == (36, 4) and scale_a.stride() == (1, 36)
        b, scale_b = ops.quantize_fp8_tiles(w, scale_dtype=E8M0)
        assert b.shape == w.shape and scale_b.shape == (3, 4) and scale_b.dtype == E8M0 and scale_b.is_contiguous()
        out = ops.fp8_gemm(a, b, scale_a, scale_b)
        assert out.shape == (4, 9, 384) and out.dtype == BF16
        out = ops.fp8_gated_gemm(a, b, b, scale_a, scale_b, scale_b)
        assert out.shape == (4, 9, 384) and out.dtype == BF16
        # tensorwise and rowwise scale shapes are accepted
        out = ops.fp8_gemm(a, b, torch.empty((), device="cuda"), torch.empty(1, 1, device="cuda"), use_fast_accum=True)
        assert out.shape == (4, 9, 384)
        out = ops.fp8_gemm(a, b, torch.empty(36, 1, device="cuda"), torch.empty(384, 1, device="cuda"))
        assert out.shape == (4, 9, 384)
        q, scale = ops.quantize_fp8_tensorwise(x)
        assert q.shape == x.shape and q.dtype == FP8 and scale.shape == () and scale.dtype == F32
        y, h = ops.fused_add_rms_norm(x, x, weight, 1e-6)
        assert y.shape == x.shape and y.dtype == BF16 and h.shape == x.shape and h.dtype == BF16
        q, scales, h = ops.fused_add_rms_norm_fp8_quant(x, x, weight, 1e-6, fp8_scaling="block128", fp8_scale_dtype=E8M0)
        assert q.dtype == FP8 and scales.shape == (36, 4) and scales.stride() == (1, 36) and scales.dtype == E8M0
        q, scales = ops.rms_norm_fp8_quant(x, weight, 1e-6, fp8_scaling="rowwise")
        assert q.dtype == FP8 and scales.shape == (36, 1) and scales.dtype == F32
        out = ops.gated_gemm(x, w, w)
        assert out.shape == (4, 9, 384) and out.dtype == BF16


def test_argument_errors_need_no_gpu():
    with FakeTensorMode():
        x = torch.empty(8, 264, device="cuda", dtype=BF16)
        a = torch.empty(8, 256, device="cuda", dtype=FP8)
        b = torch.empty(128, 256, device="cuda", dtype=FP8)
        # dtype, rank and choice checks run on fake tensors too; size checks need real ones
        with pytest.raises(ValueError):
            ops.rms_norm_fp8_quant(x, None, 1e-6, fp8_scaling="bogus")
        with pytest.raises(ValueError):
            ops.rms_norm_fp8_quant(x, None, 1e-6, fp8_scaling="rowwise", fp8_scale_dtype=E8M0)
        with pytest.raises(ValueError):
            ops.fp8_gemm(a, b, torch.empty(8, 2, device="cuda"), torch.empty(1, 2, device="cuda"), activation="relu")
        with pytest.raises(ValueError):
            ops.fp8_gemm(a, b, torch.empty(8, 2, device="cuda").to(BF16), torch.empty(1, 2, device="cuda"))
