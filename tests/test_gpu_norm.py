"""fused_add_rms_norm / rms_norm on the GPU: residual stream bit-exact, norm within the reference's bounds
(3 * 2^-7 relative for BF16 outputs and at most 1 % of elements differing in bits from the PyTorch sequence;
tests/test_rms_norm.py:52-57, :246-276 of the reference)."""

import pytest
import torch

from helpers import BF16, FP8, assert_same_bits, from_golden, same_bits
from oracle import rules

pytestmark = pytest.mark.gpu
F32 = torch.float32
EPS = 1e-6
BF16_BOUND = 3 * 2.0**-7
FP32_EXACT_BOUND = 2.0**-19
FP32_PYTORCH_BOUND = 8 * 2.0**-23
TINY = 2.0**-126
WIDTHS = [8, 64, 136, 256, 264, 520, 1000, 1032, 4088, 4104, 8200, 16384, 16392, 32768]


@pytest.fixture(scope="module")
def ops():
    import zig_cu_kernels.torch as z
    return z


def within(tensor, reference, relative, name):
    error = (tensor.double() - reference.double()).abs()
    allowed = relative * reference.double().abs() + TINY
    assert bool((error <= allowed).all()), f"{name}: max excess {float((error - allowed).max())}"


def test_golden_rows(ops, golden):
    g = golden["norm"]
    differing, total = 0, 0
    for index in range(int(g["norm_cases"])):
        x, other = from_golden(g[f"norm{index}_x"], BF16).cuda(), from_golden(g[f"norm{index}_other"], BF16).cuda()
        w_bf16 = from_golden(g[f"norm{index}_w_bf16"], BF16).cuda()
        w_f32 = from_golden(g[f"norm{index}_w_f32"], F32).cuda()
        y, h = ops.fused_add_rms_norm(x, other, w_bf16, EPS)
        assert_same_bits(h, from_golden(g[f"norm{index}_h"], BF16), "residual_out")
        for weight, zc, key in ((w_bf16, False, "y_bf16"), (None, False, "y_none"), (w_f32, False, "y_f32"),
                                (w_bf16, True, "y_zc")):
            y, _ = ops.fused_add_rms_norm(x, other, weight, EPS, zero_centered=zc)
            expected = from_golden(g[f"norm{index}_{key}"], BF16)
            within(y.cpu(), expected, BF16_BOUND, key)
            differing += int((~same_bits(y.cpu(), expected)).sum())
            total += y.numel()
    assert differing <= 0.01 * total, f"{differing} of {total} BF16 results differ in bits"


NORMS = [
    (BF16, None, False, BF16, False), (BF16, BF16, False, BF16, False), (BF16, F32, False, BF16, False),
    (BF16, BF16, True, BF16, False), (BF16, F32, True, BF16, False), (F32, None, False, F32, False),
    (F32, F32, False, F32, False), (F32, BF16, False, BF16, False), (F32, BF16, False, F32, False),
    (F32, F32, True, F32, False), (BF16, None, False, BF16, True), (BF16, BF16, False, BF16, True),
    (BF16, BF16, True, BF16, True), (F32, BF16, False, BF16, True), (F32, BF16, False, F32, True),
]


@pytest.mark.parametrize("dtype,weight_dtype,zero_centered,out_dtype,residual", NORMS)
def test_norms_meet_the_bounds_of_their_regime(ops, dtype, weight_dtype, zero_centered, out_dtype, residual):
    torch.manual_seed(0)
    differing, total = 0, 0
    for width in WIDTHS:
        weight = None if weight_dtype is None else (torch.randn(width, device="cuda") * 0.5 + 1).to(weight_dtype)
        for rows in (1, 13):
            x = (torch.randn(rows, width, device="cuda") * 2).to(dtype)
            if rows > 1:
                x[rows // 2] = 0
            if residual:
                other = (torch.randn(rows, width, device="cuda") * 2).to(dtype)
                y, h = ops.fused_add_rms_norm(x, other, weight, EPS, zero_centered=zero_centered, out_dtype=out_dtype)
                assert_same_bits(h, x + other, f"residual_out {width} {rows}")
                again = ops.rms_norm(h, weight, EPS, zero_centered=zero_centered, out_dtype=out_dtype)
                assert_same_bits(y, again, f"y against the norm of residual_out {width} {rows}")
            else:
                h = x
                y = ops.rms_norm(x, weight, EPS, zero_centered=zero_centered, out_dtype=out_dtype)
            assert (y.shape, y.dtype) == (x.shape, out_dtype)
            pytorch = rules.rms_norm(h, weight, zero_centered, EPS, out_dtype)
            if out_dtype == BF16:
                within(y, pytorch, BF16_BOUND, f"y against PyTorch {width} {rows}")
                differing += int((~same_bits(y, pytorch)).sum())
                total += y.numel()
            else:
                within(y, rules.rms_norm_exact(h, weight, zero_centered, EPS), FP32_EXACT_BOUND, f"y vs FP64 {width}")
                within(y, pytorch, FP32_PYTORCH_BOUND, f"y vs PyTorch {width}")
    if out_dtype == BF16:
        assert differing <= 0.01 * total, f"{differing} of {total} differ"


def test_config3_norm(ops):
    """BASELINE config 3 front end: x, residual (2, 512, 4096) BF16 seed 2, weight ones, eps 1e-6."""
    generator = torch.Generator().manual_seed(2)
    x = torch.randn(2, 512, 4096, generator=generator).bfloat16().cuda()
    residual = torch.randn(2, 512, 4096, generator=generator).bfloat16().cuda()
    weight = torch.ones(4096, dtype=BF16, device="cuda")
    y, h = ops.fused_add_rms_norm(x, residual, weight, EPS)
    expected_y, expected_h = rules.fused_add_rms_norm(x.cpu(), residual.cpu(), weight.cpu(), EPS)
    assert_same_bits(h, expected_h, "h")
    within(y.cpu(), expected_y, BF16_BOUND, "y")
    assert float((~same_bits(y.cpu(), expected_y)).float().mean()) <= 0.01
    relative = (y.cpu().double() - expected_y.double()).abs().max() / expected_y.double().abs().max()
    assert relative <= 1e-2


def test_exact_aliases_run_in_place_and_overlaps_go_through_temporaries(ops):
    torch.manual_seed(3)
    x = torch.randn(13, 1032, device="cuda", dtype=BF16)
    other = torch.randn(13, 1032, device="cuda", dtype=BF16)
    weight = torch.randn(1032, device="cuda", dtype=BF16)
    y, h = ops.fused_add_rms_norm(x, other, weight, EPS)
    for out_is, h_is in (("x", "other"), ("other", "x"), ("new", "x"), ("x", "new")):
        xs, os_ = x.clone(), other.clone()
        pick = {"x": xs, "other": os_}
        out = pick.get(out_is, torch.empty_like(x))
        h_out = pick.get(h_is, torch.empty_like(x))
        got_y, got_h = ops.fused_add_rms_norm(xs, os_, weight, EPS, out=out, residual_out=h_out)
        assert got_y is out and got_h is h_out
        assert_same_bits(out, y, f"y in {out_is}")
        assert_same_bits(h_out, h, f"h in {h_is}")
    # outputs that overlap an input without being the same view
    buffer = torch.empty(14 * 1032, device="cuda", dtype=BF16)
    xs = buffer[:13 * 1032].view(13, 1032).copy_(x)
    shifted = buffer[1032:].view(13, 1032)
    got_y, got_h = ops.fused_add_rms_norm(xs, other, weight, EPS, out=shifted)
    assert_same_bits(got_y, y, "overlapping out")
    # strided and misaligned inputs and outputs
    wide = torch.randn(13, 2 * 1032 + 8, device="cuda", dtype=BF16)
    xs, os_ = wide[:, 1:1033], wide[:, 1040:2072]
    ey, eh = ops.fused_add_rms_norm(xs.contiguous(), os_.contiguous(), weight, EPS)
    out = torch.empty(13, 2064, device="cuda", dtype=BF16)[:, ::2]
    got_y, got_h = ops.fused_add_rms_norm(xs, os_, weight, EPS, out=out)
    assert_same_bits(got_y.contiguous(), ey, "strided y")
    assert_same_bits(got_h, eh, "strided h")
    with pytest.raises(ValueError, match="share memory"):
        ops.fused_add_rms_norm(x, other, weight, EPS, out=x, residual_out=x)


def test_rows_do_not_depend_on_the_batch(ops):
    torch.manual_seed(4)
    x = torch.randn(257, 4096, device="cuda", dtype=BF16)
    other = torch.randn(257, 4096, device="cuda", dtype=BF16)
    weight = torch.randn(4096, device="cuda", dtype=BF16)
    y, h = ops.fused_add_rms_norm(x, other, weight, EPS)
    for rows in (1, 5, 64):
        y_part, h_part = ops.fused_add_rms_norm(x[100:100 + rows], other[100:100 + rows], weight, EPS)
        assert_same_bits(y_part, y[100:100 + rows], f"{rows} rows")
        assert_same_bits(h_part, h[100:100 + rows], f"{rows} rows")


def test_fp8_output_with_a_given_scale(ops):
    torch.manual_seed(5)
    x = torch.randn(13, 1032, device="cuda", dtype=BF16) * 3
    weight = torch.randn(1032, device="cuda", dtype=BF16)
    scale = torch.tensor(0.0371, device="cuda")
    y = ops.rms_norm(x, weight, EPS)
    q = ops.rms_norm_op(x, weight, scale, EPS, False, FP8)
    expected = (y.float() / scale).clamp(-448, 448).to(FP8)
    assert_same_bits(q, expected, "codes of the BF16 norm")


def test_empty_inputs_and_errors(ops):
    weight = torch.ones(64, device="cuda", dtype=BF16)
    y, h = ops.fused_add_rms_norm(torch.empty(0, 64, device="cuda", dtype=BF16),
                                  torch.empty(0, 64, device="cuda", dtype=BF16), weight, EPS)
    assert y.shape == (0, 64) and h.shape == (0, 64)
    x = torch.ones(2, 64, device="cuda", dtype=BF16)
    with pytest.raises(ValueError, match="multiple of 8"):
        ops.rms_norm(torch.ones(2, 12, device="cuda", dtype=BF16), None, EPS)
    with pytest.raises(ValueError, match="residual must have the shape"):
        ops.fused_add_rms_norm(x, x[:, :32], weight, EPS)
    with pytest.raises(ValueError, match="zero_centered needs a weight"):
        ops.rms_norm(x, None, EPS, zero_centered=True)
    with pytest.raises(TypeError, match="eps must be a Python number"):
        ops.rms_norm(x, None, torch.tensor(1e-6))
    with pytest.raises(OverflowError):
        ops.rms_norm(x, None, 1e39)


# ---- rms_norm_fp8_quant / fused_add_rms_norm_fp8_quant, block128 (the reference's tests/test_rms_norm.py:445-472:
# codes and scales equal the quantizer's rules applied to the BF16 result of the same norm, bit for bit) ------------

E8M0 = torch.float8_e8m0fnu
BLOCK_WIDTHS = [128, 256, 384, 1024, 2048, 4096, 8192, 16384, 32768]


@pytest.mark.parametrize("scale_dtype", [F32, E8M0])
@pytest.mark.parametrize("x_dtype,weight_dtype,zero_centered", [(BF16, BF16, False), (BF16, None, False),
                                                                (BF16, F32, True), (F32, BF16, False)])
def test_block_quantized_outputs_quantize_the_bf16_result(ops, x_dtype, weight_dtype, zero_centered, scale_dtype):
    torch.manual_seed(3)
    for width in BLOCK_WIDTHS:
        if width * (2 if x_dtype == BF16 else 4) > 131072:
            continue
        for rows in (1, 6, 13, 67):
            x = (torch.randn(rows, width, device="cuda") * 3).to(x_dtype)
            other = (torch.randn(rows, width, device="cuda") * 3).to(x_dtype)
            if rows > 1:
                x[rows // 2] = 0
                other[rows // 2] = 0
                x[1, :128] *= 2.0**-20
                other[1, :128] *= 2.0**-20
            weight = None if weight_dtype is None else (torch.randn(width, device="cuda") * 0.5 + 1).to(weight_dtype)
            # plain
            v = ops.rms_norm(x, weight, EPS, zero_centered=zero_centered, out_dtype=BF16)
            q, scales = ops.rms_norm_fp8_quant(x, weight, EPS, fp8_scaling="block128", fp8_scale_dtype=scale_dtype,
                                               zero_centered=zero_centered)
            codes, expected = rules.quantize_rows(v.cpu(), scale_dtype)
            assert_same_bits(q.cpu(), codes, f"codes {width}x{rows}")
            assert_same_bits(scales.cpu(), expected, f"scales {width}x{rows}")
            assert scales.stride() == (1, rows) or scales.shape[1] == 1
            q2, scales2 = ops.quantize_fp8_rows(v, scale_dtype=scale_dtype)
            assert_same_bits(q.cpu(), q2.cpu(), "codes vs quantize_fp8_rows")
            assert_same_bits(scales.cpu(), scales2.cpu(), "scales vs quantize_fp8_rows")
            # fused add
            v, h = ops.fused_add_rms_norm(x, other, weight, EPS, zero_centered=zero_centered, out_dtype=BF16)
            q, scales, h2 = ops.fused_add_rms_norm_fp8_quant(x, other, weight, EPS, fp8_scaling="block128",
                                                             fp8_scale_dtype=scale_dtype, zero_centered=zero_centered)
            codes, expected = rules.quantize_rows(v.cpu(), scale_dtype)
            assert_same_bits(q.cpu(), codes, f"fused codes {width}x{rows}")
            assert_same_bits(scales.cpu(), expected, f"fused scales {width}x{rows}")
            assert_same_bits(h2.cpu(), h.cpu(), "residual_out")


def test_block_quantized_golden_rows(ops, golden):
    """On the golden inputs the fused op stays within the quantizer's rules of ITS norm; where the norm has the bits of
    the PyTorch sequence (the golden one) the codes are the golden codes."""
    g = golden["norm"]
    for index in range(int(g["nq_cases"])):
        x, other = from_golden(g[f"nq{index}_x"], BF16).cuda(), from_golden(g[f"nq{index}_other"], BF16).cuda()
        w = from_golden(g[f"nq{index}_w"], BF16).cuda()
        v, _ = ops.fused_add_rms_norm(x, other, w, EPS)
        golden_v = rules.rms_norm((x + other).cpu(), w.cpu())
        for name, scale_dtype in (("f32", F32), ("e8m0", E8M0)):
            q, scales, _ = ops.fused_add_rms_norm_fp8_quant(x, other, w, EPS, fp8_scaling="block128",
                                                            fp8_scale_dtype=scale_dtype)
            rows_equal = same_bits(v.cpu(), golden_v).reshape(v.shape[0], -1, 128).all(-1)  # per (row, group)
            got = same_bits(q.cpu(), from_golden(g[f"nq{index}_codes_{name}"], FP8)).reshape(v.shape[0], -1, 128).all(-1)
            assert bool((got | ~rows_equal).all()), "a group whose norm has the golden bits has other codes"
            assert float(rows_equal.float().mean()) > 0.5


def test_block_quantized_out_variants_and_errors(ops):
    torch.manual_seed(5)
    rows, width = 9, 512
    x = torch.randn(rows, width, device="cuda", dtype=BF16)
    other = torch.randn(rows, width, device="cuda", dtype=BF16)
    w = torch.randn(width, device="cuda", dtype=BF16)
    q, scales, h = ops.fused_add_rms_norm_fp8_quant(x, other, w, EPS, fp8_scaling="block128")
    # row-major scales_out, strided codes, residual_out aliasing residual
    scales_out = torch.empty(rows, width // 128, device="cuda")
    wide = torch.empty(rows, 2 * width, device="cuda", dtype=FP8)
    residual = other.clone()
    got = ops.fused_add_rms_norm_fp8_quant(x, residual, w, EPS, fp8_scaling="block128", out=wide[:, :width],
                                           scales_out=scales_out, residual_out=residual)
    assert got[0].data_ptr() == wide.data_ptr() and got[1] is scales_out and got[2] is residual
    assert_same_bits(wide[:, :width].cpu(), q.cpu(), "strided codes")
    assert_same_bits(scales_out.cpu(), scales.cpu(), "row-major scales")
    assert_same_bits(residual.cpu(), h.cpu(), "residual in place")
    # leading dimensions
    q3, s3 = ops.rms_norm_fp8_quant(x.reshape(3, 3, width), w, EPS, fp8_scaling="block128")
    q1, s1 = ops.rms_norm_fp8_quant(x, w, EPS, fp8_scaling="block128")
    assert q3.shape == (3, 3, width) and s3.shape == (rows, width // 128)
    assert_same_bits(q3.reshape(rows, width).cpu(), q1.cpu(), "leading dims")
    # tensorwise goes through the given scale
    scale = torch.tensor([0.0123], device="cuda")
    qt, st = ops.rms_norm_fp8_quant(x, w, EPS, fp8_scaling="tensorwise", fp8_scale=scale)
    assert st.data_ptr() == scale.data_ptr() and qt.dtype == FP8
    with pytest.raises(ValueError):
        ops.rms_norm_fp8_quant(x, w, EPS, fp8_scaling="rowwise", fp8_scale_dtype=E8M0)
    with pytest.raises(ValueError):
        ops.rms_norm_fp8_quant(x[:, :264], w[:264], EPS, fp8_scaling="block128")
    with pytest.raises(ValueError):
        ops.rms_norm_fp8_quant(x, w, EPS, fp8_scaling="block128", fp8_scale=scale)
    with pytest.raises(ValueError):
        ops.rms_norm_fp8_quant(x, w, EPS, fp8_scaling="tensorwise")
    with pytest.raises(ValueError):
        ops.rms_norm_fp8_quant(x, w, EPS, fp8_scaling="nope")
    # empty
    q0, s0 = ops.rms_norm_fp8_quant(x[:0], w, EPS, fp8_scaling="block128")
    assert q0.shape == (0, width) and s0.shape == (0, width // 128)


@pytest.mark.parametrize("x_dtype,weight_dtype,zero_centered", [(BF16, BF16, False), (BF16, None, False),
                                                                (BF16, F32, True), (F32, BF16, False)])
def test_rowwise_quantized_outputs_quantize_the_bf16_result(ops, x_dtype, weight_dtype, zero_centered):
    torch.manual_seed(6)
    for width in (8, 64, 136, 256, 1000, 1032, 4104, 8192, 16392, 32768):
        if width * (2 if x_dtype == BF16 else 4) > 131072:
            continue
        for rows in (1, 6, 13, 67):
            x = (torch.randn(rows, width, device="cuda") * 3).to(x_dtype)
            other = (torch.randn(rows, width, device="cuda") * 3).to(x_dtype)
            if rows > 1:
                x[rows // 2] = 0
                other[rows // 2] = 0
            if rows > 6:
                x[5, 3] = float("nan")
            weight = None if weight_dtype is None else (torch.randn(width, device="cuda") * 0.5 + 1).to(weight_dtype)
            v = ops.rms_norm(x, weight, EPS, zero_centered=zero_centered, out_dtype=BF16)
            q, scales = ops.rms_norm_fp8_quant(x, weight, EPS, fp8_scaling="rowwise", zero_centered=zero_centered)
            codes, expected = rules.quantize_rowwise(v.cpu())
            assert scales.shape == (rows, 1) and scales.dtype == F32
            assert_same_bits(scales.cpu(), expected, f"scales {width}x{rows}")
            assert_same_bits(q.cpu(), codes, f"codes {width}x{rows}")
            v, h = ops.fused_add_rms_norm(x, other, weight, EPS, zero_centered=zero_centered, out_dtype=BF16)
            q, scales, h2 = ops.fused_add_rms_norm_fp8_quant(x, other, weight, EPS, fp8_scaling="rowwise",
                                                             zero_centered=zero_centered)
            codes, expected = rules.quantize_rowwise(v.cpu())
            assert_same_bits(scales.cpu(), expected, f"fused scales {width}x{rows}")
            assert_same_bits(q.cpu(), codes, f"fused codes {width}x{rows}")
            assert_same_bits(h2.cpu(), h.cpu(), "residual_out")
