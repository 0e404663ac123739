"""quantize_fp8_rows / quantize_fp8_tiles on the GPU against the golden vectors and the CPU oracle: bit-exact."""

import math

import pytest
import torch

from helpers import BF16, E8M0, FP8, assert_same_bits, from_golden
from oracle import rules

pytestmark = pytest.mark.gpu
SCALES = {"f32": torch.float32, "e8m0": E8M0}
INPUTS = {"f32": torch.float32, "bf16": BF16}


@pytest.fixture(scope="module")
def ops():
    import zig_cu_kernels.torch as z
    return z


@pytest.mark.parametrize("tag", INPUTS)
@pytest.mark.parametrize("stag", SCALES)
def test_rows_match_the_golden_edge_groups(ops, golden, tag, stag):
    g = golden["quantizers"]
    x = from_golden(g[f"rows_x_{tag}"], INPUTS[tag]).cuda()
    q, scales = ops.quantize_fp8_rows(x, scale_dtype=SCALES[stag])
    m, k = x.shape
    assert scales.shape == (m, k // 128) and scales.stride() == (1, m) and scales.dtype == SCALES[stag]
    assert q.dtype == FP8 and q.is_contiguous()
    assert_same_bits(scales, from_golden(g[f"rows_scales_{tag}_{stag}"], SCALES[stag]), "scales")
    assert_same_bits(q, from_golden(g[f"rows_codes_{tag}_{stag}"], FP8), "codes")


@pytest.mark.parametrize("tag", INPUTS)
@pytest.mark.parametrize("stag", SCALES)
@pytest.mark.parametrize("n", (136, 200))
def test_tiles_match_the_golden_edge_groups(ops, golden, tag, stag, n):
    g = golden["quantizers"]
    w = from_golden(g[f"tiles{n}_w_{tag}"], INPUTS[tag]).cuda()
    q, scales = ops.quantize_fp8_tiles(w, scale_dtype=SCALES[stag])
    assert scales.shape == (2, 3) and scales.is_contiguous()
    assert_same_bits(scales, from_golden(g[f"tiles{n}_scales_{tag}_{stag}"], SCALES[stag]), "tile scales")
    assert_same_bits(q, from_golden(g[f"tiles{n}_codes_{tag}_{stag}"], FP8), "tile codes")


@pytest.mark.parametrize("scale_dtype", (torch.float32, E8M0))
def test_rows_handle_strided_batched_and_given_outputs(ops, golden, scale_dtype):
    g = golden["quantizers"]
    wide = from_golden(g["rows_x_bf16"], BF16).cuda()
    cases = {"strided": wide[:, 128:], "batched": wide[:36, :256].reshape(4, 9, 256), "one row": wide[3:4, :384],
             "f32 strided": wide.float()[:, 128:512]}
    for name, x in cases.items():
        expected_q, expected_s = rules.quantize_rows(x.cpu(), scale_dtype)
        q, scales = ops.quantize_fp8_rows(x, scale_dtype=scale_dtype)
        assert_same_bits(q, expected_q, f"{name} codes")
        assert_same_bits(scales, expected_s, f"{name} scales")
        m, groups = expected_s.shape
        # given outputs: codes into a strided view (temporary path), scales into a row-major tensor (temporary path)
        holder = torch.zeros(*x.shape[:-1], 2 * x.shape[-1], device="cuda").to(FP8)
        q_out = holder[..., ::2]
        s_out = torch.empty(m, groups, device="cuda", dtype=scale_dtype)
        got_q, got_s = ops.quantize_fp8_rows(x, scale_dtype=scale_dtype, out=q_out, scales_out=s_out)
        assert got_q is q_out and got_s is s_out
        assert_same_bits(q_out.contiguous(), expected_q, f"{name} codes out")
        assert_same_bits(s_out, expected_s, f"{name} scales out")
        # scales into a padded column-major tensor: written in place, padding untouched
        padded = torch.full((groups, m + 3), 7, device="cuda", dtype=torch.uint8 if scale_dtype == E8M0 else torch.float32)
        view = (padded.view(E8M0) if scale_dtype == E8M0 else padded).t()[:m]
        ops.quantize_fp8_rows(x, scale_dtype=scale_dtype, scales_out=view)
        assert_same_bits(view.contiguous(), expected_s.contiguous(), f"{name} padded scales")
        assert bool((padded[:, m:] == 7).all())


def test_config2_sizes_are_bit_exact(ops):
    """BASELINE config 2: rows on (4096, 4096) and tiles on (11008, 4096), seed 1, FP32 and E8M0 scales."""
    generator = torch.Generator().manual_seed(1)
    x = torch.randn(4096, 4096, generator=generator).bfloat16()
    w = (torch.randn(11008, 4096, generator=generator) / 64).bfloat16()
    for scale_dtype in (torch.float32, E8M0):
        q, s = ops.quantize_fp8_rows(x.cuda(), scale_dtype=scale_dtype)
        assert s.shape == (4096, 32)
        eq, es = rules.quantize_rows(x, scale_dtype)
        assert_same_bits(s, es, "row scales")
        assert_same_bits(q, eq, "row codes")
        q, s = ops.quantize_fp8_tiles(w.cuda(), scale_dtype=scale_dtype)
        assert s.shape == (86, 32)
        eq, es = rules.quantize_tiles(w, scale_dtype)
        assert_same_bits(s, es, "tile scales")
        assert_same_bits(q, eq, "tile codes")


@pytest.mark.parametrize("dtype", (torch.float32, BF16))
def test_wide_dynamic_range_inside_groups_is_bit_exact(ops, dtype):
    """Values spread over 40 binades inside every group, scales over 80 binades across groups: the quotients land on
    every kind of E4M3 rounding boundary, underflow and zero, which pins the kernels' division against x / scale."""
    generator = torch.Generator().manual_seed(17)
    rows, k = 2048, 1024
    magnitude = torch.exp2(-40 * torch.rand(rows, k, generator=generator))
    group_scale = torch.exp2(torch.randint(-40, 41, (rows, k // 128, 1), generator=generator).float())
    x = (torch.randn(rows, k, generator=generator) * magnitude).reshape(rows, k // 128, 128) * group_scale
    x = x.reshape(rows, k).to(dtype)
    q, s = ops.quantize_fp8_rows(x.cuda())
    eq, es = rules.quantize_rows(x)
    assert_same_bits(s, es, "row scales")
    assert_same_bits(q, eq, "row codes")
    q, s = ops.quantize_fp8_tiles(x.cuda())
    eq, es = rules.quantize_tiles(x)
    assert_same_bits(s, es, "tile scales")
    assert_same_bits(q, eq, "tile codes")


def test_quantizers_are_idempotent_on_their_own_output_at_full_size(ops):
    """Size-independent property at the largest hot-path size (16384 x 8192): dequantised codes re-quantize to the
    same codes and scales with power-of-two (E8M0) scales."""
    x = torch.randn(16384, 8192, device="cuda", dtype=BF16)
    q, s = ops.quantize_fp8_rows(x, scale_dtype=E8M0)
    deq = (q.float().reshape(16384, 64, 128) * s.float()[..., None]).reshape(16384, 8192)
    q2, s2 = ops.quantize_fp8_rows(deq, scale_dtype=E8M0)
    # the amax of a group can only shrink or stay; where the scale stays the codes must stay
    same = (s2.view(torch.uint8) == s.view(torch.uint8))
    assert same.float().mean() > 0.9
    mask = same[..., None].expand(16384, 64, 128).reshape(16384, 8192)
    assert bool((q2.view(torch.uint8)[mask] == q.view(torch.uint8)[mask]).all())


def test_empty_inputs_and_errors(ops):
    q, s = ops.quantize_fp8_rows(torch.empty(0, 256, device="cuda", dtype=BF16))
    assert q.shape == (0, 256) and s.shape == (0, 2)
    q, s = ops.quantize_fp8_tiles(torch.empty(0, 128, device="cuda", dtype=BF16))
    assert q.shape == (0, 128) and s.shape == (0, 1)
    with pytest.raises(ValueError, match="multiple of 128"):
        ops.quantize_fp8_rows(torch.empty(4, 100, device="cuda", dtype=BF16))
    with pytest.raises(ValueError, match="scale_dtype"):
        ops.quantize_fp8_rows(torch.empty(4, 128, device="cuda", dtype=BF16), scale_dtype=torch.float16)
    with pytest.raises(ValueError):
        ops.quantize_fp8_rows(torch.empty(4, 128, device="cuda", dtype=torch.float16))
    with pytest.raises(ValueError, match="matrix"):
        ops.quantize_fp8_tiles(torch.empty(2, 4, 128, device="cuda", dtype=BF16))
    assert math.prod(q.shape) == 0


# ---- quantize_fp8_tensorwise / quantize_fp8_static (the reference's tests/test_fp8_gemm.py:284-306) -----------------

@pytest.mark.parametrize("dtype", (torch.bfloat16, torch.float32))
def test_tensorwise_quantizers_are_bitwise_equal_to_the_rules(ops, dtype):
    import math
    generator = torch.Generator(device="cuda").manual_seed(2)
    full = (torch.randn(37, 200, device="cuda", generator=generator) * 30).to(dtype)
    big = (torch.randn(4096, 8192, device="cuda", generator=generator) * 3).to(dtype)
    cases = {"matrix": full[:, :192], "vector": full.flatten()[:1000], "batched": full[:36].reshape(4, 9, 200),
             "zeros": torch.zeros(64, 128, device="cuda", dtype=dtype), "underflow": full[:4, :64] * 1e-44,
             "nan": torch.where(full == full.max(), math.nan, full),
             "infinity": torch.where(full == full.min(), -math.inf, full), "large": big,
             "empty rows": torch.empty(2, 0, 16, device="cuda", dtype=dtype),
             "empty matrix": torch.empty(3, 0, device="cuda", dtype=dtype)}
    given = torch.full((1, 1), 0.0371, device="cuda")
    for name, x in cases.items():
        q, scale = ops.quantize_fp8_tensorwise(x)
        codes, expected = rules.quantize_tensorwise(x.cpu())
        assert scale.shape == () and scale.dtype == torch.float32 and q.shape == x.shape, name
        assert_same_bits(scale.cpu(), expected, f"{name}: scale")
        assert_same_bits(q.cpu(), codes, f"{name}: codes")
        q, returned = ops.quantize_fp8_tensorwise(x, given)
        assert returned.shape == () and returned.data_ptr() == given.data_ptr()
        assert_same_bits(q.cpu(), rules.quantize_tensorwise(x.cpu(), given.cpu())[0], f"{name}: given scale codes")
    # outputs given by the caller, a strided destination, and the errors
    x = full[:, :192]
    wide = torch.empty(37, 400, device="cuda", dtype=FP8)
    scale_out = torch.empty(1, device="cuda")
    q, scale = ops.quantize_fp8_tensorwise(x, out=wide[:, :192], scale_out=scale_out)
    assert q.data_ptr() == wide.data_ptr() and scale.data_ptr() == scale_out.data_ptr()
    assert_same_bits(q.cpu(), rules.quantize_tensorwise(x.cpu())[0], "strided codes")
    with pytest.raises(ValueError):
        ops.quantize_fp8_tensorwise(full[:, :13])
    with pytest.raises(ValueError):
        ops.quantize_fp8_tensorwise(x, given, scale_out=scale_out)
    with pytest.raises(ValueError):
        ops.quantize_fp8_tensorwise(x, torch.ones(2, device="cuda"))
