"""Shared helpers of the tests: bit views, golden decoding, the any-NaN-equals-any-NaN comparison of the reference
(tests/checks.py:40-42 there)."""

import numpy as np
import torch

FP8 = torch.float8_e4m3fn
E8M0 = torch.float8_e8m0fnu
BF16 = torch.bfloat16
BITS = {1: torch.uint8, 2: torch.int16, 4: torch.int32, 8: torch.int64}


def from_golden(array, dtype):
    """Tensor of `dtype` from the bit-preserving numpy array of a golden file."""
    tensor = torch.from_numpy(np.ascontiguousarray(array))
    if dtype in (FP8, E8M0):
        return tensor.view(dtype)
    if dtype == BF16:
        return tensor.view(BF16)
    return tensor.to(dtype) if tensor.dtype != dtype else tensor


def same_bits(tensor, expected):
    bits = BITS[tensor.element_size()]
    return (tensor.contiguous().view(bits) == expected.contiguous().view(bits)) | (
        tensor.float().isnan() & expected.float().isnan())


def assert_same_bits(tensor, expected, name=""):
    assert tensor.shape == expected.shape, f"{name}: shape {tuple(tensor.shape)} != {tuple(expected.shape)}"
    assert tensor.dtype == expected.dtype, f"{name}: dtype {tensor.dtype} != {expected.dtype}"
    bad = ~same_bits(tensor.cpu(), expected.cpu())
    if bad.any():
        index = bad.nonzero()[0].tolist()
        raise AssertionError(f"{name}: {int(bad.sum())} of {bad.numel()} elements differ, first at {index}: "
                             f"{tensor.cpu()[tuple(index)].float().item()} != {expected.cpu()[tuple(index)].float().item()}")


def max_relative_error(out, reference):
    """max |out - ref| / max |ref|: the 1e-2 tolerance of the hot path is stated on this figure."""
    out, reference = out.double().cpu(), reference.double().cpu()
    return float((out - reference).abs().max() / reference.abs().max().clamp_min(1e-30))
