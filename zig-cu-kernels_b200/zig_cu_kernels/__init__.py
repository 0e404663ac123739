"""B200-native drop-in for the block-scaled FP8 inference ops of zig-cu-kernels.

`import zig_cu_kernels.torch` registers `torch.ops.zig_cu_kernels.{fp8_gemm, fp8_gated_gemm, quantize_fp8_rows,
quantize_fp8_tiles, fused_add_rms_norm, rms_norm}` and their `_out` variants, backed by `libzck_b200.so`
(hand-written CUDA for sm_100a behind a C ABI). There is no CPU or other-GPU fallback: a missing library raises.
"""

__version__ = "0.1.0"
