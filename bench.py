"""Benchmark of the block-scaled FP8 hot path: the Llama-70B-shaped SwiGLU MLP prefill (tokens (16384, 8192) BF16,
intermediate 28672, FP32 block scales), tensor-parallel over N GPUs of one node.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

A step is one forward pass over all tokens: quantize_fp8_rows -> fp8_gated_gemm (SwiGLU) -> quantize_fp8_rows ->
fp8_gemm, then (N > 1) the sum of the BF16 partials over NVLink. Rank 0 prints ONE JSON line. `value` is tokens/s with
the tokens resident in HBM; `e2e` is the same with the tokens copied from pinned host memory and the result read
back inside the timed region. `--impl reference` times the CPU restatement of the reference's torch path instead.
"""

import argparse
import json
import os
import pathlib
import statistics
import subprocess
import sys
import time

ROOT = pathlib.Path(__file__).resolve().parent
for entry in (ROOT / "zig-cu-kernels_b200", ROOT):
    if str(entry) not in sys.path:
        sys.path.insert(0, str(entry))

import torch  # noqa: E402

M, HIDDEN, INTER = 16384, 8192, 28672
SEED = 4
FLOPS_PER_TOKEN = 6 * HIDDEN * INTER
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
CPU_SAMPLE_TOKENS = 128
# DRAM bytes of one gated-GEMM launch on 4096 tokens (one band of the tile walk), dram__bytes_read.sum +
# dram__bytes_write.sum from the ncu capture summarised in profiles/fp8_gemm_kernel_4096_tokens_dram_traffic.md.
# A 16384-token launch walks four such bands, each streaming the weights once, so its traffic is four times this.
GATED_TRAFFIC_PER_4096_TOKENS = 640222976 + 226347008


def peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        return json.loads(path.read_text()), "measured"
    return dict(FALLBACK_PEAKS), "fallback"


def synthetic(device, rows=M):
    """Config-5 tensors: tokens ~ N(0,1), w_gate_up ~ N(0,1)/90, w_down ~ N(0,1)/170, BF16, seed 4 (same on all ranks)."""
    generator = torch.Generator(device=device).manual_seed(SEED)
    tokens = torch.randn(rows, HIDDEN, device=device, generator=generator).bfloat16()
    w_gate = (torch.randn(INTER, HIDDEN, device=device, generator=generator) / 90).bfloat16()
    w_up = (torch.randn(INTER, HIDDEN, device=device, generator=generator) / 90).bfloat16()
    w_down = (torch.randn(HIDDEN, INTER, device=device, generator=generator) / 170).bfloat16()
    return tokens, w_gate, w_up, w_down


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while a timed region runs."""

    FIELDS = ("timestamp,clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.process = None
        try:
            self.process = subprocess.Popen(
                ["nvidia-smi", f"--id={index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "20"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            pass

    def stop(self, begin=None, end=None):
        """Summary of the samples taken between the wall-clock times `begin` and `end` (all samples when None)."""
        if self.process is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.process.terminate()
        try:
            text, _ = self.process.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.process.kill()
            text, _ = self.process.communicate()
        clocks, maxima, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in text.splitlines():
            parts = [part.strip() for part in line.split(",")]
            if len(parts) != 7 or not parts[1].isdigit():
                continue
            try:
                stamp = time.mktime(time.strptime(parts[0][:19], "%Y/%m/%d %H:%M:%S")) + float("0" + parts[0][19:])
            except ValueError:
                continue
            if begin is not None and not (begin - 0.02 <= stamp <= end + 0.02):
                continue
            clocks.append(int(parts[1]))
            maxima.append(int(parts[2]))
            reasons.update(name for name, flag in zip(names, parts[3:]) if flag == "Active")
        if not clocks:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        return {"sm_mhz": statistics.median(clocks), "sm_max_mhz": max(maxima), "reasons": sorted(reasons),
                "samples": len(clocks)}


def cpu_reference_tokens_per_s(sample_tokens, repeats, warmup=0):
    """The CPU restatement of the reference's torch path (oracle/rules.py) on the first `sample_tokens` tokens of the
    workload, all host threads: rows-quantize, dequantise, FP32 matmuls, SwiGLU epilogue, rows-quantize, down."""
    from oracle import rules

    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    tokens, w_gate, w_up, w_down = synthetic("cpu", rows=sample_tokens)
    gate, s_gate = rules.quantize_tiles(w_gate)
    up, s_up = rules.quantize_tiles(w_up)
    down, s_down = rules.quantize_tiles(w_down)
    del w_gate, w_up, w_down

    def step():
        a, s_a = rules.quantize_rows(tokens)
        act = rules.fp8_gated_gemm(a, gate, up, s_a, s_gate, s_up, dtype=torch.float32)
        q, s_q = rules.quantize_rows(act)
        return rules.fp8_gemm(q, down, s_q, s_down, dtype=torch.float32)

    for _ in range(warmup):
        step()
    times = []
    for _ in range(repeats):
        start = time.perf_counter()
        step()
        times.append(time.perf_counter() - start)
    return sample_tokens / statistics.median(times), threads, statistics.median(times)


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    rate, threads, seconds = cpu_reference_tokens_per_s(CPU_SAMPLE_TOKENS, max(1, args.steps), min(args.warmup, 3))
    sample = f"first {CPU_SAMPLE_TOKENS} of {M} tokens per step, weights quantized once outside the timed region"
    print(json.dumps({
        "impl": "reference", "metric": "tp_mlp_tokens_per_s", "value": rate, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": seconds * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "fp8_e4m3", "data": "synthetic",
        "config": workload_config(args.gpus),
        "cpu_baseline": {"value": rate, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": rate, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def workload_config(gpus, exchange="reduce_scatter"):
    return {"workload": f"llama70b_swiglu_mlp_prefill M={M} H={HIDDEN} I={INTER} fp32 block128 scales (BASELINE config 5)",
            "global_batch_tokens": M, "parallelism": f"tp{gpus}", "exchange": exchange if gpus > 1 else "none",
            "l2": "weights (705 MB FP8) and activations exceed the 126 MB L2, no flush needed"}


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=10)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", default="ours", choices=("ours", "reference"))
    parser.add_argument("--chunks", type=int, default=1, help="token chunks whose exchange overlaps the next GEMMs")
    parser.add_argument("--exchange", default="reduce_scatter", choices=("reduce_scatter", "all_reduce"))
    parser.add_argument("--e2e-chunks", type=int, default=4, help="token chunks of the pipelined end-to-end step")
    parser.add_argument("--skip-e2e", action="store_true", help="profiling runs: leave the end-to-end step out")
    parser.add_argument("--no-graphs", action="store_true", help="launch every op from Python instead of replaying CUDA graphs")
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--tokens", type=int, default=M, help="token rows per step (smaller only for profiling)")
    args = parser.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    args.warmup = max(3, args.warmup)
    tokens_per_step = args.tokens

    import torch.distributed as dist

    import zig_cu_kernels.torch as ops  # noqa: F401  (fails loudly when libzck_b200.so is missing)
    from zig_cu_kernels.tp_mlp import TensorParallelMLP

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE is {world}: launch with torch.distributed.run")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    tokens, w_gate, w_up, w_down = synthetic(device, rows=tokens_per_step)
    mlp = TensorParallelMLP(w_gate, w_up, w_down, rank, world, chunks=args.chunks if world > 1 else 1,
                            exchange=args.exchange)
    del w_gate, w_up, w_down
    torch.cuda.empty_cache()
    # End-to-end step: every rank owns tokens_per_step / world rows in pinned host memory (ordered chunk after chunk),
    # copies them to the device, the ranks all-gather the token matrix over NVLink, run the MLP and each reads back what
    # the exchange left it (its rows after reduce_scatter, all rows after all_reduce). The step is pipelined over
    # --e2e-chunks token chunks: upload of chunk c+1 and download of chunk c-1 run under the kernels of chunk c.
    own = tokens_per_step // world
    out_rows = own if (world > 1 and args.exchange == "reduce_scatter") else tokens_per_step
    staged = torch.empty_like(tokens)
    device_step = mlp.graphed(tokens) if not args.no_graphs else (lambda: mlp.forward(tokens))
    pipelined = (lambda *_: None) if args.skip_e2e else mlp.graphed(staged, chunks=args.e2e_chunks)
    if args.skip_e2e:
        pipelined.finish = lambda: None
    pinned_in = torch.empty(own, HIDDEN, dtype=tokens.dtype).pin_memory()
    from zig_cu_kernels.tp_mlp import exchange_plan
    offset = 0
    for lo, hi, _, _ in exchange_plan(tokens_per_step, world, args.e2e_chunks, args.exchange):
        rows = (hi - lo) // world
        pinned_in[offset:offset + rows].copy_(tokens[lo + rank * rows:lo + (rank + 1) * rows])
        offset += rows
    pinned_out = torch.empty(out_rows, HIDDEN, dtype=tokens.dtype).pin_memory()

    def e2e_step():
        return pipelined(pinned_in, pinned_out)

    e2e_step.finish = pipelined.finish

    def eager_step():
        return mlp.forward(tokens)

    def timed(step, steps):
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        start.record()
        for _ in range(steps):
            step()
        if hasattr(step, "finish"):
            step.finish()  # copies on the side streams belong to the timed region
        end.record()
        barrier()
        seconds = torch.tensor([start.elapsed_time(end) * 1e-3], device=device, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(seconds, op=dist.ReduceOp.MAX)
        return float(seconds)

    sampler = ClockSampler(local) if rank == 0 else None  # started early: nvidia-smi needs a moment to come up
    for _ in range(args.warmup):
        device_step()
        e2e_step()
    barrier()
    wall_begin = time.time()
    device_seconds = timed(device_step, args.steps)
    wall_end = time.time()
    e2e_seconds = timed(e2e_step, args.steps)
    clocks = sampler.stop(wall_begin, wall_end) if sampler else None
    # Kernel durations for the roofline: the same K steps once more, launched op by op with CUDA events around each
    # kernel (events cannot sit inside a replayed graph).
    launches_before = mlp.launches
    mlp.kernel_events = {}
    timed(eager_step, args.steps)
    events, mlp.kernel_events = mlp.kernel_events, None
    launches = mlp.launches - launches_before  # the kernels of one pass of K steps (a replay launches the same)

    kernel_ms = {name: statistics.mean(start.elapsed_time(end) for start, end in pairs) for name, pairs in events.items()}
    launches_per_step = {name: len(pairs) // args.steps for name, pairs in events.items()}
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    measured, source = peaks()
    # FP8 runs at twice the BF16 rate on the tcgen05 pipe; the denominator is twice the measured sustained cuBLAS BF16
    # rate (the GEMM is timed inside a long step under the power cap).
    fp8_peak = 2.0 * measured["bf16_tflops_sustained"]
    gated_flops = 4.0 * tokens_per_step * (INTER // world) * HIDDEN / launches_per_step["gated_gemm"]
    gated_tflops = gated_flops / (kernel_ms["gated_gemm"] * 1e-3) / 1e12
    down_flops = 2.0 * tokens_per_step * HIDDEN * (INTER // world) / launches_per_step["down_gemm"]
    down_tflops = down_flops / (kernel_ms["down_gemm"] * 1e-3) / 1e12
    rows_bytes = (tokens_per_step / launches_per_step["quantize_tokens"]) * HIDDEN * (2 + 1 + 4 / 128)
    rows_gbs = rows_bytes / (kernel_ms["quantize_tokens"] * 1e-3) / 1e9
    result = {
        "metric": "tp_mlp_tokens_per_s", "value": tokens_per_step * args.steps / device_seconds, "unit": "tokens/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": device_seconds / args.steps * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "fp8_e4m3", "data": "synthetic",
        "config": dict(workload_config(world, args.exchange), tokens_per_step=tokens_per_step, chunks=args.chunks,
                       launch="python ops" if args.no_graphs else "cuda graph replay of the kernels, NCCL calls between replays"),
        "tflops": tokens_per_step * FLOPS_PER_TOKEN * args.steps / device_seconds / 1e12,
        "e2e": None if args.skip_e2e else {"value": tokens_per_step * args.steps / e2e_seconds, "unit": "tokens/s", "ms_per_step": e2e_seconds / args.steps * 1e3,
                "h2d_bytes_per_step": own * HIDDEN * 2 * world,
                "d2h_bytes_per_step": out_rows * HIDDEN * 2 * world},
        "gpu_launches": launches,
        "clocks": clocks,
        "roofline": {"kernel": "fp8_gemm_kernel<gated> (fp8_gated_gemm)", "bound": "tensor", "achieved": gated_tflops,
                     "peak": fp8_peak, "unit": "TFLOP/s", "frac": gated_tflops / fp8_peak,
                     "traffic": (GATED_TRAFFIC_PER_4096_TOKENS * (tokens_per_step // 4096)
                                 if world == 1 and tokens_per_step % 4096 == 0 and launches_per_step["gated_gemm"] == 1
                                 else None),
                     "algorithmic_bytes": tokens_per_step * HIDDEN + 2 * (INTER // world) * HIDDEN +
                     2 * tokens_per_step * (INTER // world),
                     "peak_source": f"2 x bf16_tflops_sustained of {source} MEASURED_PEAKS.json"},
        "kernels": {"gated_gemm_tflops": gated_tflops, "down_gemm_tflops": down_tflops,
                    "quantize_rows_gbs": rows_gbs, "hbm_peak_gbs": measured["hbm_gbs"],
                    "ms": kernel_ms, "launches_per_step": launches_per_step},
    }
    if world == 1 and not args.no_cpu_baseline:
        rate, threads, seconds = cpu_reference_tokens_per_s(CPU_SAMPLE_TOKENS, 5)
        result["cpu_baseline"] = {"value": rate, "unit": "tokens/s", "cores": threads, "kind": "port",
                                  "sample": f"first {CPU_SAMPLE_TOKENS} of {M} tokens, median of 5 passes of {seconds:.1f} s; "
                                            "weights quantized once outside the timed region"}
    print(json.dumps(result))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
