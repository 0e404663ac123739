"""Host-side logic of the tensor-parallel MLP, on CPU: shard bounds, the chunked exchange plan, and the equality of the
rank-sharded computation with the unsharded one over real `gloo` ranks (world size 2) running the CPU oracle."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import rules
from zig_cu_kernels.tp_mlp import exchange_plan, shard_bounds


def test_shard_bounds_are_multiples_of_the_scale_group():
    for world in (1, 2, 4, 8):
        edges = [shard_bounds(28672, rank, world) for rank in range(world)]
        assert edges[0][0] == 0 and edges[-1][1] == 28672
        assert all(lo % 128 == 0 and hi % 128 == 0 for lo, hi in edges)
        assert all(a[1] == b[0] for a, b in zip(edges, edges[1:]))
    with pytest.raises(ValueError):
        shard_bounds(28672 + 128, 0, 8)


def test_exchange_plan_covers_every_row_once():
    for m, world, chunks in ((16384, 8, 4), (16384, 2, 7), (64, 8, 4), (4096, 4, 1)):
        plan = exchange_plan(m, world, chunks, "all_reduce")
        assert plan[0][0] == 0 and plan[-1][1] == m
        assert all(a[1] == b[0] for a, b in zip(plan, plan[1:]))
        assert all((lo, hi) == (rlo, rhi) for lo, hi, rlo, rhi in plan)
        assert len(plan) <= chunks
    plan = exchange_plan(16384, 8, 4, "reduce_scatter")
    assert [hi - lo for lo, hi, _, _ in plan] == [4096] * 4
    assert [(rlo, rhi) for _, _, rlo, rhi in plan] == [(0, 512), (512, 1024), (1024, 1536), (1536, 2048)]
    with pytest.raises(ValueError):
        exchange_plan(16384, 8, 4, "broadcast")
    assert len(exchange_plan(64, 8, 4, "all_reduce")) == 1  # a decode batch is never chunked


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank(rank, world, port, exchange, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(2)
    generator = torch.Generator().manual_seed(4)
    m, hidden, inter = 32, 256, 512
    tokens = torch.randn(m, hidden, generator=generator).bfloat16()
    w_gate = (torch.randn(inter, hidden, generator=generator) / 16).bfloat16()
    w_up = (torch.randn(inter, hidden, generator=generator) / 16).bfloat16()
    w_down = (torch.randn(hidden, inter, generator=generator) / 22).bfloat16()
    partial = rules.mlp_shard(tokens, w_gate, w_up, w_down, rank, world)
    whole = rules.mlp(tokens, w_gate, w_up, w_down).float()
    if exchange == "all_reduce":
        total = partial.float()  # gloo has no BF16 sum; the sum of BF16 partials is taken in FP32
        dist.all_reduce(total)
        mine = whole
    else:
        plan = exchange_plan(m, world, 1, "reduce_scatter")
        (lo, hi, rlo, rhi), = plan
        pieces = list(partial.float().chunk(world))
        total = torch.empty_like(pieces[0])
        dist.reduce_scatter(total, pieces) if dist.get_backend() != "gloo" else None
        if dist.get_backend() == "gloo":  # gloo lacks reduce_scatter: all_reduce and keep this rank's share
            full = partial.float()
            dist.all_reduce(full)
            total = full.chunk(world)[rank]
        mine = whole.chunk(world)[rank]
    error = float((total - mine).abs().max() / whole.abs().max())
    results[rank] = error
    dist.destroy_process_group()


@pytest.mark.parametrize("exchange", ("all_reduce", "reduce_scatter"))
def test_two_gloo_ranks_sum_to_the_unsharded_mlp(exchange):
    world, port = 2, _free_port()
    manager = mp.get_context("spawn").Manager()
    results = manager.dict()
    mp.spawn(_rank, args=(world, port, exchange, results), nprocs=world, join=True)
    assert len(results) == world
    assert all(error <= 1e-2 for error in results.values()), dict(results)
