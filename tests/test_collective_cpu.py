"""Host-side logic of the tensor-parallel path on CPU, world_size 2 over gloo: handle
exchange, block sharding of the MLP, and the rank-order reduction contract of the oracle."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import bench
from oracle import mx_oracle as ora


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out):
    import sys
    from pathlib import Path
    root = Path(__file__).resolve().parents[1]
    for p in (root, root / "vllm-mach_b200"):
        sys.path.insert(0, str(p))
    from mach_b200 import collective
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        got = collective.exchange(dist.group.WORLD, bytes([rank]) * 64)
        assert got == [bytes([r]) * 64 for r in range(world)]
        # Tensor-parallel MLP: gate_up column-parallel, down row-parallel, partials all-reduced.
        g = torch.Generator().manual_seed(0)
        hidden, inter, m = 128, 256, 5
        x = torch.randn(m, hidden, generator=g).to(torch.bfloat16)
        w_gu = (0.05 * torch.randn(2 * inter, hidden, generator=g)).to(torch.bfloat16)
        w_d = (0.05 * torch.randn(hidden, inter, generator=g)).to(torch.bfloat16)
        residual = torch.randn(m, hidden, generator=g).to(torch.bfloat16)
        gamma = (0.1 * torch.randn(hidden, generator=g)).to(torch.bfloat16)

        def mlp(start, count):
            gu = torch.cat([w_gu[start:start + count], w_gu[inter + start:inter + start + count]])
            a_c, a_s = ora.quantize_mxfp8(x)
            gate_up = ora.mx_gemm(a_c, a_s, ora.dequantize_mx(*ora.quantize_weight_mxfp8(gu)))
            h_c, h_s = ora.swiglu_quantize(gate_up)
            wd = ora.dequantize_mx(*ora.quantize_weight_mxfp8(w_d[:, start:start + count].contiguous()))
            return ora.mx_gemm(h_c, h_s, wd)

        start, count = bench.shard_blocks(inter, world, rank)
        partial = mlp(start, count)
        gathered = [torch.empty_like(partial) for _ in range(world)]
        dist.all_gather(gathered, partial)
        norm, res = ora.allreduce_rmsnorm(gathered, residual, gamma, 1e-6)
        full_norm, full_res = ora.allreduce_rmsnorm([mlp(0, inter)], residual, gamma, 1e-6)
        rel = float((norm.float() - full_norm.float()).norm() / full_norm.float().norm())
        assert rel < 2e-2, rel
        # Row ownership between norms: the blocks tile [0, m) in rank order, and gathering every
        # rank's owned rows of the residual stream gives back the full tensor.
        first, count = collective.owner_rows(m, dist.group.WORLD)
        spans = [None] * world
        dist.all_gather_object(spans, (first, count))
        assert spans[0][0] == 0 and spans[-1][0] + spans[-1][1] == m
        assert all(a[0] + a[1] == b[0] for a, b in zip(spans, spans[1:]))
        owned = res[first:first + count].contiguous()
        assert torch.equal(collective.gather_owned_rows(owned, m, dist.group.WORLD), res)
        for tokens in (0, 1, 7, 4096):
            f, c = collective.owner_rows(tokens, dist.group.WORLD)
            assert 0 <= f <= tokens and f + c <= tokens and c <= (tokens + world - 1) // world
        out[rank] = (res.float().sum().item(), rel)
    finally:
        dist.destroy_process_group()


def test_two_rank_gloo_tensor_parallel_mlp():
    world = 2
    ctx = mp.get_context("spawn")
    with ctx.Manager() as manager:
        out = manager.dict()
        port = _free_port()
        procs = [ctx.Process(target=_worker, args=(r, world, port, out)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(timeout=300)
            assert p.exitcode == 0
        assert out[0][0] == out[1][0]  # both ranks hold the same reduced residual stream


def test_shard_blocks_cover_the_intermediate_dimension():
    for inter in (9728, 17408, 512):
        for world in (1, 2, 4, 8):
            spans = [bench.shard_blocks(inter, world, r) for r in range(world)]
            assert spans[0][0] == 0
            for (s0, c0), (s1, _) in zip(spans, spans[1:]):
                assert s0 + c0 == s1
            assert spans[-1][0] + spans[-1][1] == inter
            assert all(c % 32 == 0 for _, c in spans)
            assert max(c for _, c in spans) - min(c for _, c in spans) <= 32


def test_oracle_allreduce_rounds_the_sum_before_the_residual():
    # 1 + 2^-8 summed over two ranks is exact in FP32 but rounds in BF16 before the residual
    # is added (native/ar_norm/trtllm_allreduce_fusion_mxfp8.cuh:1470-1494).
    a = torch.tensor([[1.0] * 32], dtype=torch.bfloat16)
    b = torch.tensor([[2.0 ** -8] * 32], dtype=torch.bfloat16)
    residual = torch.tensor([[2.0 ** -8] * 32], dtype=torch.bfloat16)
    gamma = torch.zeros(32, dtype=torch.bfloat16)
    _, res = ora.allreduce_rmsnorm([a, b], residual, gamma, 1e-6)
    assert float(res[0, 0]) == 1.0
