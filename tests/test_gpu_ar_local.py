"""The fused all-reduce + residual + RMSNorm (+ MXFP8) protocols on ONE GPU.

Every rank of a 2/4/8-way group lives on the same device and the ranks run as one cooperative
grid (mach_allreduce_local_ranks): the flag protocol, slot arithmetic, rank-order sum,
rounding points and the owner form's code gather are exactly the multi-GPU ones, only the
"peer" pointers are local. Oracle: oracle.mx_oracle.allreduce_rmsnorm, the restatement of
native/ar_norm/trtllm_allreduce_fusion_mxfp8.cuh:1092-1108,1303-1342,1470-1494. Bars (those of
tests/native_mxfp6/test_moe_ar_norm.py:172-201 made exact where the arithmetic is defined):
residual_out bit-exact, norm within one BF16 ulp, codes and scales bit-exact given the
kernel's own norm.

Also here: the single-rank entry points, and the bounded wait running out (a flag nobody sets).
"""
import ctypes

import pytest
import torch

from oracle import mx_oracle as ora
from tests.gpu_util import LocalRanks, gpu_available, randn_bf16

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not gpu_available(), reason="needs a B200")]

EPS = 1e-6


def _check_rows(tag, norm, res, ref_norm, ref_res):
    assert torch.equal(res.cpu().view(torch.int16), ref_res.view(torch.int16)), tag + " residual_out"
    diff = (norm.float().cpu() - ref_norm.float()).abs()
    assert bool((diff <= ref_norm.float().abs().clamp_min(1e-30) * 2.0 ** -7).all()), \
        tag + f" norm off by {float(diff.max())}"


def _check_codes(tag, codes, scales, norm_full, m, h):
    rc, rs = ora.quantize_mxfp8(norm_full.cpu())
    assert torch.equal(codes.view(torch.uint8).cpu(), rc), tag + " codes"
    assert torch.equal(ora.unswizzle_scales(scales.cpu(), m, h), rs), tag + " scales"


def _inputs(world, m, h, seed):
    partials = [randn_bf16(m, h, seed + r) for r in range(world)]
    residual = randn_bf16(m, h, seed + 99)
    gamma = randn_bf16(1, h, 3, 0.1)[0].contiguous()
    return partials, residual, gamma


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("h", [2560, 5120])
def test_push_forms_all_ranks_on_one_device(world, h):
    from mach_b200 import native
    group = LocalRanks(world, h, 1024)
    try:
        for algo in (1, 2, 3):
            for it, m in enumerate((1, 33, 512, 7, 1000, 512)):
                partials, residual, gamma = _inputs(world, m, h, 1000 * algo + 10 * it + h)
                ref_norm, ref_res = ora.allreduce_rmsnorm(partials, residual, gamma, EPS)
                outs = group.run([p.cuda() for p in partials], [residual.cuda()] * world,
                                 gamma.cuda(), EPS, m, algo=algo)
                assert native.device_status() == 0
                for r, (norm, res, codes, scales) in enumerate(outs):
                    tag = f"world{world} h{h} algo{algo} m{m} rank{r}"
                    _check_rows(tag, norm, res, ref_norm, ref_res)
                    _check_codes(tag, codes, scales, norm, m, h)
    finally:
        group.close()


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("h", [2560, 5120, 2592])
def test_owner_form_all_ranks_on_one_device(world, h):
    """h = 2592: hidden % 128 != 0, the scale gather takes its byte path."""
    from mach_b200 import native
    group = LocalRanks(world, h, 2048)
    try:
        for it, m in enumerate((1, 5, 33, 512, 1000, 2048, 512)):
            partials, residual, gamma = _inputs(world, m, h, 77 * it + h + world)
            ref_norm, ref_res = ora.allreduce_rmsnorm(partials, residual, gamma, EPS)
            rpo = (m + world - 1) // world
            owned = [(min(r * rpo, m), max(0, min(rpo, m - min(r * rpo, m)))) for r in range(world)]
            in_buffer = it % 2 == 1   # alternate: partial tensor / written into the buffer
            in_place = (it // 2) % 2 == 1   # codes and scales read where the owners stored them
            dev_partials = []
            for r in range(world):
                if in_buffer:
                    group.partial_buffer(r, m).copy_(partials[r].cuda())
                    dev_partials.append(None)
                else:
                    dev_partials.append(partials[r].cuda())
            residual_rows = [residual[f:f + c].contiguous().cuda() for f, c in owned]
            outs = group.run(dev_partials, residual_rows, gamma.cuda(), EPS, m, owner=True,
                             in_place=in_place)
            assert native.device_status() == 0
            norm_full = torch.cat([o[0] for o in outs], 0)
            res_full = torch.cat([o[1] for o in outs], 0)
            assert norm_full.shape[0] == m
            tag = f"owner world{world} h{h} m{m}"
            _check_rows(tag, norm_full, res_full, ref_norm, ref_res)
            for r, (_, _, codes, scales) in enumerate(outs):
                _check_codes(tag + f" rank{r}", codes, scales, norm_full, m, h)
    finally:
        group.close()


@pytest.mark.parametrize("algo", [0, 1, 3])
def test_single_rank_workspace(algo):
    from mach_b200 import native
    h = 2560
    group = LocalRanks(1, h, 1024)
    try:
        for m in (1, 33, 513):
            partials, residual, gamma = _inputs(1, m, h, 5 + m)
            ref_norm, ref_res = ora.allreduce_rmsnorm(partials, residual, gamma, EPS)
            x, res_in, g = partials[0].cuda(), residual.cuda(), gamma.cuda()
            norm, res = torch.empty_like(x), torch.empty_like(x)
            codes = torch.empty((m, h), dtype=torch.uint8, device="cuda")
            scales = torch.empty(native.sf_bytes(m, h), dtype=torch.uint8, device="cuda")
            rc = group.lib.mach_allreduce_residual_rmsnorm_mxfp8(
                group.handles[0], x.data_ptr(), res_in.data_ptr(), g.data_ptr(), EPS, 1.0,
                norm.data_ptr(), res.data_ptr(), codes.data_ptr(), scales.data_ptr(), m, h, algo,
                ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
            native._check(rc, "allreduce_rmsnorm")
            torch.cuda.synchronize()
            assert native.device_status() == 0
            _check_rows(f"world1 algo{algo} m{m}", norm, res, ref_norm, ref_res)
            _check_codes(f"world1 algo{algo} m{m}", codes, scales, norm, m, h)
    finally:
        group.close()


@pytest.mark.parametrize("m", [0, 1, 33, 513])
def test_rounded_sum_norm_tail(m):
    """mach_residual_rmsnorm_rounded_mxfp8: the all-reduce's tail on an already reduced sum."""
    from mach_b200 import native
    h = 5120
    partials, residual, gamma = _inputs(1, m, h, 40 + m)
    norm, res, codes, scales = native.add_rmsnorm_mxfp8(
        partials[0].cuda(), residual.cuda(), gamma.cuda(), EPS, 1.0, rounded_sum=True)
    torch.cuda.synchronize()
    if m == 0:
        assert norm.shape == (0, h)
        return
    ref_norm, ref_res = ora.allreduce_rmsnorm(partials, residual, gamma, EPS)
    _check_rows(f"rounded tail m{m}", norm, res, ref_norm, ref_res)
    _check_codes(f"rounded tail m{m}", codes, scales, norm, m, h)


@pytest.mark.parametrize("owner", [False, True])
def test_bounded_wait_runs_out_and_reset_recovers(owner):
    """Rank 0 of a two-rank workspace is launched alone: the flag of rank 1 is never set. The
    wait must end at its limit (1 ms here), record 401, poison the outputs and mark the
    workspace; the next call returns poisoned outputs at once (403); after mach_ar_reset on
    both ranks the group works again."""
    from mach_b200 import native
    h, m = 2560, 16
    group = LocalRanks(2, h, 64)
    lib = group.lib
    try:
        assert native.device_status() == 0
        for hnd in group.handles:
            native._check(lib.mach_ar_set_wait_limit_us(hnd, 1000), "set_wait_limit")
        partials, residual, gamma = _inputs(2, m, h, 321)
        x, g = partials[0].cuda(), gamma.cuda()
        first, count = (0, m // 2) if owner else (0, m)
        res_in = residual[first:first + count].contiguous().cuda()
        stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

        def launch_rank0():
            norm = torch.zeros((count, h), dtype=torch.bfloat16, device="cuda")
            res = torch.zeros((count, h), dtype=torch.bfloat16, device="cuda")
            codes = torch.zeros((m, h), dtype=torch.uint8, device="cuda")
            scales = torch.zeros(native.sf_bytes(m, h), dtype=torch.uint8, device="cuda")
            if owner:
                rc = lib.mach_allreduce_owner_rmsnorm_mxfp8(
                    group.handles[0], x.data_ptr(), res_in.data_ptr(), g.data_ptr(), EPS, 1.0,
                    norm.data_ptr(), res.data_ptr(), codes.data_ptr(), scales.data_ptr(), m, h,
                    stream)
            else:
                rc = lib.mach_allreduce_residual_rmsnorm_mxfp8(
                    group.handles[0], x.data_ptr(), res_in.data_ptr(), g.data_ptr(), EPS, 1.0,
                    norm.data_ptr(), res.data_ptr(), codes.data_ptr(), scales.data_ptr(), m, h, 1,
                    stream)
            native._check(rc, "allreduce")
            torch.cuda.synchronize()
            return norm, res, codes, scales

        norm, res, codes, scales = launch_rank0()
        assert native.device_status() == 401
        assert bool(torch.isnan(norm.float()).all()) and bool(torch.isnan(res.float()).all())
        assert bool((codes == 0x7F).all())
        assert bool((ora.unswizzle_scales(scales.cpu(), m, h) == 0xFF).all())
        # a failed workspace answers at once, poisoned, with its own code
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        norm, res, codes, scales = launch_rank0()
        end.record()
        torch.cuda.synchronize()
        assert start.elapsed_time(end) < 500.0
        assert native.device_status() == 403
        assert bool(torch.isnan(norm.float()).all()) and bool((codes == 0x7F).all())
        # collective reset, then a healthy two-rank call
        for hnd in group.handles:
            native._check(lib.mach_ar_reset(hnd, stream), "ar_reset")
            native._check(lib.mach_ar_set_wait_limit_us(hnd, 1000000), "set_wait_limit")
        ref_norm, ref_res = ora.allreduce_rmsnorm(partials, residual, gamma, EPS)
        if owner:
            rows = [residual[:m // 2].contiguous().cuda(), residual[m // 2:].contiguous().cuda()]
            outs = group.run([p.cuda() for p in partials], rows, g, EPS, m, owner=True)
            norm_full = torch.cat([o[0] for o in outs], 0)
            res_full = torch.cat([o[1] for o in outs], 0)
        else:
            outs = group.run([p.cuda() for p in partials], [residual.cuda()] * 2, g, EPS, m, algo=1)
            norm_full, res_full = outs[0][0], outs[0][1]
        assert native.device_status() == 0
        _check_rows("after reset", norm_full, res_full, ref_norm, ref_res)
        _check_codes("after reset", outs[1][2], outs[1][3], norm_full, m, h)
    finally:
        group.close()


@pytest.mark.parametrize("h", [2560, 5120, 8192])
def test_owner_form_single_rank_prefetch_path(h):
    """One rank owns every row: the per-rank kernel (with the next-row prefetch for hidden <=
    4096, without it above) instead of the single-grid multi-rank launch."""
    from mach_b200 import native
    group = LocalRanks(1, h, 2048)
    lib = group.lib
    try:
        for it, m in enumerate((1, 700, 2048)):
            partials, residual, gamma = _inputs(1, m, h, 1234 + it + h)
            ref_norm, ref_res = ora.allreduce_rmsnorm(partials, residual, gamma, EPS)
            x, res_in, g = partials[0].cuda(), residual.cuda(), gamma.cuda()
            if it % 2:
                group.partial_buffer(0, m).copy_(x)
            norm, res = torch.empty_like(x), torch.empty_like(x)
            codes = torch.empty((m, h), dtype=torch.uint8, device="cuda")
            scales = torch.empty(native.sf_bytes(m, h), dtype=torch.uint8, device="cuda")
            rc = lib.mach_allreduce_owner_rmsnorm_mxfp8(
                group.handles[0], None if it % 2 else x.data_ptr(), res_in.data_ptr(), g.data_ptr(),
                EPS, 1.0, norm.data_ptr(), res.data_ptr(), codes.data_ptr(), scales.data_ptr(), m, h,
                ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
            native._check(rc, "allreduce_owner")
            torch.cuda.synchronize()
            assert native.device_status() == 0
            _check_rows(f"owner world1 h{h} m{m}", norm, res, ref_norm, ref_res)
            _check_codes(f"owner world1 h{h} m{m}", codes, scales, norm, m, h)
    finally:
        group.close()
