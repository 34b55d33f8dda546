"""The allocation-free entry point mach_block_fp8_gemm_ordered_static, through the C ABI.

Some callers cannot hand the library a scratch buffer: a serving worker that gave all free
HBM to its KV cache cannot count on a late cudaMalloc, and a plain C host has no caching
allocator to ask. For them the ordered block-FP8 GEMM has a variant whose scratch is an 8 MiB
array inside the library. This test calls it twice in a row on different inputs and requires
the bytes of each result to equal what the caller-scratch entry point produces; it also checks
that an oversized problem is refused instead of overrunning the array. The file name sorts
last so a run that stops at the first failure has already executed every other test.
"""
import ctypes

import pytest
import torch

from tests.gpu_util import gpu_available, randn_bf16

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not gpu_available(), reason="needs a B200")]


def _weight(n, k, seed):
    w = randn_bf16(n, k, seed, 0.02).float()
    scale = w.abs().amax().clamp_min(1e-10) / 448.0
    q = (w / scale).clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8)
    sb = torch.full(((n + 127) // 128, k // 128), float(scale), dtype=torch.float32)
    return q, sb


def test_static_scratch_matches_caller_scratch_twice_in_a_row():
    from mach_b200 import native
    lib = native.lib()
    n, k = 2560, 2048
    b, sb = _weight(n, k, 1)
    b, sb = b.cuda(), sb.cuda()
    for call, (m, seed) in enumerate(((8, 11), (5, 12))):
        x = randn_bf16(m, k, seed) * (1.0 + call)
        q, sa = native.fp8_group_quantize(x.cuda())
        raw = torch.empty((k // 128, m, n), dtype=torch.float32, device="cuda")
        expected = native.block_fp8_gemm(q, sa, b, sb, raw=raw)
        out = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
        stream = torch.cuda.current_stream().cuda_stream
        rc = lib.mach_block_fp8_gemm_ordered_static(
            q.data_ptr(), b.data_ptr(), sa.data_ptr(), sb.data_ptr(), out.data_ptr(), m, n, k,
            ctypes.c_void_p(stream))
        assert rc == 0, lib.mach_last_error().decode()
        torch.cuda.synchronize()
        assert native.device_status() == 0
        # Same kernels, same order of operations: the results agree bit for bit (tolerance 0).
        assert torch.equal(out.view(torch.int16), expected.view(torch.int16)), f"call {call}"
        assert float(out.float().abs().max()) > 0.0


def test_static_scratch_refuses_oversized_problems():
    from mach_b200 import native
    lib = native.lib()
    m, n, k = 64, 9728, 9728  # 76 * 64 * 9728 * 4 B = 189 MB > 8 MiB
    dummy = torch.zeros(16, dtype=torch.uint8, device="cuda")
    rc = lib.mach_block_fp8_gemm_ordered_static(
        dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(),
        m, n, k, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 2
    assert b"exceeds the built-in scratch" in lib.mach_last_error()


def test_static_scratch_at_its_limit():
    """A problem that fills the built-in array almost completely (16 x 51 x 2560 x 4 B =
    8 355 840 of 8 388 608 bytes) must still match the caller-scratch route bit for bit, and
    one row more (8 519 680 bytes) must be refused: the accept/refuse boundary sits where the
    header says it does, and a nearly full array does not overrun."""
    from mach_b200 import native
    lib = native.lib()
    n, k = 2560, 2048
    b, sb = _weight(n, k, 3)
    b, sb = b.cuda(), sb.cuda()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for m, accepted in ((51, True), (52, False)):
        x = randn_bf16(m, k, 20 + m)
        q, sa = native.fp8_group_quantize(x.cuda())
        out = torch.zeros((m, n), dtype=torch.bfloat16, device="cuda")
        rc = lib.mach_block_fp8_gemm_ordered_static(
            q.data_ptr(), b.data_ptr(), sa.data_ptr(), sb.data_ptr(), out.data_ptr(), m, n, k, stream)
        if not accepted:
            assert rc == 2 and b"exceeds the built-in scratch" in lib.mach_last_error()
            continue
        assert rc == 0, lib.mach_last_error().decode()
        raw = torch.empty((k // 128, m, n), dtype=torch.float32, device="cuda")
        expected = native.block_fp8_gemm(q, sa, b, sb, raw=raw)
        torch.cuda.synchronize()
        assert native.device_status() == 0
        assert torch.equal(out.view(torch.int16), expected.view(torch.int16))
