"""GPU parity of the stand-alone activation producers, through the C ABI, against the oracle.
Bar: codes and scales bit-exact; normalised values within one BF16 ulp (the FP32 sum of
squares has no canonical order), residual bit-exact."""
import pytest
import torch

from oracle import mx_oracle as ora
from tests.gpu_util import (bytes_equal, edge_activations, gpu_available, mismatch_report,
                            randn_bf16)

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not gpu_available(), reason="needs a B200")]


@pytest.fixture(scope="module")
def nat():
    from mach_b200 import native
    native.lib()
    return native


@pytest.mark.parametrize("m,k", [(1, 32), (1, 2560), (16, 2048), (33, 96), (513, 2560), (4096, 2560)])
def test_mxfp8_quantize_bit_exact(nat, m, k):
    x = edge_activations(m, k, 100 + m) if m < 4096 else randn_bf16(m, k, 5)
    codes, scales = nat.quantize_mxfp8(x.cuda())
    ref_codes, ref_scales = ora.quantize_mxfp8(x)
    assert bytes_equal(codes, ref_codes), mismatch_report(codes, ref_codes)
    got = ora.unswizzle_scales(scales.cpu(), m, k)
    assert torch.equal(got, ref_scales)
    assert torch.equal(nat.unpack_scales(scales, m, k).cpu(), ref_scales)


def test_mxfp8_quantize_zero_after_nonzero(nat):
    x = randn_bf16(16, 256, 1).cuda()
    nat.quantize_mxfp8(x)
    x.zero_()
    codes, scales = nat.quantize_mxfp8(x)
    assert int(codes.view(torch.uint8).max()) == 0
    assert set(ora.unswizzle_scales(scales.cpu(), 16, 256).flatten().tolist()) == {28}


def test_empty_inputs(nat):
    x = torch.empty((0, 256), dtype=torch.bfloat16, device="cuda")
    codes, scales = nat.quantize_mxfp8(x)
    assert codes.shape == (0, 256) and scales.numel() == 0


@pytest.mark.parametrize("m,inter", [(1, 128), (16, 9728), (33, 96), (257, 2560)])
def test_swiglu_quantize_bit_exact(nat, m, inter):
    gate_up = edge_activations(m, 2 * inter, 200 + m)
    if m >= 16:
        gate_up[5] = randn_bf16(1, 2 * inter, 9)[0] * 8.0   # saturating sigmoids
    codes, scales = nat.swiglu_quantize_mxfp8(gate_up.cuda())
    ref_codes, ref_scales = ora.swiglu_quantize(gate_up)
    assert bytes_equal(codes, ref_codes), mismatch_report(codes, ref_codes)
    assert torch.equal(ora.unswizzle_scales(scales.cpu(), m, inter), ref_scales)


@pytest.mark.parametrize("m,h", [(1, 2560), (16, 5120), (33, 128), (300, 2560), (7, 9728)])
def test_add_rmsnorm_mxfp8(nat, m, h):
    x = edge_activations(m, h, 300 + m)
    r = edge_activations(m, h, 301 + m)
    w = randn_bf16(1, h, 302, 0.1)[0].contiguous()
    eps = 1e-6
    norm, res, codes, scales = nat.add_rmsnorm_mxfp8(x.cuda(), r.cuda(), w.cuda(), eps)
    ref_norm, ref_res = ora.gemma_rmsnorm(x, r, w, eps)
    assert bytes_equal(res, ref_res), mismatch_report(res, ref_res)
    diff = (norm.float().cpu() - ref_norm.float()).abs()
    ulp = ref_norm.float().abs().clamp_min(1e-30) * 2.0 ** -7
    assert bool((diff <= ulp).all())
    assert float((diff > 0).float().mean()) < 0.01
    # Quantisation of the kernel's own normalised values is exact.
    ref_codes, ref_scales = ora.quantize_mxfp8(norm.cpu())
    assert bytes_equal(codes, ref_codes), mismatch_report(codes, ref_codes)
    assert torch.equal(ora.unswizzle_scales(scales.cpu(), m, h), ref_scales)


def test_rmsnorm_without_residual_or_quant(nat):
    x = randn_bf16(8, 2560, 1)
    w = randn_bf16(1, 2560, 2, 0.1)[0].contiguous()
    norm, res, codes, scales = nat.add_rmsnorm_mxfp8(x.cuda(), None, w.cuda(), 1e-6,
                                                    want_quant=False)
    assert res is None and codes is None and scales is None
    ref, _ = ora.gemma_rmsnorm(x, None, w, 1e-6)
    diff = (norm.float().cpu() - ref.float()).abs()
    assert bool((diff <= ref.float().abs().clamp_min(1e-30) * 2.0 ** -7).all())


@pytest.mark.parametrize("rows,k", [(1, 32), (130, 2560), (19456, 2560)])
def test_scale_pack_unpack(nat, rows, k):
    logical = torch.randint(0, 255, (rows, k // 32), dtype=torch.uint8)
    packed = nat.pack_scales(logical.cuda(), k)
    assert torch.equal(packed.cpu(), ora.swizzle_scales(logical, k, fill=127))
    assert torch.equal(nat.unpack_scales(packed, rows, k).cpu(), logical)


@pytest.mark.parametrize("m,k", [(1, 128), (19, 384), (512, 2560)])
def test_fp8_group_quantize_bit_exact(nat, m, k):
    x = edge_activations(m, k, 400 + m)
    q, s = nat.fp8_group_quantize(x.cuda())
    ref_q, ref_s = ora.fp8_group_quantize(x)
    assert s.stride() == (1, m) or m == 1
    assert bytes_equal(q, ref_q), mismatch_report(q, ref_q)
    assert bytes_equal(s.contiguous(), ref_s), mismatch_report(s.contiguous(), ref_s)


@pytest.mark.parametrize("m,inter,transposed", [(1, 128, True), (33, 256, False), (64, 9216, True)])
def test_silu_mul_fp8_group_quantize_bit_exact(nat, m, inter, transposed):
    inp = edge_activations(m, 2 * inter, 500 + m)
    q, s = nat.silu_mul_fp8_group_quantize(inp.cuda(), transposed)
    ref_q, ref_s = ora.silu_mul_fp8_group_quantize(inp)
    assert bytes_equal(s.contiguous(), ref_s), mismatch_report(s.contiguous(), ref_s)
    assert bytes_equal(q, ref_q), mismatch_report(q, ref_q)


@pytest.mark.parametrize("m,inter", [(1, 64), (16, 9216), (33, 6144), (513, 256)])
def test_champion_swiglu_contract(nat, m, inter):
    """mach_swiglu_mxfp8_quantize_champion vs the oracle's restatement of
    src/vllm_mach/mxfp8/swiglu_quant.py:46-70 (parity unpinned: see the oracle), over the
    magnitudes of tests/test_mxfp8_swiglu_quant.py:103, bit for bit."""
    import ctypes
    lib = nat.lib()
    base = randn_bf16(m, 2 * inter, 600 + m).float()
    for magnitude in (1.0, 0.0, 1.0e-15, 50.0):
        x = (base * magnitude).to(torch.bfloat16)
        dev = x.cuda()
        codes = torch.empty((m, inter), dtype=torch.uint8, device="cuda")
        scales = torch.zeros(nat.sf_bytes(m, inter), dtype=torch.uint8, device="cuda")
        nat._check(lib.mach_swiglu_mxfp8_quantize_champion(
            dev.data_ptr(), codes.data_ptr(), scales.data_ptr(), m, inter,
            ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)), "champion")
        torch.cuda.synchronize()
        ref_codes, ref_scales = ora.swiglu_quantize_champion(x)
        assert torch.equal(ora.unswizzle_scales(scales.cpu(), m, inter), ref_scales), magnitude
        assert torch.equal(codes.cpu(), ref_codes), magnitude


@pytest.mark.parametrize("m,heads,wdtype", [(1, 24, torch.bfloat16), (16, 24, torch.float32),
                                            (33, 3, torch.bfloat16), (513, 24, torch.bfloat16)])
def test_gated_rmsnorm_producer(nat, m, heads, wdtype):
    """mach_gated_rmsnorm_mxfp8_quantize vs the oracle's restatement of the unfused gated norm
    (parity unpinned: the fused form lives in the absent third-party wheel). The sum of 128
    squares has no canonical order, so a value may differ by one BF16 ulp: fewer than 1 % of
    the codes differ and never by more than one code; scales equal except where such a value
    is the block maximum."""
    core = randn_bf16(m, heads * 128, 900 + m).reshape(m, heads, 128)
    wide = randn_bf16(m, heads * 128 + 64, 901 + m)       # strided gate rows
    gate = wide[:, :heads * 128]
    weight = (1.0 + 0.1 * randn_bf16(1, 128, 902)[0].float()).to(wdtype)
    codes, scales = nat.gated_rmsnorm_quantize(core.cuda(), wide.cuda()[:, :heads * 128],
                                               weight.cuda(), 1e-6)
    torch.cuda.synchronize()
    values = ora.gated_rmsnorm_values(core, gate.contiguous().reshape(m, heads, 128), weight, 1e-6)
    ref_codes, ref_scales = ora.quantize_mxfp8(values)
    got_scales = ora.unswizzle_scales(scales.cpu(), m, heads * 128)
    assert float((got_scales != ref_scales).float().mean()) < 0.01
    same_scale = (got_scales == ref_scales).repeat_interleave(32, 1)
    got, ref = codes.view(torch.uint8).cpu(), ref_codes
    differ = (got != ref) & same_scale
    assert float(differ.float().mean()) < 0.01
    step = (got.to(torch.int16) - ref.to(torch.int16)).abs()
    assert int(step[differ].max() if differ.any() else 0) <= 1


def test_gdn_output_projection_and_projected_adapter(nat):
    """vllm::mach_gdn_norm_mxfp6_out at the reference's shape (24 heads of 128 -> 5120,
    src/vllm_mach/mxfp6/gdn_output.py:21-33) and `projected` at its QKV-like shapes."""
    from mach_b200 import ops
    ops.register()
    ops.set_mxfp6_format("e3m2")
    m, heads, n = 8, 24, 5120
    k = heads * 128
    core = randn_bf16(m, k, 950).reshape(m, heads, 128)
    gate = randn_bf16(m, k, 951)
    weight = (1.0 + 0.1 * randn_bf16(1, 128, 952)[0].float()).bfloat16()
    w = randn_bf16(n, k, 953, 0.02)
    w_codes, w_scales = ora.quantize_weight_mxfp6(w, "e3m2")
    packed_w = ora.pack_fp6(w_codes).cuda()
    packed_s = nat.pack_scales(w_scales.cuda(), k)
    out = torch.ops.vllm.mach_gdn_norm_mxfp6_out(core.cuda(), gate.cuda(), weight.cuda(), packed_w,
                                                 packed_s, 1e-6)
    values = ora.gated_rmsnorm_values(core, gate.reshape(m, heads, 128), weight, 1e-6)
    a_c, a_s = ora.quantize_mxfp8(values)
    ref = ora.mx_gemm(a_c, a_s, ora.dequantize_mxfp6(w_codes, w_scales, "e3m2"))
    assert out.shape == (m, n)
    assert torch.allclose(out.float().cpu(), ref.float(), rtol=0.01, atol=0.02)
    # projected(): activations already quantised by a fused norm
    for (rows, n2, k2) in ((4, 8192, 5120), (32, 3840, 5120)):
        x = randn_bf16(rows, k2, 960 + rows)
        w2 = randn_bf16(n2, k2, 961 + rows, 0.02)
        c2, s2 = ora.quantize_weight_mxfp6(w2, "e3m2")
        codes, scales = nat.quantize_mxfp8(x.cuda())
        y = ops.projected(codes, scales, ora.pack_fp6(c2).cuda(), nat.pack_scales(s2.cuda(), k2))
        rc, rs = ora.quantize_mxfp8(x)
        ref2 = ora.mx_gemm(rc, rs, ora.dequantize_mxfp6(c2, s2, "e3m2"))
        assert torch.allclose(y.float().cpu(), ref2.float(), rtol=0.01, atol=0.02)
