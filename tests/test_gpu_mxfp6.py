"""GPU parity of the W6A8 path: MXFP8 activations x packed MXFP6 (E2M3 / E3M2) weights.
The 6-bit codes travel packed (4 codes per 3 bytes) through TMA, which expands them to one
byte per code in shared memory for tcgen05.mma kind::mxf8f6f4. Bar: rtol 0.01 / atol 0.02 and
relative Frobenius error <= 1e-2 against dequantise -> FP32 matmul."""
import pytest
import torch

from oracle import mx_oracle as ora
from tests.gpu_util import bytes_equal, gpu_available, mismatch_report, randn_bf16, rel_fro

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not gpu_available(), reason="needs a B200")]


@pytest.fixture(scope="module")
def nat():
    from mach_b200 import native
    native.lib()
    return native


def mxfp6_weight(n, k, seed, fmt, sigma=0.015):
    w = randn_bf16(n, k, seed, sigma)
    codes, scales = ora.quantize_weight_mxfp6(w, fmt)
    return ora.pack_fp6(codes), scales, ora.dequantize_mxfp6(codes, scales, fmt)


@pytest.mark.parametrize("fmt", ["e2m3", "e3m2"])
def test_fp6_decode_through_identity_activations(nat, fmt):
    """One-hot activations read the weight back: out[i, n] == dequantised W[n, i]."""
    n = k = 128
    packed, scales, deq = mxfp6_weight(n, k, 1, fmt, sigma=1.0)
    eye = torch.eye(k, dtype=torch.bfloat16)
    a, sa = nat.quantize_mxfp8(eye.cuda())
    out = nat.mx_gemm(a, sa, packed.cuda(), nat.pack_scales(scales.cuda(), k), fmt=fmt)
    torch.cuda.synchronize()
    assert nat.device_status() == 0
    assert torch.equal(out.float().cpu(), deq.t().to(torch.bfloat16).float())


@pytest.mark.parametrize("fmt", ["e2m3", "e3m2"])
@pytest.mark.parametrize("m,n,k", [(1, 256, 128), (32, 5120, 2176), (64, 2176, 5120), (512, 4352, 5120),
                                   (300, 640, 384),
                                   # one token tile (49..128 tokens, wide matrix), and a narrow
                                   # matrix at 256 tokens (feature-major, receive slots in the ring)
                                   (100, 9728, 256), (128, 19456, 128), (256, 640, 384)])
def test_w6a8_gemm(nat, fmt, m, n, k):
    x = randn_bf16(m, k, 5000 + m)
    packed, scales, deq = mxfp6_weight(n, k, 5001 + m, fmt)
    a_c, a_s = ora.quantize_mxfp8(x)
    ref = ora.mx_gemm(a_c, a_s, deq)
    a, sa = nat.quantize_mxfp8(x.cuda())
    out = nat.mx_gemm(a, sa, packed.cuda(), nat.pack_scales(scales.cuda(), k), fmt=fmt)
    torch.cuda.synchronize()
    assert nat.device_status() == 0
    assert torch.allclose(out.float().cpu(), ref.float(), rtol=0.01, atol=0.02)
    assert rel_fro(out, ref) <= 1e-2


@pytest.mark.parametrize("m,inter,k", [(16, 1088, 640), (200, 1088, 640), (1024, 1088, 640),
                                       (100, 4864, 256)])   # the last: one-token-tile kernel
def test_w6a8_fused_swiglu(nat, m, inter, k):
    fmt = "e2m3"
    x = randn_bf16(m, k, 6000 + m)
    packed, scales, _ = mxfp6_weight(2 * inter, k, 6001 + m, fmt, sigma=0.05)
    a, sa = nat.quantize_mxfp8(x.cuda())
    wi = nat.interleave_gate_up(packed.cuda())
    si = nat.pack_scales(nat.interleave_gate_up(scales.cuda()), k)
    gate_up = nat.mx_gemm(a, sa, wi, si, fmt=fmt, layout=nat.LAYOUT_GATE_UP_32)
    codes, sc = nat.mx_gemm_swiglu(a, sa, wi, si, fmt=fmt, layout=nat.LAYOUT_GATE_UP_32)
    torch.cuda.synchronize()
    assert nat.device_status() == 0
    ref_codes, ref_scales = ora.swiglu_quantize(gate_up.cpu())
    assert torch.equal(ora.unswizzle_scales(sc.cpu(), m, inter), ref_scales)
    assert bytes_equal(codes, ref_codes), mismatch_report(codes, ref_codes)
