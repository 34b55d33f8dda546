"""The checkpoint weight quantiser on the B200 and the loaders, through the C ABI, against
the oracle (pinned to the reference's golden vector and to quantize_block itself):
codes and scales bit for bit; a converted checkpoint loads into kernel layout and the MLP it
describes matches the oracle."""
import pytest
import torch
from safetensors.torch import save_file

from oracle import mx_oracle as ora
from tests.gpu_util import gpu_available, randn_bf16, rel_fro

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not gpu_available(), reason="needs a B200")]


@pytest.mark.parametrize("n,k,sigma", [(1, 32, 1.0), (64, 2560, 0.02), (513, 96, 0.02), (2560, 9728, 0.015)])
def test_weight_quantiser_bit_exact(n, k, sigma):
    from mach_b200 import checkpoint
    w = randn_bf16(n, k, 7000 + n, sigma)
    if n > 2:
        w[1] = 0                                   # an all-zero row: scale byte 0
        w[2, :32] = torch.tensor([1.7421875, -1.7421875] * 16).bfloat16()   # golden-vector blocks
        w[2, 32:64] = torch.tensor([1.75, -1.75] * 16).bfloat16()
        w[2, 64:96] = torch.tensor([448.0, -448.0] * 16).bfloat16()
    codes, scales = checkpoint.quantize_weight_mxfp8(w.cuda())
    ref_codes, ref_scales = ora.quantize_weight_mxfp8(w)
    assert torch.equal(scales.cpu(), ref_scales)
    assert torch.equal(codes.view(torch.uint8).cpu(), ref_codes)
    if n > 2:
        assert scales[2, :3].tolist() == [119, 120, 128] and int(scales[1].max()) == 0


def test_converted_checkpoint_loads_and_runs(tmp_path):
    from mach_b200 import checkpoint
    from mach_b200.mlp import mlp_forward
    hidden, inter, m = 512, 1024, 40
    tensors = {
        "model.layers.0.mlp.gate_proj.weight": randn_bf16(inter, hidden, 1, 0.05),
        "model.layers.0.mlp.up_proj.weight": randn_bf16(inter, hidden, 2, 0.05),
        "model.layers.0.mlp.down_proj.weight": randn_bf16(hidden, inter, 3, 0.05),
    }
    src = tmp_path / "bf16.safetensors"
    save_file(tensors, str(src))
    out = tmp_path / "mxfp8"
    summary = checkpoint.convert_bf16_to_mxfp8(src, out)
    assert summary["quantised"] == 3
    reader = checkpoint.CheckpointReader(out)
    weights = checkpoint.load_mx_mlp(reader, "model.layers.0.mlp")
    x = randn_bf16(m, hidden, 4)
    got = mlp_forward(x.cuda(), weights)
    torch.cuda.synchronize()
    gu = torch.cat([tensors["model.layers.0.mlp.gate_proj.weight"],
                    tensors["model.layers.0.mlp.up_proj.weight"]], 0)
    w_gu = ora.dequantize_mx(*ora.quantize_weight_mxfp8(gu))
    w_d = ora.dequantize_mx(*ora.quantize_weight_mxfp8(tensors["model.layers.0.mlp.down_proj.weight"]))
    a_c, a_s = ora.quantize_mxfp8(x)
    h_c, h_s = ora.swiglu_quantize(ora.mx_gemm(a_c, a_s, w_gu))
    ref = ora.mx_gemm(h_c, h_s, w_d)
    assert rel_fro(got, ref) < 0.005
    w, s, k, kind = checkpoint.load_mx_linear(reader, "model.layers.0.mlp.down_proj")
    assert kind == "mxfp8" and k == inter and w.shape == (hidden, inter)
