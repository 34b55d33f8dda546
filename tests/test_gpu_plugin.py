"""The adapter classes and custom ops on a GPU: load-time packing, apply_weights against the
oracle, and the reference's capture/replay pattern (warm up, capture a CUDA graph, change the
inputs in place including all-zeros, replay; tests/native_mxfp6/test_mxfp8_sm120.py:40-58,
tests/native_mxfp6/test_mxfp8_mlp.py:37-59)."""
import pytest
import torch

from oracle import mx_oracle as ora
from tests.gpu_util import gpu_available, mxfp8_weight, randn_bf16, rel_fro

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not gpu_available(), reason="needs a B200")]


class Layer(torch.nn.Module):
    def __init__(self, weight, weight_scale):
        super().__init__()
        self.weight = torch.nn.Parameter(weight, requires_grad=False)
        self.weight_scale = torch.nn.Parameter(weight_scale, requires_grad=False)
        self.params_dtype = torch.bfloat16


def test_is_supported_on_b200():
    from mach_b200 import linear
    assert linear.Mxfp8B200LinearKernel.is_supported() == (True, None)
    assert linear.Mxfp6B200LinearKernel.is_supported(100) == (True, None)
    assert linear.Mxfp6B200LinearKernel.is_supported(120)[0] is False


def test_mxfp8_kernel_apply_and_graph_replay():
    from mach_b200 import linear
    n, k = 512, 256
    codes, scales, deq = mxfp8_weight(n, k, 1)
    layer = Layer(codes.view(torch.float8_e4m3fn).cuda(), scales.cuda())
    kernel = object.__new__(linear.Mxfp8B200LinearKernel)
    kernel.process_weights_after_loading(layer)
    assert layer.weight_scale.numel() == 512 * 2 * 4 and not layer.weight.requires_grad
    x = randn_bf16(16, k, 2).cuda()
    bias = randn_bf16(1, n, 3)[0].cuda()

    def ref(xc):
        a_c, a_s = ora.quantize_mxfp8(xc.cpu())
        return ora.mx_gemm(a_c, a_s, deq).float() + bias.float().cpu()

    y = kernel.apply_weights(layer, x.reshape(2, 8, k), bias)
    assert y.shape == (2, 8, n) and y.dtype == torch.bfloat16
    assert torch.allclose(y.reshape(16, n).float().cpu(), ref(x), rtol=0.01, atol=0.02)
    # capture, then change the input in place and replay
    static_x = x.clone()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        kernel.apply_weights(layer, static_x, bias)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        static_y = kernel.apply_weights(layer, static_x, bias)
    for new in (randn_bf16(16, k, 9).cuda() * 3.0, torch.zeros_like(x)):
        static_x.copy_(new)
        graph.replay()
        torch.cuda.synchronize()
        assert torch.allclose(static_y.float().cpu(), ref(new), rtol=0.01, atol=0.02)


def test_mxfp6_kernel_apply():
    from mach_b200 import linear
    n, k = 256, 384
    w = randn_bf16(n, k, 4, 0.02)
    codes, scales = ora.quantize_weight_mxfp6(w, "e3m2")
    layer = Layer(ora.pack_fp6(codes).cuda(), scales.cuda())
    kernel = object.__new__(linear.Mxfp6B200LinearKernel)
    kernel.process_weights_after_loading(layer)
    x = randn_bf16(5, k, 5)
    y = kernel.apply_weights(layer, x.cuda())
    a_c, a_s = ora.quantize_mxfp8(x)
    ref = ora.mx_gemm(a_c, a_s, ora.dequantize_mxfp6(codes, scales, "e3m2"))
    assert torch.allclose(y.float().cpu(), ref.float(), rtol=0.01, atol=0.02)


def test_fused_ops_match_the_oracle():
    from mach_b200 import native, ops
    ops.register()
    m, hidden, inter = 24, 256, 512
    x, r = randn_bf16(m, hidden, 6), randn_bf16(m, hidden, 7)
    norm_w = randn_bf16(1, hidden, 8, 0.1)[0].contiguous()
    gu_c, gu_s, gu_d = mxfp8_weight(2 * inter, hidden, 9, 0.05)
    d_c, d_s, d_d = mxfp8_weight(hidden, inter, 10, 0.05)
    gu_w, gu_ws = gu_c.view(torch.float8_e4m3fn).cuda(), native.pack_scales(gu_s.cuda(), hidden)
    d_w, d_ws = d_c.view(torch.float8_e4m3fn).cuda(), native.pack_scales(d_s.cuda(), inter)
    gate_up, summed = torch.ops.vllm.mach_norm_quant_mxfp8_gate_up(
        x.cuda(), r.cuda(), norm_w.cuda(), 1e-6, gu_w, gu_ws)
    y_ref, res_ref = ora.gemma_rmsnorm(x, r, norm_w, 1e-6)
    assert torch.equal(summed.cpu().view(torch.int16), res_ref.view(torch.int16))
    a_c, a_s = ora.quantize_mxfp8(y_ref)
    assert rel_fro(gate_up, ora.mx_gemm(a_c, a_s, gu_d)) < 0.005
    out = torch.ops.vllm.mach_swiglu_mxfp8_down(gate_up, d_w, d_ws)
    h_c, h_s = ora.swiglu_quantize(gate_up.cpu())
    assert rel_fro(out, ora.mx_gemm(h_c, h_s, d_d)) < 0.005
    norm, res = torch.ops.vllm.mach_gemma_norm(x.cuda(), r.cuda(), norm_w.cuda(), 1e-6)
    assert torch.equal(res.cpu().view(torch.int16), res_ref.view(torch.int16))
    assert rel_fro(norm, y_ref) < 0.002


def test_block_fp8_adapter():
    from mach_b200 import linear, ops
    from tests.test_gpu_block_fp8 import block_fp8_weight
    ops.register()
    n, k = 256, 512
    b, sb = block_fp8_weight(n, k, 11)
    w = b.view(torch.float8_e4m3fn).cuda()
    for m in (4, 40):
        x = randn_bf16(m, k, 12 + m)
        y = linear.BlockFp8B200Linear.apply(w, sb.cuda(), x.cuda())
        q, sa = ora.fp8_group_quantize(x)
        ref = ora.block_fp8_gemm(q, sa, b, sb)
        assert rel_fro(y, ref) < 0.005


def test_native_extension_ops_of_the_reference():
    """mach_fp8_activation::run, vllm_mach_block_fp8::mm and mach_norm_quant::run with the
    argument conventions of native/fp8_activation/activation.cu:60-104,
    native/block_fp8/block_fp8.cu:233-262 and native/ar_norm/binding.cu:11-80."""
    import os
    import torch.distributed as dist
    from mach_b200 import collective, native, ops
    from tests.test_gpu_block_fp8 import block_fp8_weight
    ops.register()
    # ---- SiLU * up + 1x128 FP8 quantisation straight into the caller's tensors
    m, inter = 24, 512
    gate_up = randn_bf16(m, 2 * inter, 31)
    ref_q, ref_s = ora.silu_mul_fp8_group_quantize(gate_up)
    for transposed in (True, False):
        out = torch.zeros((m, inter), dtype=torch.float8_e4m3fn, device="cuda")
        if transposed:
            scales = torch.zeros((inter // 128, m), dtype=torch.float32, device="cuda").t()
        else:
            scales = torch.zeros((m, inter // 128), dtype=torch.float32, device="cuda")
        torch.ops.mach_fp8_activation.run(out, gate_up.cuda(), scales, transposed)
        assert torch.equal(out.view(torch.uint8).cpu(), ref_q)
        assert torch.equal(scales.cpu(), ref_s)
    with pytest.raises(RuntimeError):
        torch.ops.mach_fp8_activation.run(out, gate_up.cuda().float(), scales, False)
    # ---- block-FP8 GEMM with the weight and its scales passed as [K, N] views
    n, k = 256, 512
    b, sb = block_fp8_weight(n, k, 32)
    x = randn_bf16(16, k, 33)
    q, sa = native.fp8_group_quantize(x.cuda())
    weight = b.view(torch.float8_e4m3fn).cuda()
    y = torch.ops.vllm_mach_block_fp8.mm(q, weight.t(), sa, sb.cuda().t())
    sb64 = sb.repeat_interleave(2, 0).cuda()          # the reference's 64-row variant of the scales
    y64 = torch.ops.vllm_mach_block_fp8.mm(q, weight.t(), sa, sb64.t())
    rq, rsa = ora.fp8_group_quantize(x)
    ref = ora.block_fp8_gemm(rq, rsa, b, sb)
    assert rel_fro(y, ref) < 0.005 and torch.equal(y, y64)
    # ---- all-reduce + residual + norm + MXFP8 on a one-rank group
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29533")
        dist.init_process_group("gloo", rank=0, world_size=1)
    try:
        group = dist.group.WORLD
        h, rows = 2560, 12
        hidden = randn_bf16(rows, h, 34)
        residual, gamma = randn_bf16(rows, h, 35), randn_bf16(1, h, 36, 0.1)[0].contiguous()
        ws = collective.workspace_tensor(group, h, rows, "cuda:0")
        assert collective.workspace_tensor(group, h, rows, "cuda:0") is ws
        hid = hidden.cuda()
        norm = torch.empty_like(hid)
        codes = torch.empty((rows, h), dtype=torch.uint8, device="cuda")
        scales = torch.empty(native.sf_bytes(rows, h), dtype=torch.uint8, device="cuda")
        # residual_out aliases hidden, as the reference's caller does
        torch.ops.mach_norm_quant.run(hid, residual.cuda(), gamma.cuda(), ws, norm, hid, codes,
                                      scales, 0, 1e-6, True)
        torch.cuda.synchronize()
        ref_norm, ref_res = ora.allreduce_rmsnorm([hidden], residual, gamma, 1e-6)
        assert torch.equal(hid.cpu().view(torch.int16), ref_res.view(torch.int16))
        assert rel_fro(norm, ref_norm) < 0.002
        rc, rs = ora.quantize_mxfp8(norm.cpu())
        assert torch.equal(codes.cpu(), rc)
        assert torch.equal(ora.unswizzle_scales(scales.cpu(), rows, h), rs)
        with pytest.raises(RuntimeError):
            torch.ops.mach_norm_quant.run(hid, residual.cuda(), gamma.cuda(),
                                          torch.zeros(7, dtype=torch.int64, device="cuda"), norm,
                                          hid, codes, scales, 0, 1e-6, True)
        assert torch.ops.mach_norm_quant.abi() == "ar-norm-mxfp8-b200-v1"
    finally:
        collective.close_all()
        dist.destroy_process_group()


def test_moe_shims_and_experts_class():
    """The staged shims (route -> grouped_gemm -> silu_grouped_gemm -> reduce), the whole-layer
    shim and the experts class give what `experts_forward` gives, and match the oracle
    (rtol = atol = 0.03, tests/native_mxfp6/test_moe.py:248)."""
    import types
    from mach_b200 import moe, ops
    from mach_b200.experts import Mxfp6B200Experts
    ops.register()
    ops.set_mxfp6_format("e2m3")
    try:
        m, experts, hidden, inter, top_k, fmt = 77, 8, 256, 128, 2, "e2m3"
        x = randn_bf16(m, hidden, 41)
        logits = randn_bf16(m, experts, 42)
        parts = [(ora.quantize_weight_mxfp6(randn_bf16(2 * inter, hidden, 50 + e, 0.05), fmt),
                  ora.quantize_weight_mxfp6(randn_bf16(hidden, inter, 70 + e, 0.05), fmt))
                 for e in range(experts)]
        w1 = torch.stack([ora.pack_fp6(p[0][0]) for p in parts]).cuda()
        s1 = torch.stack([p[0][1] for p in parts]).cuda()
        w2 = torch.stack([ora.pack_fp6(p[1][0]) for p in parts]).cuda()
        s2 = torch.stack([p[1][1] for p in parts]).cuda()
        topk_w, topk_ids = moe.router_topk(logits.cuda(), top_k)
        ref = ora.moe_forward(x, lambda e: ora.dequantize_mxfp6(*parts[e][0], fmt),
                              lambda e: ora.dequantize_mxfp6(*parts[e][1], fmt),
                              topk_w.cpu(), topk_ids.cpu())
        xd = x.cuda()
        # whole-layer shim
        out = torch.zeros_like(xd)
        dummy = torch.empty(1, device="cuda")
        torch.ops.vllm.mxfp6_sm120_qwen35_grouped_moe(out, xd, w1, s1, w2, s2, topk_w, topk_ids,
                                                      dummy, dummy)
        assert torch.allclose(out.float().cpu(), ref.float(), rtol=0.03, atol=0.03)
        # experts class
        cls_out = torch.zeros_like(xd)
        obj = object.__new__(Mxfp6B200Experts)
        obj.quant_config = types.SimpleNamespace(w1_scale=s1, w2_scale=s2)
        obj.apply(cls_out, xd, w1, w2, topk_w, topk_ids, "silu", experts, None, None, None, None,
                  None, None, False)
        assert torch.equal(cls_out, out)
        # staged shims
        codes, logical = torch.ops.vllm.mxfp6_sm120_quantize_mxfp8(xd)
        rc, rs = ora.quantize_mxfp8(x)
        assert torch.equal(codes.view(torch.uint8).cpu(), rc) and torch.equal(logical.cpu(), rs)
        rows = moe.permuted_rows(m, top_k, experts)
        permuted = torch.zeros((rows, hidden), dtype=torch.float8_e4m3fn, device="cuda")
        packed, expert_offsets, scale_offsets, inverse = torch.ops.vllm.mxfp6_sm120_route(
            permuted, codes, logical, topk_ids, None, experts)
        counts = torch.bincount(topk_ids.flatten().cpu(), minlength=experts)
        assert expert_offsets.cpu().tolist() == [0] + counts.cumsum(0).tolist()
        padded = ((counts + 127) // 128 * 128).cumsum(0).tolist()
        assert scale_offsets.cpu().tolist() == [0] + padded
        gemm1 = torch.zeros((rows, 2 * inter), dtype=torch.bfloat16, device="cuda")
        torch.ops.vllm.mxfp6_sm120_grouped_gemm(gemm1, permuted, packed, w1, s1, expert_offsets,
                                                scale_offsets)
        gemm2 = torch.zeros((rows, hidden), dtype=torch.bfloat16, device="cuda")
        torch.ops.vllm.mxfp6_sm120_silu_grouped_gemm(gemm2, gemm1, w2, s2, expert_offsets,
                                                     scale_offsets)
        staged = torch.zeros_like(xd)
        torch.ops.vllm.mxfp6_sm120_reduce(staged, gemm2, topk_w, inverse)
        torch.cuda.synchronize()
        assert torch.allclose(staged.float().cpu(), ref.float(), rtol=0.03, atol=0.03)
        with pytest.raises(ValueError):
            torch.ops.vllm.mxfp6_sm120_route(permuted[: m * top_k], codes, logical, topk_ids, None,
                                             experts)
    finally:
        ops.set_mxfp6_format("e3m2")


def test_warmup_walks_the_layers():
    from mach_b200 import linear, warmup
    n, k = 256, 256
    codes, scales, _ = mxfp8_weight(n, k, 91)
    layer = Layer(codes.view(torch.float8_e4m3fn).cuda(), scales.cuda())
    kernel = object.__new__(linear.Mxfp8B200LinearKernel)
    kernel.process_weights_after_loading(layer)
    layer.scheme = type("Scheme", (), {"kernel": kernel})()
    model = torch.nn.Sequential(layer)
    assert warmup.warmup(model, [1, 16, 16, 300]) == 3
    assert warmup.warmup_shapes([(256, 256)], [8, 700]) == 2
