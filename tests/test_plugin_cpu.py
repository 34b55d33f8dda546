"""Plugin-side contract on CPU with stand-in layers and a stand-in vLLM registry, the way the
reference's CPU tests exercise it (tests/test_fp8_linear_cpu.py:15-142,
tests/test_mxfp8_native_cpu.py:174-215)."""
import types

import pytest
import torch

from mach_b200 import linear, ops, plugin


class Layer:
    def __init__(self, weight, weight_scale, params_dtype=torch.bfloat16):
        self.weight = torch.nn.Parameter(weight, requires_grad=False)
        self.weight_scale = torch.nn.Parameter(weight_scale, requires_grad=False)
        self.params_dtype = params_dtype


def test_is_supported_never_raises_and_reports_a_reason():
    for cls in (linear.Mxfp8B200LinearKernel, linear.Mxfp6B200LinearKernel):
        ok, reason = cls.is_supported(120)       # the reference's SM120: not ours
        assert ok is False and "sm_100" in reason
        ok, reason = cls.is_supported()          # no GPU in this process
        assert ok is False and isinstance(reason, str)


def test_registration_prepends_once():
    cuda = object()
    registry = types.SimpleNamespace(_POSSIBLE_MXFP6_KERNELS={cuda: ["stock6"]},
                                     _POSSIBLE_MXFP8_KERNELS={cuda: ["stock8"]})
    assert plugin.register_dense_kernels(registry, cuda) == {"mxfp6": True, "mxfp8": True}
    plugin.register_dense_kernels(registry, cuda)
    assert registry._POSSIBLE_MXFP8_KERNELS[cuda] == [linear.Mxfp8B200LinearKernel, "stock8"]
    assert registry._POSSIBLE_MXFP6_KERNELS[cuda] == [linear.Mxfp6B200LinearKernel, "stock6"]
    assert plugin.register_dense_kernels(types.SimpleNamespace(), cuda) == {"mxfp6": False, "mxfp8": False}


def test_mxfp8_weight_contract_violations():
    kernel = object.__new__(linear.Mxfp8B200LinearKernel)  # vLLM's base wants a config
    good_w = torch.zeros((128, 256), dtype=torch.float8_e4m3fn)
    good_s = torch.zeros((128, 8), dtype=torch.uint8)
    for w, s, dt in ((torch.zeros((100, 256), dtype=torch.float8_e4m3fn), good_s, torch.bfloat16),
                     (torch.zeros((128, 256), dtype=torch.uint8), good_s, torch.bfloat16),
                     (good_w, torch.zeros((128, 4), dtype=torch.uint8), torch.bfloat16),
                     (good_w, good_s, torch.float16)):
        with pytest.raises(ValueError):
            kernel.process_weights_after_loading(Layer(w, s, dt))
    layer = Layer(good_w, good_s)
    with pytest.raises(ValueError):
        kernel.apply_weights(layer, torch.zeros((4, 128), dtype=torch.bfloat16))     # K mismatch
    with pytest.raises(ValueError):
        kernel.apply_weights(layer, torch.zeros((4, 256), dtype=torch.float16))      # dtype
    out = kernel.apply_weights(layer, torch.zeros((0, 256), dtype=torch.bfloat16))   # empty batch
    assert out.shape == (0, 128)
    out = kernel.apply_weights(layer, torch.zeros((2, 0, 256), dtype=torch.bfloat16))
    assert out.shape == (2, 0, 128)


def test_mxfp6_shape_rules():
    assert linear.logical_weight_shape(torch.zeros((16, 96), dtype=torch.uint8)) == (16, 128)
    for shape in ((16, 100), (12, 96), (16, 48), (16,)):
        with pytest.raises(ValueError):
            linear.logical_weight_shape(torch.zeros(shape, dtype=torch.uint8))
    kernel = object.__new__(linear.Mxfp6B200LinearKernel)
    layer = Layer(torch.zeros((16, 96), dtype=torch.uint8), torch.zeros((16, 4), dtype=torch.uint8))
    with pytest.raises(ValueError):
        kernel.apply_weights(layer, torch.zeros((3, 256), dtype=torch.bfloat16))
    assert kernel.apply_weights(layer, torch.zeros((0, 128), dtype=torch.bfloat16)).shape == (0, 16)
    cfg = types.SimpleNamespace(weight_quant_key="kMxfp6E3M2Static", activation_quant_key="kMxfp8Dynamic")
    assert linear.Mxfp6B200LinearKernel.can_implement(cfg) == (True, None)
    cfg.activation_quant_key = "kFp8Static"
    assert linear.Mxfp6B200LinearKernel.can_implement(cfg)[0] is False


def test_block_fp8_eligibility():
    w = torch.zeros((2560, 4096), dtype=torch.float8_e4m3fn)
    s = torch.zeros((20, 32), dtype=torch.float32)
    assert linear.BlockFp8B200Linear.eligible(w, s)
    assert not linear.BlockFp8B200Linear.eligible(w, s[:10])
    with pytest.raises(ValueError):
        linear.BlockFp8B200Linear.apply(w, s, torch.zeros((2, 128), dtype=torch.bfloat16))
    assert linear.BlockFp8B200Linear.apply(w, s, torch.zeros((0, 4096), dtype=torch.bfloat16)).shape == (0, 2560)


def test_custom_ops_are_defined_with_fake_impls_that_keep_the_batch_symbolic():
    ops.register()
    ops.register()  # idempotent
    assert "vllm::mach_mxfp8_sm120_gemm" in ops.op_names()
    x = torch.empty((7, 256), dtype=torch.bfloat16, device="meta")
    w = torch.empty((128, 256), dtype=torch.float8_e4m3fn, device="meta")
    s = torch.empty((4096,), dtype=torch.uint8, device="meta")
    assert torch.ops.vllm.mach_mxfp8_sm120_gemm(x, w, s).shape == (7, 128)
    w6 = torch.empty((128, 192), dtype=torch.uint8, device="meta")
    assert torch.ops.vllm.mach_mxfp6_sm120_gemm(x, w6, s, 128, torch.bfloat16).shape == (7, 128)
    gate_up = torch.empty((7, 512), dtype=torch.bfloat16, device="meta")
    assert torch.ops.vllm.mach_swiglu_mxfp8_down(gate_up, w, s).shape == (7, 128)
    norm_w = torch.empty((256,), dtype=torch.bfloat16, device="meta")
    y, summed = torch.ops.vllm.mach_norm_quant_mxfp8_gate_up(x, x, norm_w, 1e-6, w, s)
    assert y.shape == (7, 128) and summed.shape == x.shape
    n, r = torch.ops.vllm.mach_allreduce_gemma_rms_norm(x, x, norm_w, 1e-6)
    assert n.shape == x.shape and r.shape == x.shape
    a8 = torch.empty((7, 256), dtype=torch.float8_e4m3fn, device="meta")
    sa = torch.empty((7, 2), dtype=torch.float32, device="meta")
    sb = torch.empty((1, 2), dtype=torch.float32, device="meta")
    out = torch.ops.vllm_mach.block_fp8_linear(a8, w, sa, sb, sb, False, True)
    assert out.shape == (7, 128) and out.dtype == torch.bfloat16


def test_every_reference_op_name_is_defined():
    """The op names the reference's Python side and native extensions export
    (native/ar_norm/binding.cu:72-80, native/block_fp8/block_fp8.cu:257-262,
    native/fp8_activation/activation.cu:98-104, src/vllm_mach/mxfp6/moe_utils.py:47-488)."""
    ops.register()
    names = set(ops.op_names())
    for expected in ("mach_norm_quant::run", "mach_norm_quant::abi", "vllm_mach_block_fp8::mm",
                     "mach_fp8_activation::run", "vllm::mxfp6_sm120_quantize_mxfp8",
                     "vllm::mxfp6_sm120_quantize_mxfp8_packed", "vllm::mxfp6_sm120_route",
                     "vllm::mxfp6_sm120_grouped_gemm", "vllm::mxfp6_sm120_silu_grouped_gemm",
                     "vllm::mxfp6_sm120_reduce", "vllm::mxfp6_sm120_qwen35_grouped_moe"):
        assert expected in names
    assert torch.ops.mach_norm_quant.abi() == "ar-norm-mxfp8-b200-v1"
    # fake impls keep the batch symbolic
    x = torch.empty((7, 256), dtype=torch.bfloat16, device="meta")
    codes, scales = torch.ops.vllm.mxfp6_sm120_quantize_mxfp8(x)
    assert codes.shape == (7, 256) and scales.shape == (7, 8)
    codes, scales = torch.ops.vllm.mxfp6_sm120_quantize_mxfp8_packed(x)
    assert codes.shape == (7, 256) and scales.numel() == 128 * 2 * 4
    a8 = torch.empty((7, 256), dtype=torch.float8_e4m3fn, device="meta")
    b = torch.empty((128, 256), dtype=torch.float8_e4m3fn, device="meta").t()
    sa = torch.empty((7, 2), dtype=torch.float32, device="meta")
    sb = torch.empty((2, 1), dtype=torch.float32, device="meta")
    assert torch.ops.vllm_mach_block_fp8.mm(a8, b, sa, sb).shape == (7, 128)
    ids = torch.empty((7, 2), dtype=torch.int32, device="meta")
    packed, eo, so, inv = torch.ops.vllm.mxfp6_sm120_route(
        torch.empty((14, 256), dtype=torch.float8_e4m3fn, device="meta"), a8,
        torch.empty((7, 8), dtype=torch.uint8, device="meta"), ids, None, 4)
    assert eo.shape == (5,) and so.dtype == torch.int64 and inv.shape == (14,)
    assert packed.numel() == (14 + 4 * 127) * 8


def test_block_fp8_method_swap_installs_once_and_falls_through():
    calls = []

    class StockKernel:
        apply_input_quant = True
        config = types.SimpleNamespace(out_dtype=torch.bfloat16)

        def process_weights_after_loading(self, layer):
            calls.append("stock_prepare")

        def apply_weights(self, layer, x, bias=None, **kwargs):
            calls.append("stock_apply")
            return "stock"

    try:
        assert plugin.install_block_fp8(StockKernel) is True
        assert plugin.install_block_fp8(StockKernel) is False          # once
        kernel = StockKernel()
        # a CPU layer is prepared by the stock method and never marked for the B200 path
        layer = types.SimpleNamespace(weight=torch.zeros((256, 256), dtype=torch.float8_e4m3fn),
                                      weight_scale=torch.ones((2, 2)))
        kernel.process_weights_after_loading(layer)
        assert calls == ["stock_prepare"] and layer._mach_b200_block_fp8 is False
        assert kernel.apply_weights(layer, torch.zeros((2, 256), dtype=torch.bfloat16)) == "stock"
        # an ineligible layout (wrong scale shape) falls through as well
        layer2 = types.SimpleNamespace(weight=torch.zeros((256, 256), dtype=torch.float8_e4m3fn),
                                       weight_scale_inv=torch.ones((3, 2)))
        kernel.process_weights_after_loading(layer2)
        assert kernel.apply_weights(layer2, torch.zeros((2, 256), dtype=torch.bfloat16)) == "stock"
    finally:
        assert plugin.uninstall_block_fp8() is True
    assert StockKernel.apply_weights(StockKernel(), None, None) == "stock"
    assert plugin.uninstall_block_fp8() is False


def test_quark_key_and_moe_experts_registration_with_stand_ins():
    key = object()
    quark = types.SimpleNamespace(_ACTIVATION_QUANT_KEY_MAP={})
    utils = types.SimpleNamespace(kMxfp8Dynamic=key)
    assert plugin.register_quark_mxfp8_activation(quark, utils) is True
    assert quark._ACTIVATION_QUANT_KEY_MAP["mxfp8_e4m3"] is key
    assert plugin.register_quark_mxfp8_activation(types.SimpleNamespace(), utils) is False
    assert plugin.register_quark_mxfp8_activation(quark, types.SimpleNamespace()) is False

    class Method:
        experts_cls = None
    assert plugin.register_moe_experts(Method) is True
    from mach_b200.experts import Mxfp6B200Experts
    assert Method.experts_cls is Mxfp6B200Experts


def test_experts_apply_contract_violations():
    """Error behaviour of Mxfp6Sm120Experts.apply (src/vllm_mach/mxfp6/moe.py:589-615)."""
    from mach_b200.experts import Mxfp6B200Experts
    experts = object.__new__(Mxfp6B200Experts)
    experts.quant_config = types.SimpleNamespace(
        w1_scale=torch.zeros((4, 128, 4), dtype=torch.uint8),
        w2_scale=torch.zeros((4, 128, 2), dtype=torch.uint8))
    x = torch.zeros((3, 128), dtype=torch.bfloat16)
    out = torch.zeros_like(x)
    w1 = torch.zeros((4, 128, 96), dtype=torch.uint8)        # 2I = 128, K = 128
    w2 = torch.zeros((4, 128, 48), dtype=torch.uint8)        # H = 128, I = 64
    tw = torch.zeros((3, 2)); ids = torch.zeros((3, 2), dtype=torch.int32)
    args = dict(output=out, hidden_states=x, w1=w1, w2=w2, topk_weights=tw, topk_ids=ids,
                activation="silu", global_num_experts=4, expert_map=None, a1q_scale=None,
                a2_scale=None, workspace13=None, workspace2=None, expert_tokens_meta=None,
                apply_router_weight_on_input=False)
    for change in (dict(apply_router_weight_on_input=True), dict(expert_tokens_meta=object()),
                   dict(activation="gelu"), dict(global_num_experts=8),
                   dict(w1=torch.zeros((4, 128, 48), dtype=torch.uint8)),
                   dict(w2=torch.zeros((4, 64, 48), dtype=torch.uint8))):
        with pytest.raises(ValueError):
            experts.apply(**{**args, **change})
    # an empty batch returns without touching the device
    experts.apply(**{**args, "hidden_states": x[:0], "output": out[:0], "topk_weights": tw[:0],
                     "topk_ids": ids[:0]})
    assert experts.workspace_shapes(3, 128, 128, 2, 4, 4, None, "silu")[2] == (3, 128)
    assert Mxfp6B200Experts._supports_shape(2048) and not Mxfp6B200Experts._supports_shape(100)
    assert Mxfp6B200Experts._supports_activation("silu")


def test_mxfp8_can_implement_checks_the_config_keys():
    ok = types.SimpleNamespace(weight_quant_key="kMxfp8Static", activation_quant_key="kMxfp8Dynamic")
    assert linear.Mxfp8B200LinearKernel.can_implement(ok) == (True, None)
    assert linear.Mxfp8B200LinearKernel.can_implement(types.SimpleNamespace()) == (True, None)
    bad = types.SimpleNamespace(weight_quant_key="kNvfp4Static", activation_quant_key="kMxfp8Dynamic")
    assert linear.Mxfp8B200LinearKernel.can_implement(bad)[0] is False
    bad = types.SimpleNamespace(weight_quant_key="kMxfp8Static", out_dtype=torch.float16)
    assert linear.Mxfp8B200LinearKernel.can_implement(bad)[0] is False


def test_mxfp6_format_comes_from_the_layer():
    assert linear.mxfp6_format_of(types.SimpleNamespace(weight_dtype="fp6_e2m3")) == "e2m3"
    assert linear.mxfp6_format_of(types.SimpleNamespace(scheme=types.SimpleNamespace(
        weight_quant_key="kMxfp6E3M2Static"))) == "e3m2"
    assert linear.mxfp6_format_of(types.SimpleNamespace()) == "e3m2"
    ops.set_mxfp6_format("e2m3")
    assert ops.current_mxfp6_format() == "e2m3"
    ops.set_mxfp6_format("e3m2")
    with pytest.raises(ValueError):
        ops.set_mxfp6_format("e5m2")


def test_packaging_declares_the_vllm_plugin_entry_point():
    import tomllib
    from pathlib import Path
    text = (Path(__file__).resolve().parents[1] / "vllm-mach_b200" / "pyproject.toml").read_bytes()
    data = tomllib.loads(text.decode())
    assert data["project"]["entry-points"]["vllm.general_plugins"]["mach_b200"] == \
        "mach_b200.plugin:register"
    from mach_b200 import plugin as entry
    assert callable(entry.register)


def test_warmup_refuses_other_dtypes_and_orders_sizes():
    from mach_b200 import warmup
    assert warmup.normalize_sizes([8, 0, 1, 8, -3, 512]) == [512, 8, 1]
    with pytest.raises(ValueError):
        warmup.warmup(torch.nn.Linear(4, 4), [1], torch.float16)
    assert warmup.warmup(torch.nn.Linear(4, 4), [1, 8]) == 0     # no quantised layers: no launches
