"""vLLM general-plugin entry point for B200 (`vllm.general_plugins: mach = mach_b200.plugin:register`).

Mirrors src/vllm_mach/plugin.py:68-127 and the registration helpers
src/vllm_mach/mxfp6/dense.py:255-265, src/vllm_mach/mxfp6/dense_mxfp8.py:165-174: the kernel
classes are PREPENDED to vLLM's candidate lists for the CUDA platform, so vLLM's own selector
(`is_supported` / `can_implement`) picks them on sm_100 and falls through elsewhere. No CUDA
call happens at registration; the native library is loaded when the selector asks
`is_supported()` inside the GPU worker.
"""
from __future__ import annotations

import logging

logger = logging.getLogger(__name__)


def _prepend(kernels: list, cls) -> None:
    while cls in kernels:
        kernels.remove(cls)
    kernels.insert(0, cls)


def register_dense_kernels(linear_module=None, platform=None) -> dict[str, bool]:
    """Returns which candidate lists were found and extended. `linear_module` / `platform`
    default to vLLM's `vllm.model_executor.kernels.linear` and `PlatformEnum.CUDA`."""
    from .linear import Mxfp6B200LinearKernel, Mxfp8B200LinearKernel
    if linear_module is None:
        try:
            from vllm.model_executor.kernels import linear as linear_module
            from vllm.platforms import PlatformEnum
            platform = PlatformEnum.CUDA
        except Exception as error:  # noqa: BLE001
            logger.info("mach_b200: vLLM kernel registry unavailable (%s)", error)
            return {"mxfp6": False, "mxfp8": False}
    done = {}
    for key, attr, cls in (("mxfp6", "_POSSIBLE_MXFP6_KERNELS", Mxfp6B200LinearKernel),
                           ("mxfp8", "_POSSIBLE_MXFP8_KERNELS", Mxfp8B200LinearKernel)):
        table = getattr(linear_module, attr, None)
        kernels = table.get(platform) if isinstance(table, dict) else None
        if isinstance(kernels, list):
            _prepend(kernels, cls)
            done[key] = True
        else:
            done[key] = False
    return done


# ---------------------------------------------------------------- block-FP8 method swap
_BLOCK_FP8 = {"target": None, "prepare": None, "apply": None}
_FLAG = "_mach_b200_block_fp8"


def _weight_scale(layer):
    scale = getattr(layer, "weight_scale_inv", None)
    return getattr(layer, "weight_scale", None) if scale is None else scale


def _block_fp8_prepare(self, layer):
    """process_weights_after_loading of the stock kernel, then mark the layers this package
    serves (src/vllm_mach/fp8/linear.py:149-155 derives a scale buffer here; the B200 GEMM
    reads the checkpoint's [N/128, K/128] scales as they are, so nothing is derived)."""
    from .linear import BlockFp8B200Linear
    _BLOCK_FP8["prepare"](self, layer)
    import torch
    ok = (getattr(getattr(self, "config", None), "out_dtype", torch.bfloat16) == torch.bfloat16
          and BlockFp8B200Linear.eligible(getattr(layer, "weight", None), _weight_scale(layer))
          and getattr(layer.weight, "is_cuda", False))
    setattr(layer, _FLAG, bool(ok))


def _block_fp8_apply(self, layer, x, bias=None, **kwargs):
    """apply_weights: eligible layers run quantise + block-FP8 GEMM on the B200 kernels; every
    other layer, dtype or layout falls through to the stock method, silently, as the reference
    does for unsupported shapes (src/vllm_mach/fp8/linear.py:157-192)."""
    import torch
    from . import native
    from .linear import BlockFp8B200Linear
    if not getattr(layer, _FLAG, False):
        return _BLOCK_FP8["apply"](self, layer, x, bias, **kwargs)
    params = self._get_layer_params(layer) if hasattr(self, "_get_layer_params") else layer
    weight = params.weight
    scale = _weight_scale(layer)
    if not getattr(self, "apply_input_quant", True):
        # activations arrive quantised (1x128 FP32 scales): GEMM only
        q_input = x.view(-1, x.shape[-1])
        out = native.block_fp8_gemm(q_input, params.input_scale, weight, scale.contiguous())
        out = out.view(*x.shape[:-1], weight.shape[0])
        return out if bias is None else out + bias
    if x.dtype != torch.bfloat16:
        return _BLOCK_FP8["apply"](self, layer, x, bias, **kwargs)
    return BlockFp8B200Linear.apply(weight, scale, x, bias)


def install_block_fp8(target_cls=None) -> bool:
    """Replaces the two methods of vLLM's CutlassFp8BlockScaledMMKernel, once
    (src/vllm_mach/fp8/linear.py:193-216). `target_cls` is for tests."""
    if _BLOCK_FP8["target"] is not None:
        return False
    if target_cls is None:
        try:
            from importlib import import_module
            target_cls = import_module(
                "vllm.model_executor.kernels.linear.scaled_mm.cutlass").CutlassFp8BlockScaledMMKernel
        except Exception as error:  # noqa: BLE001
            logger.info("mach_b200: block-FP8 kernel class unavailable (%s)", error)
            return False
    _BLOCK_FP8.update(target=target_cls, prepare=target_cls.process_weights_after_loading,
                      apply=target_cls.apply_weights)
    target_cls.process_weights_after_loading = _block_fp8_prepare
    target_cls.apply_weights = _block_fp8_apply
    return True


def uninstall_block_fp8() -> bool:
    target = _BLOCK_FP8["target"]
    if target is None:
        return False
    target.process_weights_after_loading = _BLOCK_FP8["prepare"]
    target.apply_weights = _BLOCK_FP8["apply"]
    _BLOCK_FP8.update(target=None, prepare=None, apply=None)
    return True


# ---------------------------------------------------------------- Quark key, MoE experts
def register_quark_mxfp8_activation(quark_module=None, quant_utils=None) -> bool:
    """Quark normalises the checkpoint's dynamic E4M3 activations to "mxfp8_e4m3"; vLLM has the
    kMxfp8Dynamic key but does not map that spelling (src/vllm_mach/mxfp6/dense.py:217-241)."""
    try:
        if quark_module is None:
            from importlib import import_module
            quark_module = import_module(
                "vllm.model_executor.layers.quantization.quark.schemes.quark_ocp_mx")
            from vllm.model_executor.layers.quantization.utils import quant_utils
        key = getattr(quant_utils, "kMxfp8Dynamic", None)
        table = getattr(quark_module, "_ACTIVATION_QUANT_KEY_MAP", None)
        if key is None or not isinstance(table, dict):
            return False
        table.setdefault("mxfp8_e4m3", key)
        return table.get("mxfp8_e4m3") == key
    except Exception:  # noqa: BLE001 - optional bridge
        return False


def register_moe_experts(method_cls=None) -> bool:
    """Points the OCP-MX MoE method at the B200 experts class, which is what the reference's
    source patch does for its own class (mxfp6/profile/v034/runtime.patch:186-200)."""
    try:
        from .experts import Mxfp6B200Experts
        if method_cls is None:
            from importlib import import_module
            method_cls = import_module(
                "vllm.model_executor.layers.quantization.quark.quark_moe").QuarkOCP_MX_MoEMethod
        method_cls.experts_cls = Mxfp6B200Experts
        return True
    except Exception as error:  # noqa: BLE001
        logger.info("mach_b200: MoE method class unavailable (%s)", error)
        return False


def register() -> None:
    """Entry point (`vllm.general_plugins`). Everything is best effort and touches no CUDA
    state: the library is loaded when vLLM's selector asks `is_supported()` in the worker."""
    done = register_dense_kernels()
    done["block_fp8"] = install_block_fp8()
    done["quark_mxfp8_key"] = register_quark_mxfp8_activation()
    done["moe_experts"] = register_moe_experts()
    logger.info("mach_b200 plugin: registered %s", done)
