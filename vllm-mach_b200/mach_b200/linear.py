"""LinearKernel adapters with the reference's method contract, for B200.

`Mxfp8B200LinearKernel` / `Mxfp6B200LinearKernel` mirror `Mxfp8Sm120LinearKernel`
(src/vllm_mach/mxfp6/dense_mxfp8.py:114-162) and `Mxfp6Sm120LinearKernel`
(src/vllm_mach/mxfp6/dense.py:160-214): `is_supported` never raises and returns
(bool, reason), `can_implement(config)`, `process_weights_after_loading(layer)` replaces
`layer.weight` / `layer.weight_scale` by frozen Parameters in kernel layout,
`apply_weights(layer, x, bias)` returns `(*x.shape[:-1], N)` in x.dtype and raises
ValueError on contract violations. `BlockFp8B200Linear` carries the two methods the
reference installs on `CutlassFp8BlockScaledMMKernel` (src/vllm_mach/fp8/linear.py:157-192).

vLLM >= 0.33 provides the base classes; when it is absent (as in this repository's tests)
plain `object` bases are used, which is how the reference's own CPU tests exercise the
contract.
"""
from __future__ import annotations

import torch

from . import native, ops

try:  # vLLM 0.33 / 0.34
    from vllm.model_executor.kernels.linear.mxfp8 import Mxfp8LinearKernel as _Mxfp8Base
except Exception:  # noqa: BLE001 - any import problem means "no such vLLM"
    _Mxfp8Base = object
try:
    from vllm.model_executor.kernels.linear.mxfp6 import MxFp6LinearKernel as _Mxfp6Base
except Exception:  # noqa: BLE001
    _Mxfp6Base = object

REQUIRED_CAPABILITY = 100  # sm_100a; the reference gates on 120 (mxfp6/dense.py:95)


def b200_available(compute_capability: int | None = None) -> tuple[bool, str | None]:
    """Never raises. (True, None) when a B200 and the native library are usable."""
    try:
        if compute_capability is None:
            if not torch.cuda.is_available():
                return False, "no CUDA device"
            major, minor = torch.cuda.get_device_capability()
            compute_capability = major * 10 + minor
        if int(compute_capability) != REQUIRED_CAPABILITY:
            return False, f"requires sm_100 (got {compute_capability})"
        native.lib()
        ops.register()
    except Exception as error:  # noqa: BLE001
        return False, f"libmach_b200 unavailable: {error}"
    return True, None


def _frozen(t: torch.Tensor) -> torch.nn.Parameter:
    return torch.nn.Parameter(t, requires_grad=False)


class Mxfp8B200LinearKernel(_Mxfp8Base):
    @classmethod
    def is_supported(cls, compute_capability=None):
        return b200_available(compute_capability)

    @classmethod
    def can_implement(cls, config):
        """MXFP8 weights (E4M3 + E8M0 per 32) with dynamic MXFP8 activations and BF16 output;
        a config that names other formats is refused with a reason."""
        wq = str(getattr(config, "weight_quant_key", "") or "").lower()
        aq = str(getattr(config, "activation_quant_key", "") or "").lower()
        out = getattr(config, "out_dtype", None)
        if wq and "mxfp8" not in wq and "e4m3" not in wq:
            return False, "requires static MXFP8 E4M3 weights"
        if aq and "mxfp8" not in aq and "e4m3" not in aq:
            return False, "requires dynamic MXFP8 E4M3 activations"
        if out is not None and out != torch.bfloat16:
            return False, "requires BF16 output"
        return True, None

    def process_weights_after_loading(self, layer):
        weight = layer.weight.data
        if weight.ndim != 2 or any(d <= 0 or d % 128 for d in weight.shape):
            raise ValueError("MXFP8 requires positive N and K divisible by 128")
        if weight.dtype != torch.float8_e4m3fn:
            raise ValueError("MXFP8 requires E4M3 weights")
        if getattr(layer, "params_dtype", torch.bfloat16) != torch.bfloat16:
            raise ValueError("MXFP8 requires --dtype bfloat16")
        n, k = weight.shape
        scale = layer.weight_scale.data
        if scale.dtype != torch.uint8 or tuple(scale.shape) != (n, k // 32):
            raise ValueError("MXFP8 requires uint8 E8M0 scales shaped [N, K/32]")
        layer.weight = _frozen(weight.contiguous())
        layer.weight_scale = _frozen(native.pack_scales(scale.contiguous(), k))

    def apply_weights(self, layer, x, bias=None):
        n, k = layer.weight.shape
        if x.dtype != torch.bfloat16 or x.shape[-1] != k:
            raise ValueError("MXFP8 requires BF16 activations with matching K")
        if x.numel() == 0:
            return x.new_empty((*x.shape[:-1], n))
        y = torch.ops.vllm.mach_mxfp8_sm120_gemm(
            x.reshape(-1, k).contiguous(), layer.weight, layer.weight_scale,
        ).reshape(*x.shape[:-1], n)
        return y if bias is None else y + bias


def logical_weight_shape(weight: torch.Tensor) -> tuple[int, int]:
    """(N, K) of a packed MXFP6 weight [N, 3K/4] (src/vllm_mach/mxfp6/dense.py:61-80)."""
    if weight.ndim != 2:
        raise ValueError(f"MXFP6 requires a two-dimensional packed weight; got {tuple(weight.shape)}")
    n, packed_k = map(int, weight.shape)
    if packed_k % 3 != 0:
        raise ValueError(f"MXFP6 packs four codes into three bytes; got packed K={packed_k}")
    k = packed_k * 4 // 3
    if n % 8 != 0 or k % 128 != 0:
        raise ValueError(f"MXFP6 requires N % 8 == 0 and K % 128 == 0; got N={n}, K={k}")
    return n, k


def mxfp6_format_of(layer, default: str = "e3m2") -> str:
    """6-bit element format of a layer's weights from its quantisation config: the reference
    admits "fp6_e3m2" only (src/vllm_mach/mxfp6/dense.py:172-177); B200 also takes "fp6_e2m3"."""
    for holder in (layer, getattr(layer, "scheme", None), getattr(layer, "quant_config", None)):
        for attr in ("weight_dtype", "weight_quant_key", "ocp_mx_scheme", "weight_format"):
            text = str(getattr(holder, attr, "") or "").lower()
            if "e2m3" in text:
                return "e2m3"
            if "e3m2" in text:
                return "e3m2"
    return default


class Mxfp6B200LinearKernel(_Mxfp6Base):
    """W6A8: static MXFP6 weights (E3M2 as the reference admits, or E2M3), dynamic MXFP8
    activations."""

    weight_format = "e3m2"

    @classmethod
    def is_supported(cls, compute_capability=None):
        return b200_available(compute_capability)

    @classmethod
    def can_implement(cls, config):
        wq = str(getattr(config, "weight_quant_key", "")).lower()
        aq = str(getattr(config, "activation_quant_key", "")).lower()
        if "mxfp6" not in wq and "e3m2" not in wq and "e2m3" not in wq:
            return False, "requires static MXFP6 weights"
        if "mxfp8" not in aq and "e4m3" not in aq:
            return False, "requires dynamic MXFP8 E4M3 activations"
        return True, None

    def process_weights_after_loading(self, layer):
        n, k = logical_weight_shape(layer.weight)
        if n % 16:
            raise ValueError("the B200 W6A8 GEMM requires N % 16 == 0")
        fmt = mxfp6_format_of(layer, self.weight_format)
        ops.set_mxfp6_format(fmt)
        self.weight_format = fmt
        scale = layer.weight_scale.data
        if scale.dtype != torch.uint8 or tuple(scale.shape) != (n, k // 32):
            raise ValueError("MXFP6 requires uint8 E8M0 scales shaped [N, K/32]")
        layer.weight = _frozen(layer.weight.data.contiguous())
        layer.weight_scale = _frozen(native.pack_scales(scale.contiguous(), k))

    def apply_weights(self, layer, x, bias=None):
        n, k = logical_weight_shape(layer.weight)
        if int(x.shape[-1]) != k:
            raise ValueError(f"activation K={int(x.shape[-1])} differs from weight K={k}")
        if x.numel() == 0:
            return x.new_empty((*x.shape[:-1], n))
        y = torch.ops.vllm.mach_mxfp6_sm120_gemm(
            x.reshape(-1, k).contiguous(), layer.weight, layer.weight_scale, n, x.dtype,
        ).reshape(*x.shape[:-1], n)
        return y if bias is None else y + bias


class BlockFp8B200Linear:
    """apply/prepare pair for block-FP8 layers (E4M3 weight, FP32 scale per 128x128)."""

    @staticmethod
    def eligible(weight, scale) -> bool:
        return (weight is not None and scale is not None and weight.ndim == 2
                and weight.dtype == torch.float8_e4m3fn and scale.dtype == torch.float32
                and weight.shape[1] % 128 == 0 and weight.shape[0] % 16 == 0
                and tuple(scale.shape) == ((weight.shape[0] + 127) // 128, weight.shape[1] // 128))

    @classmethod
    def apply(cls, weight, weight_scale, x, bias=None, ordered: bool = True):
        if not cls.eligible(weight, weight_scale):
            raise ValueError("unsupported block-FP8 layout/dtype/shape")
        k = weight.shape[1]
        if x.dtype != torch.bfloat16 or x.shape[-1] != k:
            raise ValueError("block-FP8 requires BF16 activations with matching K")
        if x.numel() == 0:
            return x.new_empty((*x.shape[:-1], weight.shape[0]))
        q, sa = native.fp8_group_quantize(x.reshape(-1, k).contiguous())
        y = torch.ops.vllm_mach.block_fp8_linear(q, weight, sa, weight_scale.contiguous(),
                                                 weight_scale, False, ordered)
        y = y.reshape(*x.shape[:-1], weight.shape[0])
        return y if bias is None else y + bias
