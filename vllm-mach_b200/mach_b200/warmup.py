"""Warm-up before CUDA-graph capture.

The reference walks the model's quantised projections over the batch sizes vLLM will capture
and freezes its workspace plan (`warmup_mxfp6_sm120`, src/vllm_mach/mxfp6/warmup.py:76-116;
`warmup_mxfp8`, src/vllm_mach/mxfp6/dense_mxfp8.py:177-199). The B200 kernels keep no
workspace plan, but three things happen on the FIRST launch of a kernel variant on a device
and none of them may happen inside a capture: the opt-in to more than 48 KiB of dynamic shared
memory (`cudaFuncSetAttribute`), the occupancy query of the persistent kernels, and the lookup
of device symbols (status word, built-in scratch). Which variant runs depends on the shape
bucket (decode / mid / large batch, tile width), so `warmup` runs every distinct layer shape
once per requested batch size, on the current stream, and synchronises.
"""
from __future__ import annotations

import torch

from . import native


def _problems(model: torch.nn.Module):
    """Distinct (kind, N, K) of the layers whose kernel is one of this package's classes."""
    from .linear import BlockFp8B200Linear, Mxfp6B200LinearKernel, Mxfp8B200LinearKernel
    seen = {}
    for layer in model.modules():
        scheme = getattr(layer, "scheme", None)
        kernel = getattr(scheme, "ocp_mx_linear", None) or getattr(scheme, "kernel", None)
        weight = getattr(layer, "weight", None)
        if weight is None or weight.ndim != 2:
            continue
        if isinstance(kernel, Mxfp6B200LinearKernel):
            key = ("mxfp6", int(weight.shape[0]), int(weight.shape[1]) * 4 // 3)
        elif isinstance(kernel, Mxfp8B200LinearKernel):
            key = ("mxfp8", int(weight.shape[0]), int(weight.shape[1]))
        elif BlockFp8B200Linear.eligible(weight, getattr(layer, "weight_scale_inv", None)
                                         if getattr(layer, "weight_scale_inv", None) is not None
                                         else getattr(layer, "weight_scale", None)) \
                and getattr(layer, "_mach_b200_block_fp8", False):
            key = ("block_fp8", int(weight.shape[0]), int(weight.shape[1]))
        else:
            continue
        seen.setdefault(key, (layer, kernel))
    return seen


def normalize_sizes(token_sizes) -> list[int]:
    return sorted({int(s) for s in token_sizes if int(s) > 0}, reverse=True)


@torch.inference_mode()
def warmup(model: torch.nn.Module, token_sizes, dtype: torch.dtype = torch.bfloat16) -> int:
    """Runs every distinct quantised projection of `model` once per batch size. Returns the
    number of launches made. Call after weight loading, before graph capture."""
    if dtype != torch.bfloat16:
        raise ValueError("the B200 kernels take BF16 activations")
    if torch.cuda.is_available() and torch.cuda.is_current_stream_capturing():
        raise RuntimeError("warm up before graph capture, not inside it")
    from .linear import BlockFp8B200Linear
    launches = 0
    sizes = normalize_sizes(token_sizes)
    for (kind, n, k), (layer, kernel) in _problems(model).items():
        device = layer.weight.device
        for m in sizes:
            x = torch.empty((m, k), device=device, dtype=dtype).uniform_(-1.0, 1.0)
            if kind == "block_fp8":
                scale = getattr(layer, "weight_scale_inv", None)
                scale = layer.weight_scale if scale is None else scale
                BlockFp8B200Linear.apply(layer.weight, scale, x)
            else:
                kernel.apply_weights(layer, x)
            launches += 1
    if launches:
        torch.cuda.synchronize()
        # resolve the device symbols outside any capture as well
        native.device_status(clear=False)
    return launches


@torch.inference_mode()
def warmup_shapes(shapes, token_sizes, device="cuda", fmt: str = "e4m3") -> int:
    """The same for stand-alone users: `shapes` is an iterable of (N, K) weight shapes; random
    codes are used (only the launch path matters)."""
    launches = 0
    for n, k in shapes:
        cols = k if fmt == "e4m3" else k * 3 // 4
        w = torch.randint(0, 256, (n, cols), dtype=torch.uint8, device=device)
        s = native.pack_scales(torch.full((n, k // 32), 120, dtype=torch.uint8, device=device), k)
        for m in normalize_sizes(token_sizes):
            x = torch.empty((m, k), device=device, dtype=torch.bfloat16).uniform_(-1.0, 1.0)
            codes, scales = native.quantize_mxfp8(x)
            native.mx_gemm(codes, scales, w, s, fmt)
            launches += 1
    if launches:
        torch.cuda.synchronize()
        native.device_status(clear=False)
    return launches
