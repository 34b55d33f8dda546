"""Checkpoint-format I/O for the quantised linear layers.

What the reference does on the CPU in `reconstruct_model` (src/vllm_mach/mxfp8/
reconstruct_model.py:34-50,131-190: BF16 safetensors -> E4M3 codes + E8M0 group-32 scales in
the compressed-tensors "mxfp8-quantized" layout) runs here on the B200: the weight quantiser is
`mach_mxfp8_quantize_weight`, bit-identical to `quantize_block`. The model-specific parts of
the reference tool (pinned SHA-256 identities of one published checkpoint, the L0 code asset,
tokenizer regeneration) are not reproduced.

Also the loaders that turn checkpoint tensors into kernel-layout weights:
  * compressed-tensors MXFP8: `<name>.weight` F8_E4M3 [N, K], `<name>.weight_scale` U8 [N, K/32]
    (tests/native_mxfp6/test_mxfp8_sm120.py:33-39);
  * Quark MXFP6: `<name>.weight` U8 [N, 3K/4] (four 6-bit codes per three bytes),
    `<name>.weight_scale` U8 [N, K/32] (src/vllm_mach/mxfp6/dense.py:61-80,179-188);
  * block-FP8: `<name>.weight` F8_E4M3 [N, K], `<name>.weight_scale_inv` F32 [N/128, K/128]
    (src/vllm_mach/fp8/linear.py:120-135).
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Callable, Iterable

import torch

from . import native

MXFP8_QUANTIZATION_CONFIG = {
    "quant_method": "compressed-tensors",
    "format": "mxfp8-quantized",
    "quantization_status": "compressed",
    "config_groups": {"group_0": {
        "format": "mxfp8-quantized", "targets": ["Linear"],
        "weights": {"type": "float", "num_bits": 8, "strategy": "group", "group_size": 32,
                    "symmetric": True, "dynamic": False, "scale_dtype": "torch.uint8"},
        "input_activations": {"type": "float", "num_bits": 8, "strategy": "group",
                              "group_size": 32, "symmetric": True, "dynamic": True,
                              "scale_dtype": "torch.uint8"},
        "output_activations": None}},
}


def quantize_weight_mxfp8(weight: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """BF16 [N, K] on a B200 -> (E4M3 codes [N, K], logical E8M0 scales uint8 [N, K/32])."""
    native._require(weight, torch.bfloat16, "weight")
    n, k = weight.shape
    if k % 32:
        raise ValueError("MXFP8 weights need K % 32 == 0")
    codes = torch.empty((n, k), dtype=torch.float8_e4m3fn, device=weight.device)
    scales = torch.empty((n, k // 32), dtype=torch.uint8, device=weight.device)
    with torch.cuda.device(weight.device):
        native._check(native.lib().mach_mxfp8_quantize_weight(
            native._ptr(weight), native._ptr(codes), native._ptr(scales), n, k,
            native._stream(weight)), "mxfp8_quantize_weight")
    return codes, scales


def norm_recipe(key: str) -> str | None:
    """Which norm weights the reference re-rounds (reconstruct_model.py:53-61)."""
    if key.endswith(".linear_attn.norm.weight"):
        return "bf16"
    if (key == "model.language_model.norm.weight"
            or key.endswith((".input_layernorm.weight", ".post_attention_layernorm.weight",
                             ".self_attn.q_norm.weight", ".self_attn.k_norm.weight"))):
        return "float32_plus1_bf16_minus1"
    return None


def convert_norm(key: str, x: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """reconstruct_model.py:64-71: (1 + w) is what the Gemma-style norm multiplies by, so the
    BF16 rounding is applied to 1 + w and undone."""
    recipe = norm_recipe(key)
    if recipe == "bf16":
        return x.to(torch.bfloat16).to(dtype)
    if recipe == "float32_plus1_bf16_minus1":
        return ((x.float() + 1).to(torch.bfloat16).float() - 1).to(dtype)
    return x.to(dtype)


def is_quantised_linear(key: str, tensor: torch.Tensor, ignore: Iterable[str]) -> bool:
    if not key.endswith(".weight") or tensor.ndim != 2 or tensor.dtype != torch.bfloat16:
        return False
    module = key[: -len(".weight")]
    if any(module == name or module.endswith("." + name) or name in module.split(".")
           for name in ignore):
        return False
    if "norm" in module.rsplit(".", 1)[-1] or "embed" in module:
        return False
    return tensor.shape[1] % 32 == 0


def convert_bf16_to_mxfp8(source, output, ignore: Iterable[str] = ("lm_head",),
                          device: str = "cuda", round_norms: bool = False,
                          quantizer: Callable | None = None) -> dict:
    """BF16 safetensors checkpoint (a file or a directory of shards) -> one compressed-tensors
    MXFP8 directory: every 2-D BF16 `.weight` of a Linear that is not ignored becomes
    `<name>.weight` (F8_E4M3) + `<name>.weight_scale` (U8 [N, K/32]); everything else is copied
    (norm weights re-rounded like the reference when `round_norms`). Tensors stream through the
    device one at a time. Returns a summary. `quantizer(bf16 [N, K]) -> (codes, scales)`
    defaults to the B200 kernel."""
    from safetensors import safe_open
    from safetensors.torch import save_file
    source, output = Path(source), Path(output)
    if output.exists():
        raise FileExistsError(output)
    shards = [source] if source.is_file() else sorted(source.glob("*.safetensors"))
    if not shards:
        raise FileNotFoundError(f"no safetensors under {source}")
    quantizer = quantizer or (lambda w: quantize_weight_mxfp8(w.to(device)))
    ignore = tuple(ignore)
    output.mkdir(parents=True)
    summary = {"quantised": 0, "copied": 0, "bytes_in": 0, "bytes_out": 0, "shards": []}
    index = {}
    for number, shard in enumerate(shards):
        out_tensors = {}
        with safe_open(str(shard), framework="pt", device="cpu") as reader:
            for key in reader.keys():
                tensor = reader.get_tensor(key)
                summary["bytes_in"] += tensor.numel() * tensor.element_size()
                if is_quantised_linear(key, tensor, ignore):
                    codes, scales = quantizer(tensor.contiguous())
                    out_tensors[key] = codes.cpu()
                    out_tensors[key[: -len(".weight")] + ".weight_scale"] = scales.cpu()
                    summary["quantised"] += 1
                else:
                    out_tensors[key] = convert_norm(key, tensor, tensor.dtype) if round_norms \
                        else tensor
                    summary["copied"] += 1
        name = f"model-{number + 1:05d}-of-{len(shards):05d}.safetensors"
        save_file(out_tensors, str(output / name), metadata={"format": "pt"})
        for key, tensor in out_tensors.items():
            index[key] = name
            summary["bytes_out"] += tensor.numel() * tensor.element_size()
        summary["shards"].append(name)
    (output / "model.safetensors.index.json").write_text(json.dumps(
        {"metadata": {"total_size": summary["bytes_out"]}, "weight_map": index}, indent=1))
    config_path = (source if source.is_dir() else source.parent) / "config.json"
    config = json.loads(config_path.read_text()) if config_path.exists() else {}
    config["quantization_config"] = dict(MXFP8_QUANTIZATION_CONFIG, ignore=list(ignore))
    (output / "config.json").write_text(json.dumps(config, indent=2))
    return summary


# ------------------------------------------------------------------ loaders
class CheckpointReader:
    """Tensors of a safetensors file or sharded directory, by name."""

    def __init__(self, path):
        from safetensors import safe_open
        path = Path(path)
        self._files = [path] if path.is_file() else sorted(path.glob("*.safetensors"))
        self._where = {}
        for file in self._files:
            with safe_open(str(file), framework="pt", device="cpu") as reader:
                for key in reader.keys():
                    self._where[key] = file
        self._open = safe_open

    def keys(self):
        return self._where.keys()

    def __contains__(self, key):
        return key in self._where

    def get(self, key: str, device="cpu") -> torch.Tensor:
        if key not in self._where:
            raise KeyError(key)
        with self._open(str(self._where[key]), framework="pt", device="cpu") as reader:
            return reader.get_tensor(key).to(device)


def linear_format(reader, prefix: str) -> str:
    """"mxfp8", "mxfp6", "block_fp8" or "bf16" from the tensors a layer has."""
    weight = reader.get(prefix + ".weight")
    if prefix + ".weight_scale_inv" in reader:
        return "block_fp8"
    if prefix + ".weight_scale" in reader:
        scale = reader.get(prefix + ".weight_scale")
        if weight.dtype == torch.float8_e4m3fn:
            return "block_fp8" if scale.dtype == torch.float32 else "mxfp8"
        if weight.dtype == torch.uint8 and scale.shape[-1] * 32 * 3 == weight.shape[-1] * 4:
            return "mxfp6"
        raise ValueError(f"{prefix}: unrecognised quantised layout "
                         f"({weight.dtype} {tuple(weight.shape)}, scale {tuple(scale.shape)})")
    return "bf16"


def load_mx_linear(reader, prefix: str, device="cuda"):
    """(weight bytes [N, K or 3K/4], swizzled scales, logical K, kind) in kernel layout."""
    kind = linear_format(reader, prefix)
    if kind not in ("mxfp8", "mxfp6"):
        raise ValueError(f"{prefix} is {kind}, not an MX-format layer")
    weight = reader.get(prefix + ".weight", device).contiguous()
    scale = reader.get(prefix + ".weight_scale", device).contiguous()
    k = weight.shape[1] if kind == "mxfp8" else weight.shape[1] * 4 // 3
    if scale.dtype != torch.uint8 or tuple(scale.shape) != (weight.shape[0], k // 32):
        raise ValueError(f"{prefix}: scales must be uint8 [N, K/32]")
    return weight.view(torch.uint8), native.pack_scales(scale, k), k, kind


def load_mx_mlp(reader, prefix: str, device="cuda", fmt: str | None = None):
    """`<prefix>.gate_proj / up_proj / down_proj` (or a fused `gate_up_proj`) ->
    mlp.MxMlpWeights. `fmt` names the 6-bit element format of MXFP6 checkpoints
    ("e2m3" / "e3m2"); MXFP8 needs none."""
    from .mlp import MxMlpWeights

    def logical(name):
        return (reader.get(f"{prefix}.{name}.weight", device).contiguous().view(torch.uint8),
                reader.get(f"{prefix}.{name}.weight_scale", device).contiguous())
    if f"{prefix}.gate_up_proj.weight" in reader:
        kind = linear_format(reader, f"{prefix}.gate_up_proj")
        w_gu, s_gu = logical("gate_up_proj")
    else:
        kind = linear_format(reader, f"{prefix}.gate_proj")
        (w_g, s_g), (w_u, s_u) = logical("gate_proj"), logical("up_proj")
        w_gu, s_gu = torch.cat([w_g, w_u], 0), torch.cat([s_g, s_u], 0)
    if kind not in ("mxfp8", "mxfp6"):
        raise ValueError(f"{prefix} is {kind}, not an MX-format MLP")
    w_d, s_d = logical("down_proj")
    hidden = w_d.shape[0]
    element = "e4m3" if kind == "mxfp8" else (fmt or "e3m2")
    return MxMlpWeights.from_logical(w_gu, s_gu, w_d, s_d, hidden, fmt=element)


def load_block_fp8_linear(reader, prefix: str, device="cuda"):
    """(weight E4M3 [N, K], FP32 scales [ceil(N/128), K/128]) for mach_block_fp8_gemm."""
    weight = reader.get(prefix + ".weight", device).contiguous()
    name = prefix + (".weight_scale_inv" if prefix + ".weight_scale_inv" in reader else ".weight_scale")
    scale = reader.get(name, device).contiguous()
    n, k = weight.shape
    if weight.dtype != torch.float8_e4m3fn or scale.dtype != torch.float32 \
            or tuple(scale.shape) != ((n + 127) // 128, k // 128):
        raise ValueError(f"{prefix}: expected E4M3 [N, K] with FP32 scales [N/128, K/128]")
    return weight, scale
