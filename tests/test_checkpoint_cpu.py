"""Checkpoint I/O on CPU: file-format logic of the BF16 -> MXFP8 conversion and the loaders'
layout detection, with the oracle's weight quantiser standing in for the B200 kernel (the
kernel itself is compared with the same oracle in tests/test_gpu_checkpoint.py). Mirrors what
tests/test_mxfp8_reconstruct_model.py of the reference checks: tensor names, dtypes, shapes,
the golden scale vector, norm re-rounding."""
import json

import pytest
import torch
from safetensors.torch import save_file

from mach_b200 import checkpoint
from oracle import mx_oracle as ora


def oracle_quantizer(w):
    codes, scales = ora.quantize_weight_mxfp8(w)
    return codes.view(torch.float8_e4m3fn), scales


def tiny_checkpoint(tmp_path):
    g = torch.Generator().manual_seed(0)
    tensors = {
        "model.layers.0.mlp.gate_proj.weight": (torch.randn(64, 128, generator=g) * 0.02).bfloat16(),
        "model.layers.0.mlp.up_proj.weight": (torch.randn(64, 128, generator=g) * 0.02).bfloat16(),
        "model.layers.0.mlp.down_proj.weight": (torch.randn(128, 64, generator=g) * 0.02).bfloat16(),
        "model.layers.0.input_layernorm.weight": (torch.randn(128, generator=g) * 0.1).bfloat16(),
        "model.embed_tokens.weight": torch.randn(32, 128, generator=g).bfloat16(),
        "lm_head.weight": torch.randn(32, 128, generator=g).bfloat16(),
    }
    src = tmp_path / "bf16"
    src.mkdir()
    save_file(tensors, str(src / "model.safetensors"))
    (src / "config.json").write_text(json.dumps({"hidden_size": 128}))
    return src, tensors


def test_conversion_writes_compressed_tensors_layout(tmp_path):
    src, tensors = tiny_checkpoint(tmp_path)
    out = tmp_path / "mxfp8"
    summary = checkpoint.convert_bf16_to_mxfp8(src, out, quantizer=oracle_quantizer, round_norms=True)
    assert summary["quantised"] == 3 and summary["copied"] == 3
    reader = checkpoint.CheckpointReader(out)
    for name in ("gate_proj", "up_proj", "down_proj"):
        prefix = f"model.layers.0.mlp.{name}"
        w = reader.get(prefix + ".weight")
        s = reader.get(prefix + ".weight_scale")
        ref_c, ref_s = ora.quantize_weight_mxfp8(tensors[prefix + ".weight"])
        assert w.dtype == torch.float8_e4m3fn and torch.equal(w.view(torch.uint8), ref_c)
        assert s.dtype == torch.uint8 and torch.equal(s, ref_s)
        assert checkpoint.linear_format(reader, prefix) == "mxfp8"
    # ignored and non-linear tensors are carried over; the norm is re-rounded like the reference
    assert torch.equal(reader.get("lm_head.weight"), tensors["lm_head.weight"])
    assert torch.equal(reader.get("model.embed_tokens.weight"), tensors["model.embed_tokens.weight"])
    norm = tensors["model.layers.0.input_layernorm.weight"]
    assert torch.equal(reader.get("model.layers.0.input_layernorm.weight"),
                       ((norm.float() + 1).bfloat16().float() - 1).bfloat16())
    config = json.loads((out / "config.json").read_text())
    assert config["hidden_size"] == 128
    assert config["quantization_config"]["format"] == "mxfp8-quantized"
    assert config["quantization_config"]["ignore"] == ["lm_head"]
    index = json.loads((out / "model.safetensors.index.json").read_text())
    assert "model.layers.0.mlp.down_proj.weight_scale" in index["weight_map"]
    with pytest.raises(FileExistsError):
        checkpoint.convert_bf16_to_mxfp8(src, out, quantizer=oracle_quantizer)


def test_golden_scale_vector_survives_the_file_round_trip(tmp_path):
    """Block maxima [0, 1, 1.7421875, 1.75, 2, 3.5, 448] -> E8M0 [0, 119, 119, 120, 120, 121, 128]
    (tests/test_mxfp8_reconstruct_model.py:142-156 of the reference)."""
    maxima = [0.0, 1.0, 1.7421875, 1.75, 2.0, 3.5, 448.0]
    row = torch.cat([torch.tensor([v, -v] * 16) for v in maxima]).bfloat16()
    src = tmp_path / "one.safetensors"
    save_file({"layer.proj.weight": row[None, :].repeat(2, 1).contiguous()}, str(src))
    out = tmp_path / "out"
    checkpoint.convert_bf16_to_mxfp8(src, out, ignore=(), quantizer=oracle_quantizer)
    reader = checkpoint.CheckpointReader(out)
    assert reader.get("layer.proj.weight_scale")[0].tolist() == [0, 119, 119, 120, 120, 121, 128]


def test_layout_detection_and_norm_recipes(tmp_path):
    path = tmp_path / "mixed.safetensors"
    save_file({
        "a.weight": torch.zeros((16, 96), dtype=torch.uint8), "a.weight_scale": torch.zeros((16, 4), dtype=torch.uint8),
        "b.weight": torch.zeros((128, 256), dtype=torch.float8_e4m3fn),
        "b.weight_scale_inv": torch.ones((1, 2), dtype=torch.float32),
        "c.weight": torch.zeros((8, 32), dtype=torch.bfloat16),
        "d.weight": torch.zeros((16, 100), dtype=torch.uint8), "d.weight_scale": torch.zeros((16, 4), dtype=torch.uint8),
    }, str(path))
    reader = checkpoint.CheckpointReader(path)
    assert checkpoint.linear_format(reader, "a") == "mxfp6"
    assert checkpoint.linear_format(reader, "b") == "block_fp8"
    assert checkpoint.linear_format(reader, "c") == "bf16"
    with pytest.raises(ValueError):
        checkpoint.linear_format(reader, "d")
    with pytest.raises(KeyError):
        reader.get("missing.weight")
    assert checkpoint.norm_recipe("model.layers.3.linear_attn.norm.weight") == "bf16"
    assert checkpoint.norm_recipe("model.layers.3.self_attn.q_norm.weight") == "float32_plus1_bf16_minus1"
    assert checkpoint.norm_recipe("model.layers.3.mlp.down_proj.weight") is None
    assert not checkpoint.is_quantised_linear("x.weight", torch.zeros((4, 30), dtype=torch.bfloat16), ())
    assert not checkpoint.is_quantised_linear("lm_head.weight", torch.zeros((4, 32), dtype=torch.bfloat16), ("lm_head",))
    assert checkpoint.is_quantised_linear("m.q_proj.weight", torch.zeros((4, 32), dtype=torch.bfloat16), ("lm_head",))
