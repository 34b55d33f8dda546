"""torch custom ops with the names and schemas the reference plugin registers, implemented
on libmach_b200.so. Every op has a fake (meta) implementation that keeps the batch dimension
symbolic, so the ops trace under torch.compile(fullgraph=True, dynamic=True) exactly like
the reference's (src/vllm_mach/mxfp6/dense_mxfp8.py:100-110, mxfp6/dense.py:132-156,
mxfp6/mxfp8_mlp.py:25-30, mxfp6/mxfp8_norm_quant.py:75-80, mxfp6/gemma_norm.py:48-55,
mxfp6/compiled_ar_norm.py:7-13, fp8/linear.py:84-97, fp8/activation.py:23-27), the ops the
reference's native extensions define (native/ar_norm/binding.cu:72-80,
native/block_fp8/block_fp8.cu:257-262, native/fp8_activation/activation.cu:98-104) and the
mixture-of-experts shims of src/vllm_mach/mxfp6/moe_utils.py:47-488.

The op names keep the reference's spelling (including "sm120") so that adapters and compiled
graphs that name them keep working; the implementation is sm_100a.
"""
from __future__ import annotations

import threading

import torch

from . import native

_lock = threading.RLock()
_registered = False
_libs: list = []  # keep Library objects alive

_DTYPES = {torch.bfloat16: "bf16"}


def _mxfp8_gemm(x, weight, weight_scale):
    codes, scales = native.quantize_mxfp8(x)
    return native.mx_gemm(codes, scales, weight.view(torch.uint8), weight_scale, "e4m3")


# 6-bit element format of the checkpoint's MXFP6 weights. The reference admits E3M2 only
# (src/vllm_mach/mxfp6/dense.py:172-177) and its op schemas carry no format argument, so the
# format is process state set at load time (`set_mxfp6_format`, called by
# Mxfp6B200LinearKernel.process_weights_after_loading from the layer's quantisation config).
_mxfp6_format = "e3m2"


def set_mxfp6_format(fmt: str) -> None:
    global _mxfp6_format
    if fmt not in ("e3m2", "e2m3"):
        raise ValueError(f"unknown MXFP6 element format {fmt!r}")
    _mxfp6_format = fmt


def current_mxfp6_format() -> str:
    return _mxfp6_format


def _mxfp6_gemm(x, weight, weight_scale, n: int, dtype):
    if dtype != torch.bfloat16:
        raise ValueError("the B200 W6A8 GEMM returns BF16")
    codes, scales = native.quantize_mxfp8(x)
    out = native.mx_gemm(codes, scales, weight, weight_scale, current_mxfp6_format())
    if out.shape[1] != n:
        raise ValueError(f"weight has {out.shape[1]} rows, expected N={n}")
    return out


def _swiglu_down(gate_up, weight, weight_scale, fmt: str):
    if gate_up.shape[0] == 0:
        return gate_up.new_empty((0, weight.shape[0]))
    codes, scales = native.swiglu_quantize_mxfp8(gate_up)
    return native.mx_gemm(codes, scales, weight.view(torch.uint8), weight_scale, fmt)


def _norm_quant_gate_up(x, residual, norm_w, eps: float, weight, weight_scale):
    _, summed, codes, scales = native.add_rmsnorm_mxfp8(x, residual, norm_w, eps, 1.0,
                                                       want_norm=False)
    if x.shape[0] == 0:
        return x.new_empty((0, weight.shape[0])), summed
    return native.mx_gemm(codes, scales, weight.view(torch.uint8), weight_scale, "e4m3"), summed


def _gemma_norm(x, residual, weight, eps: float):
    norm, summed, _, _ = native.add_rmsnorm_mxfp8(x, residual, weight, eps, 1.0, want_quant=False)
    return norm, (summed if summed is not None else x.new_empty((0,)))


def _allreduce_gemma_rms_norm(hidden, residual, weight, eps: float):
    from . import collective, parallel_state
    return collective.allreduce_add_rmsnorm(hidden, residual, weight, eps,
                                            parallel_state.get_tp_group())


def _mlp(x, w_gate_up, s_gate_up, w_down, s_down):
    from .mlp import MxMlpWeights, mlp_forward
    return mlp_forward(x, MxMlpWeights(w_gate_up, s_gate_up, w_down, s_down, "e4m3"))


def _block_fp8_linear(a, b, sa, sb, sb64, n64: bool, ordered: bool):
    m = a.shape[0]
    if ordered and 1 <= m <= 8:
        raw = torch.empty((a.shape[1] // 128, m, b.shape[0]), dtype=torch.float32, device=a.device)
        return native.block_fp8_gemm(a, sa, b, sb, raw=raw)
    return native.block_fp8_gemm(a, sa, b, sb)


def _silu_and_mul_per_block_quant(out, input, scales, group_size: int, scale_ub,
                                  is_scale_transposed: bool):
    if group_size != 128 or scale_ub is not None:
        raise ValueError("the B200 SiLU/FP8 producer implements group 128 without an upper bound")
    _fp8_activation_run(out, input, scales, is_scale_transposed)


def _fp8_activation_run(out, input, scales, is_scale_transposed: bool):
    """mach_fp8_activation::run: writes straight into the caller's `out` and `scales`."""
    rows, two_i = input.shape
    inter = two_i // 2
    if (input.dtype != torch.bfloat16 or out.dtype != torch.float8_e4m3fn
            or scales.dtype != torch.float32):
        raise RuntimeError("Expected BF16, E4M3, FP32 tensors")
    if tuple(out.shape) != (rows, inter) or tuple(scales.shape) != (rows, inter // 128):
        raise RuntimeError("out must be [M, I] and scales [M, I/128]")
    if not input.is_contiguous() or not out.is_contiguous():
        raise RuntimeError("input and out must be contiguous")
    ok = (scales.stride() == (1, rows) or rows == 1) if is_scale_transposed else scales.is_contiguous()
    if not ok:
        raise RuntimeError("Unexpected scale layout")
    native.silu_mul_fp8_group_quantize(input, transposed=is_scale_transposed, out=out,
                                       scales=scales)


def _block_fp8_mm(a, b, sa, sb):
    """vllm_mach_block_fp8::mm: `b` is the weight viewed [K, N] (column-major, i.e. the
    checkpoint's [N, K] transposed) and `sb` its scales viewed [K/128, N/128] or, as the
    reference's 64-row variant passes them, [K/128, N/64] with every value repeated."""
    if b.ndim != 2 or b.stride(0) != 1:
        raise RuntimeError("b must be the column-major [K, N] view of an [N, K] weight")
    weight = b.t()
    k = a.shape[1]
    n = weight.shape[0]
    scale = sb.t()
    if scale.shape[0] == (n + 63) // 64 and scale.shape[0] != (n + 127) // 128:
        scale = scale[::2]
    return native.block_fp8_gemm(a, sa, weight, scale.contiguous())


_NORM_QUANT_ABI = "ar-norm-mxfp8-b200-v1"


def _norm_quant_run(hidden, residual, gamma, workspace, norm, residual_out, quant, scales,
                    rank: int, eps: float, fused: bool):
    """mach_norm_quant::run on the B200 reduce. `workspace` is the int64 tensor
    `collective.workspace_tensor` returns (the reference passes FlashInfer's pointer table in
    the same argument). `residual_out` may alias `hidden`, as the reference's caller does
    (src/vllm_mach/mxfp6/ar_norm.py:136-140)."""
    from . import collective
    m, h = hidden.shape
    for t in (hidden, residual, gamma, norm, residual_out):
        if t.dtype != torch.bfloat16 or not t.is_contiguous() or t.device != hidden.device:
            raise RuntimeError("mach_norm_quant.run BF16 tensors must be contiguous and on "
                               "hidden's device")
    if residual.shape != hidden.shape or norm.shape != hidden.shape \
            or residual_out.shape != hidden.shape or gamma.numel() != h:
        raise RuntimeError("mach_norm_quant.run requires residual, norm and residual_out to "
                           "match hidden and gamma.numel() == hidden size")
    ws = collective.workspace_from_tensor(workspace)
    if ws.rank != rank:
        raise RuntimeError(f"mach_norm_quant.run: workspace belongs to rank {ws.rank}, not {rank}")
    if fused:
        if quant.dtype not in (torch.uint8, torch.float8_e4m3fn) or quant.shape != hidden.shape \
                or not quant.is_contiguous():
            raise RuntimeError("mach_norm_quant.run requires a contiguous one-byte quant tensor "
                               "matching hidden")
        if scales.dtype != torch.uint8 or scales.numel() < native.sf_bytes(m, h):
            raise RuntimeError("mach_norm_quant.run requires a uint8 scale tensor with "
                               f"{native.sf_bytes(m, h)} entries")
    if m == 0:
        return
    with torch.cuda.device(hidden.device):
        native._check(native.lib().mach_allreduce_residual_rmsnorm_mxfp8(
            ws.handle, native._ptr(hidden), native._ptr(residual), native._ptr(gamma), eps, 1.0,
            native._ptr(norm), native._ptr(residual_out),
            native._ptr(quant) if fused else None, native._ptr(scales) if fused else None,
            m, h, 0, native._stream(hidden)), "mach_norm_quant.run")


def _gdn_norm_out(core, gate, norm_weight, weight, weight_scale, eps: float):
    """vllm::mach_gdn_norm_mxfp6_out (src/vllm_mach/mxfp6/gdn_output.py:11-19,56-64): gated
    RMSNorm + MXFP8 producer, then the W6A8 output projection."""
    codes, scales = native.gated_rmsnorm_quantize(core, gate, norm_weight, eps)
    if core.shape[0] == 0:
        return core.new_empty((0, weight.shape[0]))
    return native.mx_gemm(codes, scales, weight.view(torch.uint8), weight_scale,
                          current_mxfp6_format())


def projected(codes, scales, weight, weight_scale, fmt: str | None = None):
    """The reference's `projected(codes, scales, layer)` (src/vllm_mach/mxfp6/ar_norm.py:144-147):
    a projection fed by activations that a fused norm already quantised (QKV / QKVZ / gate_up
    after the all-reduce + norm + MXFP8 kernel)."""
    return native.mx_gemm(codes, scales, weight.view(torch.uint8), weight_scale,
                          fmt or current_mxfp6_format())


# ---- mixture-of-experts shims (src/vllm_mach/mxfp6/moe_utils.py:47-488)
def _moe_quantize_mxfp8(input):
    codes, scales = native.quantize_mxfp8(input)
    return codes, native.unpack_scales(scales, input.shape[0], input.shape[1])


def _moe_quantize_mxfp8_packed(input):
    return native.quantize_mxfp8(input)


def _moe_reduce(output, routed_output, topk_weights, inverse_permutation):
    from . import moe
    moe.combine(routed_output, topk_weights, inverse_permutation, output)


def _moe_whole_layer(output, hidden_states, w1, w1_scale, w2, w2_scale, topk_weights, topk_ids,
                     workspace13, workspace2):
    from . import moe
    weights = moe.cached_weights(w1, w1_scale, w2, w2_scale, current_mxfp6_format())
    moe.experts_forward(hidden_states, weights, topk_weights, topk_ids, out=output)


def _moe_route(permuted_activation, activation, logical_scales, topk_ids, expert_map,
               local_experts: int):
    from . import moe
    return moe.route_quantized(permuted_activation, activation, logical_scales, topk_ids,
                               expert_map, local_experts)


def _moe_grouped_gemm(output, activation, packed_scales, weight, weight_scales, expert_offsets,
                      scale_offsets):
    from . import moe
    moe.grouped_gemm_stage(output, activation, packed_scales, weight, weight_scales,
                           expert_offsets, scale_offsets, fmt=current_mxfp6_format())


def _moe_silu_grouped_gemm(output, gate_up, weight, weight_scales, expert_offsets, scale_offsets):
    from . import moe
    moe.grouped_gemm_stage(output, None, None, weight, weight_scales, expert_offsets,
                           scale_offsets, swiglu_input=gate_up, fmt=current_mxfp6_format())


def _moe_route_fake(permuted_activation, activation, logical_scales, topk_ids, expert_map,
                    local_experts: int):
    routes = activation.shape[0] * topk_ids.shape[1]
    scale_rows = routes + local_experts * 127
    dev = activation.device
    offsets = torch.empty(local_experts + 1, dtype=torch.int64, device=dev)
    return (torch.empty(scale_rows * (activation.shape[1] // 32), dtype=torch.uint8, device=dev),
            offsets, torch.empty_like(offsets), torch.empty(routes, dtype=torch.int32, device=dev))


def _empty_rows(x, n):
    return x.new_empty((x.shape[0], n))


_SCHEMAS = [
    ("vllm", "mach_mxfp8_sm120_gemm(Tensor x, Tensor weight, Tensor weight_scale) -> Tensor",
     _mxfp8_gemm, lambda x, w, s: _empty_rows(x, w.shape[0])),
    ("vllm", "mach_mxfp6_sm120_gemm(Tensor x, Tensor weight, Tensor weight_scale, int n, "
             "ScalarType dtype) -> Tensor",
     _mxfp6_gemm, lambda x, w, s, n, dtype: x.new_empty((x.shape[0], n), dtype=dtype)),
    ("vllm", "mach_swiglu_mxfp8_down(Tensor gate_up, Tensor weight, Tensor weight_scale) -> Tensor",
     lambda g, w, s: _swiglu_down(g, w, s, "e4m3"), lambda g, w, s: _empty_rows(g, w.shape[0])),
    ("vllm", "mach_swiglu_mxfp6_down(Tensor gate_up, Tensor weight, Tensor weight_scale) -> Tensor",
     lambda g, w, s: _swiglu_down(g, w, s, current_mxfp6_format()),
     lambda g, w, s: _empty_rows(g, w.shape[0])),
    ("vllm", "mach_norm_quant_mxfp8_gate_up(Tensor x, Tensor residual, Tensor norm_weight, "
             "float eps, Tensor weight, Tensor weight_scale) -> (Tensor, Tensor)",
     _norm_quant_gate_up,
     lambda x, r, nw, eps, w, s: (_empty_rows(x, w.shape[0]), torch.empty_like(x))),
    ("vllm", "mach_gemma_norm(Tensor x, Tensor? residual, Tensor weight, float eps) -> (Tensor, Tensor)",
     _gemma_norm,
     lambda x, r, w, eps: (torch.empty_like(x),
                           torch.empty_like(x) if r is not None else x.new_empty((0,)))),
    ("vllm", "mach_allreduce_gemma_rms_norm(Tensor hidden, Tensor residual, Tensor weight, "
             "float eps) -> (Tensor, Tensor)",
     _allreduce_gemma_rms_norm, lambda h, r, w, eps: (torch.empty_like(h), torch.empty_like(h))),
    ("vllm", "mach_mxfp8_mlp(Tensor x, Tensor w_gate_up, Tensor s_gate_up, Tensor w_down, "
             "Tensor s_down) -> Tensor",
     _mlp, lambda x, wg, sg, wd, sd: _empty_rows(x, wd.shape[0])),
    ("vllm_mach", "block_fp8_linear(Tensor a, Tensor b, Tensor sa, Tensor sb, Tensor sb64, "
                  "bool n64, bool ordered) -> Tensor",
     _block_fp8_linear,
     lambda a, b, sa, sb, sb64, n64, ordered: a.new_empty((a.shape[0], b.shape[0]),
                                                           dtype=torch.bfloat16)),
    ("vllm_mach_fp8", "silu_and_mul_per_block_quant(Tensor(a!) out, Tensor input, Tensor(b!) scales, "
                      "int group_size, Tensor? scale_ub, bool is_scale_transposed) -> ()",
     _silu_and_mul_per_block_quant, lambda *a: None),
    ("vllm", "mach_gdn_norm_mxfp6_out(Tensor core, Tensor gate, Tensor norm_weight, Tensor weight, "
             "Tensor weight_scale, float eps) -> Tensor",
     _gdn_norm_out, lambda c, g, nw, w, ws, eps: c.new_empty((c.shape[0], w.shape[0]))),
    ("mach_fp8_activation", "run(Tensor(a!) out, Tensor input, Tensor(b!) scales, "
                            "bool is_scale_transposed) -> ()",
     _fp8_activation_run, lambda *a: None),
    ("vllm_mach_block_fp8", "mm(Tensor a, Tensor b, Tensor sa, Tensor sb) -> Tensor",
     _block_fp8_mm, lambda a, b, sa, sb: a.new_empty((a.shape[0], b.shape[1]),
                                                     dtype=torch.bfloat16)),
    ("mach_norm_quant", "run(Tensor hidden, Tensor residual, Tensor gamma, Tensor workspace, "
                        "Tensor(a!) norm, Tensor(b!) residual_out, Tensor(c!) quant, "
                        "Tensor(d!) scales, int rank, float eps, bool fused) -> ()",
     _norm_quant_run, lambda *a: None),
    ("vllm", "mxfp6_sm120_quantize_mxfp8(Tensor input) -> (Tensor, Tensor)",
     _moe_quantize_mxfp8,
     lambda x: (torch.empty_like(x, dtype=torch.float8_e4m3fn),
                torch.empty((x.shape[0], x.shape[1] // 32), dtype=torch.uint8, device=x.device))),
    ("vllm", "mxfp6_sm120_quantize_mxfp8_packed(Tensor input) -> (Tensor, Tensor)",
     _moe_quantize_mxfp8_packed,
     lambda x: (torch.empty_like(x, dtype=torch.float8_e4m3fn),
                torch.empty(((x.shape[0] + 127) // 128 * 128 * ((x.shape[1] + 127) // 128) * 4,),
                            dtype=torch.uint8, device=x.device))),
    ("vllm", "mxfp6_sm120_route(Tensor(a!) permuted_activation, Tensor activation, "
             "Tensor logical_scales, Tensor topk_ids, Tensor? expert_map, int local_experts) "
             "-> (Tensor, Tensor, Tensor, Tensor)",
     _moe_route, _moe_route_fake),
    ("vllm", "mxfp6_sm120_grouped_gemm(Tensor(a!) output, Tensor activation, Tensor packed_scales, "
             "Tensor weight, Tensor weight_scales, Tensor expert_offsets, Tensor scale_offsets) -> ()",
     _moe_grouped_gemm, lambda *a: None),
    ("vllm", "mxfp6_sm120_silu_grouped_gemm(Tensor(a!) output, Tensor gate_up, Tensor weight, "
             "Tensor weight_scales, Tensor expert_offsets, Tensor scale_offsets) -> ()",
     _moe_silu_grouped_gemm, lambda *a: None),
    ("vllm", "mxfp6_sm120_reduce(Tensor(a!) output, Tensor routed_output, Tensor topk_weights, "
             "Tensor inverse_permutation) -> ()",
     _moe_reduce, lambda *a: None),
    ("vllm", "mxfp6_sm120_qwen35_grouped_moe(Tensor(a!) output, Tensor hidden_states, Tensor w1, "
             "Tensor w1_scale, Tensor w2, Tensor w2_scale, Tensor topk_weights, Tensor topk_ids, "
             "Tensor(b!) workspace13, Tensor(c!) workspace2) -> ()",
     _moe_whole_layer, lambda *a: None),
]

_DEFS_ONLY = [
    # (namespace, schema, python implementation registered for every backend)
    ("mach_norm_quant", "abi() -> str", lambda: _NORM_QUANT_ABI),
]


def op_names() -> list[str]:
    return ([f"{ns}::{schema.split('(')[0]}" for ns, schema, _, _ in _SCHEMAS]
            + [f"{ns}::{schema.split('(')[0]}" for ns, schema, _ in _DEFS_ONLY])


def register() -> None:
    """Idempotent. Defines the ops, their CUDA implementations and fake implementations."""
    global _registered
    with _lock:
        if _registered:
            return
        for ns, schema, impl, fake in _SCHEMAS:
            name = schema.split("(")[0]
            if hasattr(getattr(torch.ops, ns), name):
                continue  # another copy of the plugin already owns the name
            lib = torch.library.Library(ns, "FRAGMENT")
            lib.define(schema)
            lib.impl(name, impl, "CUDA")
            torch.library.register_fake(f"{ns}::{name}", fake, lib=lib)
            _libs.append(lib)
        for ns, schema, impl in _DEFS_ONLY:
            name = schema.split("(")[0]
            if hasattr(getattr(torch.ops, ns), name):
                continue
            lib = torch.library.Library(ns, "FRAGMENT")
            lib.define(schema)
            lib.impl(name, impl, "CompositeExplicitAutograd")
            _libs.append(lib)
        _registered = True
