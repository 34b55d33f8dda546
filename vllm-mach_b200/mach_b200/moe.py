"""Mixture-of-experts layer on the B200 kernels (W6A8 / W8A8 expert weights).

Follows the stage order of `Mxfp6Sm120Experts.apply` (src/vllm_mach/mxfp6/moe.py:574-702):
route -> gather + MXFP8 quantise -> grouped GEMM W1 with SwiGLU + requant -> grouped GEMM W2
-> top-k weighted reduce. `expert_map` keeps the reference's expert-parallel hook
(src/vllm_mach/mxfp6/moe.py:655-669): pairs routed to non-local experts are skipped and the
output is this rank's partial sum, reduced by the fused all-reduce + RMSNorm that follows.
"""
from __future__ import annotations

import torch

from . import native


class MoeWeights:
    """Stacked expert weights in kernel layout: w13 [E*2I, K(bytes)] with gate/up rows
    interleaved by 32 inside each expert, w2 [E*H, I(bytes)], swizzled scales packed over the
    stacked matrices."""

    def __init__(self, w13, s13, w2, s2, experts: int, hidden: int, inter: int, fmt: str):
        self.w13, self.s13, self.w2, self.s2 = w13, s13, w2, s2
        self.experts, self.hidden, self.inter, self.fmt = experts, hidden, inter, fmt

    @classmethod
    def from_logical(cls, w13, s13, w2, s2, fmt: str = "e2m3"):
        """w13 uint8 [E, 2I, K or 3K/4] ([gate | up] rows), s13 uint8 [E, 2I, K/32],
        w2 uint8 [E, H, I or 3I/4], s2 uint8 [E, H, I/32] (checkpoint layout,
        src/vllm_mach/mxfp6/moe.py:380-387)."""
        experts, two_i, _ = w13.shape
        hidden = w2.shape[1]
        inter = two_i // 2
        if two_i % 128 or hidden % 128 or inter % 32:
            raise ValueError("expert shapes must satisfy 2I % 128 == 0 and H % 128 == 0")
        w13 = w13.contiguous().view(torch.uint8)
        w13_il = torch.stack([native.interleave_gate_up(w13[e]) for e in range(experts)])
        s13_il = torch.stack([native.interleave_gate_up(s13[e].contiguous()) for e in range(experts)])
        packed13 = native.pack_scales(s13_il.reshape(experts * two_i, -1), hidden)
        packed2 = native.pack_scales(s2.contiguous().reshape(experts * hidden, -1), inter)
        return cls(w13_il.reshape(experts * two_i, -1), packed13,
                   w2.contiguous().view(torch.uint8).reshape(experts * hidden, -1), packed2,
                   experts, hidden, inter, fmt)

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.w13, self.s13, self.w2, self.s2))


def router_topk(logits: torch.Tensor, top_k: int):
    """BF16 [M, E] -> (weights FP32 [M, k] renormalised, ids int32 [M, k])."""
    native._require(logits, torch.bfloat16, "logits")
    m, e = logits.shape
    w = torch.empty((m, top_k), dtype=torch.float32, device=logits.device)
    ids = torch.empty((m, top_k), dtype=torch.int32, device=logits.device)
    with torch.cuda.device(logits.device):
        native._check(native.lib().mach_moe_router_topk(native._ptr(logits), native._ptr(w),
                                                        native._ptr(ids), m, e, top_k,
                                                        native._stream(logits)), "moe_router_topk")
    return w, ids


# Largest batch that takes the small-batch schedule (three CUDA-core launches; see
# mach_moe_small_batch; the entry point itself accepts up to 8 tokens). Measured on B200,
# 256 experts / top-8 / hidden 2048 / intermediate 512, CUDA-graph replay: one token 21.6 us
# against 28.9 us for route + gather + two grouped GEMMs + combine; the CUDA-core products cost
# about 17 us per further token (instruction-bound), the grouped path about 1-3 us (4 tokens:
# 67.8 against 32.7 us), so only single-token decode takes it.
SMALL_BATCH_MAX_TOKENS = 1


def chunk_rows_for(tokens: int, top_k: int, experts: int) -> int:
    if tokens <= 16:
        return 16
    # Measured cross-over on B200: below about 20 routed rows per expert the feature-major
    # grouped kernel (64-row chunks) streams the weights fastest, above it the token-major one.
    avg = tokens * top_k / experts
    return 64 if avg <= 20 else 128


def experts_forward(hidden, weights: MoeWeights, topk_weights, topk_ids, expert_map=None,
                    out: torch.Tensor | None = None):
    """BF16 [M, H] -> BF16 [M, H] (weighted sum over this rank's experts), into `out` when
    given."""
    native._require(hidden, torch.bfloat16, "hidden_states")
    native._require(topk_ids, torch.int32, "topk_ids")
    native._require(topk_weights, torch.float32, "topk_weights")
    m, h = hidden.shape
    top_k = topk_ids.shape[1]
    if h != weights.hidden:
        raise ValueError("w1 K does not match the activation")
    if out is None:
        out = torch.empty_like(hidden)
    elif out.shape != hidden.shape or out.dtype != torch.bfloat16 or not out.is_contiguous():
        raise ValueError("out must be a contiguous BF16 tensor shaped like hidden_states")
    if m == 0:
        return out
    lib, dev = native.lib(), hidden.device
    e = weights.experts
    if m <= SMALL_BATCH_MAX_TOKENS and top_k <= 16 and h <= 10240 and weights.inter <= 640:
        nbytes = int(lib.mach_moe_small_scratch_bytes(m, top_k, h, weights.inter))
        scratch = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        with torch.cuda.device(dev):
            native._check(lib.mach_moe_small_batch(
                native._ptr(hidden), native._ptr(topk_weights), native._ptr(topk_ids),
                native._ptr(expert_map), native._ptr(weights.w13), native._ptr(weights.s13),
                native._ptr(weights.w2), native._ptr(weights.s2), native._ptr(scratch),
                native._ptr(out), m, top_k, e, h, weights.inter, native._FORMATS[weights.fmt],
                native._stream(hidden)), "moe_small_batch")
        return out
    chunk = chunk_rows_for(m, top_k, e)
    rows_cap = int(lib.mach_moe_rows_cap(m, top_k, e))
    work_cap = int(lib.mach_moe_work_cap(m, top_k, e, chunk))
    i32 = dict(dtype=torch.int32, device=dev)
    counts, offsets = torch.empty(e, **i32), torch.empty(e + 1, **i32)
    pos_of, src_of = torch.empty(m * top_k, **i32), torch.empty(rows_cap, **i32)
    work, num_work = torch.empty(3 * work_cap, **i32), torch.empty(1, **i32)
    a_codes = torch.empty((rows_cap, h), dtype=torch.uint8, device=dev)
    a_scales = torch.empty(native.sf_bytes(rows_cap, h), dtype=torch.uint8, device=dev)
    act_codes = torch.empty((rows_cap, weights.inter), dtype=torch.uint8, device=dev)
    act_scales = torch.empty(native.sf_bytes(rows_cap, weights.inter), dtype=torch.uint8, device=dev)
    y = torch.empty((rows_cap, h), dtype=torch.bfloat16, device=dev)
    fmt = native._FORMATS[weights.fmt]
    p, st = native._ptr, native._stream(hidden)
    with torch.cuda.device(dev):
        native._check(lib.mach_moe_route(p(topk_ids), p(expert_map), m, top_k, e, chunk, rows_cap,
                                         work_cap, p(counts), p(offsets), p(pos_of), p(src_of),
                                         p(work), p(num_work), st), "moe_route")
        if m >= 512:
            # large batches: every token is read and quantised once, then stored top-k times
            native._check(lib.mach_moe_scatter_quantize(p(hidden), p(pos_of), m, top_k, h,
                                                        p(a_codes), p(a_scales), st),
                          "moe_scatter_quantize")
        else:
            # small batches: one warp per permuted row keeps more of the machine busy
            native._check(lib.mach_moe_gather_quantize(p(hidden), p(src_of), p(offsets), e, rows_cap,
                                                       h, p(a_codes), p(a_scales), st),
                          "moe_gather_quantize")
        native._check(lib.mach_moe_grouped_gemm(p(a_codes), p(a_scales), p(weights.w13),
                                                p(weights.s13), p(act_codes), p(act_scales),
                                                p(work), p(num_work), work_cap, rows_cap, e,
                                                2 * weights.inter, h, chunk, fmt, 1, st),
                      "moe_grouped_gemm(w1)")
        native._check(lib.mach_moe_grouped_gemm(p(act_codes), p(act_scales), p(weights.w2),
                                                p(weights.s2), p(y), None, p(work), p(num_work),
                                                work_cap, rows_cap, e, h, weights.inter, chunk,
                                                fmt, 0, st), "moe_grouped_gemm(w2)")
        native._check(lib.mach_moe_combine(p(y), p(topk_weights), p(pos_of), p(out), m, h, top_k,
                                           st), "moe_combine")
    return out


# ------------------------------------------------------------------ checkpoint-layout weights
_weight_cache: dict = {}


def cached_weights(w1, w1_scale, w2, w2_scale, fmt: str = "e2m3") -> MoeWeights:
    """Kernel-layout weights of a (w1, w2) pair in checkpoint layout, converted once and kept
    for as long as the source tensors live at the same addresses (weights are static after
    loading; the reference repacks at load too, src/vllm_mach/mxfp6/moe.py:380-387).
    Scales: uint8 E8M0, logical [E, rows, K/32] (a flat [E, rows * K/32] tensor is viewed)."""
    key = (w1.data_ptr(), w2.data_ptr(), w1_scale.data_ptr(), w2_scale.data_ptr(), fmt,
           tuple(w1.shape), tuple(w2.shape))
    hit = _weight_cache.get(key)
    if hit is not None:
        return hit
    experts, two_i, _ = w1.shape
    hidden = w2.shape[1]
    k1 = w1.shape[2] if fmt == "e4m3" else w1.shape[2] * 4 // 3
    k2 = w2.shape[2] if fmt == "e4m3" else w2.shape[2] * 4 // 3
    s1 = w1_scale.reshape(experts, two_i, k1 // 32)
    s2 = w2_scale.reshape(experts, hidden, k2 // 32)
    weights = MoeWeights.from_logical(w1, s1, w2, s2, fmt)
    _weight_cache[key] = weights
    return weights


def combine(routed_output, topk_weights, inverse_permutation, output) -> None:
    """out[m] = bf16(sum_k w[m, k] * routed_output[inverse_permutation[m, k]]), FP32, k ascending
    (mxfp6_sm120_reduce, src/vllm_mach/mxfp6/moe_utils.py:445-488)."""
    native._require(routed_output, torch.bfloat16, "routed_output")
    native._require(topk_weights, torch.float32, "topk_weights")
    native._require(inverse_permutation, torch.int32, "inverse_permutation")
    m, h = output.shape
    top_k = topk_weights.shape[1]
    with torch.cuda.device(output.device):
        native._check(native.lib().mach_moe_combine(
            native._ptr(routed_output), native._ptr(topk_weights), native._ptr(inverse_permutation),
            native._ptr(output), m, h, top_k, native._stream(output)), "moe_combine")


def permuted_rows(tokens: int, top_k: int, experts: int) -> int:
    """Rows the permuted buffers of the staged interface need: every expert's segment is padded
    to 128 rows (the reference pads only its scale rows, src/vllm_mach/mxfp6/moe_utils.py:232-243)."""
    return int(native.lib().mach_moe_rows_cap(tokens, top_k, experts))


def route_quantized(permuted_activation, activation, logical_scales, topk_ids, expert_map,
                    local_experts: int):
    """mxfp6_sm120_route on the B200 layout. activation: E4M3 codes [M, K]; logical_scales:
    uint8 [M, K/32]. Writes the permuted codes into `permuted_activation` (at least
    `permuted_rows(M, topk, local_experts)` rows of K bytes) and returns (packed scales in the
    swizzled layout, expert_offsets int64 [E+1] = routed rows before each expert,
    scale_offsets int64 [E+1] = first row of each expert's padded segment,
    inverse_permutation int32 [M * topk] = permuted row of every (token, k) pair, -1 when the
    expert is not local)."""
    lib = native.lib()
    native._require(activation, native._U8, "activation")
    native._require(logical_scales, torch.uint8, "logical_scales")
    native._require(topk_ids, torch.int32, "topk_ids")
    m, k = activation.shape
    top_k = topk_ids.shape[1]
    e = int(local_experts)
    rows_cap = permuted_rows(m, top_k, e)
    if permuted_activation.numel() * permuted_activation.element_size() < rows_cap * k:
        raise ValueError(f"permuted_activation must hold {rows_cap} rows of {k} bytes "
                         "(expert segments are padded to 128 rows)")
    dev = activation.device
    chunk = 128
    work_cap = int(lib.mach_moe_work_cap(m, top_k, e, chunk))
    i32 = dict(dtype=torch.int32, device=dev)
    counts, offsets = torch.empty(e, **i32), torch.empty(e + 1, **i32)
    pos_of, src_of = torch.empty(m * top_k, **i32), torch.empty(rows_cap, **i32)
    work, num_work = torch.empty(3 * work_cap, **i32), torch.empty(1, **i32)
    packed = torch.empty(native.sf_bytes(rows_cap, k), dtype=torch.uint8, device=dev)
    expert_offsets = torch.empty(e + 1, dtype=torch.int64, device=dev)
    scale_offsets = torch.empty(e + 1, dtype=torch.int64, device=dev)
    p, st = native._ptr, native._stream(activation)
    with torch.cuda.device(dev):
        native._check(lib.mach_moe_route(p(topk_ids), p(expert_map), m, top_k, e, chunk, rows_cap,
                                         work_cap, p(counts), p(offsets), p(pos_of), p(src_of),
                                         p(work), p(num_work), st), "moe_route")
        native._check(lib.mach_moe_scatter_codes(p(activation), p(logical_scales), p(pos_of), m,
                                                 top_k, k, p(permuted_activation), p(packed), st),
                      "moe_scatter_codes")
        native._check(lib.mach_moe_stage_offsets(p(counts), p(offsets), e, p(expert_offsets),
                                                 p(scale_offsets), st), "moe_stage_offsets")
    return packed, expert_offsets, scale_offsets, pos_of


_stage_cache: dict = {}


def _stage_weight(weight, weight_scales, fmt: str):
    """[E, rows, K bytes] checkpoint-layout expert weights -> stacked matrix + swizzled scales
    packed over the stack (no gate/up interleave: the staged GEMMs have no fused epilogue)."""
    key = (weight.data_ptr(), weight_scales.data_ptr(), fmt, tuple(weight.shape))
    hit = _stage_cache.get(key)
    if hit is None:
        experts, rows, cols = weight.shape
        k = cols if fmt == "e4m3" else cols * 4 // 3
        logical = weight_scales.reshape(experts * rows, k // 32).contiguous()
        hit = (weight.contiguous().view(torch.uint8).reshape(experts * rows, cols),
               native.pack_scales(logical, k), experts, rows, k)
        _stage_cache[key] = hit
    return hit


def grouped_gemm_stage(output, activation, packed_scales, weight, weight_scales, expert_offsets,
                       scale_offsets, swiglu_input=None, fmt: str = "e2m3") -> None:
    """mxfp6_sm120_grouped_gemm (swiglu_input is None) and mxfp6_sm120_silu_grouped_gemm
    (swiglu_input = the BF16 [rows, 2I] output of the first stage): one grouped W6A8 GEMM over
    the permuted rows into `output` BF16 [rows, N]."""
    lib = native.lib()
    w, ws, experts, w_rows, k = _stage_weight(weight, weight_scales, fmt)
    if swiglu_input is not None:
        activation, packed_scales = native.swiglu_quantize_mxfp8(swiglu_input)
    rows_cap = activation.shape[0]
    if output.shape[0] < rows_cap or output.shape[1] != w_rows or output.dtype != torch.bfloat16:
        raise ValueError("output must be BF16 [permuted rows, N]")
    avg = max(0, rows_cap - 127 * experts) / experts
    chunk = 64 if avg <= 20 else 128
    work_cap = int(lib.mach_moe_work_cap(rows_cap, 1, experts, chunk))
    dev = activation.device
    work = torch.empty(3 * work_cap, dtype=torch.int32, device=dev)
    num_work = torch.empty(1, dtype=torch.int32, device=dev)
    p, st = native._ptr, native._stream(activation)
    with torch.cuda.device(dev):
        native._check(lib.mach_moe_work_from_offsets(p(expert_offsets), p(scale_offsets), experts,
                                                     chunk, work_cap, p(work), p(num_work), st),
                      "moe_work_from_offsets")
        native._check(lib.mach_moe_grouped_gemm(p(activation), p(packed_scales), p(w), p(ws),
                                                p(output), None, p(work), p(num_work), work_cap,
                                                rows_cap, experts, w_rows, k, chunk,
                                                native._FORMATS[fmt], 0, st), "moe_grouped_gemm")
