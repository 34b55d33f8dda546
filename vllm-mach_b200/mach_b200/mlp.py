"""Dense decoder MLP block on the B200 kernels: dynamic MXFP8 activation quantisation ->
gate_up GEMM with fused SwiGLU + requant -> down GEMM -> (all-reduce +) residual + RMSNorm.

Mirrors the producers the reference installs over `Qwen2MoeMLP.forward` /
`Qwen3_5DecoderLayer.forward` (src/vllm_mach/mxfp6/mxfp8_mlp.py:62-84,
src/vllm_mach/mxfp6/mxfp8_norm_quant.py:83-130, src/vllm_mach/mxfp6/ar_norm.py:150-190):
column-parallel gate_up, row-parallel down with the reduce deferred into the next norm.
"""
from __future__ import annotations

import torch

from . import native


class MxMlpWeights:
    """Kernel-layout weights of one MLP shard: gate_up rows interleaved in groups of 32
    (gate and up of a feature meet in one GEMM tile) and swizzled E8M0 scales."""

    def __init__(self, w_gate_up, s_gate_up, w_down, s_down, fmt: str = "e4m3",
                 layout: int = native.LAYOUT_GATE_UP_32):
        self.w_gate_up, self.s_gate_up = w_gate_up, s_gate_up
        self.w_down, self.s_down = w_down, s_down
        self.fmt = fmt
        self.layout = layout
        self.intermediate = w_gate_up.shape[0] // 2
        self.hidden = w_down.shape[0]

    @classmethod
    def from_logical(cls, w_gate_up, s_gate_up, w_down, s_down, hidden: int, fmt: str = "e4m3"):
        """Checkpoint layout (codes [gate rows | up rows] + uint8 [N, K/32] scales) -> kernel
        layout; the load-time step of process_weights_after_loading
        (src/vllm_mach/mxfp6/dense_mxfp8.py:137-151, src/vllm_mach/mxfp6/dense.py:179-188)."""
        inter = w_gate_up.shape[0] // 2
        if inter % 32:
            raise ValueError("intermediate size must be a multiple of 32")
        w_gu = native.interleave_gate_up(w_gate_up.contiguous().view(torch.uint8))
        s_gu = native.interleave_gate_up(s_gate_up.contiguous())
        return cls(w_gu, native.pack_scales(s_gu, hidden), w_down.contiguous(),
                   native.pack_scales(s_down.contiguous(), inter), fmt)

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size()
                   for t in (self.w_gate_up, self.s_gate_up, self.w_down, self.s_down))


def mlp_forward(x: torch.Tensor, w: MxMlpWeights, out: torch.Tensor | None = None) -> torch.Tensor:
    """BF16 [M, H] -> BF16 [M, H] (this rank's partial sum when the MLP is sharded)."""
    if x.shape[0] == 0:
        return x.new_empty((0, w.hidden))
    codes, scales = native.quantize_mxfp8(x)
    return mlp_forward_quantized(codes, scales, w, out)


def mlp_forward_quantized(codes, scales, w: MxMlpWeights, out: torch.Tensor | None = None):
    """The same from MXFP8 activations (codes [M, H] + swizzled scales), which is what a
    preceding fused norm + quantise hands over (src/vllm_mach/mxfp6/mxfp8_norm_quant.py:83-130)."""
    h_codes, h_scales = native.mx_gemm_swiglu(codes, scales, w.w_gate_up, w.s_gate_up, w.fmt,
                                              w.layout)
    return native.mx_gemm(h_codes, h_scales, w.w_down, w.s_down, w.fmt, out=out)


def mlp_block(x, residual, norm_weight, eps: float, w: MxMlpWeights, group=None):
    """MLP + deferred row-parallel reduce + residual add + RMSNorm of the following layer.
    Returns (norm BF16, residual_out BF16). `group`: torch.distributed group of the TP ranks
    (None or size 1: no reduce)."""
    if group is not None and torch.distributed.get_world_size(group) > 1:
        from . import collective
        if collective.FUSED_SCATTER and x.shape[0] >= collective.FUSED_SCATTER_MIN_TOKENS:
            # Large batches: the down projection stores its partial rows straight into the
            # owners' all-reduce buffers (reduce-scatter in the GEMM epilogue).
            codes, scales = native.quantize_mxfp8(x)
            h_codes, h_scales = native.mx_gemm_swiglu(codes, scales, w.w_gate_up, w.s_gate_up,
                                                      w.fmt, w.layout)
            if collective.gemm_reduce_scatter(h_codes, h_scales, w.w_down, w.s_down, w.fmt, group):
                return collective.allreduce_add_rmsnorm(None, residual, norm_weight, eps, group)
            partial = native.mx_gemm(h_codes, h_scales, w.w_down, w.s_down, w.fmt)
        else:
            partial = mlp_forward(x, w)
        return collective.allreduce_add_rmsnorm(partial, residual, norm_weight, eps, group)
    partial = mlp_forward(x, w)
    norm, res, _, _ = native.add_rmsnorm_mxfp8(partial, residual, norm_weight, eps,
                                               want_quant=False)
    return norm, res


def mlp_block_owner(x, residual_rows, norm_weight, eps: float, w: MxMlpWeights, group=None,
                    want_norm: bool = True, codes_in_workspace: bool = False):
    """MLP + deferred reduce with row ownership between norms (native/owner_prefill/owner.cu:
    64-160): the residual stream is row-owned (`collective.owner_rows`), the down projection
    writes its partial sums straight into this rank's communication buffer, every owner reduces,
    normalises and quantises its rows, and every rank receives the MXFP8 codes + scales of all
    rows for the next layer's GEMM. `x`: BF16 [M, H], or a (codes, scales) pair from the
    previous block. Returns (codes [M, H], scales, residual_out_rows, norm_rows | None)."""
    from . import collective
    quantized = isinstance(x, tuple)
    m = (x[0] if quantized else x).shape[0]
    world = torch.distributed.get_world_size(group) if group is not None else 1
    if world == 1:
        partial = mlp_forward_quantized(x[0], x[1], w) if quantized else mlp_forward(x, w)
        norm, res, codes, scales = native.add_rmsnorm_mxfp8(partial, residual_rows, norm_weight,
                                                            eps, want_norm=want_norm)
        return codes, scales, res, norm
    dev = residual_rows.device
    target = collective.owner_partial_buffer(group, w.hidden, m, dev) if m else None
    partial = (mlp_forward_quantized(x[0], x[1], w, out=target) if quantized
               else mlp_forward(x, w, out=target))
    return collective.allreduce_owner_add_rmsnorm(None if target is not None else partial,
                                                  residual_rows, norm_weight, eps, group, m,
                                                  want_norm=want_norm,
                                                  codes_in_workspace=codes_in_workspace)
