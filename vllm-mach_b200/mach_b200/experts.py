"""The experts class vLLM's modular MoE kernel drives, on the B200 kernels.

Mirrors `Mxfp6Sm120Experts` (src/vllm_mach/mxfp6/moe.py:478-702): same constructor checks, same
capability predicates, same `workspace_shapes` / `apply` signatures and error behaviour. `apply`
runs the whole routed-experts layer (`mach_b200.moe.experts_forward`): route -> quantise +
permute -> grouped GEMM W1 with SwiGLU + requant -> grouped GEMM W2 -> top-k weighted reduce
into `output`. The checkpoint-layout weights are converted to the kernel layout once per
(w1, w2) pair and cached (`moe.cached_weights`), the way the reference repacks at load.

vLLM >= 0.33 supplies the base class; without it (this repository's tests) a plain object
base keeps the contract testable.
"""
from __future__ import annotations

import torch

from . import moe

try:  # vLLM 0.33 / 0.34
    import vllm.model_executor.layers.fused_moe.modular_kernel as mk
    _Base = mk.FusedMoEPermuteExpertsUnpermute
except Exception:  # noqa: BLE001
    mk = None
    _Base = object

try:
    from vllm.model_executor.layers.fused_moe.activation import MoEActivation
    _SILU = MoEActivation.SILU
except Exception:  # noqa: BLE001
    _SILU = "silu"


def _is_silu(activation) -> bool:
    return activation == _SILU or str(getattr(activation, "value", activation)).lower() == "silu"


class Mxfp6B200Experts(_Base):
    """W6A8 (or W8A8) routed experts: static MXFP6 / MXFP8 weights, dynamic MXFP8 activations."""

    weight_format = "e2m3"

    def __init__(self, moe_config=None, quant_config=None, max_num_tokens=None,
                 num_dispatchers=None):
        if _Base is not object:
            super().__init__(moe_config, quant_config, max_num_tokens=max_num_tokens,
                             num_dispatchers=num_dispatchers)
        else:
            self.moe_config, self.quant_config = moe_config, quant_config
        if quant_config is not None:
            if getattr(quant_config, "w1_scale", None) is None or \
                    getattr(quant_config, "w2_scale", None) is None:
                raise ValueError("MXFP6 B200 MoE requires packed weight scales")
            if getattr(quant_config, "w1_bias", None) is not None or \
                    getattr(quant_config, "w2_bias", None) is not None:
                raise ValueError("MXFP6 B200 MoE does not support expert bias")
            if getattr(quant_config, "gemm1_clamp_limit", None) is not None:
                raise ValueError("MXFP6 B200 MoE does not support SwiGLU clamping")

    # ---- capability predicates (src/vllm_mach/mxfp6/moe.py:503-540)
    @property
    def expects_unquantized_inputs(self) -> bool:
        return True

    @staticmethod
    def activation_format():
        return mk.FusedMoEActivationFormat.Standard if mk is not None else "standard"

    @staticmethod
    def _supports_current_device() -> bool:
        from .linear import b200_available
        return b200_available()[0]

    @staticmethod
    def _supports_no_act_and_mul() -> bool:
        return False

    @staticmethod
    def _supports_quant_scheme(weight_key, activation_key) -> bool:
        return True

    @staticmethod
    def _supports_activation(activation) -> bool:
        return _is_silu(activation)

    @staticmethod
    def _supports_parallel_config(moe_parallel_config) -> bool:
        return not getattr(moe_parallel_config, "use_batched_activation_format", False)

    @staticmethod
    def _supports_shape(hidden_dim: int) -> bool:
        return hidden_dim % 128 == 0

    def finalize_weight_and_reduce_impl(self):
        from vllm.model_executor.layers.fused_moe.topk_weight_and_reduce import (
            TopKWeightAndReduceNoOP)
        return TopKWeightAndReduceNoOP()

    @property
    def w1_scale(self):
        return getattr(self.quant_config, "w1_scale", None)

    @property
    def w2_scale(self):
        return getattr(self.quant_config, "w2_scale", None)

    def workspace_shapes(self, M, N, K, topk, global_num_experts, local_num_experts,
                         expert_tokens_meta, activation):
        """The kernels allocate their own permuted buffers (their row count depends on the
        128-row padding per expert); the workspaces vLLM hands over are not used, so the
        smallest legal shapes are requested. Output is (M, K) as in the reference."""
        del N, topk, global_num_experts, local_num_experts, expert_tokens_meta, activation
        return (1, 1), (1, 1), (M, K)

    def apply(self, output, hidden_states, w1, w2, topk_weights, topk_ids, activation,
              global_num_experts, expert_map, a1q_scale, a2_scale, workspace13, workspace2,
              expert_tokens_meta, apply_router_weight_on_input) -> None:
        del a1q_scale, a2_scale, workspace13, workspace2
        if apply_router_weight_on_input:
            raise ValueError("MXFP6 B200 MoE requires router weights on output")
        if expert_tokens_meta is not None:
            raise ValueError("MXFP6 B200 MoE requires standard routed activations")
        if not _is_silu(activation):
            raise ValueError("MXFP6 B200 MoE currently supports only SiLU")
        tokens, hidden_size = hidden_states.shape
        w1_scale, w2_scale = self.w1_scale, self.w2_scale
        if w1_scale is None or w2_scale is None:
            raise ValueError("MXFP6 B200 MoE requires packed weight scales")
        if (expert_map is None and w1.shape[0] == global_num_experts + 1
                and w2.shape[0] == global_num_experts + 1):
            # a shared expert appended as one more row by the small-batch specialisation
            w1, w2 = w1[:global_num_experts], w2[:global_num_experts]
            w1_scale, w2_scale = w1_scale[:global_num_experts], w2_scale[:global_num_experts]
        local_experts = w1.shape[0]
        packed = self.weight_format != "e4m3"
        k_of = (lambda t: t.shape[2] * 4 // 3) if packed else (lambda t: t.shape[2])
        if k_of(w1) != hidden_size:
            raise ValueError("w1 packed K does not match the activation")
        intermediate_size = k_of(w2)
        if w1.shape[1] != 2 * intermediate_size or w2.shape[1] != hidden_size:
            raise ValueError("MXFP6 MoE weight shapes are inconsistent")
        if expert_map is None and global_num_experts != local_experts:
            raise ValueError("global and local expert counts require an expert_map")
        if tokens == 0:
            return
        weights = moe.cached_weights(w1, w1_scale, w2, w2_scale, self.weight_format)
        ids = topk_ids if topk_ids.dtype == torch.int32 else topk_ids.to(torch.int32)
        tw = topk_weights if topk_weights.dtype == torch.float32 else topk_weights.float()
        emap = None
        if expert_map is not None:
            emap = expert_map if expert_map.dtype == torch.int32 else expert_map.to(torch.int32)
        moe.experts_forward(hidden_states, weights, tw.contiguous(), ids.contiguous(), emap,
                            out=output)
