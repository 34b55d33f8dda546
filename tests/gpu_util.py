"""Helpers shared by the GPU parity tests (seeded inputs per benchmark configuration, comparisons)."""
from __future__ import annotations

import numpy as np
import torch

from oracle import mx_oracle as ora


def gpu_available() -> bool:
    return torch.cuda.is_available() and torch.cuda.get_device_capability(0) == (10, 0)


def randn_bf16(m, k, seed, sigma=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(m, k, generator=g) * sigma).to(torch.bfloat16)


def edge_activations(m, k, seed):
    """Rows cycle through magnitudes {1, 0, 1e-15, 50}; half of row 2 is exactly zero."""
    x = randn_bf16(m, k, seed).float()
    mags = [1.0, 0.0, 1.0e-15, 50.0]
    for r in range(m):
        x[r] *= mags[r % 4]
    if m > 2:
        x[2, : k // 2] = 0.0
    return x.to(torch.bfloat16)


def mxfp8_weight(n, k, seed, sigma=0.02):
    """Seeded BF16 weight quantised with the reference checkpoint rule.
    Returns (codes uint8 [N,K], logical scales uint8 [N,K/32], dequantised FP32 [N,K])."""
    w = randn_bf16(n, k, seed, sigma)
    codes, scales = ora.quantize_weight_mxfp8(w)
    return codes, scales, ora.dequantize_mx(codes, scales)


def bytes_equal(a: torch.Tensor, b: torch.Tensor) -> bool:
    return torch.equal(a.contiguous().view(torch.uint8).cpu(), b.contiguous().view(torch.uint8).cpu())


def mismatch_report(a: torch.Tensor, b: torch.Tensor) -> str:
    a8, b8 = a.contiguous().view(torch.uint8).cpu(), b.contiguous().view(torch.uint8).cpu()
    bad = (a8 != b8).nonzero()
    return f"{bad.shape[0]} of {a8.numel()} bytes differ; first {bad[:5].tolist()}"


def rel_fro(a: torch.Tensor, b: torch.Tensor) -> float:
    a, b = a.float().cpu(), b.float().cpu()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))


class LocalRanks:
    """All ranks of a tensor-parallel group on ONE device: `world` communication buffers and
    workspaces, driven through mach_allreduce_local_ranks (one cooperative grid)."""

    def __init__(self, world: int, hidden: int, tokens_cap: int):
        import ctypes
        from mach_b200 import native
        self.lib, self.world, self.hidden, self.tokens_cap = native.lib(), world, hidden, tokens_cap
        self.native = native
        nbytes = self.lib.mach_ar_buffer_bytes(world, tokens_cap, hidden)
        assert nbytes > 0
        self.buffers = []
        for _ in range(world):
            p = ctypes.c_void_p()
            native._check(self.lib.mach_ar_buffer_alloc(nbytes, ctypes.byref(p)), "ar_buffer_alloc")
            self.buffers.append(p.value)
        arr = (ctypes.c_void_p * world)(*self.buffers)
        self.handles = []
        for r in range(world):
            ws = ctypes.c_void_p()
            native._check(self.lib.mach_ar_create(world, r, tokens_cap, hidden, arr, ctypes.byref(ws)),
                          "ar_create")
            self.handles.append(ws.value)

    def partial_buffer(self, rank: int, m: int) -> torch.Tensor:
        import ctypes
        p = ctypes.c_void_p()
        self.native._check(self.lib.mach_ar_partial_ptr(self.handles[rank], ctypes.byref(p)),
                           "ar_partial_ptr")
        return self.native.tensor_from_ptr(p.value, (m, self.hidden), torch.bfloat16, "cuda:0")

    def codes_buffer(self, rank: int, m: int):
        import ctypes
        c, s = ctypes.c_void_p(), ctypes.c_void_p()
        self.native._check(self.lib.mach_ar_codes_ptr(self.handles[rank], ctypes.byref(c),
                                                      ctypes.byref(s)), "ar_codes_ptr")
        return (self.native.tensor_from_ptr(c.value, (m, self.hidden), torch.uint8, "cuda:0"),
                self.native.tensor_from_ptr(s.value, (self.native.sf_bytes(m, self.hidden),),
                                            torch.uint8, "cuda:0"))

    def run(self, partials, residuals, gamma, eps, m, algo=0, owner=False, weight_bias=1.0,
            in_place=False):
        """partials / residuals: per-rank CUDA tensors (partials[r] may be None in the owner
        form). in_place (owner form): the codes and scales are the views of each rank's own
        communication buffer. Returns per-rank (norm, residual_out, codes, scales)."""
        import ctypes
        native, world, h = self.native, self.world, self.hidden
        outs = []
        for r in range(world):
            rows = m
            if owner:
                first, count = ctypes.c_int64(), ctypes.c_int64()
                self.lib.mach_ar_owner_rows(world, r, m, ctypes.byref(first), ctypes.byref(count))
                rows = count.value
            if in_place:
                codes, scales = self.codes_buffer(r, m)
                codes.zero_()
                scales.zero_()
            else:
                codes = torch.zeros((m, h), dtype=torch.uint8, device="cuda")
                scales = torch.zeros(native.sf_bytes(m, h), dtype=torch.uint8, device="cuda")
            outs.append((torch.full((rows, h), 7.0, dtype=torch.bfloat16, device="cuda"),
                         torch.full((rows, h), 7.0, dtype=torch.bfloat16, device="cuda"),
                         codes, scales))

        def ptrs(tensors):
            return (ctypes.c_void_p * world)(*[None if t is None else t.data_ptr() for t in tensors])
        rc = self.lib.mach_allreduce_local_ranks(
            world, (ctypes.c_void_p * world)(*self.handles), ptrs(partials), ptrs(residuals),
            gamma.data_ptr(), eps, weight_bias, ptrs([o[0] for o in outs]),
            ptrs([o[1] for o in outs]), ptrs([o[2] for o in outs]), ptrs([o[3] for o in outs]),
            m, h, algo, int(owner), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
        native._check(rc, "allreduce_local_ranks")
        torch.cuda.synchronize()
        return outs

    def close(self):
        torch.cuda.synchronize()
        for hnd in self.handles:
            self.lib.mach_ar_destroy(hnd)
        for b in self.buffers:
            self.lib.mach_ar_buffer_free(b)
        self.handles, self.buffers = [], []
