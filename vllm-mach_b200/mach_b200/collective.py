"""Row-parallel reduce fused with residual add + RMSNorm over NVLink peer memory.

`allreduce_add_rmsnorm` is the public call; it follows the contract of
torch.ops.mach_norm_quant.run / compiled_allreduce_gemma_rms_norm
(native/ar_norm/binding.cu:11-70, src/vllm_mach/mxfp6/compiled_ar_norm.py:7-84):
a = bf16(sum over ranks, FP32, rank order); res = bf16(a + residual);
norm = bf16(res * rsqrt(mean(res^2) + eps) * (1 + gamma)).

`allreduce_owner_add_rmsnorm` is the same reduce with row ownership between norms
(native/owner_prefill/owner.cu:64-160): the residual stream and the BF16 norm stay with the
rank that owns the rows, every rank receives the MXFP8 codes and scales of all rows.

One process per GPU. The communication buffers are CUDA allocations shared through IPC
handles that travel over the torch.distributed group (the reference exchanges its FlashInfer
workspace handles over the TP cpu_group the same way, src/vllm_mach/mxfp6/ar_norm.py:113-128).

Failure behaviour: a device-side wait for a peer that gives up poisons the outputs (NaN /
0x7F / 0xFF) and marks the workspace as failed on the device. `poll_status()` (call it at a
host synchronisation point, e.g. the end of a step) turns that into host state: the failed
workspaces then route `allreduce_add_rmsnorm` through NCCL `all_reduce` + the local
rounded-sum norm kernel (the always-correct route of compiled_ar_norm.py:38-48) until
`reset_failed()` has been called collectively. Shapes the fused kernel does not take
(hidden > 8192) and groups whose buffers cannot be shared over IPC use the same route.
"""
from __future__ import annotations

import ctypes
import logging
import threading

import torch
import torch.distributed as dist

from . import native

logger = logging.getLogger(__name__)
_lock = threading.RLock()
_workspaces: dict = {}
_unavailable: set = set()     # (group id, hidden, device index) whose IPC set-up failed

MAX_FUSED_HIDDEN = 8192


class ArWorkspace:
    """Peer-mapped buffers of one TP group for a fixed hidden size and token capacity."""

    def __init__(self, group, hidden: int, tokens_cap: int, device: torch.device):
        lib = native.lib()
        self.group, self.hidden, self.tokens_cap, self.device = group, hidden, tokens_cap, device
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self._peers: list[int] = []
        self._opened: list[int] = []
        self.handle = None
        self.failed = False
        with torch.cuda.device(device):
            nbytes = lib.mach_ar_buffer_bytes(self.world, tokens_cap, hidden)
            if nbytes == 0:
                raise ValueError("unsupported all-reduce workspace shape")
            own = ctypes.c_void_p()
            native._check(lib.mach_ar_buffer_alloc(nbytes, ctypes.byref(own)), "ar_buffer_alloc")
            self.own = own.value
            raw = ctypes.create_string_buffer(64)
            native._check(lib.mach_ar_ipc_export(self.own, raw), "ar_ipc_export")
            handles = exchange(group, raw.raw)
            error = None
            for r, h in enumerate(handles):
                if r == self.rank:
                    self._peers.append(self.own)
                    continue
                ptr = ctypes.c_void_p()
                rc = lib.mach_ar_ipc_open(h, ctypes.byref(ptr))
                if rc != 0:
                    error = lib.mach_last_error().decode(errors="replace")
                    break
                self._peers.append(ptr.value)
                self._opened.append(ptr.value)
            # every rank learns whether every rank could map every buffer
            oks = exchange(group, b"\x00" if error else b"\x01")
            if any(o != b"\x01" for o in oks):
                for p in self._opened:
                    lib.mach_ar_ipc_close(p)
                dist.barrier(group)
                lib.mach_ar_buffer_free(self.own)
                raise RuntimeError(f"all-reduce buffers cannot be shared over CUDA IPC: {error}")
            arr = (ctypes.c_void_p * self.world)(*self._peers)
            ws = ctypes.c_void_p()
            native._check(lib.mach_ar_create(self.world, self.rank, tokens_cap, hidden, arr,
                                             ctypes.byref(ws)), "ar_create")
            self.handle = ws.value
            ptr = ctypes.c_void_p()
            native._check(lib.mach_ar_partial_ptr(self.handle, ctypes.byref(ptr)), "ar_partial_ptr")
            self._partial_ptr = ptr.value
        dist.barrier(group)

    def partial_buffer(self, m: int) -> torch.Tensor:
        """BF16 [m, hidden] inside this rank's communication buffer: a GEMM that writes its
        partial sums here spares the owner-form reduce one local copy."""
        if m > self.tokens_cap:
            raise ValueError("more tokens than the workspace holds")
        return native.tensor_from_ptr(self._partial_ptr, (m, self.hidden), torch.bfloat16,
                                      self.device)

    def codes_buffer(self, m: int):
        """(E4M3 [m, hidden], swizzled E8M0 scales) INSIDE this rank's communication buffer:
        where the owners of the rows store them. Passing them as the outputs of the owner-form
        reduce skips the copy into caller tensors; they are overwritten by the next reduce on
        this workspace."""
        if m > self.tokens_cap:
            raise ValueError("more tokens than the workspace holds")
        codes, scales = native._P(), native._P()
        native._check(native.lib().mach_ar_codes_ptr(self.handle, ctypes.byref(codes),
                                                     ctypes.byref(scales)), "ar_codes_ptr")
        return (native.tensor_from_ptr(codes.value, (m, self.hidden), torch.float8_e4m3fn,
                                       self.device),
                native.tensor_from_ptr(scales.value, (native.sf_bytes(m, self.hidden),),
                                       torch.uint8, self.device))

    def set_wait_limit_us(self, microseconds: int) -> None:
        native._check(native.lib().mach_ar_set_wait_limit_us(self.handle, int(microseconds)),
                      "ar_set_wait_limit_us")

    def reset(self) -> None:
        """Collective: clears epoch, flags and the failed mark on every rank."""
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)
        with torch.cuda.device(self.device):
            native._check(native.lib().mach_ar_reset(
                self.handle, torch.cuda.current_stream(self.device).cuda_stream), "ar_reset")
        dist.barrier(self.group)
        self.failed = False

    def close(self):
        """Collective: every rank stops using the buffers before any is unmapped or freed."""
        if self.handle is None:
            return
        lib = native.lib()
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)
        with torch.cuda.device(self.device):
            lib.mach_ar_destroy(self.handle)
            for p in self._opened:
                lib.mach_ar_ipc_close(p)
            dist.barrier(self.group)
            lib.mach_ar_buffer_free(self.own)
        self.handle = None


def exchange(group, payload: bytes) -> list[bytes]:
    """All-gather of one small byte string per rank (rank order)."""
    out = [None] * dist.get_world_size(group)
    dist.all_gather_object(out, payload, group=group)
    return out


def workspace_for(group, hidden: int, tokens: int, device) -> ArWorkspace | None:
    """Cached per (group, hidden, device); grows collectively (every rank sees the same sizes).
    None when the fused kernel cannot serve this group or shape (the caller reduces with
    NCCL)."""
    key = (id(group), hidden, torch.device(device).index)
    with _lock:
        if key in _unavailable or hidden > MAX_FUSED_HIDDEN or hidden % 32:
            return None
        ws = _workspaces.get(key)
        if ws is None or ws.tokens_cap < tokens:
            if ws is not None:
                ws.close()
                del _workspaces[key]
            cap = max(4096, 1 << (max(tokens, 1) - 1).bit_length())
            try:
                ws = ArWorkspace(group, hidden, cap, torch.device(device))
            except RuntimeError as error:
                logger.warning("mach_b200: fused all-reduce unavailable, using NCCL (%s)", error)
                _unavailable.add(key)
                return None
            _workspaces[key] = ws
        return ws


def close_all():
    with _lock:
        for ws in _workspaces.values():
            ws.close()
        _workspaces.clear()
        _tensors.clear()


# The reference hands its FlashInfer workspace to `mach_norm_quant.run` as an int64 CUDA tensor
# (a table of 7 device pointers, src/vllm_mach/mxfp6/ar_norm.py:113-128). The same argument
# carries a B200 workspace: a 7-entry int64 CUDA tensor whose identity (its address) names the
# ArWorkspace, so the op never reads device memory to find it.
_tensors: dict = {}


def workspace_tensor(group, hidden: int, tokens: int, device) -> torch.Tensor:
    ws = workspace_for(group, hidden, tokens, device)
    if ws is None:
        raise RuntimeError("the fused all-reduce is unavailable for this group or shape")
    with _lock:
        for tensor, owner in _tensors.values():
            if owner is ws:
                return tensor
        tensor = torch.zeros(7, dtype=torch.int64, device=ws.device)
        tensor[0] = ws.handle
        _tensors[tensor.data_ptr()] = (tensor, ws)
        return tensor


def workspace_from_tensor(tensor: torch.Tensor) -> ArWorkspace:
    if tensor.dtype != torch.int64 or tensor.numel() != 7 or not tensor.is_contiguous():
        raise RuntimeError("mach_norm_quant.run requires a contiguous int64 workspace with 7 entries")
    with _lock:
        hit = _tensors.get(tensor.data_ptr())
    if hit is None or hit[1].handle is None:
        raise RuntimeError("workspace tensor was not created by collective.workspace_tensor "
                           "(or its workspace has been closed)")
    return hit[1]


def poll_status() -> int:
    """Reads (and clears) the device status word; call at a host synchronisation point.
    Non-zero (401 / 402: a wait for a peer gave up; 403: a failed workspace was used): every
    workspace of this process is marked failed and the public calls reduce through NCCL until
    `reset_failed()`; the outputs of the failing call were poisoned on the device."""
    code = native.device_status()
    if code in (401, 402, 403):
        with _lock:
            for ws in _workspaces.values():
                ws.failed = True
    return code


def reset_failed() -> None:
    """Collective over every group that has a failed workspace."""
    with _lock:
        for ws in _workspaces.values():
            if ws.failed:
                ws.reset()


# Reduce-scatter from the down projection's epilogue (`mach_mx_gemm_reduce_scatter`). Off by
# default: measured on 2 B200s at M = 4096 the fused pair (GEMM with peer stores 67 us +
# reduce/norm 49 us) ties with GEMM 44 us + one-shot all-reduce 76 us, because 128-byte peer
# stores from the epilogue move ~450 GB/s and are not hidden behind the MMAs; results are
# bit-identical either way. Every rank must use the same setting.
FUSED_SCATTER = False
# Smallest batch for the fused form (below it the GEMM does not take the CTA-pair kernel, and
# the payload is latency-bound anyway).
FUSED_SCATTER_MIN_TOKENS = 512


def gemm_reduce_scatter(h_codes, h_scales, w_down, s_down, fmt: str, group) -> bool:
    """Row-parallel down projection with the reduce-scatter in its epilogue
    (`mach_mx_gemm_reduce_scatter`). Returns False when the shape does not qualify: the caller
    then runs the plain GEMM and passes its output to `allreduce_add_rmsnorm`. The decision
    depends only on shapes, so every rank takes the same branch."""
    world = dist.get_world_size(group) if group is not None else 1
    m = h_codes.shape[0]
    hidden = w_down.shape[0]
    if not FUSED_SCATTER or world < 2 or m < FUSED_SCATTER_MIN_TOKENS or hidden % 128:
        return False
    ws = workspace_for(group, hidden, m, h_codes.device)
    if ws is None or ws.failed:
        return False
    k = h_codes.shape[1]
    with torch.cuda.device(h_codes.device):
        native._check(native.lib().mach_mx_gemm_reduce_scatter(
            ws.handle, native._ptr(h_codes), native._ptr(h_scales), native._ptr(w_down),
            native._ptr(s_down), m, hidden, k, native._FORMATS[fmt], native._stream(h_codes)),
            "mx_gemm_reduce_scatter")
    return True


def _nccl_route(partial, residual, gamma, eps, group, weight_bias, want_quant):
    """NCCL all_reduce (BF16 wire; NCCL's own summation order) + the rounded-sum norm kernel.
    Always available; not bit-identical to the fused kernel's rank-order FP32 sum."""
    summed = partial.clone()
    dist.all_reduce(summed, group=group)
    norm, res, codes, scales = native.add_rmsnorm_mxfp8(
        summed, residual, gamma, eps, weight_bias, want_quant=want_quant, rounded_sum=True)
    return (norm, res, codes, scales) if want_quant else (norm, res)


def allreduce_add_rmsnorm(partial, residual, gamma, eps: float, group, weight_bias: float = 1.0,
                          want_quant: bool = False, algo: int = 0, checked: bool = False):
    """Returns (norm, residual_out) or (norm, residual_out, codes, scales) with want_quant.
    algo: 0 choose, 1 one-shot, 2 two-shot (every rank must pass the same value).
    partial=None: the partial sums were scattered by `gemm_reduce_scatter` on this stream.
    checked=True synchronises the device after the call and raises RuntimeError when a wait
    for a peer gave up (debugging; production code calls `poll_status()` once per step)."""
    for t, name in ((residual, "residual"), (gamma, "gamma")):
        native._require(t, torch.bfloat16, name)
    if partial is None:
        partial_like = residual
    else:
        native._require(partial, torch.bfloat16, "partial")
        partial_like = partial
    m, h = partial_like.shape
    world = dist.get_world_size(group) if group is not None else 1
    if world == 1:
        norm, res, codes, scales = native.add_rmsnorm_mxfp8(
            partial, residual, gamma, eps, weight_bias, want_quant=want_quant, rounded_sum=True)
        return (norm, res, codes, scales) if want_quant else (norm, res)
    dev = partial_like.device
    ws = workspace_for(group, h, m, dev) if m else None
    if m and (ws is None or ws.failed):
        if partial is None:
            raise RuntimeError("the fused all-reduce is unavailable and the partial sums were "
                               "scattered into its buffers")
        return _nccl_route(partial, residual, gamma, eps, group, weight_bias, want_quant)
    norm = torch.empty_like(partial_like)
    res = torch.empty_like(partial_like)
    codes = scales = None
    if want_quant:
        codes = torch.empty((m, h), dtype=torch.float8_e4m3fn, device=dev)
        scales = torch.empty((native.sf_bytes(m, h),), dtype=torch.uint8, device=dev)
    if m:
        with torch.cuda.device(dev):
            native._check(native.lib().mach_allreduce_residual_rmsnorm_mxfp8(
                ws.handle, native._ptr(partial), native._ptr(residual), native._ptr(gamma), eps,
                weight_bias, native._ptr(norm), native._ptr(res), native._ptr(codes),
                native._ptr(scales), m, h, algo, native._stream(partial_like)),
                "allreduce_rmsnorm")
        if checked:
            _raise_on_failure(dev)
    return (norm, res, codes, scales) if want_quant else (norm, res)


def _raise_on_failure(dev) -> None:
    torch.cuda.synchronize(dev)
    code = poll_status()
    if code:
        raise RuntimeError(f"fused all-reduce: a device-side wait gave up (status {code}); the "
                           "outputs are poisoned and the workspace needs reset_failed()")


def owner_rows(m: int, group) -> tuple[int, int]:
    """(first row, row count) of the block this rank owns in an [m, H] activation."""
    world = dist.get_world_size(group) if group is not None else 1
    rank = dist.get_rank(group) if group is not None else 0
    first, count = ctypes.c_int64(), ctypes.c_int64()
    native._check(native.lib().mach_ar_owner_rows(world, rank, m, ctypes.byref(first),
                                                  ctypes.byref(count)), "ar_owner_rows")
    return first.value, count.value


def owner_partial_buffer(group, hidden: int, m: int, device) -> torch.Tensor | None:
    """BF16 [m, hidden] view into this rank's communication buffer for the producing GEMM
    (pass partial=None to `allreduce_owner_add_rmsnorm` afterwards); None when the fused
    kernel is unavailable."""
    ws = workspace_for(group, hidden, m, device)
    if ws is None or ws.failed:
        return None
    return ws.partial_buffer(m)


def allreduce_owner_add_rmsnorm(partial, residual_rows, gamma, eps: float, group, m: int,
                                weight_bias: float = 1.0, want_norm: bool = True,
                                checked: bool = False, codes_in_workspace: bool = False):
    """Owner form. residual_rows: BF16 [count, H], this rank's rows (see `owner_rows`).
    partial: BF16 [m, H], or None when the GEMM wrote into `owner_partial_buffer`.
    codes_in_workspace: return the codes and scales as views of this rank's communication
    buffer (no copy; valid until the next reduce of this group and hidden size is launched).
    Returns (codes [m, H], scales, residual_out_rows [count, H], norm_rows [count, H] | None)."""
    native._require(residual_rows, torch.bfloat16, "residual_rows")
    native._require(gamma, torch.bfloat16, "gamma")
    if partial is not None:
        native._require(partial, torch.bfloat16, "partial")
        if partial.shape[0] != m:
            raise ValueError("partial must have m rows")
    h = gamma.shape[0]
    dev = residual_rows.device
    world = dist.get_world_size(group) if group is not None else 1
    first, count = owner_rows(m, group)
    if residual_rows.shape != (count, h):
        raise ValueError(f"residual_rows must be [{count}, {h}]")
    if world == 1:
        if partial is None:
            raise ValueError("one rank: a partial tensor is required")
        norm, res, codes, scales = native.add_rmsnorm_mxfp8(
            partial, residual_rows, gamma, eps, weight_bias, want_norm=want_norm,
            want_quant=True, rounded_sum=True)
        return codes, scales, res, norm
    res = torch.empty_like(residual_rows)
    norm = torch.empty_like(residual_rows) if want_norm else None
    ws = workspace_for(group, h, m, dev) if m else None
    if codes_in_workspace and ws is not None and not ws.failed:
        codes, scales = ws.codes_buffer(m)
    else:
        codes = torch.empty((m, h), dtype=torch.float8_e4m3fn, device=dev)
        scales = torch.empty((native.sf_bytes(m, h),), dtype=torch.uint8, device=dev)
    if m == 0:
        return codes, scales, res, norm
    if ws is None or ws.failed:
        if partial is None:
            raise RuntimeError("the fused all-reduce is unavailable and the partial sums were "
                               "written into its buffers")
        full_norm, full_res, codes, scales = _nccl_route(
            partial, _gather_rows(residual_rows, m, group), gamma, eps, group, weight_bias, True)
        return (codes, scales, full_res[first:first + count].contiguous(),
                full_norm[first:first + count].contiguous() if want_norm else None)
    with torch.cuda.device(dev):
        native._check(native.lib().mach_allreduce_owner_rmsnorm_mxfp8(
            ws.handle, native._ptr(partial), native._ptr(residual_rows), native._ptr(gamma), eps,
            weight_bias, native._ptr(norm), native._ptr(res), native._ptr(codes),
            native._ptr(scales), m, h, native._stream(residual_rows)), "allreduce_owner_rmsnorm")
    if checked:
        _raise_on_failure(dev)
    return codes, scales, res, norm


def _gather_rows(rows: torch.Tensor, m: int, group) -> torch.Tensor:
    """All-gather of row-owned blocks into the full [m, H] tensor (NCCL; off the hot path:
    entering or leaving the row-owned residual stream, and the fallback route)."""
    world = dist.get_world_size(group)
    rpo = (m + world - 1) // world
    padded = rows.new_zeros((rpo, rows.shape[1]))
    padded[:rows.shape[0]] = rows
    out = rows.new_empty((world * rpo, rows.shape[1]))
    dist.all_gather_into_tensor(out, padded, group=group)
    return out[:m].contiguous()


def gather_owned_rows(rows: torch.Tensor, m: int, group) -> torch.Tensor:
    """Public form of the gather: the full [m, H] tensor from every rank's owned rows."""
    if group is None or dist.get_world_size(group) == 1:
        return rows
    return _gather_rows(rows, m, group)
