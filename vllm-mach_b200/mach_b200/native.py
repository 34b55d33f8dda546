"""ctypes binding of libmach_b200.so plus thin torch-tensor wrappers.

The library is the product: when it is missing or cannot be loaded every wrapper raises
RuntimeError; there is no CPU or PyTorch fallback on this path.
"""
from __future__ import annotations

import ctypes
import threading
from pathlib import Path

import torch

_PKG = Path(__file__).resolve().parent
LIB_PATH = _PKG / "libmach_b200.so"

FMT_E4M3, FMT_E2M3, FMT_E3M2 = 0, 3, 4
LAYOUT_ROWS, LAYOUT_GATE_UP_32 = 0, 1
_FORMATS = {"e4m3": FMT_E4M3, "e2m3": FMT_E2M3, "e3m2": FMT_E3M2}

_lock = threading.RLock()
_lib = None

_P, _I64, _INT, _F = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_float
_SIGNATURES = {
    "mach_abi_version": (_INT, []),
    "mach_last_error": (ctypes.c_char_p, []),
    "mach_device_status": (_INT, [ctypes.POINTER(_INT), _INT]),
    "mach_mx_sf_bytes": (ctypes.c_size_t, [_I64, _I64]),
    "mach_mxfp8_quantize": (_INT, [_P, _I64, _P, _P, _I64, _I64, _P]),
    "mach_swiglu_mxfp8_quantize": (_INT, [_P, _P, _P, _I64, _I64, _P]),
    "mach_swiglu_mxfp8_quantize_champion": (_INT, [_P, _P, _P, _I64, _I64, _P]),
    "mach_mxfp8_quantize_weight": (_INT, [_P, _P, _P, _I64, _I64, _P]),
    "mach_gated_rmsnorm_mxfp8_quantize": (_INT, [_P, _P, _I64, _P, _INT, _F, _P, _P, _I64, _I64, _P]),
    "mach_add_rmsnorm_mxfp8": (_INT, [_P, _P, _P, _F, _F, _P, _P, _P, _P, _I64, _I64, _P]),
    "mach_residual_rmsnorm_rounded_mxfp8": (_INT, [_P, _P, _P, _F, _F, _P, _P, _P, _P, _I64, _I64, _P]),
    "mach_mx_pack_scales": (_INT, [_P, _P, _I64, _I64, _P]),
    "mach_mx_unpack_scales": (_INT, [_P, _P, _I64, _I64, _P]),
    "mach_mx_gemm": (_INT, [_P, _P, _P, _P, _P, _I64, _I64, _I64, _INT, _INT, _P]),
    "mach_mx_gemm_swiglu": (_INT, [_P, _P, _P, _P, _P, _P, _I64, _I64, _I64, _INT, _INT, _P]),
    "mach_mx_interleave_gate_up": (_INT, [_P, _P, _I64, _I64, _P]),
    "mach_fp8_group_quantize": (_INT, [_P, _P, _P, _I64, _I64, _P]),
    "mach_silu_mul_fp8_group_quantize": (_INT, [_P, _P, _P, _I64, _I64, _INT, _P]),
    "mach_block_fp8_gemm": (_INT, [_P, _P, _P, _P, _P, _I64, _I64, _I64, _P]),
    "mach_block_fp8_gemm_ordered": (_INT, [_P, _P, _P, _P, _P, _P, _I64, _I64, _I64, _P]),
    "mach_block_fp8_gemm_ordered_static": (_INT, [_P, _P, _P, _P, _P, _I64, _I64, _I64, _P]),
    "mach_ar_buffer_bytes": (ctypes.c_size_t, [_INT, _I64, _I64]),
    "mach_ar_buffer_alloc": (_INT, [ctypes.c_size_t, ctypes.POINTER(_P)]),
    "mach_ar_buffer_free": (_INT, [_P]),
    "mach_ar_ipc_export": (_INT, [_P, ctypes.c_char_p]),
    "mach_ar_ipc_open": (_INT, [ctypes.c_char_p, ctypes.POINTER(_P)]),
    "mach_ar_ipc_close": (_INT, [_P]),
    "mach_ar_create": (_INT, [_INT, _INT, _I64, _I64, ctypes.POINTER(_P), ctypes.POINTER(_P)]),
    "mach_ar_destroy": (_INT, [_P]),
    "mach_ar_set_wait_limit_us": (_INT, [_P, _I64]),
    "mach_ar_reset": (_INT, [_P, _P]),
    "mach_ar_owner_rows": (_INT, [_INT, _INT, _I64, ctypes.POINTER(_I64), ctypes.POINTER(_I64)]),
    "mach_ar_partial_ptr": (_INT, [_P, ctypes.POINTER(_P)]),
    "mach_ar_codes_ptr": (_INT, [_P, ctypes.POINTER(_P), ctypes.POINTER(_P)]),
    "mach_allreduce_owner_rmsnorm_mxfp8": (_INT, [_P, _P, _P, _P, _F, _F, _P, _P, _P, _P, _I64,
                                                  _I64, _P]),
    "mach_allreduce_local_ranks": (_INT, [_INT, ctypes.POINTER(_P), ctypes.POINTER(_P),
                                          ctypes.POINTER(_P), _P, _F, _F, ctypes.POINTER(_P),
                                          ctypes.POINTER(_P), ctypes.POINTER(_P),
                                          ctypes.POINTER(_P), _I64, _I64, _INT, _INT, _P]),
    "mach_allreduce_residual_rmsnorm_mxfp8": (_INT, [_P, _P, _P, _P, _F, _F, _P, _P, _P, _P, _I64,
                                                     _I64, _INT, _P]),
    "mach_mx_gemm_reduce_scatter": (_INT, [_P, _P, _P, _P, _P, _I64, _I64, _I64, _INT, _P]),
    "mach_moe_router_topk": (_INT, [_P, _P, _P, _I64, _I64, _I64, _P]),
    "mach_moe_rows_cap": (_I64, [_I64, _I64, _I64]),
    "mach_moe_work_cap": (_I64, [_I64, _I64, _I64, _I64]),
    "mach_moe_route": (_INT, [_P, _P, _I64, _I64, _I64, _I64, _I64, _I64, _P, _P, _P, _P, _P, _P, _P]),
    "mach_moe_gather_quantize": (_INT, [_P, _P, _P, _I64, _I64, _I64, _P, _P, _P]),
    "mach_moe_scatter_quantize": (_INT, [_P, _P, _I64, _I64, _I64, _P, _P, _P]),
    "mach_moe_grouped_gemm": (_INT, [_P, _P, _P, _P, _P, _P, _P, _P, _I64, _I64, _I64, _I64, _I64,
                                     _I64, _INT, _INT, _P]),
    "mach_moe_combine": (_INT, [_P, _P, _P, _P, _I64, _I64, _I64, _P]),
    "mach_moe_small_scratch_bytes": (ctypes.c_size_t, [_I64, _I64, _I64, _I64]),
    "mach_moe_small_batch": (_INT, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I64, _I64, _I64, _I64,
                                    _I64, _INT, _P]),
    "mach_moe_scatter_codes": (_INT, [_P, _P, _P, _I64, _I64, _I64, _P, _P, _P]),
    "mach_moe_stage_offsets": (_INT, [_P, _P, _I64, _P, _P, _P]),
    "mach_moe_work_from_offsets": (_INT, [_P, _P, _I64, _I64, _I64, _P, _P, _P]),
    "mach_tune_set": (_INT, [ctypes.c_char_p, _INT]),
    "mach_tune_get": (_INT, [ctypes.c_char_p]),
}
ABI_VERSION = 3


def exported_symbols() -> list[str]:
    return sorted(_SIGNATURES)


def lib() -> ctypes.CDLL:
    """Loads the library once; raises RuntimeError when it is absent or has the wrong ABI."""
    global _lib
    with _lock:
        if _lib is None:
            if not LIB_PATH.exists():
                raise RuntimeError(
                    f"{LIB_PATH} is missing: build it with `python -m mach_b200.build` "
                    "(there is no fallback for this path)")
            handle = ctypes.CDLL(str(LIB_PATH))
            for name, (res, args) in _SIGNATURES.items():
                fn = getattr(handle, name)
                fn.restype, fn.argtypes = res, args
            if handle.mach_abi_version() != ABI_VERSION:
                raise RuntimeError("libmach_b200.so ABI mismatch: rebuild the library")
            _lib = handle
        return _lib


def _check(rc: int, what: str) -> None:
    if rc == 0:
        return
    msg = lib().mach_last_error().decode(errors="replace")
    if rc in (1, 2):
        raise ValueError(f"{what}: {msg}")
    raise RuntimeError(f"{what}: {msg} (code {rc})")


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _require(t: torch.Tensor, dtype, name: str) -> None:
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor")
    if dtype is not None and t.dtype not in (dtype if isinstance(dtype, tuple) else (dtype,)):
        raise ValueError(f"{name} has dtype {t.dtype}")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")


_U8 = (torch.uint8, torch.float8_e4m3fn)


def device_status(clear: bool = True) -> int:
    out = _INT(0)
    _check(lib().mach_device_status(ctypes.byref(out), int(clear)), "device_status")
    return out.value


def tune(name: str, value: int) -> None:
    _check(lib().mach_tune_set(name.encode(), int(value)), "tune_set")


def sf_bytes(rows: int, k: int) -> int:
    return int(lib().mach_mx_sf_bytes(rows, k))


def quantize_mxfp8(x: torch.Tensor):
    """BF16 [M, K] -> (E4M3 codes [M, K], swizzled E8M0 scales uint8 [sf_bytes])."""
    _require(x, torch.bfloat16, "x")
    m, k = x.shape
    codes = torch.empty((m, k), dtype=torch.float8_e4m3fn, device=x.device)
    scales = torch.empty((sf_bytes(m, k),), dtype=torch.uint8, device=x.device)
    with torch.cuda.device(x.device):
        _check(lib().mach_mxfp8_quantize(_ptr(x), k, _ptr(codes), _ptr(scales), m, k, _stream(x)),
               "mxfp8_quantize")
    return codes, scales


def swiglu_quantize_mxfp8(gate_up: torch.Tensor):
    _require(gate_up, torch.bfloat16, "gate_up")
    m, two_i = gate_up.shape
    inter = two_i // 2
    codes = torch.empty((m, inter), dtype=torch.float8_e4m3fn, device=gate_up.device)
    scales = torch.empty((sf_bytes(m, inter),), dtype=torch.uint8, device=gate_up.device)
    with torch.cuda.device(gate_up.device):
        _check(lib().mach_swiglu_mxfp8_quantize(_ptr(gate_up), _ptr(codes), _ptr(scales), m, inter,
                                                _stream(gate_up)), "swiglu_mxfp8_quantize")
    return codes, scales


def add_rmsnorm_mxfp8(x, residual, weight, eps: float, weight_bias: float = 1.0,
                      want_norm: bool = True, want_quant: bool = True, rounded_sum: bool = False):
    """Returns (norm BF16 | None, residual_out BF16 | None, codes | None, scales | None).
    rounded_sum=True normalises the BF16-rounded sum (all-reduce contract) instead of the
    FP32 sum (single-GPU Gemma contract)."""
    _require(x, torch.bfloat16, "x")
    _require(weight, torch.bfloat16, "weight")
    if residual is not None:
        _require(residual, torch.bfloat16, "residual")
    m, h = x.shape
    norm = torch.empty_like(x) if want_norm else None
    res_out = torch.empty_like(x) if residual is not None else None
    codes = scales = None
    if want_quant:
        codes = torch.empty((m, h), dtype=torch.float8_e4m3fn, device=x.device)
        scales = torch.empty((sf_bytes(m, h),), dtype=torch.uint8, device=x.device)
    with torch.cuda.device(x.device):
        fn = lib().mach_residual_rmsnorm_rounded_mxfp8 if rounded_sum else lib().mach_add_rmsnorm_mxfp8
        _check(fn(_ptr(x), _ptr(residual), _ptr(weight), eps, weight_bias, _ptr(norm),
                  _ptr(res_out), _ptr(codes), _ptr(scales), m, h, _stream(x)), "add_rmsnorm_mxfp8")
    return norm, res_out, codes, scales


def gated_rmsnorm_quantize(core: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor, eps: float):
    """core BF16 [M, heads, 128]; gate BF16 [M, heads, 128] (rows may be strided); weight [128]
    BF16 or FP32 -> (E4M3 codes [M, heads * 128], swizzled E8M0 scales)."""
    _require(core, torch.bfloat16, "core")
    if core.ndim != 3 or core.shape[2] != 128:
        raise ValueError("core must be [M, heads, 128]")
    m, heads, _ = core.shape
    gate2 = gate.reshape(m, -1) if gate.is_contiguous() else gate
    if gate2.dtype != torch.bfloat16 or gate2.shape[-1] != heads * 128 and gate2.ndim == 2:
        raise ValueError("gate must be BF16 [M, heads * 128]")
    if gate2.ndim == 3:
        gate2 = gate2.reshape(m, heads * 128)
    if gate2.stride(-1) != 1:
        raise ValueError("gate rows must be dense")
    if weight.dtype not in (torch.bfloat16, torch.float32) or weight.numel() != 128:
        raise ValueError("norm weight must be BF16 or FP32 [128]")
    k = heads * 128
    codes = torch.empty((m, k), dtype=torch.float8_e4m3fn, device=core.device)
    scales = torch.empty((sf_bytes(m, k),), dtype=torch.uint8, device=core.device)
    with torch.cuda.device(core.device):
        _check(lib().mach_gated_rmsnorm_mxfp8_quantize(
            _ptr(core), _ptr(gate2), gate2.stride(0) if m > 1 else k, _ptr(weight.contiguous()),
            int(weight.dtype == torch.float32), eps, _ptr(codes), _ptr(scales), m, heads,
            _stream(core)), "gated_rmsnorm_mxfp8_quantize")
    return codes, scales


def pack_scales(logical: torch.Tensor, k: int) -> torch.Tensor:
    """uint8 [rows, K/32] -> swizzled uint8 [sf_bytes(rows, K)] (pad bytes = 127)."""
    _require(logical, torch.uint8, "logical")
    rows = logical.shape[0]
    if logical.shape[1] != k // 32:
        raise ValueError("logical scales must be [rows, K/32]")
    out = torch.empty((sf_bytes(rows, k),), dtype=torch.uint8, device=logical.device)
    with torch.cuda.device(logical.device):
        _check(lib().mach_mx_pack_scales(_ptr(logical), _ptr(out), rows, k, _stream(logical)),
               "pack_scales")
    return out


def unpack_scales(swizzled: torch.Tensor, rows: int, k: int) -> torch.Tensor:
    _require(swizzled, torch.uint8, "swizzled")
    if swizzled.numel() < sf_bytes(rows, k):
        raise ValueError("swizzled scale buffer is too small")
    out = torch.empty((rows, k // 32), dtype=torch.uint8, device=swizzled.device)
    with torch.cuda.device(swizzled.device):
        _check(lib().mach_mx_unpack_scales(_ptr(swizzled), _ptr(out), rows, k, _stream(swizzled)),
               "unpack_scales")
    return out


def _weight_k(w: torch.Tensor, fmt: int) -> int:
    return w.shape[1] if fmt == FMT_E4M3 else w.shape[1] * 4 // 3


def interleave_gate_up(t: torch.Tensor) -> torch.Tensor:
    """[2I, row_bytes] bytes, rows [gate | up] -> rows interleaved in groups of 32."""
    _require(t, _U8, "t")
    out = torch.empty_like(t)
    with torch.cuda.device(t.device):
        _check(lib().mach_mx_interleave_gate_up(_ptr(t), _ptr(out), t.shape[0], t.shape[1],
                                                _stream(t)), "interleave_gate_up")
    return out


class _DevicePointer:
    """Adapter that lets torch.as_tensor alias raw device memory (CUDA array interface)."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False),
                                         "version": 2}


def tensor_from_ptr(ptr: int, shape, dtype: torch.dtype, device) -> torch.Tensor:
    """A tensor that aliases `ptr` (memory owned by the library, e.g. an all-reduce buffer).
    The caller keeps the owner alive for as long as the tensor is used."""
    numel = 1
    for d in shape:
        numel *= int(d)
    nbytes = numel * torch.empty((), dtype=dtype).element_size()
    with torch.cuda.device(device):
        flat = torch.as_tensor(_DevicePointer(ptr, max(nbytes, 1)), device=torch.device(device))
    return flat[:nbytes].view(dtype).view(*shape)


def mx_gemm(a_codes, a_scales, w, w_scales, fmt: str = "e4m3", out: torch.Tensor | None = None,
            layout: int = LAYOUT_ROWS):
    """BF16 [M, N] = dq(A) dq(W)^T. W: [N, K] E4M3 bytes or [N, 3K/4] packed 6-bit."""
    f = _FORMATS[fmt]
    _require(a_codes, _U8, "a_codes")
    _require(w, _U8, "w")
    _require(a_scales, torch.uint8, "a_scales")
    _require(w_scales, torch.uint8, "w_scales")
    m, k = a_codes.shape
    n = w.shape[0]
    if _weight_k(w, f) != k:
        raise ValueError(f"K mismatch: activations {k}, weight {_weight_k(w, f)}")
    if a_scales.numel() < sf_bytes(m, k) or w_scales.numel() < sf_bytes(n, k):
        raise ValueError("scale buffer is too small")
    if out is None:
        out = torch.empty((m, n), dtype=torch.bfloat16, device=a_codes.device)
    elif out.shape != (m, n) or out.dtype != torch.bfloat16 or not out.is_contiguous():
        raise ValueError("out must be a contiguous BF16 [M, N] tensor")
    with torch.cuda.device(a_codes.device):
        _check(lib().mach_mx_gemm(_ptr(a_codes), _ptr(a_scales), _ptr(w), _ptr(w_scales), _ptr(out),
                                  m, n, k, f, layout, _stream(a_codes)), "mx_gemm")
    return out


def mx_gemm_swiglu(a_codes, a_scales, w, w_scales, fmt: str = "e4m3", layout: int = LAYOUT_ROWS):
    """Fused gate_up GEMM + SwiGLU + MXFP8 requant -> (codes [M, I], swizzled scales)."""
    f = _FORMATS[fmt]
    _require(a_codes, _U8, "a_codes")
    _require(w, _U8, "w")
    m, k = a_codes.shape
    inter = w.shape[0] // 2
    if _weight_k(w, f) != k:
        raise ValueError(f"K mismatch: activations {k}, weight {_weight_k(w, f)}")
    codes = torch.empty((m, inter), dtype=torch.float8_e4m3fn, device=a_codes.device)
    scales = torch.empty((sf_bytes(m, inter),), dtype=torch.uint8, device=a_codes.device)
    with torch.cuda.device(a_codes.device):
        _check(lib().mach_mx_gemm_swiglu(_ptr(a_codes), _ptr(a_scales), _ptr(w), _ptr(w_scales),
                                         _ptr(codes), _ptr(scales), m, inter, k, f, layout,
                                         _stream(a_codes)), "mx_gemm_swiglu")
    return codes, scales


def fp8_group_quantize(x: torch.Tensor):
    """BF16 [M, K] -> (E4M3 [M, K], FP32 scales [M, K/128] with stride (1, M))."""
    _require(x, torch.bfloat16, "x")
    m, k = x.shape
    q = torch.empty((m, k), dtype=torch.float8_e4m3fn, device=x.device)
    s = torch.empty((k // 128, m), dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        _check(lib().mach_fp8_group_quantize(_ptr(x), _ptr(q), _ptr(s), m, k, _stream(x)),
               "fp8_group_quantize")
    return q, s.t()


def silu_mul_fp8_group_quantize(inp: torch.Tensor, transposed: bool = True,
                                out: torch.Tensor | None = None,
                                scales: torch.Tensor | None = None):
    """`out` (E4M3 [M, I]) and `scales` (FP32 [M, I/128], stride (1, M) when transposed) may be
    supplied by the caller; the kernel then writes straight into them."""
    _require(inp, torch.bfloat16, "input")
    m, two_i = inp.shape
    inter = two_i // 2
    if out is None:
        out = torch.empty((m, inter), dtype=torch.float8_e4m3fn, device=inp.device)
    if scales is not None:
        view = scales
    elif transposed:
        view = torch.empty((inter // 128, m), dtype=torch.float32, device=inp.device).t()
    else:
        view = torch.empty((m, inter // 128), dtype=torch.float32, device=inp.device)
    with torch.cuda.device(inp.device):
        _check(lib().mach_silu_mul_fp8_group_quantize(_ptr(inp), _ptr(out), _ptr(view), m, inter,
                                                      int(transposed), _stream(inp)),
               "silu_mul_fp8_group_quantize")
    return out, view


def block_fp8_gemm(a, sa, b, sb, raw: torch.Tensor | None = None):
    """a E4M3 [M,K]; sa FP32 [M,K/128] stride (1,M); b E4M3 [N,K]; sb FP32 [ceil(N/128),K/128].
    With `raw` (FP32 [K/128, M, N] scratch) the ordered small-batch route is taken."""
    _require(a, _U8, "a")
    _require(b, _U8, "b")
    m, k = a.shape
    n = b.shape[0]
    if sa.shape != (m, k // 128) or sa.dtype != torch.float32 or (m > 1 and sa.stride() != (1, m)):
        if not (sa.shape == (m, k // 128) and sa.dtype == torch.float32 and m == 1):
            raise ValueError("sa must be FP32 [M, K/128] with stride (1, M)")
    if sb.dtype != torch.float32 or not sb.is_contiguous() or sb.shape != ((n + 127) // 128, k // 128):
        raise ValueError("sb must be contiguous FP32 [ceil(N/128), K/128]")
    out = torch.empty((m, n), dtype=torch.bfloat16, device=a.device)
    with torch.cuda.device(a.device):
        if raw is None:
            _check(lib().mach_block_fp8_gemm(_ptr(a), _ptr(b), _ptr(sa), _ptr(sb), _ptr(out), m, n,
                                             k, _stream(a)), "block_fp8_gemm")
        else:
            if raw.dtype != torch.float32 or raw.numel() < (k // 128) * m * n or not raw.is_contiguous():
                raise ValueError("raw scratch must be contiguous FP32 [K/128, M, N]")
            _check(lib().mach_block_fp8_gemm_ordered(_ptr(a), _ptr(b), _ptr(sa), _ptr(sb), _ptr(out),
                                                     _ptr(raw), m, n, k, _stream(a)),
                   "block_fp8_gemm_ordered")
    return out
