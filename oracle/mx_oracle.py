"""CPU oracle for the quantized-linear hot path. TEST INFRASTRUCTURE ONLY.

This module restates, in plain torch-CPU / numpy arithmetic, the numerical contracts of the
reference (troycheng/vllm-mach) for the path the CUDA library implements. Only tests, the
smoke check and the CPU-baseline leg of the benchmark may import it; the product path never
does and fails loudly when the CUDA library is missing.

Parity pins (checked in tests/test_oracle_cpu.py against fixtures under tests/golden/):
  * weight quantiser  <- golden vector of tests/test_mxfp8_reconstruct_model.py:142-156
  * activation MXFP8 / SwiGLU / residual+RMSNorm / 1x128 FP8 quantisers and the ordered
    block-FP8 GEMM <- outputs of the reference's own Triton kernels executed on CPU with
    TRITON_INTERPRET=1 (tests/golden/make_golden.py is the generating script).
  * all-reduce + residual + RMSNorm (+ MXFP8) <- the reference's own device code
    (FusedOp / rms_norm / allreduce_sum / the MXFP8 branch of
    native/ar_norm/trtllm_allreduce_fusion_mxfp8.cuh) cut out of the header where it lies and
    compiled for the host by oracle/build_ref.py: rounding points bit for bit, the norm within
    one BF16 ulp (summation tree), codes and scale swizzle bit for bit. Its fast-math rsqrt is
    the one step replaced (1 / sqrt).
  * parity unpinned: the 6-bit packing order and the MXFP6 weight quantiser (they live in the
    third-party wheel mxfp6-sm120==0.3.2, Nekofish-L/mxfp6_sm120@dd9752fb, whose source is
    not part of the reference tree), and the MoE stage order for the same reason.

Every function cites the reference file:line it follows (paths relative to the reference).
"""
from __future__ import annotations

import numpy as np
import torch

E4M3_MAX = 448.0


# --------------------------------------------------------------------------- bit helpers
def _f32_bits(x: torch.Tensor) -> torch.Tensor:
    return x.contiguous().view(torch.int32)


def _bits_f32(b: torch.Tensor) -> torch.Tensor:
    return b.contiguous().view(torch.float32)


def bf16(x: torch.Tensor) -> torch.Tensor:
    """Round FP32 to BF16 (RTNE) and return it widened back to FP32."""
    return x.to(torch.bfloat16).to(torch.float32)


# --------------------------------------------------------------------------- MXFP8 activations
def mx_scale_from_amax(amax: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """E8M0 byte and inverse scale for block maxima.

    src/vllm_mach/mxfp6/mxfp8_norm_quant.py:32-34 (== mxfp8_mlp.py:101-104 ==
    native/ar_norm/trtllm_allreduce_fusion_mxfp8.cuh:1261-1289):
      raw = max(amax / 448, 1e-30); bits = (bits(raw) + 0x007fffff) & 0x7f800000
    """
    raw = torch.maximum(amax.float() / 448.0, torch.tensor(1.0e-30, dtype=torch.float32))
    bits = (_f32_bits(raw) + 0x007FFFFF) & 0x7F800000
    inverse = 1.0 / _bits_f32(bits)
    return (bits >> 23).to(torch.uint8), inverse


def quantize_mxfp8(values: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """BF16/FP32 [M, K] -> (E4M3 codes uint8 [M, K], logical E8M0 scales uint8 [M, K/32]).

    src/vllm_mach/mxfp6/mxfp8_norm_quant.py:31-36.
    """
    m, k = values.shape
    assert k % 32 == 0
    v = values.float().reshape(m, k // 32, 32)
    scale, inverse = mx_scale_from_amax(v.abs().amax(-1))
    codes = (v * inverse[..., None]).to(torch.float8_e4m3fn).view(torch.uint8).reshape(m, k)
    return codes, scale


def sf_offsets(rows: int, k: int) -> np.ndarray:
    """Byte offset of (row, group) in the 128x4 swizzled layout.

    src/vllm_mach/mxfp6/mxfp8_mlp.py:107-110.
    """
    groups = k // 32
    tiles = (groups + 3) // 4
    row = np.arange(rows, dtype=np.int64)[:, None]
    g = np.arange(groups, dtype=np.int64)[None, :]
    return (((row // 128 * tiles + g // 4) * 32 + row % 32) * 4 + row % 128 // 32) * 4 + g % 4


def sf_bytes(rows: int, k: int) -> int:
    """Size of the swizzled buffer (src/vllm_mach/mxfp6/mxfp8_mlp.py:122-123)."""
    return (rows + 127) // 128 * 128 * ((k // 32 + 3) // 4) * 4


def swizzle_scales(logical: torch.Tensor, k: int, fill: int = 127) -> torch.Tensor:
    rows = logical.shape[0]
    out = np.full(sf_bytes(rows, k), fill, dtype=np.uint8)
    if rows:
        out[sf_offsets(rows, k).reshape(-1)] = logical.numpy().reshape(-1)
    return torch.from_numpy(out)


def unswizzle_scales(swizzled: torch.Tensor, rows: int, k: int) -> torch.Tensor:
    if rows == 0:
        return torch.empty((0, k // 32), dtype=torch.uint8)
    return torch.from_numpy(swizzled.numpy()[sf_offsets(rows, k)])


def dequantize_mx(codes: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    """codes.float() * 2^(scale-127) per 32 (tests/native_mxfp6/test_mxfp8_sm120.py:53-56)."""
    v = codes.view(torch.float8_e4m3fn).float()
    s = torch.exp2(scales.float() - 127.0).repeat_interleave(32, -1)
    return v * s


def mx_gemm(a_codes, a_scales, w_values: torch.Tensor) -> torch.Tensor:
    """(dq(A) @ dq(W)^T) in FP32, rounded to BF16 (tests/native_mxfp6/test_mxfp8_sm120.py:57)."""
    a = dequantize_mx(a_codes, a_scales)
    return (a @ w_values.t()).to(torch.bfloat16)


# --------------------------------------------------------------------------- weight quantisers
def quantize_weight_mxfp8(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """BF16 [N, K] -> (E4M3 codes, E8M0 scales [N, K/32]) for checkpoints.

    src/vllm_mach/mxfp8/reconstruct_model.py:34-50: BF16 maximum, mantissa rounded with
    (bits + 32) & 0xFF80, scale = 127 + floor(log2(.)) - 8, codes = RTNE(x / 2^(scale-127)).
    """
    assert x.dtype == torch.bfloat16 and x.ndim == 2 and x.shape[1] % 32 == 0
    maximum = x.reshape(x.shape[0], -1, 32).abs().amax(-1)
    bits = maximum.view(torch.uint16).to(torch.int32)
    rounded = ((bits + 32) & 0xFF80).to(torch.uint16).view(torch.bfloat16)
    scales = (127 + torch.floor(torch.log2(rounded)) - 8).to(torch.uint8)
    expanded = torch.exp2(scales.float() - 127).repeat_interleave(32, -1)
    codes = (x.float() / expanded).to(torch.float8_e4m3fn)
    return codes.view(torch.uint8), scales


# --------------------------------------------------------------------------- SwiGLU + requant
def exp_cr(x: torch.Tensor) -> torch.Tensor:
    """FP32 exponential, correctly rounded (evaluated in FP64, rounded once)."""
    return torch.exp(x.double()).float()


def swiglu_values(gate_up: torch.Tensor) -> torch.Tensor:
    """bf16( bf16(silu(gate)) * up ) as FP32, gate_up = [gate | up] BF16.

    src/vllm_mach/mxfp6/mxfp8_mlp.py:96-99: act = (gate / (1 + exp(-gate))).bf16; v = (act*up).bf16.
    """
    inter = gate_up.shape[1] // 2
    gate = gate_up[:, :inter].float()
    up = gate_up[:, inter:].float()
    act = bf16(gate / (1.0 + exp_cr(-gate)))
    return bf16(act * up)


def swiglu_quantize(gate_up: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """src/vllm_mach/mxfp6/mxfp8_mlp.py:87-110 (codes + logical scales)."""
    return quantize_mxfp8(swiglu_values(gate_up))


def swiglu_quantize_champion(gate_up: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """The "champion" SwiGLU producer: BF16 [M, 2I] -> (E4M3 codes [M, I], E8M0 [M, I/32]).

    src/vllm_mach/mxfp8/swiglu_quant.py:46-70: values = bf16((gate / (1 + exp(-gate))) * up)
    with ONE BF16 rounding; raw = amax * rcp(448); scale byte = cvt.rp.satfinite.ue8m0 of raw
    (smallest power of two >= raw; 0 for raw == 0); inverse = rcp(2^(e-127)), 0 when e == 0;
    codes = e4m3(clamp(values * inverse, +-448)).
    PARITY UNPINNED: the reference states this kernel with inline PTX (rcp.approx.ftz,
    cvt.rp...ue8m0x2) that the Triton interpreter rejects, and its only test compares with
    FlashInfer on an SM120 GPU (tests/test_mxfp8_swiglu_quant.py:89-109). Taken here: exp
    correctly rounded, IEEE division, rcp.approx(448) = the FP32 nearest 1/448 and exact
    reciprocals of powers of two."""
    m, two_i = gate_up.shape
    inter = two_i // 2
    g = gate_up[:, :inter].float()
    u = gate_up[:, inter:].float()
    values = bf16((g / (1.0 + exp_cr(-g))) * u)
    v = values.reshape(m, inter // 32, 32)
    amax = v.abs().amax(-1)
    raw = amax * torch.tensor(1.0 / 448.0, dtype=torch.float32)
    bits = _f32_bits(raw)
    exponent = (bits >> 23) & 0xFF
    mantissa = bits & 0x7FFFFF
    byte = exponent + (mantissa != 0).to(torch.int32)
    # subnormal raw: (2^-127, 2^-126) -> 2^-126 (byte 1); (0, 2^-127] -> 2^-127 (byte 0)
    sub = exponent == 0
    byte = torch.where(sub, (mantissa > 0x400000).to(torch.int32), byte)
    byte = torch.clamp(byte, 0, 254)
    inverse = torch.where(byte > 0, torch.exp2(127.0 - byte.float()), torch.zeros_like(raw))
    inverse = torch.where(byte >= 254, torch.zeros_like(raw), inverse)   # 2^-127 flushes to zero
    q = torch.clamp(v * inverse[..., None], -E4M3_MAX, E4M3_MAX)
    codes = q.to(torch.float8_e4m3fn).view(torch.uint8).reshape(m, inter)
    return codes, byte.to(torch.uint8)


def gated_rmsnorm_values(core, gate, weight, eps: float) -> torch.Tensor:
    """Gated RMSNorm over 128-wide heads (the producer of the linear-attention output
    projection): core, gate BF16 [M, heads, 128], weight [128] -> BF16 [M, heads * 128].

    The fused form is mxfp6.gemm_from_gdn (src/vllm_mach/mxfp6/gdn_output.py:11-13), in the
    third-party wheel whose source is absent: PARITY UNPINNED. Restated from the unfused path
    the reference falls back to (gdn_output.py:62-64: RMSNormGated with norm_before_gate and
    SiLU, written back as BF16, then out_proj): rstd = 1/sqrt(mean(x^2) + eps),
    v = bf16(((x * rstd) * w) * (z / (1 + exp(-z)))), one BF16 rounding."""
    x, z = core.float(), gate.float().reshape(core.shape)
    variance = (x * x).sum(-1, keepdim=True) / 128.0
    rstd = 1.0 / torch.sqrt(variance + eps)
    n = (x * rstd) * weight.float()
    v = bf16(n * (z / (1.0 + exp_cr(-z))))
    return v.reshape(core.shape[0], -1).to(torch.bfloat16)


# --------------------------------------------------------------------------- norms
def gemma_rmsnorm(x, residual, weight, eps: float, weight_bias: float = 1.0):
    """Residual + RMSNorm on the UNROUNDED sum.

    src/vllm_mach/mxfp6/gemma_norm.py:18-29 and mxfp8_norm_quant.py:20-28.
    Returns (y BF16, residual_out BF16 or None).
    """
    s = x.float()
    res_out = None
    if residual is not None:
        s = s + residual.float()
        res_out = s.to(torch.bfloat16)
    w = weight.float() + weight_bias
    n = s.shape[-1]
    variance = (s * s).sum(-1, keepdim=True) / n
    rs = 1.0 / torch.sqrt(variance + eps)
    y = ((s * rs) * w).to(torch.bfloat16)
    return y, res_out


def allreduce_rmsnorm(partials, residual, gamma, eps: float, weight_bias: float = 1.0):
    """All-reduce + residual + RMSNorm with the rounding points of the fused kernel.

    native/ar_norm/trtllm_allreduce_fusion_mxfp8.cuh:1470-1494 (FP32 sum over ranks in rank
    order, rounded to BF16), :1092-1108 (residual add in FP32, rounded to BF16 = residual_out),
    :1303-1342 (norm of the BF16-ROUNDED sum, scale weight_bias + gamma).
    Returns (norm BF16, residual_out BF16).
    """
    acc = torch.zeros_like(partials[0], dtype=torch.float32)
    for part in partials:
        acc = acc + part.float()
    a = bf16(acc)
    res = (a + residual.float()).to(torch.bfloat16)
    r = res.float()
    n = r.shape[-1]
    variance = (r * r).sum(-1, keepdim=True) / n
    rs = 1.0 / torch.sqrt(variance + eps)
    norm = ((r * rs) * (weight_bias + gamma.float())).to(torch.bfloat16)
    return norm, res


# --------------------------------------------------------------------------- block FP8
def fp8_group_quantize(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """BF16 [M, K] -> (E4M3 codes uint8 [M, K], FP32 scales [M, K/128]).

    src/vllm_mach/fp8/_quantize_kernel.py:12-16: scale = max(amax, 1e-10) / 448 (RN division),
    q = clamp(x / scale, +-448) (RN division) -> E4M3. The reference stores the scales
    column-major (stride (1, M)); this returns the logical [M, K/128] view.
    """
    m, k = x.shape
    v = x.float().reshape(m, k // 128, 128)
    maximum = torch.clamp(v.abs().amax(-1), min=1.0e-10)
    scale = maximum / 448.0
    q = torch.clamp(v / scale[..., None], -448.0, 448.0)
    return q.to(torch.float8_e4m3fn).view(torch.uint8).reshape(m, k), scale


def silu_mul_fp8_group_quantize(inp: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """BF16 [M, 2I] -> (E4M3 [M, I], FP32 scales [M, I/128]); no BF16 intermediate.

    native/fp8_activation/activation.cu:31-59: sigmoid = 1/(1+exp(-g)); v = (g*sigmoid)*u;
    scale = max(amax/448, 1/(448*512)); q = clamp(v/scale, +-448). exp is taken as the
    correctly rounded FP32 exponential.
    """
    m = inp.shape[0]
    inter = inp.shape[1] // 2
    gate = inp[:, :inter].float()
    up = inp[:, inter:].float()
    sig = 1.0 / (1.0 + exp_cr(-gate))
    v = ((gate * sig) * up).reshape(m, inter // 128, 128)
    scale = torch.clamp(v.abs().amax(-1) / 448.0, min=1.0 / (448.0 * 512.0))
    q = torch.clamp(v / scale[..., None], -448.0, 448.0)
    return q.to(torch.float8_e4m3fn).view(torch.uint8).reshape(m, inter), scale


def block_fp8_gemm(a_codes, sa, b_codes, sb) -> torch.Tensor:
    """Ordered block-FP8 GEMM, BF16 out.

    src/vllm_mach/fp8/ordered.py:9-35: per 128-K group an FP32 dot, then
    total = fma(dot, sa[m,g] * sb[n//128, g], total) for ascending g, one BF16 rounding.
    a_codes [M,K], sa [M,K/128], b_codes [N,K], sb [ceil(N/128), K/128]. The FMA is evaluated
    in FP64 and rounded to FP32 (exact for a single fused multiply-add of FP32 inputs up to
    double rounding, which cannot occur here: the FP64 product-sum of FP32 values is exact
    to within 2^-53 and ties at FP32 precision would need 29 trailing zero bits).
    """
    a = a_codes.view(torch.float8_e4m3fn).float()
    b = b_codes.view(torch.float8_e4m3fn).float()
    m, k = a.shape
    n = b.shape[0]
    total = torch.zeros((m, n), dtype=torch.float32)
    sb_rows = sb.repeat_interleave(128, 0)[:n]  # [N, G]
    for g in range(k // 128):
        dot = a[:, g * 128:(g + 1) * 128] @ b[:, g * 128:(g + 1) * 128].t()
        scale = sa[:, g:g + 1].float() * sb_rows[:, g][None, :].float()  # FP32 product, rounded
        total = (dot.double() * scale.double() + total.double()).float()
    return total.to(torch.bfloat16)


# --------------------------------------------------------------------------- MXFP6
# Element formats of the 6-bit weights. E2M3: 1 sign, 2 exponent (bias 1), 3 mantissa, max 7.5;
# E3M2: 1 sign, 3 exponent (bias 3), 2 mantissa, max 28 (OCP Microscaling Formats v1.0).
_FP6 = {"e2m3": (2, 3, 1, 7.5), "e3m2": (3, 2, 3, 28.0)}


def fp6_decode_table(fmt: str) -> torch.Tensor:
    ebits, mbits, bias, _ = _FP6[fmt]
    vals = []
    for code in range(64):
        sign = -1.0 if code & 0x20 else 1.0
        e = (code >> mbits) & ((1 << ebits) - 1)
        man = code & ((1 << mbits) - 1)
        if e == 0:
            v = man / (1 << mbits) * 2.0 ** (1 - bias)
        else:
            v = (1.0 + man / (1 << mbits)) * 2.0 ** (e - bias)
        vals.append(sign * v)
    return torch.tensor(vals, dtype=torch.float32)


def pack_fp6(codes: torch.Tensor) -> torch.Tensor:
    """6-bit codes uint8 [N, K] -> packed uint8 [N, 3K/4]; element i of every group of four
    occupies bits [6i, 6i+6) of a little-endian 24-bit word (packing order: parity unpinned,
    defined here and isolated in this one function pair)."""
    n, k = codes.shape
    c = codes.to(torch.int32).reshape(n, k // 4, 4)
    word = c[..., 0] | (c[..., 1] << 6) | (c[..., 2] << 12) | (c[..., 3] << 18)
    out = torch.stack([word & 0xFF, (word >> 8) & 0xFF, (word >> 16) & 0xFF], -1)
    return out.to(torch.uint8).reshape(n, k * 3 // 4)


def unpack_fp6(packed: torch.Tensor, k: int) -> torch.Tensor:
    n = packed.shape[0]
    b = packed.to(torch.int32).reshape(n, k // 4, 3)
    word = b[..., 0] | (b[..., 1] << 8) | (b[..., 2] << 16)
    out = torch.stack([(word >> (6 * i)) & 0x3F for i in range(4)], -1)
    return out.to(torch.uint8).reshape(n, k)


def quantize_weight_mxfp6(x: torch.Tensor, fmt: str = "e2m3"):
    """Synthetic-weight generator for MXFP6 (not part of the parity contract: GEMM parity is
    judged on the packed codes). OCP rule: E8M0 = floor(log2 amax) - emax_fmt, RTNE, saturate.
    Returns (codes uint8 [N,K] in 0..63, scales uint8 [N,K/32])."""
    ebits, mbits, bias, fmax = _FP6[fmt]
    emax = int(np.floor(np.log2(fmax)))
    n, k = x.shape
    v = x.float().reshape(n, k // 32, 32)
    amax = v.abs().amax(-1)
    e = torch.floor(torch.log2(torch.clamp(amax, min=2.0 ** -120))) - emax
    e = torch.clamp(e, -127, 127)
    scale = (e + 127).to(torch.uint8)
    scaled = (v / torch.exp2(e)[..., None]).reshape(n, k)
    table = fp6_decode_table(fmt)
    pos = table[:32]  # non-negative codes, ascending
    mag = torch.clamp(scaled.abs(), max=fmax)
    idx = torch.bucketize(mag, pos)  # first pos >= mag
    idx = torch.clamp(idx, 1, 31)
    lo, hi = pos[idx - 1], pos[idx]
    pick_hi = (mag - lo) > (hi - mag)
    tie = (mag - lo) == (hi - mag)
    pick_hi = pick_hi | (tie & (idx % 2 == 0))  # ties to even code
    code = torch.where(pick_hi, idx, idx - 1)
    code = torch.where(mag <= 0, torch.zeros_like(code), code)
    code = code | torch.where(scaled < 0, 32, 0)
    return code.to(torch.uint8), scale


def dequantize_mxfp6(codes: torch.Tensor, scales: torch.Tensor, fmt: str) -> torch.Tensor:
    v = fp6_decode_table(fmt)[codes.long()]
    return v * torch.exp2(scales.float() - 127.0).repeat_interleave(32, -1)


# --------------------------------------------------------------------------- MoE routing
def route_topk(logits: torch.Tensor, top_k: int):
    """softmax (FP32) -> top-k -> renormalise (benchmark configuration 5; vLLM fused_topk semantics
    used by src/vllm_mach/mxfp6/moe.py:574-702 through topk_weights/topk_ids inputs)."""
    probs = torch.softmax(logits.float(), -1)
    w, ids = torch.topk(probs, top_k, dim=-1)
    w = w / w.sum(-1, keepdim=True)
    return w, ids.to(torch.int32)


def moe_forward(hidden, expert_w13, expert_w2, topk_weights, topk_ids, expert_map=None):
    """Routed experts on CPU with the rounding points of the reference path
    (src/vllm_mach/mxfp6/moe.py:574-702; tests/native_mxfp6/test_moe.py:225-248):
    MXFP8 of the hidden rows -> W1 GEMM -> BF16 -> SwiGLU + MXFP8 -> W2 GEMM -> BF16 ->
    out[m] = bf16(sum_k w[m,k] * y[m,k]) accumulated in FP32 with one FMA per k, k ascending.
    expert_w13(e) / expert_w2(e) return the dequantised FP32 weights [2I, H] / [H, I] of local
    expert e ([gate | up] row order). Pairs whose expert is not local are skipped."""
    m, h = hidden.shape
    top_k = topk_ids.shape[1]
    a_codes, a_scales = quantize_mxfp8(hidden)
    local = topk_ids.long()
    if expert_map is not None:
        local = torch.where(local >= 0, expert_map.long()[local.clamp_min(0)], local)
    y_pairs = torch.zeros((m, top_k, h), dtype=torch.float32)
    for e in local[local >= 0].unique().tolist():
        tok, kk = (local == e).nonzero(as_tuple=True)
        gate_up = mx_gemm(a_codes[tok], a_scales[tok], expert_w13(e))
        h_codes, h_scales = swiglu_quantize(gate_up)
        y_pairs[tok, kk] = mx_gemm(h_codes, h_scales, expert_w2(e)).float()
    acc = torch.zeros((m, h), dtype=torch.float64)
    for k in range(top_k):
        keep = (local[:, k] >= 0).double()[:, None]
        term = topk_weights[:, k].double()[:, None] * y_pairs[:, k].double()
        acc = torch.where(keep > 0, (term + acc).float().double(), acc)
    return acc.float().to(torch.bfloat16)
