// Device arithmetic shared by the stand-alone quantisers and the GEMM epilogues.
//
// The MXFP8 activation rule follows the reference producers
// (src/vllm_mach/mxfp6/mxfp8_norm_quant.py:29-39, src/vllm_mach/mxfp6/mxfp8_mlp.py:100-110,
// native/ar_norm/trtllm_allreduce_fusion_mxfp8.cuh:1261-1289): per 32 consecutive K,
//   raw   = max(amax / 448, 1e-30)            (IEEE division)
//   bits  = (f32bits(raw) + 0x007fffff) & 0x7f800000   -> next power of two >= raw
//   E8M0  = bits >> 23,  inverse = 1 / pow2,  code = RTNE e4m3(v * inverse)
// Every step here is an exactly-rounded FP32 operation or an integer operation, so the
// codes and scale bytes are reproducible bit for bit on any IEEE machine.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <cstdint>

namespace mach {

__device__ __forceinline__ float bf16_round(float x) {
  return __bfloat162float(__float2bfloat16_rn(x));
}

// Power-of-two scale (as FP32 bit pattern) for a block whose absolute maximum is `amax`.
__device__ __forceinline__ uint32_t mx_scale_bits(float amax) {
  const float raw = fmaxf(__fdiv_rn(amax, 448.0f), 1.0e-30f);
  return (__float_as_uint(raw) + 0x007fffffu) & 0x7f800000u;
}
__device__ __forceinline__ float mx_inverse(uint32_t scale_bits) {
  return __fdiv_rn(1.0f, __uint_as_float(scale_bits));
}
// Two values -> two E4M3 bytes (low byte = a), round-to-nearest-even, saturating.
__device__ __forceinline__ uint32_t e4m3x2(float a, float b) {
  return static_cast<uint32_t>(
      __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3));
}
__device__ __forceinline__ uint32_t e4m3x4(float a, float b, float c, float d) {
  return e4m3x2(a, b) | (e4m3x2(c, d) << 16);
}

// Byte offset of the E8M0 scale of (row, 32-K group) in the 128-row x 4-group swizzled
// layout the block-scaled MMA consumes (src/vllm_mach/mxfp6/mxfp8_mlp.py:107-110).
// k_tiles = ceil(K / 128).
__device__ __forceinline__ size_t sf_offset(int row, int group, int k_tiles) {
  return ((((size_t)(row >> 7) * k_tiles + (group >> 2)) * 32 + (row & 31)) * 4 +
          ((row & 127) >> 5)) * 4 + (group & 3);
}

// bf16( g / (1 + exp(-g)) ) with the FP32 sequence of the reference
// (t = exp(-g); s = 1 + t; r = g / s, each rounded to FP32; mxfp8_mlp.py:98).
// exp is taken as the correctly rounded FP32 exponential. Three tiers keep the common case
// cheap without ever letting the hardware's approximations reach the result:
//   1. ex2.approx / rcp.approx (a handful of instructions). Their combined error stays below
//      about 2 + |g| / 8 FP32 ulps for |g| <= 32; outside that range, or whenever the result
//      lies within 96 ulps of a BF16 rounding tie (0.3 % of values), fall through to
//   2. expf (<= 2 ulp) and an IEEE division, error <= 4 ulps; if the result lies within 16 ulps
//      of a tie (0.05 %), fall through to
//   3. the exponential evaluated in FP64 and rounded once, which is exact.
// Tiers 2 and 3, kept out of line: the epilogues evaluate silu_bf16 dozens of times per thread
// fully unrolled, and inlining this rarely taken path into every copy makes the loop body far
// larger than the instruction cache (measured: warps stalled on instruction fetch).
static __device__ __noinline__ float silu_f32_slow(float g) {
  float r = __fdiv_rn(g, __fadd_rn(1.0f, expf(-g)));
  const int low = static_cast<int>(__float_as_uint(r) & 0xFFFFu);
  if (abs(low - 0x8000) <= 16) {
    const float t = static_cast<float>(exp(static_cast<double>(-g)));
    r = __fdiv_rn(g, __fadd_rn(1.0f, t));
  }
  return r;
}
__device__ __forceinline__ float silu_bf16(float g) {
  float r = __fdividef(g, 1.0f + __expf(-g));
  const int low = static_cast<int>(__float_as_uint(r) & 0xFFFFu);
  if (abs(low - 0x8000) <= 96 || fabsf(g) > 32.0f) r = silu_f32_slow(g);
  return bf16_round(r);
}
// v = bf16( bf16(silu(gate)) * up ), gate and up already BF16-representable.
__device__ __forceinline__ float swiglu_bf16(float gate, float up) {
  return bf16_round(__fmul_rn(silu_bf16(gate), up));
}

// ---- The "champion" SwiGLU producer contract (src/vllm_mach/mxfp8/swiglu_quant.py:46-70): ONE
// BF16 rounding of silu(gate) * up, the scale exponent from cvt.rp.satfinite.ue8m0x2 of
// amax * rcp.approx(448), the inverse from rcp.approx of the power of two, and an all-zero
// block stored as scale byte 0 with inverse 0.
static __device__ __noinline__ float swiglu_once_slow(float g, float up) {
  float v = __fmul_rn(__fdiv_rn(g, __fadd_rn(1.0f, expf(-g))), up);
  const int low = static_cast<int>(__float_as_uint(v) & 0xFFFFu);
  if (abs(low - 0x8000) <= 16) {
    const float t = static_cast<float>(exp(static_cast<double>(-g)));
    v = __fmul_rn(__fdiv_rn(g, __fadd_rn(1.0f, t)), up);
  }
  return v;
}
// bf16( (gate / (1 + exp(-gate))) * up ): the same three tiers as silu_bf16, the tie test
// applied to the product, which is the only value that is rounded.
__device__ __forceinline__ float swiglu_once_bf16(float g, float up) {
  float v = __fmul_rn(__fdividef(g, 1.0f + __expf(-g)), up);
  const int low = static_cast<int>(__float_as_uint(v) & 0xFFFFu);
  if (abs(low - 0x8000) <= 96 || fabsf(g) > 32.0f) v = swiglu_once_slow(g, up);
  return bf16_round(v);
}
__device__ __forceinline__ float rcp_approx_ftz(float x) {
  float r;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}
// E8M0 byte of the smallest power of two >= raw (0 for raw == 0, 254 at most).
__device__ __forceinline__ uint32_t ue8m0_round_up(float raw) {
  uint16_t packed;
  asm("{cvt.rp.satfinite.ue8m0x2.f32 %0, 0f00000000, %1;}" : "=h"(packed) : "f"(raw));
  return static_cast<uint32_t>(packed) & 255u;
}

}  // namespace mach
