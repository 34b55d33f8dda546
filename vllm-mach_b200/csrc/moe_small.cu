// Small-batch schedule of the MoE expert layer (decode, M <= 8 tokens): three launches instead of
// route -> gather -> grouped GEMM -> grouped GEMM -> combine. The reference has the same idea
// for its decode batches ("router + quant, split-K W1 + SiLU, W2 + reduce",
// src/vllm_mach/mxfp6/moe.py:74-88,126-188). With a handful of routed rows per expert the layer
// is a set of matrix-vector products bound by the expert-weight stream, so the 128-row MMA
// tile, the 128-row padded permutation and the work list buy nothing; here every (token, expert)
// pair is its own row and the products run on the CUDA cores straight from the kernel-layout
// weights (gate/up-interleaved W1, swizzled E8M0 scales).
//
//   front:  x -> MXFP8 (the activation quantiser) -> dequantised FP32 row; expert_map applied
//   w1:     per pair and output feature: gate/up dot products (FP32, weights decoded from E4M3 /
//           6-bit codes x 2^(scale-127)), BF16, SwiGLU v = bf16(bf16(silu(g)) * u)
//   w2:     per token and output feature: the MXFP8 requant of v (blocks of 32, on load), then
//           for k ascending y_k = bf16(dot), acc = fma(w_k, y_k, acc)
//
// Rounding points are those of the large-batch path (quantise, BF16 between the stages, FP32
// combine); only the summation order inside a dot product differs (lane-strided + shuffle tree
// instead of the tensor core's), which the layer's tolerance (rtol = atol = 0.03,
// tests/native_mxfp6/test_moe.py:248 of the reference) covers.
#include <cuda_bf16.h>
#include <cuda_fp6.h>
#include <cuda_fp8.h>
#include "host_util.h"
#include "ptx.cuh"
#include "quant_math.cuh"

namespace mach {
namespace {

constexpr int kMaxSmallTokens = 8;
constexpr int kMaxSmallTopk = 16;

__device__ __forceinline__ float e4m3_to_float(uint32_t byte) {
  const __half_raw h = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>(byte), __NV_E4M3);
  return __half2float(*reinterpret_cast<const __half*>(&h));
}

// One unit = 16 consecutive K indices of one weight row: 16 bytes (E4M3) or 12 bytes (6-bit,
// four 24-bit words with element i of a word in bits [6i, 6i + 6)).
struct WeightUnit {
  uint32_t w[4];
};
template <int kFmt>
__device__ __forceinline__ WeightUnit load_unit(const uint8_t* __restrict__ row, int unit) {
  WeightUnit u;
  if (kFmt == MACH_FMT_E4M3) {
    const uint4 v = __ldg(reinterpret_cast<const uint4*>(row + (size_t)unit * 16));
    u.w[0] = v.x; u.w[1] = v.y; u.w[2] = v.z; u.w[3] = v.w;
  } else {
    const uint32_t* p = reinterpret_cast<const uint32_t*>(row + (size_t)unit * 12);
    const uint32_t a = __ldg(p), b = __ldg(p + 1), c = __ldg(p + 2);
    u.w[0] = a & 0xFFFFFFu;
    u.w[1] = (a >> 24) | ((b & 0xFFFFu) << 8);
    u.w[2] = (b >> 16) | ((c & 0xFFu) << 16);
    u.w[3] = c >> 8;
  }
  return u;
}
// Two codes -> two FP32 values with the hardware conversions (cvt.rn.f16x2.{e4m3x2, e2m3x2,
// e3m2x2}; every code value is exact in FP16).
template <int kFmt>
__device__ __forceinline__ float2 decode2(uint32_t pair16) {
  __half2_raw h;
  if (kFmt == MACH_FMT_E4M3)
    h = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(pair16), __NV_E4M3);
  else
    h = __nv_cvt_fp6x2_to_halfraw2(static_cast<__nv_fp6x2_storage_t>(pair16),
                                   kFmt == MACH_FMT_E2M3 ? __NV_E2M3 : __NV_E3M2);
  return __half22float2(*reinterpret_cast<const __half2*>(&h));
}
// Dot product of a unit with its 16 activation values (registers); the unit's E8M0 scale
// (32-element groups: two units per group) is applied by the caller.
template <int kFmt>
__device__ __forceinline__ float dot16(const WeightUnit& u, const float (&act)[16]) {
  float acc = 0.0f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint32_t lo, hi;  // codes (0, 1) and (2, 3) of word i, one code per byte
    if (kFmt == MACH_FMT_E4M3) {
      lo = u.w[i] & 0xFFFFu;
      hi = u.w[i] >> 16;
    } else {
      lo = (u.w[i] & 0x3Fu) | ((u.w[i] << 2) & 0x3F00u);
      hi = ((u.w[i] >> 12) & 0x3Fu) | ((u.w[i] >> 10) & 0x3F00u);
    }
    const float2 a = decode2<kFmt>(lo), b = decode2<kFmt>(hi);
    acc = __fmaf_rn(a.x, act[4 * i], acc);
    acc = __fmaf_rn(a.y, act[4 * i + 1], acc);
    acc = __fmaf_rn(b.x, act[4 * i + 2], acc);
    acc = __fmaf_rn(b.y, act[4 * i + 3], acc);
  }
  return acc;
}
__device__ __forceinline__ void load_act16(const float* __restrict__ p, float (&act)[16]) {
  const float4* v = reinterpret_cast<const float4*>(p);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float4 t = __ldg(v + i);
    act[4 * i] = t.x; act[4 * i + 1] = t.y; act[4 * i + 2] = t.z; act[4 * i + 3] = t.w;
  }
}

__device__ __forceinline__ float pow2_of_byte(uint32_t byte) {
  // 2^(byte - 127); byte 0 is 2^-127 (a subnormal float)
  return byte > 0 ? __uint_as_float(byte << 23) : 5.877471754111438e-39f;
}

// ---- front: one CTA per token. Quantises the row exactly as mach_mxfp8_quantize does and
// writes the DEQUANTISED values; maps every pair's expert through expert_map.
__global__ void __launch_bounds__(256)
moe_small_front_kernel(const __nv_bfloat16* __restrict__ hidden, const int* __restrict__ topk_ids,
                       const int* __restrict__ expert_map, int experts, int topk, int k,
                       float* __restrict__ act, int* __restrict__ pair_expert) {
  pdl_launch_dependents();
  pdl_wait();
  const int token = blockIdx.x;
  const int sub = threadIdx.x & 3;
  for (int g = threadIdx.x >> 2; g < (k >> 5); g += blockDim.x >> 2) {
    const uint4 v = __ldg(reinterpret_cast<const uint4*>(hidden + (size_t)token * k + g * 32 + sub * 8));
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    float f[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      f[2 * i] = __uint_as_float(w[i] << 16);
      f[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
    }
    float a = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) a = fmaxf(a, fabsf(f[i]));
    a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, 1));
    a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, 2));
    const uint32_t bits = mx_scale_bits(a);
    const float inv = mx_inverse(bits);
    const float scale = __uint_as_float(bits);
    float d[8];
#pragma unroll
    for (int i = 0; i < 8; i += 2) {
      const uint32_t q = e4m3x2(__fmul_rn(f[i], inv), __fmul_rn(f[i + 1], inv));
      d[i] = __fmul_rn(e4m3_to_float(q & 0xFFu), scale);
      d[i + 1] = __fmul_rn(e4m3_to_float((q >> 8) & 0xFFu), scale);
    }
    float4* dst = reinterpret_cast<float4*>(act + (size_t)token * k + g * 32 + sub * 8);
    dst[0] = make_float4(d[0], d[1], d[2], d[3]);
    dst[1] = make_float4(d[4], d[5], d[6], d[7]);
  }
  for (int j = threadIdx.x; j < topk; j += blockDim.x) {
    int e = topk_ids[(size_t)token * topk + j];
    if (expert_map != nullptr) e = e >= 0 ? expert_map[e] : -1;
    pair_expert[(size_t)token * topk + j] = (e >= 0 && e < experts) ? e : -1;
  }
}

// ---- w1: one warp per (pair, output feature): the gate row and the up row of the feature in
// the expert's gate/up-interleaved W1, both rows' loads in flight together. A lane keeps its
// slice of the token's activation row in registers (up to four units = 64 values: K <= 2048
// per pass). Writes v = bf16(bf16(silu(gate)) * up) as FP32; the MXFP8 requant of v (blocks of
// 32 features) happens where the down projection loads it.
template <int kFmt>
__global__ void __launch_bounds__(128)
moe_small_w1_kernel(const float* __restrict__ act, const int* __restrict__ pair_expert,
                    const uint8_t* __restrict__ w13, const uint8_t* __restrict__ s13, int topk,
                    int k, int inter, int row_bytes, float* __restrict__ h_val) {
  pdl_launch_dependents();
  const int pair = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int token = pair / topk;
  const int k_tiles = (k + 127) >> 7;
  const int units = k >> 4;
  const int feat = blockIdx.x * 4 + warp;
  pdl_wait();
  const int e = pair_expert[pair];
  if (e < 0 || feat >= inter) return;  // warp-uniform
  // physical rows inside the stacked, interleaved W1: gate feature f at 64 * (f / 32) + f % 32
  const int64_t g_row = (int64_t)e * 2 * inter + 64 * (feat >> 5) + (feat & 31);
  const int64_t u_row = g_row + 32;
  const uint8_t* g_ptr = w13 + g_row * row_bytes;
  const uint8_t* u_ptr = w13 + u_row * row_bytes;
  const float* a_row = act + (size_t)token * k;
  float gate = 0.0f, up = 0.0f;
  for (int base = 0; base < units; base += 128) {
    WeightUnit gw[4], uw[4];
    float gs[4], us[4];
    float a[4][16];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int unit = base + 32 * i + lane;
      if (unit < units) {
        gw[i] = load_unit<kFmt>(g_ptr, unit);
        uw[i] = load_unit<kFmt>(u_ptr, unit);
        gs[i] = pow2_of_byte(__ldg(s13 + sf_offset((int)g_row, unit >> 1, k_tiles)));
        us[i] = pow2_of_byte(__ldg(s13 + sf_offset((int)u_row, unit >> 1, k_tiles)));
        load_act16(a_row + unit * 16, a[i]);
      }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if (base + 32 * i + lane < units) {
        gate = __fmaf_rn(dot16<kFmt>(gw[i], a[i]), gs[i], gate);
        up = __fmaf_rn(dot16<kFmt>(uw[i], a[i]), us[i], up);
      }
    }
  }
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) {
    gate = __fadd_rn(gate, __shfl_xor_sync(0xffffffffu, gate, d));
    up = __fadd_rn(up, __shfl_xor_sync(0xffffffffu, up, d));
  }
  if (lane == 0) h_val[(size_t)pair * inter + feat] = swiglu_bf16(bf16_round(gate), bf16_round(up));
}

// 16 SwiGLU values of a unit -> what the MXFP8 requant leaves of them: the block of 32 is this
// lane's unit and the neighbouring lane's (units 2g and 2g + 1 sit in lanes that differ in bit
// 0), so the block maximum is one shuffle away.
__device__ __forceinline__ void requant16(float (&v)[16]) {
  float amax = 0.0f;
#pragma unroll
  for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
  const uint32_t bits = mx_scale_bits(amax);
  const float inv = mx_inverse(bits);
  const float scale = __uint_as_float(bits);
#pragma unroll
  for (int i = 0; i < 16; i += 2) {
    const uint32_t q = e4m3x2(__fmul_rn(v[i], inv), __fmul_rn(v[i + 1], inv));
    const float2 d = decode2<MACH_FMT_E4M3>(q);
    v[i] = __fmul_rn(d.x, scale);
    v[i + 1] = __fmul_rn(d.y, scale);
  }
}

// ---- w2: one warp per (token, output feature): for every pair of the token, y_k = bf16(dot of
// the pair's requantised SwiGLU row with the expert's W2 row), four pairs' loads in flight
// together, then acc = fma(w_k, y_k, acc) in k order.
template <int kFmt>
__global__ void __launch_bounds__(128)
moe_small_w2_kernel(const float* __restrict__ h_val, const int* __restrict__ pair_expert,
                    const float* __restrict__ topk_weights, const uint8_t* __restrict__ w2,
                    const uint8_t* __restrict__ s2, int topk, int hidden, int inter,
                    int row_bytes, __nv_bfloat16* __restrict__ out) {
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int token = blockIdx.y;
  const int feat = blockIdx.x * 4 + warp;
  const int k_tiles = (inter + 127) >> 7;
  const int units = inter >> 4;   // even: inter % 32 == 0
  pdl_wait();
  if (feat >= hidden) return;
  float acc = 0.0f;
  for (int j0 = 0; j0 < topk; j0 += 4) {
    int e[4];
    float dots[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
    for (int q = 0; q < 4; ++q) e[q] = j0 + q < topk ? pair_expert[token * topk + j0 + q] : -1;
    for (int base = 0; base < units; base += 32) {
      const int unit = base + lane;
      const bool in_range = unit < units;   // pairs of lanes (one 32-block) are in range together
      WeightUnit w[4];
      float sc[4];
      float a[4][16];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        if (e[q] >= 0 && in_range) {
          const int64_t row = (int64_t)e[q] * hidden + feat;
          w[q] = load_unit<kFmt>(w2 + row * row_bytes, unit);
          sc[q] = pow2_of_byte(__ldg(s2 + sf_offset((int)row, unit >> 1, k_tiles)));
          load_act16(h_val + (size_t)(token * topk + j0 + q) * inter + unit * 16, a[q]);
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i) a[q][i] = 0.0f;
        }
      }
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        if (e[q] >= 0) {   // warp-uniform: the shuffle inside sees every lane
          requant16(a[q]);
          if (in_range) dots[q] = __fmaf_rn(dot16<kFmt>(w[q], a[q]), sc[q], dots[q]);
        }
      }
    }
#pragma unroll
    for (int q = 0; q < 4; ++q) {
#pragma unroll
      for (int d = 16; d > 0; d >>= 1) dots[q] = __fadd_rn(dots[q], __shfl_xor_sync(0xffffffffu, dots[q], d));
      if (e[q] >= 0) acc = __fmaf_rn(topk_weights[token * topk + j0 + q], bf16_round(dots[q]), acc);
    }
  }
  if (lane == 0) out[(size_t)token * hidden + feat] = __float2bfloat16_rn(acc);
}

int launched(cudaError_t e, const char* what) {
  if (e == cudaSuccess) return MACH_OK;
  return fail(MACH_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

}  // namespace
}  // namespace mach

using namespace mach;

extern "C" size_t mach_moe_small_scratch_bytes(int64_t tokens, int64_t topk, int64_t hidden,
                                               int64_t inter) {
  if (tokens < 0 || topk < 1 || hidden < 1 || inter < 1) return 0;
  // dequantised activations, dequantised SwiGLU outputs, local expert of every pair
  return (size_t)tokens * hidden * 4 + (size_t)tokens * topk * inter * 4 + (size_t)tokens * topk * 4;
}

extern "C" int mach_moe_small_batch(const void* hidden_bf16, const void* topk_weights_f32,
                                    const void* topk_ids_i32, const void* expert_map_i32,
                                    const void* w13, const void* s13, const void* w2,
                                    const void* s2, void* scratch, void* out_bf16, int64_t m,
                                    int64_t topk, int64_t experts, int64_t hidden, int64_t inter,
                                    int w_format, void* stream) {
  if (m < 0) return fail(MACH_ERR_INVALID, "moe_small_batch: negative size");
  if (m == 0) return MACH_OK;
  if (!hidden_bf16 || !topk_weights_f32 || !topk_ids_i32 || !w13 || !s13 || !w2 || !s2 || !scratch ||
      !out_bf16)
    return fail(MACH_ERR_INVALID, "moe_small_batch: null pointer");
  if (m > kMaxSmallTokens || topk < 1 || topk > kMaxSmallTopk)
    return fail(MACH_ERR_UNSUPPORTED, "moe_small_batch: M <= 8 and topk <= 16 required");
  if (w_format != MACH_FMT_E4M3 && w_format != MACH_FMT_E2M3 && w_format != MACH_FMT_E3M2)
    return fail(MACH_ERR_INVALID, "moe_small_batch: unknown weight format %d", w_format);
  if (hidden % 128 || inter % 32 || (2 * inter) % 128 || experts < 1 ||
      experts * 2 * inter > INT32_MAX || experts * hidden > INT32_MAX)
    return fail(MACH_ERR_UNSUPPORTED,
                "moe_small_batch: hidden %% 128 == 0, intermediate %% 64 == 0 required");
  if (!aligned16(hidden_bf16) || !aligned16(w13) || !aligned16(w2) || !aligned16(scratch))
    return fail(MACH_ERR_UNSUPPORTED, "moe_small_batch: 16-byte aligned tensors required");
  const bool six = w_format != MACH_FMT_E4M3;
  const int row1 = (int)(six ? hidden * 3 / 4 : hidden);
  const int row2 = (int)(six ? inter * 3 / 4 : inter);
  float* act = reinterpret_cast<float*>(scratch);
  float* h_deq = act + m * hidden;
  int* pair_expert = reinterpret_cast<int*>(h_deq + m * topk * inter);
  cudaStream_t st = (cudaStream_t)stream;
  int rc = launched(launch_ex(moe_small_front_kernel, dim3((unsigned)m), dim3(256), 0, st,
                              dim3(1, 1, 1), pdl_enabled(), (const __nv_bfloat16*)hidden_bf16,
                              (const int*)topk_ids_i32, (const int*)expert_map_i32, (int)experts,
                              (int)topk, (int)hidden, act, pair_expert),
                    "moe_small_front");
  if (rc != MACH_OK) return rc;
  const dim3 g1((unsigned)((inter + 3) / 4), (unsigned)(m * topk));
  const dim3 g2((unsigned)((hidden + 3) / 4), (unsigned)m);
#define MACH_SMALL_LAUNCH(FMT)                                                                     \
  do {                                                                                             \
    rc = launched(launch_ex(moe_small_w1_kernel<FMT>, g1, dim3(128), 0, st, dim3(1, 1, 1),         \
                            pdl_enabled(), (const float*)act, (const int*)pair_expert,             \
                            (const uint8_t*)w13, (const uint8_t*)s13, (int)topk, (int)hidden,      \
                            (int)inter, row1, h_deq),                                              \
                  "moe_small_w1");                                                                 \
    if (rc != MACH_OK) return rc;                                                                  \
    return launched(launch_ex(moe_small_w2_kernel<FMT>, g2, dim3(128), 0, st, dim3(1, 1, 1),       \
                              pdl_enabled(), (const float*)h_deq, (const int*)pair_expert,         \
                              (const float*)topk_weights_f32, (const uint8_t*)w2,                  \
                              (const uint8_t*)s2, (int)topk, (int)hidden, (int)inter, row2,        \
                              (__nv_bfloat16*)out_bf16),                                           \
                    "moe_small_w2");                                                               \
  } while (0)
  if (w_format == MACH_FMT_E4M3) MACH_SMALL_LAUNCH(MACH_FMT_E4M3);
  if (w_format == MACH_FMT_E2M3) MACH_SMALL_LAUNCH(MACH_FMT_E2M3);
  MACH_SMALL_LAUNCH(MACH_FMT_E3M2);
#undef MACH_SMALL_LAUNCH
}
