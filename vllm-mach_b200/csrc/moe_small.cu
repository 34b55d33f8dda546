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
//   w1:     per pair and 32 output features: gate/up dot products (FP32, weights decoded from
//           E4M3 / 6-bit codes x 2^(scale-127)), BF16, SwiGLU (bf16(bf16(silu(g)) * u)), MXFP8
//           requant of the 32 values -> dequantised FP32 (what the down projection multiplies)
//   w2:     per token and output feature: for k ascending y_k = bf16(dot), acc = fma(w_k, y_k, acc)
//
// Rounding points are those of the large-batch path (quantise, BF16 between the stages, FP32
// combine); only the summation order inside a dot product differs (lane-strided + shuffle tree
// instead of the tensor core's), which the layer's tolerance (rtol = atol = 0.03,
// tests/native_mxfp6/test_moe.py:248 of the reference) covers.
#include <cuda_bf16.h>
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

// Value of a weight code: E4M3 byte, or a 6-bit code (sign, 2/3 exponent bits, 3/2 mantissa bits).
__device__ __forceinline__ float decode_weight(uint32_t code, int fmt) {
  if (fmt == MACH_FMT_E4M3) return e4m3_to_float(code);
  const int mbits = fmt == MACH_FMT_E2M3 ? 3 : 2;
  const int bias = fmt == MACH_FMT_E2M3 ? 1 : 3;
  const uint32_t e = (code >> mbits) & ((1u << (5 - mbits)) - 1u);
  const uint32_t man = code & ((1u << mbits) - 1u);
  const float frac = (float)man / (float)(1u << mbits);
  const float mag = e == 0 ? frac * exp2f((float)(1 - bias)) : (1.0f + frac) * exp2f((float)((int)e - bias));
  return (code & 0x20u) ? -mag : mag;
}

// One unit = 16 consecutive K indices of one weight row: 16 bytes (E4M3) or 12 bytes (6-bit).
struct WeightUnit {
  uint32_t w[4];
};
__device__ __forceinline__ WeightUnit load_unit(const uint8_t* __restrict__ row, int unit, int fmt) {
  WeightUnit u;
  if (fmt == MACH_FMT_E4M3) {
    const uint4 v = __ldg(reinterpret_cast<const uint4*>(row + (size_t)unit * 16));
    u.w[0] = v.x; u.w[1] = v.y; u.w[2] = v.z; u.w[3] = v.w;
  } else {
    const uint32_t* p = reinterpret_cast<const uint32_t*>(row + (size_t)unit * 12);
    const uint32_t a = __ldg(p), b = __ldg(p + 1), c = __ldg(p + 2);
    // four 24-bit words, element i of a word in bits [6i, 6i + 6)
    u.w[0] = a & 0xFFFFFFu;
    u.w[1] = (a >> 24) | ((b & 0xFFFFu) << 8);
    u.w[2] = (b >> 16) | ((c & 0xFFu) << 16);
    u.w[3] = c >> 8;
  }
  return u;
}
// Dot product of a unit with its 16 activation values; the unit's E8M0 scale (32-element
// groups: two units per group) is applied by the caller. lut: decoded code values in shared
// memory. The activations sit in shared memory TRANSPOSED, element j of unit u at
// act_t[j * units + u], so the lanes of a warp (consecutive units) read consecutive words.
__device__ __forceinline__ float dot16(const WeightUnit& u, int fmt, const float* __restrict__ lut,
                                       const float* __restrict__ act_t, int units, int unit) {
  float acc = 0.0f;
  const int bits = fmt == MACH_FMT_E4M3 ? 8 : 6;
  const uint32_t mask = fmt == MACH_FMT_E4M3 ? 0xFFu : 0x3Fu;
#pragma unroll
  for (int i = 0; i < 16; ++i)
    acc = __fmaf_rn(lut[(u.w[i >> 2] >> ((i & 3) * bits)) & mask], act_t[i * units + unit], acc);
  return acc;
}
// Copies one activation row (n floats, n % 16 == 0) from global memory into the transposed
// shared layout above; all threads of the CTA.
__device__ __forceinline__ void stage_transposed(float* act_t, const float* __restrict__ row, int n) {
  const int units = n >> 4;
  for (int i = threadIdx.x; i < n; i += blockDim.x) act_t[(i & 15) * units + (i >> 4)] = __ldg(row + i);
}

__device__ __forceinline__ void load_lut(float* lut, int fmt) {
  const int entries = fmt == MACH_FMT_E4M3 ? 256 : 64;
  for (int i = threadIdx.x; i < entries; i += blockDim.x) lut[i] = decode_weight((uint32_t)i, fmt);
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

// ---- w1: one CTA per (pair, 32 output features); warp w computes feature 32 * block + w:
// its gate row and its up row of the expert's gate/up-interleaved W1. Dynamic shared memory:
// the token's dequantised activation row, k floats.
__global__ void __launch_bounds__(1024)
moe_small_w1_kernel(const float* __restrict__ act, const int* __restrict__ pair_expert,
                    const uint8_t* __restrict__ w13, const uint8_t* __restrict__ s13, int topk,
                    int k, int inter, int fmt, int row_bytes, float* __restrict__ h_deq) {
  extern __shared__ float act_t[];
  __shared__ float lut[256];
  __shared__ float vals[32];
  pdl_launch_dependents();
  load_lut(lut, fmt);
  const int pair = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int feat = blockIdx.x * 32 + warp;                 // < inter (inter % 32 == 0)
  const int token = pair / topk;
  const int k_tiles = (k + 127) >> 7;
  const int units = k >> 4;
  pdl_wait();
  const int e = pair_expert[pair];
  if (e < 0) return;  // block-uniform
  // physical rows inside the stacked, interleaved W1: gate feature f at 64 * (f / 32) + f % 32
  const int64_t g_row = (int64_t)e * 2 * inter + 64 * (feat >> 5) + (feat & 31);
  const int64_t u_row = g_row + 32;
  const uint8_t* g_ptr = w13 + g_row * row_bytes;
  const uint8_t* u_ptr = w13 + u_row * row_bytes;
  // the first pass's weights go out before the activation row is staged
  WeightUnit gw[4], uw[4];
  float gs[4], us[4];
  auto fetch = [&](int base) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int unit = base + 32 * i + lane;
      if (unit < units) {
        gw[i] = load_unit(g_ptr, unit, fmt);
        uw[i] = load_unit(u_ptr, unit, fmt);
        gs[i] = pow2_of_byte(__ldg(s13 + sf_offset((int)g_row, unit >> 1, k_tiles)));
        us[i] = pow2_of_byte(__ldg(s13 + sf_offset((int)u_row, unit >> 1, k_tiles)));
      }
    }
  };
  fetch(0);
  stage_transposed(act_t, act + (size_t)token * k, k);
  __syncthreads();
  float gate = 0.0f, up = 0.0f;
  // Four units per lane and pass (2048 K indices per warp), all loads of a pass in flight
  // together: one memory round trip per pass.
  for (int base = 0; base < units; base += 128) {
    if (base > 0) fetch(base);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int unit = base + 32 * i + lane;
      if (unit < units) {
        gate = __fmaf_rn(dot16(gw[i], fmt, lut, act_t, units, unit), gs[i], gate);
        up = __fmaf_rn(dot16(uw[i], fmt, lut, act_t, units, unit), us[i], up);
      }
    }
  }
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) {
    gate = __fadd_rn(gate, __shfl_xor_sync(0xffffffffu, gate, d));
    up = __fadd_rn(up, __shfl_xor_sync(0xffffffffu, up, d));
  }
  if (lane == 0) vals[warp] = swiglu_bf16(bf16_round(gate), bf16_round(up));
  __syncthreads();
  if (warp == 0) {
    const float v = vals[lane];
    float amax = fabsf(v);
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, d));
    const uint32_t bits = mx_scale_bits(amax);
    const uint32_t q = e4m3x2(__fmul_rn(v, mx_inverse(bits)), 0.0f) & 0xFFu;
    h_deq[(size_t)pair * inter + blockIdx.x * 32 + lane] =
        __fmul_rn(e4m3_to_float(q), __uint_as_float(bits));
  }
}

// ---- w2: one CTA per (token, group of features); warp (f, j) computes y = bf16(dot) of feature
// f with the token's j-th pair, all pairs of a feature at the same time; then one thread per
// feature folds them in k order: acc = fma(w_k, y_k, acc). Dynamic shared memory: the
// dequantised SwiGLU rows of the token's pairs, topk_pad x inter floats.
__global__ void __launch_bounds__(1024)
moe_small_w2_kernel(const float* __restrict__ h_deq, const int* __restrict__ pair_expert,
                    const float* __restrict__ topk_weights, const uint8_t* __restrict__ w2,
                    const uint8_t* __restrict__ s2, int topk, int topk_pad, int hidden, int inter,
                    int fmt, int row_bytes, __nv_bfloat16* __restrict__ out) {
  extern __shared__ float h_t[];
  __shared__ float lut[256];
  __shared__ float ys[32];
  pdl_launch_dependents();
  load_lut(lut, fmt);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int feats = 32 / topk_pad;             // features per CTA
  const int f_local = warp / topk_pad;
  const int j = warp - f_local * topk_pad;
  const int token = blockIdx.y;
  const int feat = blockIdx.x * feats + f_local;
  const int k_tiles = (inter + 127) >> 7;
  const int units = inter >> 4;
  pdl_wait();
  const int pair = token * topk + j;
  const int e = (j < topk && feat < hidden) ? pair_expert[pair] : -1;  // warp-uniform
  const int64_t row = (int64_t)max(e, 0) * hidden + feat;
  const uint8_t* r_ptr = w2 + row * row_bytes;
  WeightUnit w[4];
  float ws[4];
  auto fetch = [&](int base) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int unit = base + 32 * i + lane;
      if (e >= 0 && unit < units) {
        w[i] = load_unit(r_ptr, unit, fmt);
        ws[i] = pow2_of_byte(__ldg(s2 + sf_offset((int)row, unit >> 1, k_tiles)));
      }
    }
  };
  fetch(0);
  for (int q = 0; q < topk; ++q)
    if (pair_expert[token * topk + q] >= 0)   // block-uniform
      stage_transposed(h_t + (size_t)q * inter, h_deq + (size_t)(token * topk + q) * inter, inter);
  __syncthreads();
  float y = 0.0f;
  if (e >= 0) {
    const float* mine = h_t + (size_t)j * inter;
    float dot = 0.0f;
    for (int base = 0; base < units; base += 128) {
      if (base > 0) fetch(base);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int unit = base + 32 * i + lane;
        if (unit < units) dot = __fmaf_rn(dot16(w[i], fmt, lut, mine, units, unit), ws[i], dot);
      }
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) dot = __fadd_rn(dot, __shfl_xor_sync(0xffffffffu, dot, d));
    y = bf16_round(dot);
  }
  if (lane == 0) ys[warp] = y;
  __syncthreads();
  if ((int)threadIdx.x < feats) {
    const int f = blockIdx.x * feats + threadIdx.x;
    if (f < hidden) {
      float acc = 0.0f;
      for (int q = 0; q < topk; ++q) {
        const int pr = token * topk + q;
        if (pair_expert[pr] < 0) continue;
        acc = __fmaf_rn(topk_weights[pr], ys[threadIdx.x * topk_pad + q], acc);
      }
      out[(size_t)token * hidden + f] = __float2bfloat16_rn(acc);
    }
  }
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
  if (hidden * 4 > 40 * 1024 || 16 * inter * 4 > 40 * 1024)
    return fail(MACH_ERR_UNSUPPORTED, "moe_small_batch: hidden <= 10240, intermediate <= 640 required");
  rc = launched(launch_ex(moe_small_w1_kernel, dim3((unsigned)(inter / 32), (unsigned)(m * topk)),
                          dim3(1024), (size_t)hidden * 4, st, dim3(1, 1, 1), pdl_enabled(),
                          (const float*)act,
                          (const int*)pair_expert, (const uint8_t*)w13, (const uint8_t*)s13,
                          (int)topk, (int)hidden, (int)inter, w_format, row1, h_deq),
                "moe_small_w1");
  if (rc != MACH_OK) return rc;
  int topk_pad = 1;
  while (topk_pad < topk) topk_pad <<= 1;       // 1, 2, 4, 8, 16: divides the 32 warps of a CTA
  const int feats = 32 / topk_pad;
  return launched(launch_ex(moe_small_w2_kernel,
                            dim3((unsigned)((hidden + feats - 1) / feats), (unsigned)m), dim3(1024),
                            (size_t)topk_pad * inter * 4, st, dim3(1, 1, 1), pdl_enabled(),
                            (const float*)h_deq,
                            (const int*)pair_expert, (const float*)topk_weights_f32,
                            (const uint8_t*)w2, (const uint8_t*)s2, (int)topk, topk_pad,
                            (int)hidden, (int)inter, w_format, row2, (__nv_bfloat16*)out_bf16),
                  "moe_small_w2");
}
