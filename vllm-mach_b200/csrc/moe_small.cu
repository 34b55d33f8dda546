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

// 16 consecutive weights of one row (unit u covers K indices [16u, 16u + 16)) times 16 activation
// values; the weights' common E8M0 scale (32-element groups: two units per group) is applied by
// the caller. lut: decoded code values in shared memory.
__device__ __forceinline__ float dot16(const uint8_t* __restrict__ row, int unit, int fmt,
                                       const float* __restrict__ lut, const float* __restrict__ act) {
  float acc = 0.0f;
  if (fmt == MACH_FMT_E4M3) {
    const uint4 v = __ldg(reinterpret_cast<const uint4*>(row + (size_t)unit * 16));
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 16; ++i)
      acc = __fmaf_rn(lut[(w[i >> 2] >> (8 * (i & 3))) & 0xFFu], act[i], acc);
  } else {
    const uint32_t* p = reinterpret_cast<const uint32_t*>(row + (size_t)unit * 12);
    const uint32_t a = __ldg(p), b = __ldg(p + 1), c = __ldg(p + 2);
    // four 24-bit words, element i of a word in bits [6i, 6i + 6)
    const uint32_t word[4] = {a & 0xFFFFFFu, (a >> 24) | ((b & 0xFFFFu) << 8),
                              (b >> 16) | ((c & 0xFFu) << 16), c >> 8};
#pragma unroll
    for (int i = 0; i < 16; ++i)
      acc = __fmaf_rn(lut[(word[i >> 2] >> (6 * (i & 3))) & 0x3Fu], act[i], acc);
  }
  return acc;
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
// its gate row and its up row of the expert's gate/up-interleaved W1.
__global__ void __launch_bounds__(1024)
moe_small_w1_kernel(const float* __restrict__ act, const int* __restrict__ pair_expert,
                    const uint8_t* __restrict__ w13, const uint8_t* __restrict__ s13, int topk,
                    int k, int inter, int fmt, int row_bytes, float* __restrict__ h_deq) {
  __shared__ float lut[256];
  __shared__ float vals[32];
  pdl_launch_dependents();
  load_lut(lut, fmt);
  pdl_wait();
  const int pair = blockIdx.y;
  const int e = pair_expert[pair];
  if (e < 0) return;  // block-uniform
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int feat = blockIdx.x * 32 + warp;                 // < inter (inter % 32 == 0)
  const int token = pair / topk;
  const int k_tiles = (k + 127) >> 7;
  // physical rows inside the stacked, interleaved W1: gate feature f at 64 * (f / 32) + f % 32
  const int64_t g_row = (int64_t)e * 2 * inter + 64 * (feat >> 5) + (feat & 31);
  const int64_t u_row = g_row + 32;
  const uint8_t* g_ptr = w13 + g_row * row_bytes;
  const uint8_t* u_ptr = w13 + u_row * row_bytes;
  const float* a_row = act + (size_t)token * k;
  float gate = 0.0f, up = 0.0f;
  for (int unit = lane; unit < (k >> 4); unit += 32) {
    float a[16];
    const float4* ap = reinterpret_cast<const float4*>(a_row + unit * 16);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float4 t = __ldg(ap + i);
      a[4 * i] = t.x; a[4 * i + 1] = t.y; a[4 * i + 2] = t.z; a[4 * i + 3] = t.w;
    }
    const int group = unit >> 1;
    const float gs = pow2_of_byte(__ldg(s13 + sf_offset((int)g_row, group, k_tiles)));
    const float us = pow2_of_byte(__ldg(s13 + sf_offset((int)u_row, group, k_tiles)));
    gate = __fmaf_rn(dot16(g_ptr, unit, fmt, lut, a), gs, gate);
    up = __fmaf_rn(dot16(u_ptr, unit, fmt, lut, a), us, up);
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

// ---- w2: one warp per (token, output feature); the top-k pairs of the token in k order.
__global__ void __launch_bounds__(1024)
moe_small_w2_kernel(const float* __restrict__ h_deq, const int* __restrict__ pair_expert,
                    const float* __restrict__ topk_weights, const uint8_t* __restrict__ w2,
                    const uint8_t* __restrict__ s2, int topk, int hidden, int inter, int fmt,
                    int row_bytes, __nv_bfloat16* __restrict__ out) {
  __shared__ float lut[256];
  pdl_launch_dependents();
  load_lut(lut, fmt);
  pdl_wait();
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int token = blockIdx.y;
  const int feat = blockIdx.x * 32 + warp;
  if (feat >= hidden) return;
  const int k_tiles = (inter + 127) >> 7;
  float acc = 0.0f;
  for (int j = 0; j < topk; ++j) {
    const int pair = token * topk + j;
    const int e = pair_expert[pair];
    if (e < 0) continue;  // warp-uniform
    const int64_t row = (int64_t)e * hidden + feat;
    const uint8_t* r_ptr = w2 + row * row_bytes;
    const float* h_row = h_deq + (size_t)pair * inter;
    float dot = 0.0f;
    for (int unit = lane; unit < (inter >> 4); unit += 32) {
      float a[16];
      const float4* ap = reinterpret_cast<const float4*>(h_row + unit * 16);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float4 t = __ldg(ap + i);
        a[4 * i] = t.x; a[4 * i + 1] = t.y; a[4 * i + 2] = t.z; a[4 * i + 3] = t.w;
      }
      const float ws = pow2_of_byte(__ldg(s2 + sf_offset((int)row, unit >> 1, k_tiles)));
      dot = __fmaf_rn(dot16(r_ptr, unit, fmt, lut, a), ws, dot);
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) dot = __fadd_rn(dot, __shfl_xor_sync(0xffffffffu, dot, d));
    acc = __fmaf_rn(topk_weights[pair], bf16_round(dot), acc);
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
  rc = launched(launch_ex(moe_small_w1_kernel, dim3((unsigned)(inter / 32), (unsigned)(m * topk)),
                          dim3(1024), 0, st, dim3(1, 1, 1), pdl_enabled(), (const float*)act,
                          (const int*)pair_expert, (const uint8_t*)w13, (const uint8_t*)s13,
                          (int)topk, (int)hidden, (int)inter, w_format, row1, h_deq),
                "moe_small_w1");
  if (rc != MACH_OK) return rc;
  return launched(launch_ex(moe_small_w2_kernel, dim3((unsigned)((hidden + 31) / 32), (unsigned)m),
                            dim3(1024), 0, st, dim3(1, 1, 1), pdl_enabled(), (const float*)h_deq,
                            (const int*)pair_expert, (const float*)topk_weights_f32,
                            (const uint8_t*)w2, (const uint8_t*)s2, (int)topk, (int)hidden,
                            (int)inter, w_format, row2, (__nv_bfloat16*)out_bf16),
                  "moe_small_w2");
}
