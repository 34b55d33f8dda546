// Stand-alone activation producers: BF16 -> MXFP8, SwiGLU -> MXFP8, residual + RMSNorm
// -> MXFP8, 1x128 block-FP8 quantisers, and E8M0 scale (un)packing. All are HBM-bound
// byte work: 16-byte loads, 8/16-byte stores, grids sized in multiples of the SM count.
#include "host_util.h"
#include "ptx.cuh"
#include "quant_math.cuh"

namespace mach {

namespace {

__device__ __forceinline__ void unpack_bf16x8(const uint4& v, float (&f)[8]) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
  }
}

// amax of 8 values, then across the 4 adjacent lanes that share one 32-element block.
__device__ __forceinline__ float amax8_quad(const float (&f)[8]) {
  float a = 0.0f;
#pragma unroll
  for (int i = 0; i < 8; ++i) a = fmaxf(a, fabsf(f[i]));
  a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, 1));
  a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, 2));
  return a;
}

__device__ __forceinline__ uint2 quantize8(const float (&f)[8], float inv) {
  uint2 q;
  q.x = e4m3x4(__fmul_rn(f[0], inv), __fmul_rn(f[1], inv), __fmul_rn(f[2], inv),
               __fmul_rn(f[3], inv));
  q.y = e4m3x4(__fmul_rn(f[4], inv), __fmul_rn(f[5], inv), __fmul_rn(f[6], inv),
               __fmul_rn(f[7], inv));
  return q;
}

// One unit = one (row, 32-K block); four threads per unit, eight values per thread.
// kMode: 0 plain BF16 input; 1 SwiGLU with the rounding points of
// src/vllm_mach/mxfp6/mxfp8_mlp.py:87-110; 2 SwiGLU with the champion contract of
// src/vllm_mach/mxfp8/swiglu_quant.py:46-70.
template <int kMode>
__global__ void __launch_bounds__(256)
mx_quantize_kernel(const __nv_bfloat16* __restrict__ x, int64_t ldx, uint8_t* __restrict__ codes,
                   uint8_t* __restrict__ scales, int64_t m, int k, int k_tiles) {
  pdl_launch_dependents();
  pdl_wait();
  const int groups = k >> 5;
  const int64_t units = m * groups;
  const int64_t units_per_pass = (int64_t)gridDim.x * (blockDim.x >> 2);
  const int sub = threadIdx.x & 3;
  // Two units per thread and pass: both 16-byte loads are in flight before either is used
  // (one load per thread leaves the kernel latency-bound at ~40 % of the HBM rate).
  for (int64_t base = 0; base < units; base += 2 * units_per_pass) {
    int64_t row[2];
    int g[2];
    bool valid[2];
    uint4 raw[2], raw_up[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int64_t unit = base + u * units_per_pass + (int64_t)blockIdx.x * (blockDim.x >> 2) +
                           (threadIdx.x >> 2);
      valid[u] = unit < units;
      row[u] = valid[u] ? unit / groups : 0;
      g[u] = valid[u] ? (int)(unit - row[u] * groups) : 0;
      raw[u] = raw_up[u] = make_uint4(0u, 0u, 0u, 0u);
      if (valid[u]) {
        const __nv_bfloat16* src = x + row[u] * ldx + g[u] * 32 + sub * 8;
        raw[u] = __ldg(reinterpret_cast<const uint4*>(src));
        if (kMode != 0) raw_up[u] = __ldg(reinterpret_cast<const uint4*>(src + k));
      }
    }
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      float f[8];
      if (kMode != 0) {
        float gate[8], up[8];
        unpack_bf16x8(raw[u], gate);
        unpack_bf16x8(raw_up[u], up);
#pragma unroll
        for (int i = 0; i < 8; ++i)
          f[i] = kMode == 1 ? swiglu_bf16(gate[i], up[i]) : swiglu_once_bf16(gate[i], up[i]);
      } else {
        unpack_bf16x8(raw[u], f);
      }
      const float amax = amax8_quad(f);
      uint32_t scale_byte;
      float inv;
      if (kMode == 2) {
        scale_byte = ue8m0_round_up(__fmul_rn(amax, rcp_approx_ftz(448.0f)));
        inv = scale_byte > 0 ? rcp_approx_ftz(__uint_as_float(scale_byte << 23)) : 0.0f;
      } else {
        const uint32_t bits = mx_scale_bits(amax);
        inv = mx_inverse(bits);
        scale_byte = bits >> 23;
      }
      if (valid[u]) {
        *reinterpret_cast<uint2*>(codes + row[u] * k + g[u] * 32 + sub * 8) = quantize8(f, inv);
        if (sub == 0) scales[sf_offset((int)row[u], g[u], k_tiles)] = (uint8_t)scale_byte;
      }
    }
  }
}


// Checkpoint weight quantiser (src/vllm_mach/mxfp8/reconstruct_model.py:34-50): per row and 32 K,
// BF16 maximum m; rounded = bf16 bits (m + 32) & 0xFF80 (the mantissa rounded up from 0.75);
// E8M0 = 127 + floor(log2(rounded)) - 8 = exponent field of `rounded` - 8; codes =
// RTNE e4m3(x / 2^(E8M0 - 127)). Logical (row-major) scales out, as checkpoints store them.
// A zero block gives scale 0 and zero codes. Blocks whose maximum is below 2^-119 would need a
// negative exponent byte, which the reference leaves to an out-of-range float -> uint8
// conversion; here the byte is clamped to 0.
__global__ void __launch_bounds__(256)
mx_quantize_weight_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ codes,
                          uint8_t* __restrict__ scales, int64_t n, int k) {
  const int groups = k >> 5;
  const int64_t units = n * groups;
  const int sub = threadIdx.x & 3;
  for (int64_t unit = (int64_t)blockIdx.x * (blockDim.x >> 2) + (threadIdx.x >> 2); unit < units;
       unit += (int64_t)gridDim.x * (blockDim.x >> 2)) {
    const int64_t row = unit / groups;
    const int g = (int)(unit - row * groups);
    float f[8];
    unpack_bf16x8(__ldg(reinterpret_cast<const uint4*>(x + row * k + g * 32 + sub * 8)), f);
    const float amax = amax8_quad(f);
    const uint32_t bits = __float_as_uint(amax) >> 16;         // BF16 bit pattern (amax >= 0)
    const uint32_t rounded = (bits + 32u) & 0xFF80u;
    const int exponent = (int)(rounded >> 7);                  // biased exponent field
    const int byte = exponent > 8 ? exponent - 8 : 0;
    // x / 2^(byte - 127): division by a power of two, exact unless the quotient is subnormal
    const float scale = byte > 0 ? __uint_as_float((uint32_t)byte << 23) : 5.877471754111438e-39f;
    uint2 q;
    q.x = e4m3x4(__fdiv_rn(f[0], scale), __fdiv_rn(f[1], scale), __fdiv_rn(f[2], scale),
                 __fdiv_rn(f[3], scale));
    q.y = e4m3x4(__fdiv_rn(f[4], scale), __fdiv_rn(f[5], scale), __fdiv_rn(f[6], scale),
                 __fdiv_rn(f[7], scale));
    *reinterpret_cast<uint2*>(codes + row * k + g * 32 + sub * 8) = q;
    if (sub == 0) scales[row * groups + g] = (uint8_t)byte;
  }
}


// Gated RMSNorm over 128-wide heads + MXFP8 quantisation: the producer in front of the
// linear-attention output projection (gemm_from_gdn, src/vllm_mach/mxfp6/gdn_output.py:11-13,56-64;
// unfused form: RMSNormGated with norm_before_gate and SiLU, then out_proj):
//   rstd = 1 / sqrt(mean_128(x^2) + eps);  n = (x * rstd) * w;  v = bf16(n * (z / (1 + exp(-z))))
// followed by the activation quantiser on v along K = heads * 128. Sixteen threads per
// (token, head), eight values each; the sum of squares is a fixed shuffle tree.
template <typename W>
__global__ void __launch_bounds__(256)
gated_rmsnorm_mx_kernel(const __nv_bfloat16* __restrict__ core, const __nv_bfloat16* __restrict__ gate,
                        int64_t ld_gate, const W* __restrict__ weight, float eps,
                        uint8_t* __restrict__ codes, uint8_t* __restrict__ scales, int64_t m,
                        int heads, int k_tiles) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane16 = threadIdx.x & 15;
  const int64_t units = m * heads;
  const int k = heads * 128;
  float w[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) w[i] = static_cast<float>(weight[lane16 * 8 + i]);
  for (int64_t unit = (int64_t)blockIdx.x * (blockDim.x >> 4) + (threadIdx.x >> 4);
       unit < ((units + 1) & ~(int64_t)1); unit += (int64_t)gridDim.x * (blockDim.x >> 4)) {
    const bool valid = unit < units;   // units are paired in a warp: keep both halves in step
    const int64_t row = valid ? unit / heads : 0;
    const int head = valid ? (int)(unit - row * heads) : 0;
    float x[8], z[8];
    unpack_bf16x8(__ldg(reinterpret_cast<const uint4*>(core + row * k + head * 128 + lane16 * 8)), x);
    unpack_bf16x8(__ldg(reinterpret_cast<const uint4*>(gate + row * ld_gate + head * 128 + lane16 * 8)), z);
    float sq = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) sq = __fadd_rn(sq, __fmul_rn(x[i], x[i]));
#pragma unroll
    for (int d = 8; d > 0; d >>= 1) sq = __fadd_rn(sq, __shfl_xor_sync(0xffffffffu, sq, d));
    const float rstd = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(sq, 128.0f), eps)));
    float v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
      v[i] = swiglu_once_bf16(z[i], __fmul_rn(__fmul_rn(x[i], rstd), w[i]));
    const float amax = amax8_quad(v);
    const uint32_t bits = mx_scale_bits(amax);
    const float inv = mx_inverse(bits);
    if (valid) {
      *reinterpret_cast<uint2*>(codes + row * k + head * 128 + lane16 * 8) = quantize8(v, inv);
      if ((lane16 & 3) == 0)
        scales[sf_offset((int)row, head * 4 + (lane16 >> 2), k_tiles)] = (uint8_t)(bits >> 23);
    }
  }
}

// One CTA per row; thread t owns elements [8t, 8t+8) (+ 8*blockDim per extra vector).
template <int kVecs>
__global__ void __launch_bounds__(1024)
add_rmsnorm_mx_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
                      const __nv_bfloat16* __restrict__ w, float eps, float weight_bias,
                      __nv_bfloat16* norm_out, __nv_bfloat16* res_out, uint8_t* codes,
                      uint8_t* scales, int h, int k_tiles, bool norm_rounded_sum) {
  __shared__ float warp_sums[32];
  pdl_launch_dependents();
  pdl_wait();
  const int64_t row = blockIdx.x;
  float s[kVecs][8];
  bool have[kVecs];
  float sq = 0.0f;
#pragma unroll
  for (int v = 0; v < kVecs; ++v) {
    const int col = (v * blockDim.x + threadIdx.x) * 8;
    have[v] = col < h;
    if (have[v]) {
      unpack_bf16x8(*reinterpret_cast<const uint4*>(x + row * h + col), s[v]);
      if (res != nullptr) {
        float r[8];
        unpack_bf16x8(*reinterpret_cast<const uint4*>(res + row * h + col), r);
        uint32_t packed[4];
#pragma unroll
        for (int i = 0; i < 8; ++i) s[v][i] = __fadd_rn(s[v][i], r[i]);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const __nv_bfloat16 lo = __float2bfloat16_rn(s[v][2 * i]);
          const __nv_bfloat16 hi = __float2bfloat16_rn(s[v][2 * i + 1]);
          packed[i] = (uint32_t)__bfloat16_as_ushort(lo) | ((uint32_t)__bfloat16_as_ushort(hi) << 16);
          if (norm_rounded_sum) {
            s[v][2 * i] = __bfloat162float(lo);
            s[v][2 * i + 1] = __bfloat162float(hi);
          }
        }
        if (res_out != nullptr)
          *reinterpret_cast<uint4*>(res_out + row * h + col) =
              make_uint4(packed[0], packed[1], packed[2], packed[3]);
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) sq = __fadd_rn(sq, __fmul_rn(s[v][i], s[v][i]));
    }
  }
  // Fixed-order block reduction of the sum of squares.
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) sq = __fadd_rn(sq, __shfl_xor_sync(0xffffffffu, sq, d));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) warp_sums[warp] = sq;
  __syncthreads();
  if (warp == 0) {
    float t = lane < (int)(blockDim.x >> 5) ? warp_sums[lane] : 0.0f;
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) t = __fadd_rn(t, __shfl_xor_sync(0xffffffffu, t, d));
    if (lane == 0) warp_sums[0] = t;
  }
  __syncthreads();
  const float var = __fdiv_rn(warp_sums[0], (float)h);
  const float rs = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(var, eps)));
#pragma unroll
  for (int v = 0; v < kVecs; ++v) {
    const int col = (v * blockDim.x + threadIdx.x) * 8;
    float y[8];
    if (have[v]) {
      float wf[8];
      unpack_bf16x8(__ldg(reinterpret_cast<const uint4*>(w + col)), wf);
#pragma unroll
      for (int i = 0; i < 8; ++i)
        y[i] = bf16_round(__fmul_rn(__fmul_rn(s[v][i], rs), __fadd_rn(wf[i], weight_bias)));
      if (norm_out != nullptr) {
        uint32_t p[4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
          p[i] = (__float_as_uint(y[2 * i]) >> 16) | (__float_as_uint(y[2 * i + 1]) & 0xFFFF0000u);
        *reinterpret_cast<uint4*>(norm_out + row * h + col) = make_uint4(p[0], p[1], p[2], p[3]);
      }
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) y[i] = 0.0f;
    }
    if (codes != nullptr) {  // uniform across the block
      const float amax = amax8_quad(y);
      const uint32_t bits = mx_scale_bits(amax);
      const float inv = mx_inverse(bits);
      if (have[v]) {
        *reinterpret_cast<uint2*>(codes + row * h + col) = quantize8(y, inv);
        if ((threadIdx.x & 3) == 0)
          scales[sf_offset((int)row, col >> 5, k_tiles)] = (uint8_t)(bits >> 23);
      }
    }
  }
}

// 1x128 block FP8: sixteen threads per block of 128 values.
__global__ void __launch_bounds__(256)
fp8_group_quantize_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ q,
                          float* __restrict__ scales, int64_t m, int k) {
  const int groups = k >> 7;
  const int64_t units = m * groups;
  const int64_t units_per_pass = (int64_t)gridDim.x * (blockDim.x >> 4);
  const int sub = threadIdx.x & 15;
  pdl_launch_dependents();
  pdl_wait();
  // Two units per thread and pass (both loads in flight before either is used).
  for (int64_t base = 0; base < units; base += 2 * units_per_pass) {
    int64_t unit[2];
    bool valid[2];
    uint4 raw[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      unit[u] = base + u * units_per_pass + (int64_t)blockIdx.x * (blockDim.x >> 4) +
                (threadIdx.x >> 4);
      valid[u] = unit[u] < units;
      raw[u] = valid[u] ? __ldg(reinterpret_cast<const uint4*>(x + unit[u] * 128 + sub * 8))
                        : make_uint4(0u, 0u, 0u, 0u);
    }
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      float f[8];
      unpack_bf16x8(raw[u], f);
      float a = 0.0f;
#pragma unroll
      for (int i = 0; i < 8; ++i) a = fmaxf(a, fabsf(f[i]));
#pragma unroll
      for (int d = 1; d < 16; d <<= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, d));
      const float scale = __fdiv_rn(fmaxf(a, 1.0e-10f), 448.0f);
      if (valid[u]) {
        float v[8];
#pragma unroll
        for (int i = 0; i < 8; ++i)
          v[i] = fminf(fmaxf(__fdiv_rn(f[i], scale), -448.0f), 448.0f);
        uint2 out;
        out.x = e4m3x4(v[0], v[1], v[2], v[3]);
        out.y = e4m3x4(v[4], v[5], v[6], v[7]);
        *reinterpret_cast<uint2*>(q + unit[u] * 128 + sub * 8) = out;
        if (sub == 0) {
          const int64_t row = unit[u] / groups;
          const int64_t g = unit[u] - row * groups;
          scales[g * m + row] = scale;
        }
      }
    }
  }
}

// silu(g) * u in FP32 with the exponential taken as correctly rounded: the fast expf
// result is kept unless it could change an output bit (see callers).
__device__ __forceinline__ float silu_mul_fast(float g, float u) {
  const float sig = __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-g)));
  return __fmul_rn(__fmul_rn(g, sig), u);
}
__device__ __forceinline__ float silu_mul_exact(float g, float u) {
  const float t = static_cast<float>(exp(static_cast<double>(-g)));
  const float sig = __fdiv_rn(1.0f, __fadd_rn(1.0f, t));
  return __fmul_rn(__fmul_rn(g, sig), u);
}
// True when q lies so close to the midpoint of two adjacent E4M3 values that an error of a
// few FP32 ulps in q could change its rounding.
__device__ __forceinline__ bool near_e4m3_tie(float q) {
  const float a = fabsf(q);
  if (a >= 464.0f) return false;  // saturates either way (clamped to 448 before conversion)
  int e;
  frexpf(a, &e);                                   // a = f * 2^e, f in [0.5, 1)
  const int step_exp = max(e - 1 - 3, -9);         // spacing of E4M3 values around a
  const float t = ldexpf(a, -step_exp);            // a in units of the spacing
  const float frac = t - floorf(t);
  return fabsf(frac - 0.5f) < 1.0e-4f;
}

// Block-FP8 SwiGLU producer: sixteen threads per (row, 128 block).
__global__ void __launch_bounds__(256)
silu_mul_fp8_group_kernel(const __nv_bfloat16* __restrict__ in, uint8_t* __restrict__ out,
                          float* __restrict__ scales, int64_t m, int inter, bool transposed) {
  const int groups = inter >> 7;
  const int64_t units = m * groups;
  const int64_t units_per_pass = (int64_t)gridDim.x * (blockDim.x >> 4);
  const int sub = threadIdx.x & 15;
  pdl_launch_dependents();
  pdl_wait();
  for (int64_t base = 0; base < units; base += units_per_pass) {
    const int64_t unit = base + (int64_t)blockIdx.x * (blockDim.x >> 4) + (threadIdx.x >> 4);
    const bool valid = unit < units;
    const int64_t row = valid ? unit / groups : 0;
    const int g = valid ? (int)(unit - row * groups) : 0;
    float gate[8], up[8], v[8];
    if (valid) {
      const __nv_bfloat16* src = in + row * 2 * inter + g * 128 + sub * 8;
      unpack_bf16x8(__ldg(reinterpret_cast<const uint4*>(src)), gate);
      unpack_bf16x8(__ldg(reinterpret_cast<const uint4*>(src + inter)), up);
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) gate[i] = up[i] = 0.0f;
    }
    float a = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      v[i] = silu_mul_fast(gate[i], up[i]);
      a = fmaxf(a, fabsf(v[i]));
    }
#pragma unroll
    for (int d = 1; d < 16; d <<= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, d));
    // Candidates for the block maximum are recomputed exactly so the FP32 scale is exact.
    float a_exact = 0.0f;
    const float floor_a = a * (1.0f - 1.0e-5f);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (fabsf(v[i]) >= floor_a && a > 0.0f) {
        v[i] = silu_mul_exact(gate[i], up[i]);
        a_exact = fmaxf(a_exact, fabsf(v[i]));
      }
    }
#pragma unroll
    for (int d = 1; d < 16; d <<= 1)
      a_exact = fmaxf(a_exact, __shfl_xor_sync(0xffffffffu, a_exact, d));
    const float scale = fmaxf(__fdiv_rn(a_exact, 448.0f), 1.0f / (448.0f * 512.0f));
    if (valid) {
      float qv[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float qi = __fdiv_rn(v[i], scale);
        if (near_e4m3_tie(qi)) qi = __fdiv_rn(silu_mul_exact(gate[i], up[i]), scale);
        qv[i] = fmaxf(-448.0f, fminf(qi, 448.0f));
      }
      uint2 o;
      o.x = e4m3x4(qv[0], qv[1], qv[2], qv[3]);
      o.y = e4m3x4(qv[4], qv[5], qv[6], qv[7]);
      *reinterpret_cast<uint2*>(out + row * inter + g * 128 + sub * 8) = o;
      if (sub == 0) scales[transposed ? (int64_t)g * m + row : unit] = scale;
    }
  }
}

__global__ void pack_scales_kernel(const uint8_t* __restrict__ logical,
                                   uint8_t* __restrict__ swizzled, int64_t rows, int groups,
                                   int k_tiles, int64_t total) {
  // One thread per swizzled byte: total = ceil(rows/128)*128 * k_tiles*4.
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int g4 = (int)(i & 3);
    const int quad = (int)((i >> 2) & 3);
    const int r32 = (int)((i >> 4) & 31);
    const int64_t atom = i >> 9;
    const int kt = (int)(atom % k_tiles);
    const int64_t rb = atom / k_tiles;
    const int64_t row = rb * 128 + quad * 32 + r32;
    const int g = kt * 4 + g4;
    swizzled[i] = (row < rows && g < groups) ? logical[row * groups + g] : (uint8_t)127;
  }
}
__global__ void unpack_scales_kernel(const uint8_t* __restrict__ swizzled,
                                     uint8_t* __restrict__ logical, int64_t rows, int groups,
                                     int k_tiles) {
  const int64_t total = rows * groups;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = i / groups;
    const int g = (int)(i - row * groups);
    logical[i] = swizzled[sf_offset((int)row, g, k_tiles)];
  }
}

// dst physical row r  <-  src row (is_up ? I : 0) + feature, feature = (r / 64) * 32 + r % 32.
__global__ void interleave_rows_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst,
                                       int64_t two_i, int64_t row_bytes) {
  const int64_t total = two_i * row_bytes;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / row_bytes;
    const int64_t b = i - r * row_bytes;
    const int64_t feature = (r >> 6) * 32 + (r & 31);
    const int64_t src_row = ((r >> 5) & 1) * (two_i >> 1) + feature;
    dst[i] = src[src_row * row_bytes + b];
  }
}

int grid_for(int64_t work_items, int items_per_block) {
  const int64_t blocks = (work_items + items_per_block - 1) / items_per_block;
  const int64_t cap = (int64_t)sm_count() * 8;
  return (int)std::max<int64_t>(1, std::min(blocks, cap));
}

}  // namespace

}  // namespace mach

using namespace mach;

extern "C" size_t mach_mx_sf_bytes(int64_t rows, int64_t k) {
  if (rows < 0 || k < 0) return 0;
  return (size_t)((rows + 127) / 128) * 128 * (size_t)((k + 127) / 128) * 4;
}

extern "C" int mach_mxfp8_quantize(const void* x, int64_t ldx, void* codes, void* scales,
                                   int64_t m, int64_t k, void* stream) {
  if (m < 0 || k < 0) return fail(MACH_ERR_INVALID, "mxfp8_quantize: negative size");
  if (m == 0 || k == 0) return MACH_OK;
  if (!x || !codes || !scales) return fail(MACH_ERR_INVALID, "mxfp8_quantize: null pointer");
  if (k % 32 || ldx % 8 || ldx < k || !aligned16(x) || !aligned16(codes))
    return fail(MACH_ERR_UNSUPPORTED, "mxfp8_quantize: K %% 32, ldx %% 8 and 16-byte alignment required");
  if (m > INT32_MAX || k > INT32_MAX) return fail(MACH_ERR_UNSUPPORTED, "mxfp8_quantize: size");
  const int64_t units = m * (k / 32);
  const cudaError_t e = launch_ex(mx_quantize_kernel<0>, dim3(grid_for(units, 64)), dim3(256), 0,
                                  (cudaStream_t)stream, dim3(1, 1, 1), pdl_enabled(),
                                  (const __nv_bfloat16*)x, ldx, (uint8_t*)codes, (uint8_t*)scales, m,
                                  (int)k, (int)((k + 127) / 128));
  if (e != cudaSuccess) return fail(MACH_ERR_CUDA, "mxfp8_quantize: %s", cudaGetErrorString(e));
  return MACH_OK;
}

extern "C" int mach_swiglu_mxfp8_quantize(const void* gate_up, void* codes, void* scales,
                                          int64_t m, int64_t inter, void* stream) {
  if (m < 0 || inter < 0) return fail(MACH_ERR_INVALID, "swiglu_mxfp8_quantize: negative size");
  if (m == 0 || inter == 0) return MACH_OK;
  if (!gate_up || !codes || !scales)
    return fail(MACH_ERR_INVALID, "swiglu_mxfp8_quantize: null pointer");
  if (inter % 32 || !aligned16(gate_up) || !aligned16(codes) || m > INT32_MAX ||
      inter > INT32_MAX / 2)
    return fail(MACH_ERR_UNSUPPORTED, "swiglu_mxfp8_quantize: I %% 32 and 16-byte alignment required");
  const int64_t units = m * (inter / 32);
  mx_quantize_kernel<1><<<grid_for(units, 64), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)gate_up, 2 * inter, (uint8_t*)codes, (uint8_t*)scales, m, (int)inter,
      (int)((inter + 127) / 128));
  return check_launch("swiglu_mxfp8_quantize");
}

extern "C" int mach_gated_rmsnorm_mxfp8_quantize(const void* core_bf16, const void* gate_bf16,
                                                 int64_t ld_gate, const void* norm_weight,
                                                 int weight_is_f32, float eps, void* codes,
                                                 void* scales, int64_t m, int64_t heads,
                                                 void* stream) {
  if (m < 0 || heads < 0) return fail(MACH_ERR_INVALID, "gated_rmsnorm_mxfp8: negative size");
  if (m == 0 || heads == 0) return MACH_OK;
  if (!core_bf16 || !gate_bf16 || !norm_weight || !codes || !scales)
    return fail(MACH_ERR_INVALID, "gated_rmsnorm_mxfp8: null pointer");
  if (!aligned16(core_bf16) || !aligned16(gate_bf16) || !aligned16(codes) || ld_gate % 8 ||
      ld_gate < heads * 128 || m > INT32_MAX || heads > 4096)
    return fail(MACH_ERR_UNSUPPORTED,
                "gated_rmsnorm_mxfp8: 16-byte aligned rows of heads x 128 required");
  const int64_t units = m * heads;
  const int blocks = (int)std::max<int64_t>(1, std::min<int64_t>((units + 15) / 16, (int64_t)sm_count() * 8));
  const int k_tiles = (int)heads;   // K = heads * 128
  cudaError_t e;
  if (weight_is_f32)
    e = launch_ex(gated_rmsnorm_mx_kernel<float>, dim3((unsigned)blocks), dim3(256), 0,
                  (cudaStream_t)stream, dim3(1, 1, 1), pdl_enabled(),
                  (const __nv_bfloat16*)core_bf16, (const __nv_bfloat16*)gate_bf16, ld_gate,
                  (const float*)norm_weight, eps, (uint8_t*)codes, (uint8_t*)scales, m, (int)heads,
                  k_tiles);
  else
    e = launch_ex(gated_rmsnorm_mx_kernel<__nv_bfloat16>, dim3((unsigned)blocks), dim3(256), 0,
                  (cudaStream_t)stream, dim3(1, 1, 1), pdl_enabled(),
                  (const __nv_bfloat16*)core_bf16, (const __nv_bfloat16*)gate_bf16, ld_gate,
                  (const __nv_bfloat16*)norm_weight, eps, (uint8_t*)codes, (uint8_t*)scales, m,
                  (int)heads, k_tiles);
  if (e != cudaSuccess)
    return fail(MACH_ERR_CUDA, "gated_rmsnorm_mxfp8: %s", cudaGetErrorString(e));
  return MACH_OK;
}

extern "C" int mach_mxfp8_quantize_weight(const void* w_bf16, void* codes, void* logical_scales,
                                          int64_t n, int64_t k, void* stream) {
  if (n < 0 || k < 0) return fail(MACH_ERR_INVALID, "mxfp8_quantize_weight: negative size");
  if (n == 0 || k == 0) return MACH_OK;
  if (!w_bf16 || !codes || !logical_scales)
    return fail(MACH_ERR_INVALID, "mxfp8_quantize_weight: null pointer");
  if (k % 32 || !aligned16(w_bf16) || !aligned16(codes) || k > INT32_MAX)
    return fail(MACH_ERR_UNSUPPORTED, "mxfp8_quantize_weight: K %% 32 and 16-byte alignment required");
  const int64_t units = n * (k / 32);
  mx_quantize_weight_kernel<<<grid_for(units, 64), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)w_bf16, (uint8_t*)codes, (uint8_t*)logical_scales, n, (int)k);
  return check_launch("mxfp8_quantize_weight");
}

extern "C" int mach_swiglu_mxfp8_quantize_champion(const void* gate_up, void* codes, void* scales,
                                                   int64_t m, int64_t inter, void* stream) {
  if (m < 0 || inter < 0)
    return fail(MACH_ERR_INVALID, "swiglu_mxfp8_quantize_champion: negative size");
  if (m == 0 || inter == 0) return MACH_OK;
  if (!gate_up || !codes || !scales)
    return fail(MACH_ERR_INVALID, "swiglu_mxfp8_quantize_champion: null pointer");
  if (inter % 32 || !aligned16(gate_up) || !aligned16(codes) || m > INT32_MAX ||
      inter > INT32_MAX / 2)
    return fail(MACH_ERR_UNSUPPORTED,
                "swiglu_mxfp8_quantize_champion: I %% 32 and 16-byte alignment required");
  const int64_t units = m * (inter / 32);
  mx_quantize_kernel<2><<<grid_for(units, 64), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)gate_up, 2 * inter, (uint8_t*)codes, (uint8_t*)scales, m, (int)inter,
      (int)((inter + 127) / 128));
  return check_launch("swiglu_mxfp8_quantize_champion");
}

namespace mach {
int launch_add_rmsnorm(const void* x, const void* residual, const void* weight, float eps,
                       float weight_bias, void* norm_out, void* residual_out, void* codes,
                       void* scales, int64_t m, int64_t h, bool norm_rounded_sum,
                       cudaStream_t stream) {
  if (m < 0 || h < 0) return fail(MACH_ERR_INVALID, "add_rmsnorm: negative size");
  if (m == 0 || h == 0) return MACH_OK;
  if (!x || !weight) return fail(MACH_ERR_INVALID, "add_rmsnorm: null pointer");
  if ((codes == nullptr) != (scales == nullptr))
    return fail(MACH_ERR_INVALID, "add_rmsnorm: codes and scales go together");
  if (h % 32 || h > 16384 || m > INT32_MAX || !aligned16(x) || !aligned16(weight) ||
      (residual && !aligned16(residual)) || (norm_out && !aligned16(norm_out)) ||
      (residual_out && !aligned16(residual_out)) || (codes && !aligned16(codes)))
    return fail(MACH_ERR_UNSUPPORTED, "add_rmsnorm: H %% 32, H <= 16384, 16-byte alignment");
  const int vec_threads = (int)(h / 8);
  const int vecs = vec_threads > 1024 ? 2 : 1;
  int threads = (vec_threads + vecs - 1) / vecs;
  threads = ((threads + 31) / 32) * 32;
  const int k_tiles = (int)((h + 127) / 128);
  auto args = [&](auto kernel) {
    return launch_ex(kernel, dim3((unsigned)m), dim3(threads), 0, stream, dim3(1, 1, 1),
                     pdl_enabled(), (const __nv_bfloat16*)x, (const __nv_bfloat16*)residual,
                     (const __nv_bfloat16*)weight, eps, weight_bias, (__nv_bfloat16*)norm_out,
                     (__nv_bfloat16*)residual_out, (uint8_t*)codes, (uint8_t*)scales, (int)h, k_tiles,
                     norm_rounded_sum);
  };
  const cudaError_t e = vecs == 1 ? args(add_rmsnorm_mx_kernel<1>) : args(add_rmsnorm_mx_kernel<2>);
  if (e != cudaSuccess) return fail(MACH_ERR_CUDA, "add_rmsnorm: %s", cudaGetErrorString(e));
  return MACH_OK;
}
}  // namespace mach

extern "C" int mach_add_rmsnorm_mxfp8(const void* x, const void* residual, const void* weight,
                                      float eps, float weight_bias, void* norm_out,
                                      void* residual_out, void* codes, void* scales, int64_t m,
                                      int64_t h, void* stream) {
  return launch_add_rmsnorm(x, residual, weight, eps, weight_bias, norm_out, residual_out, codes,
                            scales, m, h, false, (cudaStream_t)stream);
}

extern "C" int mach_residual_rmsnorm_rounded_mxfp8(const void* a, const void* residual,
                                                   const void* gamma, float eps,
                                                   float weight_bias, void* norm_out,
                                                   void* residual_out, void* codes, void* scales,
                                                   int64_t m, int64_t h, void* stream) {
  if (m == 0) return MACH_OK;
  if (!residual) return fail(MACH_ERR_INVALID, "residual_rmsnorm_rounded: residual is required");
  return launch_add_rmsnorm(a, residual, gamma, eps, weight_bias, norm_out, residual_out, codes,
                            scales, m, h, true, (cudaStream_t)stream);
}

extern "C" int mach_mx_pack_scales(const void* logical, void* swizzled, int64_t rows, int64_t k,
                                   void* stream) {
  if (rows < 0 || k < 0) return fail(MACH_ERR_INVALID, "pack_scales: negative size");
  if (rows == 0 || k == 0) return MACH_OK;
  if (!logical || !swizzled) return fail(MACH_ERR_INVALID, "pack_scales: null pointer");
  if (k % 32) return fail(MACH_ERR_UNSUPPORTED, "pack_scales: K %% 32");
  const int64_t total = (int64_t)mach_mx_sf_bytes(rows, k);
  pack_scales_kernel<<<grid_for(total, 256), 256, 0, (cudaStream_t)stream>>>(
      (const uint8_t*)logical, (uint8_t*)swizzled, rows, (int)(k / 32), (int)((k + 127) / 128),
      total);
  return check_launch("pack_scales");
}

extern "C" int mach_mx_unpack_scales(const void* swizzled, void* logical, int64_t rows, int64_t k,
                                     void* stream) {
  if (rows < 0 || k < 0) return fail(MACH_ERR_INVALID, "unpack_scales: negative size");
  if (rows == 0 || k == 0) return MACH_OK;
  if (!logical || !swizzled) return fail(MACH_ERR_INVALID, "unpack_scales: null pointer");
  if (k % 32) return fail(MACH_ERR_UNSUPPORTED, "unpack_scales: K %% 32");
  unpack_scales_kernel<<<grid_for(rows * (k / 32), 256), 256, 0, (cudaStream_t)stream>>>(
      (const uint8_t*)swizzled, (uint8_t*)logical, rows, (int)(k / 32), (int)((k + 127) / 128));
  return check_launch("unpack_scales");
}

extern "C" int mach_mx_interleave_gate_up(const void* src, void* dst, int64_t two_i,
                                          int64_t row_bytes, void* stream) {
  if (two_i < 0 || row_bytes < 0) return fail(MACH_ERR_INVALID, "interleave_gate_up: negative size");
  if (two_i == 0 || row_bytes == 0) return MACH_OK;
  if (!src || !dst || src == dst) return fail(MACH_ERR_INVALID, "interleave_gate_up: bad pointers");
  if (two_i % 64) return fail(MACH_ERR_UNSUPPORTED, "interleave_gate_up: I %% 32 == 0 required");
  interleave_rows_kernel<<<grid_for(two_i * row_bytes, 256), 256, 0, (cudaStream_t)stream>>>(
      (const uint8_t*)src, (uint8_t*)dst, two_i, row_bytes);
  return check_launch("interleave_gate_up");
}

extern "C" int mach_fp8_group_quantize(const void* x, void* q, void* scales, int64_t m, int64_t k,
                                       void* stream) {
  if (m < 0 || k < 0) return fail(MACH_ERR_INVALID, "fp8_group_quantize: negative size");
  if (m == 0 || k == 0) return MACH_OK;
  if (!x || !q || !scales) return fail(MACH_ERR_INVALID, "fp8_group_quantize: null pointer");
  if (k % 128 || !aligned16(x) || !aligned16(q) || k > INT32_MAX)
    return fail(MACH_ERR_UNSUPPORTED, "fp8_group_quantize: K %% 128 and 16-byte alignment");
  const cudaError_t e = launch_ex(fp8_group_quantize_kernel, dim3((unsigned)grid_for(m * (k / 128), 16)),
                                  dim3(256), 0, (cudaStream_t)stream, dim3(1, 1, 1), pdl_enabled(),
                                  (const __nv_bfloat16*)x, (uint8_t*)q, (float*)scales, m, (int)k);
  if (e != cudaSuccess) return fail(MACH_ERR_CUDA, "fp8_group_quantize launch: %s", cudaGetErrorString(e));
  return MACH_OK;
}

extern "C" int mach_silu_mul_fp8_group_quantize(const void* input, void* out, void* scales,
                                                int64_t m, int64_t inter, int transposed,
                                                void* stream) {
  if (m < 0 || inter < 0) return fail(MACH_ERR_INVALID, "silu_mul_fp8: negative size");
  if (m == 0 || inter == 0) return MACH_OK;
  if (!input || !out || !scales) return fail(MACH_ERR_INVALID, "silu_mul_fp8: null pointer");
  if (inter % 128 || !aligned16(input) || !aligned16(out) || inter > INT32_MAX / 2)
    return fail(MACH_ERR_UNSUPPORTED, "silu_mul_fp8: I %% 128 and 16-byte alignment");
  const cudaError_t e =
      launch_ex(silu_mul_fp8_group_kernel, dim3((unsigned)grid_for(m * (inter / 128), 16)), dim3(256),
                0, (cudaStream_t)stream, dim3(1, 1, 1), pdl_enabled(), (const __nv_bfloat16*)input,
                (uint8_t*)out, (float*)scales, m, (int)inter, transposed != 0);
  if (e != cudaSuccess) return fail(MACH_ERR_CUDA, "silu_mul_fp8 launch: %s", cudaGetErrorString(e));
  return MACH_OK;
}
