// MoE routing around the grouped block-scaled GEMM: top-k router, expert-major permutation
// with 128-row padded expert segments, gather + MXFP8 quantisation of the routed rows, and the
// top-k weighted combine. Mirrors the stages of Mxfp6Sm120Experts.apply
// (src/vllm_mach/mxfp6/moe.py:574-702): quantize -> route -> grouped GEMM (W1) -> SiLU*mul +
// MXFP8 -> grouped GEMM (W2) -> reduce. Everything is device-side; the host never reads a
// count back, so the whole sequence is stream-ordered and capturable.
#include <cuda_bf16.h>
#include "host_util.h"
#include "ptx.cuh"
#include "quant_math.cuh"

namespace mach {
namespace {

constexpr int kMaxExperts = 1024;

// softmax (FP32) -> top-k -> renormalise; one warp per token. logits BF16 [M, E].
template <int kPerLane>  // experts <= 32 * kPerLane
__global__ void __launch_bounds__(256)
router_topk_kernel(const __nv_bfloat16* __restrict__ logits, float* __restrict__ weights,
                   int* __restrict__ ids, int m, int experts, int topk) {
  const int lane = threadIdx.x & 31;
  const int token = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  pdl_launch_dependents();
  pdl_wait();
  if (token >= m) return;
  float v[kPerLane];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < kPerLane; ++i) {
    const int e = i * 32 + lane;
    v[i] = e < experts ? __bfloat162float(logits[(size_t)token * experts + e]) : -INFINITY;
    mx = fmaxf(mx, v[i]);
  }
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, d));
  float sum = 0.0f;
#pragma unroll
  for (int i = 0; i < kPerLane; ++i) {
    v[i] = (i * 32 + lane) < experts ? expf(v[i] - mx) : 0.0f;
    sum += v[i];
  }
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, d);
  const float inv_sum = 1.0f / sum;
  float picked = 0.0f;
  float my_w = 0.0f;
  int my_id = 0;
  for (int k = 0; k < topk; ++k) {
    float best = -1.0f;
    int best_e = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < kPerLane; ++i) {
      const int e = i * 32 + lane;
      if (v[i] > best || (v[i] == best && e < best_e)) { best = v[i]; best_e = e; }
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, d);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, d);
      if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
    }
    if ((best_e & 31) == lane) v[best_e >> 5] = -1.0f;  // remove from further rounds
    const float prob = best * inv_sum;
    picked += prob;
    if (lane == k) { my_w = prob; my_id = best_e; }
  }
  if (lane < topk) {
    weights[(size_t)token * topk + lane] = my_w / picked;
    ids[(size_t)token * topk + lane] = my_id;
  }
}

__device__ __forceinline__ int ld_cluster_s32(uint32_t addr) {
  int v;
  asm volatile("ld.shared::cluster.s32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
  return v;
}

// Expert-major routing by one thread-block cluster (1, 2, 4 or 8 CTAs of 1024 threads; each CTA
// owns a contiguous slice of the (token, k) pairs):
//   1. per-CTA histogram of local expert ids in shared memory;
//   2. every CTA reads all histograms over distributed shared memory: totals, and the number
//      of rows the lower-ranked CTAs claim in each expert segment (its own base there);
//   3. scans over the experts (128-row padded segment offsets, work-item indices); CTA 0
//      writes counts, offsets, the work list and num_work;
//   4. every CTA scatters its pairs into its private range of each segment and marks its
//      share of the padding rows.
// Outputs: counts[E], offsets[E + 1], pos_of[M * topk] (-1: expert not local), src_of[row]
// for row < offsets[E] (-1: padding), work[3 * max_work], num_work[1].
// Slots inside a CTA's range are claimed with shared-memory atomics, so equal-expert pairs may
// swap places between runs. Row order inside a segment never changes a result: rows are
// independent in the GEMMs and the combine follows each token's own k order.
__global__ void __launch_bounds__(1024)
moe_route_kernel(const int* __restrict__ ids, const int* __restrict__ expert_map, int pairs,
                 int experts, int topk, int chunk_rows, int p_cap, int max_work,
                 int* __restrict__ counts, int* __restrict__ offsets, int* __restrict__ pos_of,
                 int* __restrict__ src_of, int* __restrict__ work, int* __restrict__ num_work) {
  __shared__ int s_count[kMaxExperts];       // this CTA's histogram (read by the peers)
  __shared__ int s_total[kMaxExperts];       // rows per expert over the whole cluster
  __shared__ int s_base[kMaxExperts];        // first row of this CTA's range in each segment
  __shared__ int s_cursor[kMaxExperts];
  __shared__ int s_offset[kMaxExperts + 1];  // padded segment offsets
  __shared__ int s_wbase[kMaxExperts + 1];   // first work item of each expert
  __shared__ int s_warp[32];
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int wid = tid >> 5;
  const int ncta = (int)gridDim.x;  // the whole grid is one cluster
  const int rank = (int)cluster_ctarank();
  pdl_launch_dependents();
  pdl_wait();
  for (int e = tid; e < experts; e += blockDim.x) { s_count[e] = 0; s_cursor[e] = 0; }
  __syncthreads();
  const int slice = (pairs + ncta - 1) / ncta;
  const int begin = min(pairs, rank * slice);
  const int end = min(pairs, begin + slice);
  for (int i = begin + tid; i < end; i += blockDim.x) {
    int e = ids[i];
    if (expert_map != nullptr) e = (e >= 0) ? expert_map[e] : -1;
    if (e >= 0 && e < experts) atomicAdd(&s_count[e], 1);
  }
  __syncthreads();
  if (ncta > 1) cluster_sync_all();
  for (int e = tid; e < experts; e += blockDim.x) {
    int total = 0, base = 0;
    for (int c = 0; c < ncta; ++c) {
      const int v = ncta > 1 ? ld_cluster_s32(map_to_cta(smem_u32(&s_count[e]), (uint32_t)c))
                             : s_count[e];
      if (c < rank) base += v;
      total += v;
    }
    s_total[e] = total;
    s_base[e] = base;
  }
  __syncthreads();
  // Exclusive scans over the experts: padded rows and work items (kMaxExperts == blockDim.x).
  {
    const int c = tid < experts ? s_total[tid] : 0;
    int rows = (c + 127) & ~127;
    int items = (c + chunk_rows - 1) / chunk_rows;
    int r = rows, w = items;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int ro = __shfl_up_sync(0xffffffffu, r, d);
      const int wo = __shfl_up_sync(0xffffffffu, w, d);
      if (lane >= d) { r += ro; w += wo; }
    }
    if (lane == 31) { s_warp[wid] = r; s_offset[wid] = w; }  // s_offset doubles as scratch here
    __syncthreads();
    int r_before = 0, w_before = 0;
    for (int j = 0; j < wid; ++j) { r_before += s_warp[j]; w_before += s_offset[j]; }
    __syncthreads();
    const int r_excl = r_before + r - rows;
    const int w_excl = w_before + w - items;
    if (tid < experts) { s_offset[tid] = r_excl; s_wbase[tid] = w_excl; }
    if (tid == experts - 1) { s_offset[experts] = r_excl + rows; s_wbase[experts] = w_excl + items; }
    __syncthreads();
  }
  if (rank == 0) {
    for (int e = tid; e <= experts; e += blockDim.x) {
      offsets[e] = s_offset[e];
      if (e < experts) {
        const int c = s_total[e];
        counts[e] = c;
        int nw = s_wbase[e];
        for (int r = 0; r < c; r += chunk_rows, ++nw) {
          if (nw < max_work) {
            work[3 * nw] = e;
            work[3 * nw + 1] = s_offset[e] + r;
            work[3 * nw + 2] = min(chunk_rows, c - r);
          }
        }
      }
    }
    if (tid == 0) *num_work = min(s_wbase[experts], max_work);
  }
  // Scatter this CTA's pairs.
  for (int i = begin + tid; i < end; i += blockDim.x) {
    int e = ids[i];
    if (expert_map != nullptr) e = (e >= 0) ? expert_map[e] : -1;
    int pos = -1;
    if (e >= 0 && e < experts) {
      pos = s_offset[e] + s_base[e] + atomicAdd(&s_cursor[e], 1);
      if (pos < p_cap) src_of[pos] = i / topk; else pos = -1;
    }
    pos_of[i] = pos;
  }
  // Padding rows: one warp per expert, experts dealt round-robin over all warps of the cluster.
  for (int e = rank * 32 + wid; e < experts; e += ncta * 32) {
    const int first = s_offset[e] + s_total[e];
    const int last = min(s_offset[e + 1], p_cap);
    for (int r = first + lane; r < last; r += 32) src_of[r] = -1;
  }
  if (ncta > 1) cluster_sync_all();  // peers may still be reading this CTA's histogram
}

// Gather the routed BF16 rows and quantise them to MXFP8 in permuted order. One warp per
// permuted row (padding rows cost one load and are left untouched: the GEMMs never store the
// columns they feed); inside a row four lanes share a 32-element block, as in the stand-alone
// quantiser.
__global__ void __launch_bounds__(256)
moe_gather_quantize_kernel(const __nv_bfloat16* __restrict__ hidden, const int* __restrict__ src_of,
                           const int* __restrict__ offsets, int experts,
                           uint8_t* __restrict__ codes, uint8_t* __restrict__ scales, int k,
                           int k_tiles) {
  const int groups = k >> 5;
  pdl_launch_dependents();
  pdl_wait();
  const int total_rows = offsets[experts];
  const int lane = threadIdx.x & 31;
  const int sub = lane & 3;
  const int warps = (int)((gridDim.x * blockDim.x) >> 5);
  for (int row = (int)((blockIdx.x * blockDim.x + threadIdx.x) >> 5); row < total_rows; row += warps) {
    const int src = src_of[row];
    if (src < 0) continue;  // warp-uniform
    for (int g0 = 0; g0 < groups; g0 += 8) {
      const int g = g0 + (lane >> 2);
      const bool in_range = g < groups;
      float f[8];
      if (in_range) {
        const uint4 v =
            __ldg(reinterpret_cast<const uint4*>(hidden + (size_t)src * k + g * 32 + sub * 8));
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          f[2 * i] = __uint_as_float(w[i] << 16);
          f[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
        }
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = 0.0f;
      }
      float a = 0.0f;
#pragma unroll
      for (int i = 0; i < 8; ++i) a = fmaxf(a, fabsf(f[i]));
      a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, 1));
      a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, 2));
      const uint32_t bits = mx_scale_bits(a);
      const float inv = mx_inverse(bits);
      if (in_range) {
        uint2 q;
        q.x = e4m3x4(__fmul_rn(f[0], inv), __fmul_rn(f[1], inv), __fmul_rn(f[2], inv), __fmul_rn(f[3], inv));
        q.y = e4m3x4(__fmul_rn(f[4], inv), __fmul_rn(f[5], inv), __fmul_rn(f[6], inv), __fmul_rn(f[7], inv));
        *reinterpret_cast<uint2*>(codes + (size_t)row * k + g * 32 + sub * 8) = q;
        if (sub == 0) scales[sf_offset(row, g, k_tiles)] = (uint8_t)(bits >> 23);
      }
    }
  }
}

// Same result as the gather form, token-major: one warp per TOKEN quantises the row once and
// stores the codes and scale bytes into each of its top-k permuted rows (pos_of < 0: expert not
// local). Reads the activations once instead of top-k times and quantises 1/top-k as much.
__global__ void __launch_bounds__(256)
moe_scatter_quantize_kernel(const __nv_bfloat16* __restrict__ hidden, const int* __restrict__ pos_of,
                            int m, int topk, uint8_t* __restrict__ codes,
                            uint8_t* __restrict__ scales, int k, int k_tiles) {
  const int groups = k >> 5;
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int sub = lane & 3;
  const int warps = (int)((gridDim.x * blockDim.x) >> 5);
  for (int token = (int)((blockIdx.x * blockDim.x + threadIdx.x) >> 5); token < m; token += warps) {
    for (int g0 = 0; g0 < groups; g0 += 8) {
      const int g = g0 + (lane >> 2);
      const bool in_range = g < groups;
      float f[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] = 0.0f;
      if (in_range) {
        const uint4 v =
            __ldg(reinterpret_cast<const uint4*>(hidden + (size_t)token * k + g * 32 + sub * 8));
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          f[2 * i] = __uint_as_float(w[i] << 16);
          f[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
        }
      }
      float a = 0.0f;
#pragma unroll
      for (int i = 0; i < 8; ++i) a = fmaxf(a, fabsf(f[i]));
      a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, 1));
      a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, 2));
      const uint32_t bits = mx_scale_bits(a);
      const float inv = mx_inverse(bits);
      uint2 q;
      q.x = e4m3x4(__fmul_rn(f[0], inv), __fmul_rn(f[1], inv), __fmul_rn(f[2], inv), __fmul_rn(f[3], inv));
      q.y = e4m3x4(__fmul_rn(f[4], inv), __fmul_rn(f[5], inv), __fmul_rn(f[6], inv), __fmul_rn(f[7], inv));
      if (in_range) {
        for (int j = 0; j < topk; ++j) {
          const int row = __ldg(pos_of + (size_t)token * topk + j);
          if (row < 0) continue;
          *reinterpret_cast<uint2*>(codes + (size_t)row * k + g * 32 + sub * 8) = q;
          if (sub == 0) scales[sf_offset(row, g, k_tiles)] = (uint8_t)(bits >> 23);
        }
      }
    }
  }
}

// out[m] = bf16( sum_k w[m,k] * f32(y[pos_of[m,k]]) ), k ascending; pairs of non-local experts
// are skipped. Eight features per thread.
__global__ void __launch_bounds__(256)
moe_combine_kernel(const __nv_bfloat16* __restrict__ y, const float* __restrict__ weights,
                   const int* __restrict__ pos_of, __nv_bfloat16* __restrict__ out, int m, int h,
                   int topk) {
  const int vecs = h >> 3;
  const int64_t total = (int64_t)m * vecs;
  pdl_launch_dependents();
  pdl_wait();
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int token = (int)(i / vecs);
    const int col = (int)(i - (int64_t)token * vecs) * 8;
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.0f;
    for (int k = 0; k < topk; ++k) {
      const int pos = pos_of[(size_t)token * topk + k];
      if (pos < 0) continue;
      const float w = weights[(size_t)token * topk + k];
      const uint4 v = *reinterpret_cast<const uint4*>(y + (size_t)pos * h + col);
      const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        acc[2 * j] = __fmaf_rn(w, __uint_as_float(u[j] << 16), acc[2 * j]);
        acc[2 * j + 1] = __fmaf_rn(w, __uint_as_float(u[j] & 0xFFFF0000u), acc[2 * j + 1]);
      }
    }
    uint32_t p[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const __nv_bfloat162 b = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
      p[j] = *reinterpret_cast<const uint32_t*>(&b);
    }
    *reinterpret_cast<uint4*>(out + (size_t)token * h + col) = make_uint4(p[0], p[1], p[2], p[3]);
  }
}

// Staged interface (the reference's route / grouped_gemm / silu_grouped_gemm / reduce shims,
// src/vllm_mach/mxfp6/moe_utils.py:205-488): the activation arrives ALREADY quantised (codes
// [M, K] + logical scales [M, K/32]). One warp per token copies its row into each of its top-k
// permuted rows and writes the scale bytes at their swizzled offsets.
__global__ void __launch_bounds__(256)
moe_scatter_codes_kernel(const uint8_t* __restrict__ codes_in, const uint8_t* __restrict__ scales_in,
                         const int* __restrict__ pos_of, int m, int topk,
                         uint8_t* __restrict__ codes, uint8_t* __restrict__ scales, int k,
                         int k_tiles) {
  const int groups = k >> 5;
  const int vecs = k >> 4;
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int warps = (int)((gridDim.x * blockDim.x) >> 5);
  for (int token = (int)((blockIdx.x * blockDim.x + threadIdx.x) >> 5); token < m; token += warps) {
    for (int j = 0; j < topk; ++j) {
      const int row = pos_of[(size_t)token * topk + j];
      if (row < 0) continue;  // warp-uniform
      for (int v = lane; v < vecs; v += 32)
        *reinterpret_cast<uint4*>(codes + (size_t)row * k + (size_t)v * 16) =
            __ldg(reinterpret_cast<const uint4*>(codes_in + (size_t)token * k + (size_t)v * 16));
      for (int g = lane; g < groups; g += 32)
        scales[sf_offset(row, g, k_tiles)] = __ldg(scales_in + (size_t)token * groups + g);
    }
  }
}

// int64 offsets of the staged interface from the route kernel's int32 outputs:
// expert_offsets[e] = routed rows of experts < e (true counts), scale_offsets[e] = first row of
// expert e's 128-row padded segment (the row index space of the permuted activation here).
__global__ void __launch_bounds__(1024)
moe_stage_offsets_kernel(const int* __restrict__ counts, const int* __restrict__ offsets,
                         int experts, long long* __restrict__ expert_offsets,
                         long long* __restrict__ scale_offsets) {
  __shared__ int s_warp[32];
  const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
  pdl_launch_dependents();
  pdl_wait();
  const int c = tid < experts ? counts[tid] : 0;
  int r = c;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const int o = __shfl_up_sync(0xffffffffu, r, d);
    if (lane >= d) r += o;
  }
  if (lane == 31) s_warp[wid] = r;
  __syncthreads();
  int before = 0;
  for (int j = 0; j < wid; ++j) before += s_warp[j];
  if (tid < experts) {
    expert_offsets[tid] = before + r - c;
    scale_offsets[tid] = offsets[tid];
  }
  if (tid == experts - 1) {
    expert_offsets[experts] = before + r;
    scale_offsets[experts] = offsets[experts];
  }
}

// Work list (expert, first row, rows <= chunk_rows) from the staged interface's offsets.
__global__ void __launch_bounds__(1024)
moe_work_from_offsets_kernel(const long long* __restrict__ expert_offsets,
                             const long long* __restrict__ scale_offsets, int experts,
                             int chunk_rows, int max_work, int* __restrict__ work,
                             int* __restrict__ num_work) {
  __shared__ int s_warp[32];
  const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
  pdl_launch_dependents();
  pdl_wait();
  const int c = tid < experts ? (int)(expert_offsets[tid + 1] - expert_offsets[tid]) : 0;
  const int items = (c + chunk_rows - 1) / chunk_rows;
  int w = items;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const int o = __shfl_up_sync(0xffffffffu, w, d);
    if (lane >= d) w += o;
  }
  if (lane == 31) s_warp[wid] = w;
  __syncthreads();
  int before = 0;
  for (int j = 0; j < wid; ++j) before += s_warp[j];
  int nw = before + w - items;
  if (tid < experts) {
    const int first = (int)scale_offsets[tid];
    for (int r = 0; r < c; r += chunk_rows, ++nw) {
      if (nw < max_work) {
        work[3 * nw] = tid;
        work[3 * nw + 1] = first + r;
        work[3 * nw + 2] = min(chunk_rows, c - r);
      }
    }
  }
  if (tid == experts - 1) *num_work = min(before + w, max_work);
}

}  // namespace
}  // namespace mach

using namespace mach;

namespace {
int launched(cudaError_t e, const char* what) {
  if (e != cudaSuccess) return fail(MACH_ERR_CUDA, "%s launch: %s", what, cudaGetErrorString(e));
  return MACH_OK;
}
}  // namespace

extern "C" int mach_moe_router_topk(const void* logits_bf16, void* topk_weights_f32,
                                    void* topk_ids_i32, int64_t m, int64_t experts, int64_t topk,
                                    void* stream) {
  if (m < 0) return fail(MACH_ERR_INVALID, "moe_router_topk: negative size");
  if (m == 0) return MACH_OK;
  if (!logits_bf16 || !topk_weights_f32 || !topk_ids_i32)
    return fail(MACH_ERR_INVALID, "moe_router_topk: null pointer");
  if (experts < 1 || experts > kMaxExperts || topk < 1 || topk > 32 || topk > experts)
    return fail(MACH_ERR_UNSUPPORTED, "moe_router_topk: experts <= %d and top-k <= 32 required",
                kMaxExperts);
  const int warps = 8;
  auto kernel = experts <= 128 ? router_topk_kernel<4>
              : experts <= 256 ? router_topk_kernel<8>
              : experts <= 512 ? router_topk_kernel<16> : router_topk_kernel<kMaxExperts / 32>;
  return launched(launch_ex(kernel, dim3((unsigned)((m + warps - 1) / warps)),
                            dim3(warps * 32), 0, (cudaStream_t)stream, dim3(1, 1, 1), pdl_enabled(),
                            (const __nv_bfloat16*)logits_bf16, (float*)topk_weights_f32,
                            (int*)topk_ids_i32, (int)m, (int)experts, (int)topk),
                  "moe_router_topk");
}

extern "C" int64_t mach_moe_rows_cap(int64_t tokens, int64_t topk, int64_t experts) {
  // Every non-empty expert segment is padded to 128 rows.
  const int64_t pairs = tokens * topk;
  return pairs + std::min<int64_t>(experts, pairs) * 127;
}

extern "C" int64_t mach_moe_work_cap(int64_t tokens, int64_t topk, int64_t experts,
                                     int64_t chunk_rows) {
  const int64_t pairs = tokens * topk;
  return std::min<int64_t>(experts, pairs) + pairs / std::max<int64_t>(1, chunk_rows);
}

extern "C" int mach_moe_route(const void* topk_ids_i32, const void* expert_map_i32, int64_t m,
                              int64_t topk, int64_t experts, int64_t chunk_rows, int64_t rows_cap,
                              int64_t work_cap, void* counts, void* offsets, void* pos_of,
                              void* src_of, void* work, void* num_work, void* stream) {
  if (m < 0 || topk < 1) return fail(MACH_ERR_INVALID, "moe_route: bad sizes");
  if (!topk_ids_i32 || !counts || !offsets || !pos_of || !src_of || !work || !num_work)
    return fail(MACH_ERR_INVALID, "moe_route: null pointer");
  if (experts < 1 || experts > kMaxExperts || m * topk > (1 << 22) ||
      (chunk_rows != 16 && chunk_rows != 64 && chunk_rows != 128 && chunk_rows != 256))
    return fail(MACH_ERR_UNSUPPORTED, "moe_route: unsupported expert count, pair count or chunk");
  if (rows_cap < mach_moe_rows_cap(m, topk, experts) ||
      work_cap < mach_moe_work_cap(m, topk, experts, chunk_rows))
    return fail(MACH_ERR_INVALID, "moe_route: workspace capacities are too small");
  // One cluster: about 4096 pairs per CTA, at most 8 CTAs.
  const int64_t pairs = m * topk;
  unsigned ncta = 1;
  while (ncta < 8 && pairs > (int64_t)ncta * 4096) ncta <<= 1;
  return launched(launch_ex(moe_route_kernel, dim3(ncta), dim3(1024), 0, (cudaStream_t)stream,
                            dim3(ncta, 1, 1), pdl_enabled(), (const int*)topk_ids_i32,
                            (const int*)expert_map_i32, (int)(m * topk), (int)experts, (int)topk,
                            (int)chunk_rows, (int)rows_cap, (int)work_cap, (int*)counts,
                            (int*)offsets, (int*)pos_of, (int*)src_of, (int*)work, (int*)num_work),
                  "moe_route");
}

extern "C" int mach_moe_gather_quantize(const void* hidden_bf16, const void* src_of,
                                        const void* offsets, int64_t experts, int64_t rows_cap,
                                        int64_t k, void* codes, void* scales, void* stream) {
  if (!hidden_bf16 || !src_of || !offsets || !codes || !scales)
    return fail(MACH_ERR_INVALID, "moe_gather_quantize: null pointer");
  if (k % 32 || k <= 0 || rows_cap < 0 || !aligned16(hidden_bf16) || !aligned16(codes))
    return fail(MACH_ERR_UNSUPPORTED, "moe_gather_quantize: K %% 32 and 16-byte alignment");
  if (rows_cap == 0) return MACH_OK;
  const int blocks = (int)std::max<int64_t>(1, std::min<int64_t>((rows_cap + 7) / 8, (int64_t)sm_count() * 8));
  return launched(launch_ex(moe_gather_quantize_kernel, dim3((unsigned)blocks), dim3(256), 0,
                            (cudaStream_t)stream, dim3(1, 1, 1), pdl_enabled(),
                            (const __nv_bfloat16*)hidden_bf16, (const int*)src_of,
                            (const int*)offsets, (int)experts, (uint8_t*)codes, (uint8_t*)scales,
                            (int)k, (int)((k + 127) / 128)),
                  "moe_gather_quantize");
}

extern "C" int mach_moe_scatter_quantize(const void* hidden_bf16, const void* pos_of, int64_t m,
                                         int64_t topk, int64_t k, void* codes, void* scales,
                                         void* stream) {
  if (!hidden_bf16 || !pos_of || !codes || !scales)
    return fail(MACH_ERR_INVALID, "moe_scatter_quantize: null pointer");
  if (k % 32 || k <= 0 || m < 0 || topk < 1 || !aligned16(hidden_bf16) || !aligned16(codes))
    return fail(MACH_ERR_UNSUPPORTED, "moe_scatter_quantize: K %% 32 and 16-byte alignment");
  if (m == 0) return MACH_OK;
  const int blocks = (int)std::max<int64_t>(1, std::min<int64_t>((m + 7) / 8, (int64_t)sm_count() * 8));
  return launched(launch_ex(moe_scatter_quantize_kernel, dim3((unsigned)blocks), dim3(256), 0,
                            (cudaStream_t)stream, dim3(1, 1, 1), pdl_enabled(),
                            (const __nv_bfloat16*)hidden_bf16, (const int*)pos_of, (int)m, (int)topk,
                            (uint8_t*)codes, (uint8_t*)scales, (int)k, (int)((k + 127) / 128)),
                  "moe_scatter_quantize");
}

extern "C" int mach_moe_combine(const void* y_bf16, const void* topk_weights_f32,
                                const void* pos_of, void* out_bf16, int64_t m, int64_t h,
                                int64_t topk, void* stream) {
  if (m < 0 || h < 0) return fail(MACH_ERR_INVALID, "moe_combine: negative size");
  if (m == 0 || h == 0) return MACH_OK;
  if (!y_bf16 || !topk_weights_f32 || !pos_of || !out_bf16)
    return fail(MACH_ERR_INVALID, "moe_combine: null pointer");
  if (h % 8 || !aligned16(y_bf16) || !aligned16(out_bf16))
    return fail(MACH_ERR_UNSUPPORTED, "moe_combine: H %% 8 and 16-byte alignment");
  const int64_t total = m * (h / 8);
  const int blocks = (int)std::max<int64_t>(1, std::min<int64_t>((total + 255) / 256, (int64_t)sm_count() * 8));
  return launched(launch_ex(moe_combine_kernel, dim3((unsigned)blocks), dim3(256), 0,
                            (cudaStream_t)stream, dim3(1, 1, 1), pdl_enabled(),
                            (const __nv_bfloat16*)y_bf16, (const float*)topk_weights_f32,
                            (const int*)pos_of, (__nv_bfloat16*)out_bf16, (int)m, (int)h, (int)topk),
                  "moe_combine");
}

extern "C" int mach_moe_scatter_codes(const void* codes_in, const void* logical_scales,
                                      const void* pos_of, int64_t m, int64_t topk, int64_t k,
                                      void* codes, void* scales, void* stream) {
  if (!codes_in || !logical_scales || !pos_of || !codes || !scales)
    return fail(MACH_ERR_INVALID, "moe_scatter_codes: null pointer");
  if (k % 32 || k <= 0 || m < 0 || topk < 1 || !aligned16(codes_in) || !aligned16(codes))
    return fail(MACH_ERR_UNSUPPORTED, "moe_scatter_codes: K %% 32 and 16-byte alignment");
  if (m == 0) return MACH_OK;
  const int blocks = (int)std::max<int64_t>(1, std::min<int64_t>((m + 7) / 8, (int64_t)sm_count() * 8));
  return launched(launch_ex(moe_scatter_codes_kernel, dim3((unsigned)blocks), dim3(256), 0,
                            (cudaStream_t)stream, dim3(1, 1, 1), pdl_enabled(),
                            (const uint8_t*)codes_in, (const uint8_t*)logical_scales,
                            (const int*)pos_of, (int)m, (int)topk, (uint8_t*)codes,
                            (uint8_t*)scales, (int)k, (int)((k + 127) / 128)),
                  "moe_scatter_codes");
}

extern "C" int mach_moe_stage_offsets(const void* counts, const void* offsets, int64_t experts,
                                      void* expert_offsets_i64, void* scale_offsets_i64,
                                      void* stream) {
  if (!counts || !offsets || !expert_offsets_i64 || !scale_offsets_i64)
    return fail(MACH_ERR_INVALID, "moe_stage_offsets: null pointer");
  if (experts < 1 || experts > kMaxExperts)
    return fail(MACH_ERR_UNSUPPORTED, "moe_stage_offsets: 1 <= experts <= 1024");
  return launched(launch_ex(moe_stage_offsets_kernel, dim3(1), dim3(1024), 0, (cudaStream_t)stream,
                            dim3(1, 1, 1), pdl_enabled(), (const int*)counts, (const int*)offsets,
                            (int)experts, (long long*)expert_offsets_i64,
                            (long long*)scale_offsets_i64),
                  "moe_stage_offsets");
}

extern "C" int mach_moe_work_from_offsets(const void* expert_offsets_i64,
                                          const void* scale_offsets_i64, int64_t experts,
                                          int64_t chunk_rows, int64_t work_cap, void* work,
                                          void* num_work, void* stream) {
  if (!expert_offsets_i64 || !scale_offsets_i64 || !work || !num_work)
    return fail(MACH_ERR_INVALID, "moe_work_from_offsets: null pointer");
  if (experts < 1 || experts > kMaxExperts || chunk_rows < 1 || work_cap < 1)
    return fail(MACH_ERR_UNSUPPORTED, "moe_work_from_offsets: bad sizes");
  return launched(launch_ex(moe_work_from_offsets_kernel, dim3(1), dim3(1024), 0,
                            (cudaStream_t)stream, dim3(1, 1, 1), pdl_enabled(),
                            (const long long*)expert_offsets_i64,
                            (const long long*)scale_offsets_i64, (int)experts, (int)chunk_rows,
                            (int)work_cap, (int*)work, (int*)num_work),
                  "moe_work_from_offsets");
}
