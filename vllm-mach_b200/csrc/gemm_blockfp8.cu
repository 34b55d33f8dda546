// Block-FP8 GEMM for sm_100a: E4M3 x E4M3 with FP32 scales, one per token per 128 K for
// the activations and one per 128x128 block for the weights:
//
//   y[m,n] = bf16( sum_g fma( dot_f32(A[m, g*128:(g+1)*128], B[n, same]), sa[m,g]*sb[n/128,g], acc ) )
//
// (src/vllm_mach/fp8/ordered.py:23-35). The 128-K dots run on tcgen05.mma kind::f8f6f4 into
// one of two TMEM accumulators (ping-pong); while the tensor core works on K group g+1 the
// four epilogue warps pull group g out of TMEM and fold it into FP32 registers with the
// exact `fma(dot, sa*sb, acc)` of the reference, ascending g.
//
// Orientation and K split follow gemm_mx.cu: token-major tiles (128 tokens x 128 features)
// for M > 64; feature-major tiles (128 features x padded batch) with a thread-block cluster
// splitting K for M <= 64, partial chains added in rank order through distributed shared
// memory.
#include <cuda.h>
#include <cuda_bf16.h>
#include "host_util.h"
#include "ptx.cuh"

namespace mach {

int make_operand_map(CUtensorMap* map, const void* base, int64_t rows, int64_t k, int format,
                     int box_rows);
int tuned_split();
int tuned_stages();
int tuned_pair();
int tuned_tile_width();
int run_block_fp8_tm(const void* a, const void* b, const float* sa, const float* sb,
                     __nv_bfloat16* out, int64_t m, int64_t n, int64_t k, int bn,
                     cudaStream_t stream);

namespace {

constexpr int kTileRows = 128;
constexpr int kTileK = 128;
constexpr int kTileBytes = kTileRows * kTileK;
constexpr int kThreads = 192;
constexpr int kMaxStages = 12;
constexpr int kMaxSwapCols = 64;

enum { kWaitEmpty = 201, kWaitFull = 202, kWaitAccFull = 203, kWaitAccEmpty = 204 };

struct BlockFp8Params {
  const float* sa;  // [K/128][M] (column-major per-token scales)
  const float* sb;  // [ceil(N/128)][K/128]
  __nv_bfloat16* out;
  int* status;
  int m, n, k;
  int groups;      // K / 128
  int bn;          // accumulator columns (token-major: 128; feature-major: padded batch)
  int stages;
  int split;
  int tmem_cols;
  uint32_t idesc;
  int stream_weights;
  float* raw;      // ordered mode: unscaled per-group dots [K/128][M][N]; grid.y = K/128
};

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}
__device__ __forceinline__ void named_barrier_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

template <bool kSwap>
__global__ void __launch_bounds__(kThreads, 1)
block_fp8_gemm_kernel(const __grid_constant__ CUtensorMap tm_p,
                      const __grid_constant__ CUtensorMap tm_q, const BlockFp8Params p) {
  constexpr int kAccRegs = kSwap ? kMaxSwapCols : 128;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int bn = p.bn;
  const int q_bytes = bn * kTileK;
  const int stage_bytes = (kTileBytes + q_bytes + 1023) & ~1023;
  const int tx_bytes = kTileBytes + q_bytes;
  const int stages = p.stages;
  const int split = kSwap ? p.split : 1;
  const int rows_owned = kTileRows / split;

  int m0 = 0, n0 = 0, rank = 0;
  if (kSwap) {
    n0 = blockIdx.x * kTileRows;
    rank = blockIdx.y;
  } else {
    const int tiles_m = (p.m + kTileRows - 1) / kTileRows;
    m0 = (blockIdx.x % tiles_m) * kTileRows;
    n0 = (blockIdx.x / tiles_m) * bn;
  }
  const bool raw_mode = kSwap && p.raw != nullptr;
  const int g_begin = raw_mode ? rank : (int)(((long long)rank * p.groups) / split);
  const int g_end = raw_mode ? rank + 1 : (int)(((long long)(rank + 1) * p.groups) / split);
  const int my_groups = g_end - g_begin;

  float* recv = reinterpret_cast<float*>(smem + (size_t)stages * stage_bytes);
  const int recv_bytes = kSwap ? kTileRows * bn * 4 : 0;
  float* scale_tbl = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(recv) + recv_bytes);
  const int tbl_bytes = kSwap ? ((p.groups + split - 1) / split + 1) * bn * 4 : 0;
  uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(scale_tbl) + tbl_bytes);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kMaxStages + 4);
  const uint32_t full0 = smem_u32(bars);
  const uint32_t empty0 = smem_u32(bars + kMaxStages);
  const uint32_t acc_full0 = smem_u32(bars + 2 * kMaxStages);
  const uint32_t acc_empty0 = smem_u32(bars + 2 * kMaxStages + 2);

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full0 + 8 * b, 1);
      mbar_init(acc_empty0 + 8 * b, 4);  // one arrival per epilogue warp
    }
    fence_mbar_init();
    prefetch_tensormap(&tm_p);
    prefetch_tensormap(&tm_q);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), (uint32_t)p.tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (kSwap && split > 1) cluster_sync_all();
  if (threadIdx.x == 0) pdl_launch_dependents();

  if (warp == 0) {
    // TMA producer: warp-uniform loop, one elected lane issues.
    const uint64_t pol_w = p.stream_weights ? policy_evict_first() : policy_evict_normal();
    const uint64_t pol_a = policy_evict_last();
    const uint32_t base0 = smem_u32(smem);
    // The weights do not depend on the preceding kernel: fill the ring with them first, then
    // wait for the predecessor (programmatic dependent launch) and add the activations.
    const int pre = min(stages, my_groups);
    if (elect_one()) {
      for (int it = 0; it < pre; ++it) {
        const uint32_t full = full0 + 8 * it;
        mbar_expect_tx(full, (uint32_t)tx_bytes);
        const uint32_t base = base0 + (uint32_t)(it * stage_bytes);
        const int k0 = (g_begin + it) * kTileK;
        if (kSwap) tma_load_2d(base, &tm_p, full, k0, n0, pol_w);
        else tma_load_2d(base + kTileBytes, &tm_q, full, k0, n0, pol_w);
      }
      pdl_wait();
      for (int it = 0; it < pre; ++it) {
        const uint32_t full = full0 + 8 * it;
        const uint32_t base = base0 + (uint32_t)(it * stage_bytes);
        const int k0 = (g_begin + it) * kTileK;
        if (kSwap) tma_load_2d(base + kTileBytes, &tm_q, full, k0, 0, pol_a);
        else tma_load_2d(base, &tm_p, full, k0, m0, pol_a);
      }
    }
    __syncwarp();
    int s = pre % stages;
    uint32_t ph = pre == stages ? 1u : 0u;
    for (int it = pre; it < my_groups; ++it) {
      if (!mbar_wait(empty0 + 8 * s, ph ^ 1u, p.status, kWaitEmpty)) break;
      if (elect_one()) {
        const uint32_t full = full0 + 8 * s;
        mbar_expect_tx(full, (uint32_t)tx_bytes);
        const uint32_t base = base0 + (uint32_t)(s * stage_bytes);
        const int k0 = (g_begin + it) * kTileK;
        tma_load_2d(base, &tm_p, full, k0, kSwap ? n0 : m0, kSwap ? pol_w : pol_a);
        tma_load_2d(base + kTileBytes, &tm_q, full, k0, kSwap ? 0 : n0, kSwap ? pol_a : pol_w);
      }
      __syncwarp();
      if (++s == stages) { s = 0; ph ^= 1u; }
    }
  } else if (warp == 1) {
    // MMA issuer: warp-uniform loop, one elected lane issues.
    const uint32_t lo_stage0 = desc_lo(smem_u32(smem));
    const uint32_t lo_step = (uint32_t)stage_bytes >> 4;
    const uint32_t lo_q = (uint32_t)kTileBytes >> 4;
    int s = 0;
    uint32_t ph = 0;
    for (int it = 0; it < my_groups; ++it) {
      const int buf = it & 1;
      // The accumulator buffer must have been drained (two groups ago).
      if (!mbar_wait(acc_empty0 + 8 * buf, (((uint32_t)it >> 1) & 1u) ^ 1u, p.status, kWaitAccEmpty))
        break;
      if (!mbar_wait(full0 + 8 * s, ph, p.status, kWaitFull)) break;
      tc_fence_after();
      if (elect_one()) {
        const uint32_t lo = lo_stage0 + (uint32_t)s * lo_step;
#pragma unroll
        for (int sub = 0; sub < 4; ++sub)
          tc_mma_f8_lo(tmem_base + buf * bn, lo + 2 * sub, lo + lo_q + 2 * sub, p.idesc,
                       sub > 0 ? 1u : 0u);
        tc_commit(empty0 + 8 * s);
        tc_commit(acc_full0 + 8 * buf);
      }
      __syncwarp();
      if (++s == stages) { s = 0; ph ^= 1u; }
    }
  } else {
    const int quad = warp & 3;
    const uint32_t t_lane = tmem_base + ((uint32_t)(quad * 32) << 16);
    float acc[kAccRegs];
#pragma unroll
    for (int i = 0; i < kAccRegs; ++i) acc[i] = 0.0f;
    pdl_wait();  // activation scales are read and outputs written only after the predecessor

    if (kSwap) {
      // Scale table of this CTA's K range: tbl[g - g_begin][col] = sa[g, col] * sb[n0/128, g].
      const int et = threadIdx.x - 64;
      for (int idx = et; idx < my_groups * bn; idx += 128) {
        const int gl = idx / bn;
        const int col = idx - gl * bn;
        const int g = g_begin + gl;
        const float a = col < p.m ? p.sa[(size_t)g * p.m + col] : 0.0f;
        scale_tbl[idx] = raw_mode ? 1.0f : __fmul_rn(a, p.sb[(size_t)(n0 >> 7) * p.groups + g]);
      }
      named_barrier_sync(1, 128);
    }
    const int row = m0 + quad * 32 + lane;  // token-major: token index
    bool ok = true;
    // Token-major scales: fetched one group ahead, multiplied only when used.
    float sa_next = 0.0f, sb_next = 0.0f;
    if (!kSwap && my_groups > 0) {
      sa_next = row < p.m ? __ldg(p.sa + (size_t)g_begin * p.m + row) : 0.0f;
      sb_next = __ldg(p.sb + (size_t)(n0 >> 7) * p.groups + g_begin);
    }
    for (int it = 0; it < my_groups && ok; ++it) {
      const int buf = it & 1;
      const float sa_cur = sa_next, sb_cur = sb_next;
      if (!kSwap && it + 1 < my_groups) {
        const int g = g_begin + it + 1;
        sa_next = row < p.m ? __ldg(p.sa + (size_t)g * p.m + row) : 0.0f;
        sb_next = __ldg(p.sb + (size_t)(n0 >> 7) * p.groups + g);
      }
      ok = mbar_wait(acc_full0 + 8 * buf, ((uint32_t)it >> 1) & 1u, p.status, kWaitAccFull);
      tc_fence_after();
      if (!kSwap) {
        const float s = __fmul_rn(sa_cur, sb_cur);
        // 64 columns per round trip to TMEM; the buffer goes back to the MMA thread as soon
        // as its last values are in registers.
        uint32_t ra[32], rb[32];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          tmem_ld_x32(t_lane + buf * bn + h * 64, ra);
          tmem_ld_x32(t_lane + buf * bn + h * 64 + 32, rb);
          tmem_ld_wait();
          if (h == 1) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty0 + 8 * buf);
          }
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            acc[h * 64 + i] = __fmaf_rn(__uint_as_float(ra[i]), s, acc[h * 64 + i]);
            acc[h * 64 + 32 + i] = __fmaf_rn(__uint_as_float(rb[i]), s, acc[h * 64 + 32 + i]);
          }
        }
      } else {
        // All of the (at most 64) columns in flight at once, one wait.
        const float* tbl = scale_tbl + it * bn;
        uint32_t r[kMaxSwapCols];
#pragma unroll
        for (int c = 0; c < kMaxSwapCols / 16; ++c)
          if (c * 16 < bn) tmem_ld_x16(t_lane + buf * bn + c * 16, *reinterpret_cast<uint32_t(*)[16]>(r + c * 16));
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(acc_empty0 + 8 * buf);
#pragma unroll
        for (int c = 0; c < kMaxSwapCols / 16; ++c) {
          if (c * 16 < bn) {
#pragma unroll
            for (int i = 0; i < 16; ++i)
              acc[c * 16 + i] = __fmaf_rn(__uint_as_float(r[c * 16 + i]), tbl[c * 16 + i], acc[c * 16 + i]);
          }
        }
      }
    }


    if (!kSwap) {
      if (ok && row < p.m) {
#pragma unroll
        for (int c = 0; c < 128; c += 8) {
          const int n = n0 + c;
          if (n < p.n) {  // N % 8 == 0
            *reinterpret_cast<uint4*>(p.out + (size_t)row * p.n + n) =
                make_uint4(pack_bf16x2(acc[c], acc[c + 1]), pack_bf16x2(acc[c + 2], acc[c + 3]),
                           pack_bf16x2(acc[c + 4], acc[c + 5]), pack_bf16x2(acc[c + 6], acc[c + 7]));
          }
        }
      }
    } else if (raw_mode) {
      // Ordered mode: the unscaled dot of this K group goes to scratch; the chain over the
      // groups is evaluated afterwards in one ascending pass.
      const int n = n0 + quad * 32 + lane;
#pragma unroll
      for (int c = 0; c < kMaxSwapCols; ++c)
        if (c < p.m && n < p.n) p.raw[((size_t)rank * p.m + c) * p.n + n] = acc[c];
    } else {
      const int trow = quad * 32 + lane;
      const int owner = trow / rows_owned;
      const int rl = trow - owner * rows_owned;
      const uint32_t recv_local = smem_u32(recv);
      const uint32_t recv_dst = split > 1 ? map_to_cta(recv_local, (uint32_t)owner) : recv_local;
#pragma unroll
      for (int c = 0; c < kMaxSwapCols; ++c) {
        if (c < bn) {
          const uint32_t off = (uint32_t)((((rank * bn) + c) * rows_owned + rl) * 4);
          st_cluster_f32(recv_dst + off, acc[c]);
        }
      }
    }
  }

  if (kSwap) {
    if (split > 1) cluster_sync_all(); else __syncthreads();
    if (warp >= 2 && !raw_mode) {
      const int et = threadIdx.x - 64;
      const int row_base = n0 + rank * rows_owned;
      const int total = rows_owned * bn;
      for (int idx = et; idx < total; idx += 128) {
        const int col = idx / rows_owned;
        const int rl = idx - col * rows_owned;
        float v = 0.0f;
        for (int c = 0; c < split; ++c)
          v = __fadd_rn(v, recv[((size_t)c * bn + col) * rows_owned + rl]);
        const int n = row_base + rl;
        if (col < p.m && n < p.n) p.out[(size_t)col * p.n + n] = __float2bfloat16_rn(v);
      }
    }
  } else {
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, (uint32_t)p.tmem_cols);
  }
}

template <bool kSwap>
int launch(const CUtensorMap& tm_p, const CUtensorMap& tm_q, BlockFp8Params& prm, dim3 grid,
           int smem_bytes, cudaStream_t stream) {
  auto kernel = block_fp8_gemm_kernel<kSwap>;
  static int configured_smem_dev[kMaxDeviceSlots] = {};  // the attribute is per device
  int& configured_smem = configured_smem_dev[device_slot()];
  if (smem_bytes > configured_smem) {
    const cudaError_t e =
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
    if (e != cudaSuccess)
      return fail(MACH_ERR_CUDA, "block_fp8_gemm: shared memory opt-in failed: %s",
                  cudaGetErrorString(e));
    configured_smem = smem_bytes;
  }
  const cudaError_t e =
      launch_ex(kernel, grid, dim3(kThreads), (size_t)smem_bytes, stream,
                dim3(1, (kSwap && prm.split > 1) ? (unsigned)prm.split : 1u, 1), pdl_enabled(), tm_p,
                tm_q, prm);
  if (e != cudaSuccess) return fail(MACH_ERR_CUDA, "block_fp8_gemm launch: %s", cudaGetErrorString(e));
  return MACH_OK;
}

}  // namespace
}  // namespace mach

using namespace mach;

namespace mach {
namespace {

// out[m][n] = bf16( fma chain over ascending g of raw[g][m][n] * (sa[g][m] * sb[n/128][g]) ).
__global__ void __launch_bounds__(256)
ordered_reduce_kernel(const float* __restrict__ raw, const float* __restrict__ sa,
                      const float* __restrict__ sb, __nv_bfloat16* __restrict__ out, int m, int n,
                      int groups) {
  const int64_t total = (int64_t)m * n;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int row = (int)(i / n);
    const int col = (int)(i - (int64_t)row * n);
    float acc = 0.0f;
    for (int g = 0; g < groups; ++g) {
      const float s = __fmul_rn(sa[(size_t)g * m + row], sb[(size_t)(col >> 7) * groups + g]);
      acc = __fmaf_rn(raw[(size_t)g * total + i], s, acc);
    }
    out[i] = __float2bfloat16_rn(acc);
  }
}

int run_block_fp8(const void* a, const void* b, const void* sa, const void* sb, void* out,
                  float* raw, int64_t m, int64_t n, int64_t k, cudaStream_t stream);

}  // namespace
}  // namespace mach

extern "C" int mach_block_fp8_gemm(const void* a, const void* b, const void* sa, const void* sb,
                                   void* out, int64_t m, int64_t n, int64_t k, void* stream) {
  return run_block_fp8(a, b, sa, sb, out, nullptr, m, n, k, (cudaStream_t)stream);
}

// ---- Scratch that ships with the library (mach_block_fp8_gemm_ordered_static).
// kStaticScratchBytes of FP32 per-group dots; resident on every GPU that loads the library
// for as long as the process lives. The name below is only meaningful to device code: host
// code must translate it with cudaGetSymbolAddress, once per device, while that device is
// current, and hand the translated pointer to the kernels.
constexpr size_t kStaticScratchBytes = 8u << 20;
static __device__ __align__(256) float g_ordered_scratch[kStaticScratchBytes / sizeof(float)];

namespace mach {
namespace {
constexpr int kMaxScratchDevices = 64;
float* g_scratch_ptr[kMaxScratchDevices];  // device addresses, filled on first use per device

// Device address of the built-in scratch for the current device (NULL + error text on failure).
float* static_scratch_for_current_device() {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxScratchDevices) {
    fail(MACH_ERR_CUDA, "block_fp8_gemm_ordered_static: cannot identify the current device");
    return nullptr;
  }
  if (g_scratch_ptr[dev] == nullptr) {
    float* p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_ordered_scratch);
    if (e != cudaSuccess || p == nullptr) {
      fail(MACH_ERR_CUDA, "block_fp8_gemm_ordered_static: cudaGetSymbolAddress failed: %s",
           cudaGetErrorString(e));
      return nullptr;
    }
    g_scratch_ptr[dev] = p;
  }
  return g_scratch_ptr[dev];
}
}  // namespace
}  // namespace mach

extern "C" int mach_block_fp8_gemm_ordered_static(const void* a, const void* b, const void* sa,
                                                  const void* sb, void* out, int64_t m, int64_t n,
                                                  int64_t k, void* stream) {
  if (m < 0 || n < 0 || k < 0)
    return fail(MACH_ERR_INVALID, "block_fp8_gemm_ordered_static: negative size");
  if (m > kMaxSwapCols)
    return fail(MACH_ERR_UNSUPPORTED, "block_fp8_gemm_ordered_static: M <= %d required",
                kMaxSwapCols);
  const unsigned long long need =
      (unsigned long long)(k / 128) * (unsigned long long)m * (unsigned long long)n * sizeof(float);
  if (need > kStaticScratchBytes)
    return fail(MACH_ERR_UNSUPPORTED,
                "block_fp8_gemm_ordered_static: (K/128) * M * N * 4 = %llu bytes exceeds the "
                "built-in scratch of %llu bytes; use mach_block_fp8_gemm_ordered with your own "
                "scratch", need, (unsigned long long)kStaticScratchBytes);
  float* scratch = static_scratch_for_current_device();
  if (!scratch) return MACH_ERR_CUDA;
  return run_block_fp8(a, b, sa, sb, out, scratch, m, n, k, (cudaStream_t)stream);
}

extern "C" int mach_block_fp8_gemm_ordered(const void* a, const void* b, const void* sa,
                                           const void* sb, void* out, void* raw_scratch,
                                           int64_t m, int64_t n, int64_t k, void* stream) {
  if (!raw_scratch) return fail(MACH_ERR_INVALID, "block_fp8_gemm_ordered: null scratch");
  if (m > kMaxSwapCols)
    return fail(MACH_ERR_UNSUPPORTED, "block_fp8_gemm_ordered: M <= %d required", kMaxSwapCols);
  return run_block_fp8(a, b, sa, sb, out, reinterpret_cast<float*>(raw_scratch), m, n, k,
                       (cudaStream_t)stream);
}

namespace mach {
namespace {
int run_block_fp8(const void* a, const void* b, const void* sa, const void* sb, void* out,
                        float* raw, int64_t m, int64_t n, int64_t k, cudaStream_t stream) {
  if (m < 0 || n < 0 || k < 0) return fail(MACH_ERR_INVALID, "block_fp8_gemm: negative size");
  if (m == 0 || n == 0) return MACH_OK;
  if (!a || !b || !sa || !sb || !out) return fail(MACH_ERR_INVALID, "block_fp8_gemm: null pointer");
  if (k < 128 || k % 128 || n % 16)
    return fail(MACH_ERR_UNSUPPORTED, "block_fp8_gemm: K %% 128 == 0 and N %% 16 == 0 required");
  if (!aligned16(a) || !aligned16(b) || !aligned16(out))
    return fail(MACH_ERR_UNSUPPORTED, "block_fp8_gemm: 16-byte aligned operands required");
  if (m > (1 << 24) || n > (1 << 24) || k > (1 << 24))
    return fail(MACH_ERR_UNSUPPORTED, "block_fp8_gemm: dimension too large");
  BlockFp8Params prm = {};
  prm.sa = (const float*)sa;
  prm.sb = (const float*)sb;
  prm.out = (__nv_bfloat16*)out;
  prm.status = device_status_ptr();
  if (!prm.status) return fail(MACH_ERR_CUDA, "block_fp8_gemm: cannot resolve the status word");
  prm.m = (int)m;
  prm.n = (int)n;
  prm.k = (int)k;
  prm.groups = (int)(k / 128);
  const bool swap = m <= kMaxSwapCols;
  if (!swap && tuned_pair() != 0) {
    // Persistent kernel with 128 x 256 tiles once those occupy about half of the SMs (measured
    // cross-over against one 128 x 128 tile per CTA); forced by a tile-width setting.
    const int64_t tiles256 = ((m + 127) / 128) * ((n + 255) / 256);
    const int forced = tuned_tile_width();
    if (forced == 128 || forced == 256 || tiles256 * 7 >= (int64_t)sm_count() * 3)
      return run_block_fp8_tm(a, b, prm.sa, prm.sb, prm.out, m, n, k, forced == 128 ? 128 : 256,
                              stream);
  }
  dim3 grid;
  if (swap) {
    prm.bn = (int)((m + 15) / 16) * 16;
    const int64_t tiles = (n + 127) / 128;
    int split = 1;
    if (tuned_split() > 0) split = tuned_split();
    else while (split < 8 && tiles * split < sm_count()) split <<= 1;  // about one CTA per SM (measured)
    split = std::min(split, 8);
    while (split > 1 && split > prm.groups) split >>= 1;
    if (split != 1 && split != 2 && split != 4 && split != 8)
      return fail(MACH_ERR_INVALID, "block_fp8_gemm: cluster split must be 1, 2, 4 or 8");
    if (raw) split = 1;
    prm.split = split;
    prm.raw = raw;
    grid = dim3((unsigned)tiles, (unsigned)(raw ? prm.groups : split), 1);
    prm.stream_weights = 1;
    prm.idesc = idesc_f8(kFmtE4M3, kFmtE4M3, (uint32_t)prm.bn);
  } else {
    prm.bn = 128;
    prm.split = 1;
    grid = dim3((unsigned)(((m + 127) / 128) * ((n + 127) / 128)), 1, 1);
    prm.stream_weights = m <= 128 ? 1 : 0;
    prm.idesc = idesc_f8(kFmtE4M3, kFmtE4M3, 128);
  }
  int cols = 32;
  while (cols < 2 * prm.bn) cols <<= 1;
  prm.tmem_cols = cols;
  const int stage_bytes = (kTileBytes + prm.bn * kTileK + 1023) & ~1023;
  const int recv_bytes = swap ? kTileRows * prm.bn * 4 : 0;
  const int tbl_bytes = swap ? ((prm.groups + prm.split - 1) / prm.split + 1) * prm.bn * 4 : 0;
  const int fixed = recv_bytes + tbl_bytes + (2 * kMaxStages + 4) * 8 + 16 + 1024;
  int budget = max_smem_optin();
  if (swap) budget = std::min(budget, std::max(70 * 1024, fixed + 3 * stage_bytes));
  int stages = (budget - fixed) / stage_bytes;
  stages = std::min(stages, kMaxStages);
  if (tuned_stages() > 0) stages = std::min(stages, tuned_stages());
  if (stages < 1) return fail(MACH_ERR_UNSUPPORTED, "block_fp8_gemm: tile does not fit in shared memory");
  stages = std::max(1, std::min(stages, raw ? 1 : (prm.groups + prm.split - 1) / prm.split));
  prm.stages = stages;
  int smem_bytes = stages * stage_bytes + fixed;
  const int max_resident = 512 / prm.tmem_cols;
  const int sm_smem = 228 * 1024;
  if ((sm_smem / (smem_bytes + 1024)) > max_resident) smem_bytes = sm_smem / (max_resident + 1) + 1;

  CUtensorMap tm_a, tm_b;
  int rc = make_operand_map(&tm_a, a, m, k, MACH_FMT_E4M3, swap ? prm.bn : kTileRows);
  if (rc) return rc;
  rc = make_operand_map(&tm_b, b, n, k, MACH_FMT_E4M3, kTileRows);
  if (rc) return rc;
  if (swap) {
    rc = launch<true>(tm_b, tm_a, prm, grid, smem_bytes, stream);
    if (rc || !raw) return rc;
    const int64_t total = m * n;
    const int blocks = (int)std::min<int64_t>((total + 255) / 256, (int64_t)sm_count() * 8);
    ordered_reduce_kernel<<<blocks, 256, 0, stream>>>(raw, prm.sa, prm.sb, prm.out, (int)m, (int)n,
                                                      prm.groups);
    return check_launch("block_fp8_gemm_ordered");
  }
  return launch<false>(tm_a, tm_b, prm, grid, smem_bytes, stream);
}

}  // namespace
}  // namespace mach
