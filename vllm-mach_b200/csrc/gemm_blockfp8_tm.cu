// Block-FP8 GEMM, token-major persistent kernel for batches above 64 tokens:
//
//   y[m,n] = bf16( sum_g fma( dot_f32(A[m, g*128:(g+1)*128], B[n, same]), sa[m,g]*sb[n/128,g], acc ) )
//
// with g ascending (src/vllm_mach/fp8/ordered.py:23-35). The scales are arbitrary FP32 values,
// so the hardware's power-of-two block scaling cannot apply them: every 128-K dot leaves the
// tensor core unscaled and is folded into FP32 registers with the reference's exact fma.
//
// One CTA per SM walks 128-token x BN-feature tiles (BN = 256 or 128). Per K group the
// tcgen05.mma sequence (4 x K32, kind::f8f6f4) writes the group's dots into one of TWO
// accumulator buffers in TMEM (2 x BN columns). Eight epilogue warps (two per TMEM lane
// quadrant, BN/2 columns each; registers rebalanced towards them with setmaxnreg) pull group g
// out of one buffer while the tensor core fills the other with group g+1. The running sums stay
// in registers until the tile's last group, then go to shared memory and leave with a TMA
// store, so the next tile's MMAs and folds start while the previous tile drains.
//
// A cta_group::2 variant of this kernel (256-token tiles, half the weight traffic per SM) was
// measured and dropped: the buffer hand-back has to cross CTAs once per K group, and that
// round trip, not operand delivery, set its pace.
#include <cuda.h>
#include <cuda_bf16.h>
#include <algorithm>
#include "host_util.h"
#include "ptx.cuh"

namespace mach {

int make_operand_map(CUtensorMap* map, const void* base, int64_t rows, int64_t k, int format,
                     int box_rows);
int make_bf16_store_map(CUtensorMap* map, const void* base, int64_t rows, int64_t cols,
                        int box_rows);

namespace {

constexpr int kTileRows = 128;
constexpr int kTileK = 128;
constexpr int kABytes = kTileRows * kTileK;
constexpr int kEpiWarps = 8;  // two per TMEM lane quadrant
constexpr int kThreads = (4 + kEpiWarps) * 32;  // warps 0-3: TMA, MMA, two idle; 4-11: epilogue
constexpr int kMaxStages = 8;
constexpr int kAccRegs = 128;      // BN / 2 columns per epilogue warp, BN <= 256
constexpr int kOutBoxCols = 64;    // BF16 columns per TMA store box (128 bytes, 128B swizzle)
constexpr int kOutBoxBytes = kTileRows * kOutBoxCols * 2;

enum { kWaitEmpty = 701, kWaitFull = 702, kWaitAccFull = 703, kWaitAccEmpty = 704 };

struct TmFp8Params {
  const float* sa;  // [K/128][M]
  const float* sb;  // [ceil(N/128)][K/128]
  int* status;
  int m, n, groups;
  int bn, stages;
  int tiles_m, tiles_n, panel_m;
  uint32_t idesc;
};

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}
__device__ __forceinline__ void named_barrier_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
// 2-D tiled store shared -> global (bulk async group of the issuing thread).
__device__ __forceinline__ void tma_store_2d(const void* desc, uint32_t src, int c0, int c1) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(desc)),
               "r"(src), "r"(c0), "r"(c1)
               : "memory");
}
__device__ __forceinline__ void bulk_commit_group() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
// Every bulk store of this thread has finished READING shared memory.
__device__ __forceinline__ void bulk_wait_read_all() {
  asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}
__device__ __forceinline__ void bulk_wait_all() {
  asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}

struct TileCoord {
  int m0, n0;
};
__device__ __forceinline__ TileCoord tile_coord(const TmFp8Params& p, int t) {
  const int per_panel = p.panel_m * p.tiles_n;
  const int panel = t / per_panel;
  const int in_panel = t - panel * per_panel;
  const int rows_here = min(p.panel_m, p.tiles_m - panel * p.panel_m);
  TileCoord c;
  c.m0 = (panel * p.panel_m + in_panel % rows_here) * kTileRows;
  c.n0 = (in_panel / rows_here) * p.bn;
  return c;
}

// acc[32 * c + i] = fma(dot, s, acc) for one 32-column chunk just read from TMEM.
#define MACH_FOLD32(r, c)                                                        \
  _Pragma("unroll") for (int i_ = 0; i_ < 32; ++i_)                              \
      acc[(c) * 32 + i_] = __fmaf_rn(__uint_as_float((r)[i_]), s, acc[(c) * 32 + i_]);

__global__ void __launch_bounds__(kThreads, 1)
block_fp8_tm_kernel(const __grid_constant__ CUtensorMap tm_a,
                    const __grid_constant__ CUtensorMap tm_b,
                    const __grid_constant__ CUtensorMap tm_out, const TmFp8Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int bn = p.bn;
  const int stage_bytes = kABytes + bn * kTileK;  // multiple of 1024
  const int stages = p.stages;
  uint8_t* out_stage = smem + (size_t)stages * stage_bytes;  // bn / 64 boxes of 128 x 64 BF16
  uint64_t* bars = reinterpret_cast<uint64_t*>(out_stage + (bn / kOutBoxCols) * kOutBoxBytes);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kMaxStages + 4);
  const uint32_t full0 = smem_u32(bars);
  const uint32_t empty0 = smem_u32(bars + kMaxStages);
  const uint32_t acc_full0 = smem_u32(bars + 2 * kMaxStages);
  const uint32_t acc_empty0 = smem_u32(bars + 2 * kMaxStages + 2);
  const int num_tiles = p.tiles_m * p.tiles_n;
  const uint32_t tmem_cols = (uint32_t)(2 * bn);

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full0 + 8 * b, 1);
      mbar_init(acc_empty0 + 8 * b, kEpiWarps);
    }
    fence_mbar_init();
    prefetch_tensormap(&tm_a);
    prefetch_tensormap(&tm_b);
    prefetch_tensormap(&tm_out);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (threadIdx.x == 0) pdl_launch_dependents();

  // Register split: an epilogue thread keeps a 128-value running sum plus 64 values in flight
  // from TMEM; the first warpgroup gives its share away. (setmaxnreg sits inside each branch
  // so that the compiler sees one limit per role.)
  if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
    if (warp == 0) {
      // ---- TMA producer
      if (elect_one()) pdl_wait();
      __syncwarp();
      const uint64_t pol = policy_evict_normal();
      const uint32_t base0 = smem_u32(smem);
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        const TileCoord c = tile_coord(p, t);
        for (int g = 0; g < p.groups; ++g) {
          ok = mbar_wait(empty0 + 8 * s, ph ^ 1u, p.status, kWaitEmpty);
          if (!ok) break;
          if (elect_one()) {
            mbar_expect_tx(full0 + 8 * s, (uint32_t)stage_bytes);
            const uint32_t base = base0 + (uint32_t)s * (uint32_t)stage_bytes;
            tma_load_2d(base, &tm_a, full0 + 8 * s, g * kTileK, c.m0, pol);
            tma_load_2d(base + kABytes, &tm_b, full0 + 8 * s, g * kTileK, c.n0, pol);
          }
          __syncwarp();
          if (++s == stages) { s = 0; ph ^= 1u; }
        }
      }
      __syncwarp();
    } else if (warp == 1) {
      // ---- MMA issuer: one accumulator buffer per K group, alternating
      const uint32_t lo_stage0 = (smem_u32(smem) & 0x3FFFF) >> 4;
      const uint32_t lo_step = (uint32_t)stage_bytes >> 4;
      const uint32_t lo_b = (uint32_t)kABytes >> 4;
      int s = 0;
      uint32_t ph = 0;
      uint32_t gi = 0;  // K groups issued so far, over all tiles
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        for (int g = 0; g < p.groups; ++g, ++gi) {
          const uint32_t buf = gi & 1u;
          ok = mbar_wait(acc_empty0 + 8 * buf, ((gi >> 1) & 1u) ^ 1u, p.status, kWaitAccEmpty);
          if (!ok) break;
          ok = mbar_wait(full0 + 8 * s, ph, p.status, kWaitFull);
          if (!ok) break;
          tc_fence_after();
          if (elect_one()) {
            const uint32_t lo = lo_stage0 + (uint32_t)s * lo_step;
            const uint32_t d = tmem_base + buf * (uint32_t)bn;
#pragma unroll
            for (int sub = 0; sub < 4; ++sub)
              tc_mma_f8_lo(d, lo + 2 * sub, lo + lo_b + 2 * sub, p.idesc, sub > 0 ? 1u : 0u);
            tc_commit(empty0 + 8 * s);
            tc_commit(acc_full0 + 8 * buf);
          }
          __syncwarp();
          if (++s == stages) { s = 0; ph ^= 1u; }
        }
      }
      __syncwarp();
    }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 224;");
    // ---- epilogue warps: 32 tokens x BN/2 columns each
    const int ew = warp - 4;
    const int quad = warp & 3;
    const int part = ew >> 2;
    const int half = bn >> 1;  // columns per warp: 128 or 64
    const int row_in_tile = quad * 32 + lane;
    const uint32_t t_lane = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(part * half);
    const bool store_leader = warp == 4 && lane == 0;
    float acc[kAccRegs];
    uint32_t gi = 0;
    bool ok = true;
    pdl_wait();  // the activation scales come from the preceding kernel
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
      const TileCoord c = tile_coord(p, t);
      const int row = c.m0 + row_in_tile;
      const int col0 = c.n0 + part * half;
      const bool live = row < p.m && col0 < p.n;
      const float* sa_row = p.sa + (live ? row : 0);
      const float* sb_row = p.sb + (size_t)((live ? col0 : 0) >> 7) * p.groups;
#pragma unroll
      for (int i = 0; i < kAccRegs; ++i) acc[i] = 0.0f;
      // Scales are fetched two groups ahead and multiplied only when used, so their L2 latency
      // never sits on the per-group path.
      float sa0 = __ldg(sa_row), sb0 = __ldg(sb_row);
      float sa1 = 0.0f, sb1 = 0.0f;
      if (p.groups > 1) {
        sa1 = __ldg(sa_row + (size_t)p.m);
        sb1 = __ldg(sb_row + 1);
      }
      for (int g = 0; g < p.groups; ++g, ++gi) {
        const uint32_t buf = gi & 1u;
        const float sa_cur = sa0, sb_cur = sb0;
        sa0 = sa1;
        sb0 = sb1;
        if (g + 2 < p.groups) {
          sa1 = __ldg(sa_row + (size_t)(g + 2) * p.m);
          sb1 = __ldg(sb_row + g + 2);
        }
        ok = mbar_wait(acc_full0 + 8 * buf, (gi >> 1) & 1u, p.status, kWaitAccFull);
        tc_fence_after();
        if (!ok) break;
        const uint32_t t_acc = t_lane + buf * (uint32_t)bn;
        const float s = __fmul_rn(sa_cur, sb_cur);
        // 64 columns per round trip to TMEM (two x32 loads in flight, one wait); the buffer
        // goes back to the MMA thread as soon as its last values are in registers.
        uint32_t ra[32], rb[32];
#pragma unroll
        for (int h = 0; h < kAccRegs / 64; ++h) {
          if (h * 64 < half) {
            tmem_ld_x32(t_acc + h * 64, ra);
            tmem_ld_x32(t_acc + h * 64 + 32, rb);
            tmem_ld_wait();
            if ((h + 1) * 64 >= half) {
              tc_fence_before();
              __syncwarp();
              if (lane == 0) mbar_arrive(acc_empty0 + 8 * buf);
            }
            MACH_FOLD32(ra, 2 * h)
            MACH_FOLD32(rb, 2 * h + 1)
          }
        }
      }
      // Tile done: BF16 rows into the swizzled staging boxes, then one TMA store per box.
      if (store_leader) bulk_wait_read_all();  // the previous tile's stores have left smem
      named_barrier_sync(1, kEpiWarps * 32);
      if (ok) {
#pragma unroll
        for (int cc = 0; cc < kAccRegs; cc += 8) {
          if (cc < half) {
            const int col = part * half + cc;        // column inside the tile
            const int box = col >> 6;                // 64-column box
            const int chunk = (col & 63) >> 3;       // 16-byte chunk inside the 128-byte row
            uint8_t* dst = out_stage + box * kOutBoxBytes + row_in_tile * 128 +
                           ((chunk ^ (row_in_tile & 7)) << 4);
            *reinterpret_cast<uint4*>(dst) = make_uint4(
                pack_bf16x2(acc[cc], acc[cc + 1]), pack_bf16x2(acc[cc + 2], acc[cc + 3]),
                pack_bf16x2(acc[cc + 4], acc[cc + 5]), pack_bf16x2(acc[cc + 6], acc[cc + 7]));
          }
        }
      }
      fence_proxy_async_smem();
      named_barrier_sync(1, kEpiWarps * 32);
      if (store_leader && ok) {
        for (int box = 0; box < bn / kOutBoxCols; ++box)
          if (c.n0 + box * kOutBoxCols < p.n)
            tma_store_2d(&tm_out, smem_u32(out_stage + box * kOutBoxBytes),
                         c.n0 + box * kOutBoxCols, c.m0);
        bulk_commit_group();
      }
    }
    if (store_leader) bulk_wait_all();  // the last stores are complete before the CTA exits
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, tmem_cols);
  }
}

}  // namespace

// Token-major persistent block-FP8 GEMM; called by the block-FP8 dispatcher for M > 64.
int run_block_fp8_tm(const void* a, const void* b, const float* sa, const float* sb,
                     __nv_bfloat16* out, int64_t m, int64_t n, int64_t k, int bn,
                     cudaStream_t stream) {
  TmFp8Params prm = {};
  prm.sa = sa;
  prm.sb = sb;
  prm.status = device_status_ptr();
  if (!prm.status) return fail(MACH_ERR_CUDA, "block_fp8_gemm: cannot resolve the status word");
  prm.m = (int)m;
  prm.n = (int)n;
  prm.groups = (int)(k / 128);
  prm.bn = bn;
  prm.tiles_m = (int)((m + kTileRows - 1) / kTileRows);
  prm.tiles_n = (int)((n + bn - 1) / bn);
  prm.panel_m = 16;
  prm.idesc = idesc_f8(kFmtE4M3, kFmtE4M3, (uint32_t)bn);
  const int stage_bytes = kABytes + bn * kTileK;
  const int out_bytes = (bn / kOutBoxCols) * kOutBoxBytes;
  const int fixed = out_bytes + (2 * kMaxStages + 4) * 8 + 16 + 1024;
  const int stages = std::min((max_smem_optin() - fixed) / stage_bytes, kMaxStages);
  if (stages < 2) return fail(MACH_ERR_UNSUPPORTED, "block_fp8_gemm: tile does not fit in shared memory");
  prm.stages = stages;
  const int smem_bytes = stages * stage_bytes + fixed;
  CUtensorMap tm_a, tm_b, tm_out;
  int rc = make_operand_map(&tm_a, a, m, k, MACH_FMT_E4M3, kTileRows);
  if (rc) return rc;
  rc = make_operand_map(&tm_b, b, n, k, MACH_FMT_E4M3, bn);
  if (rc) return rc;
  rc = make_bf16_store_map(&tm_out, out, m, n, kTileRows);
  if (rc) return rc;

  auto kernel = block_fp8_tm_kernel;
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
  const int ctas = std::max(1, std::min(prm.tiles_m * prm.tiles_n, sm_count()));
  const cudaError_t e = launch_ex(kernel, dim3((unsigned)ctas), dim3(kThreads), (size_t)smem_bytes,
                                  stream, dim3(1, 1, 1), pdl_enabled(), tm_a, tm_b, tm_out, prm);
  if (e != cudaSuccess) return fail(MACH_ERR_CUDA, "block_fp8_gemm launch: %s", cudaGetErrorString(e));
  return MACH_OK;
}

}  // namespace mach
