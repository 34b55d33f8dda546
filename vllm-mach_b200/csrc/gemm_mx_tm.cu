// Token-major block-scaled GEMM for large batches: persistent CTAs, 256-token x BN-feature
// tiles.
//
// At M >= 512 the tcgen05 pipe is fed from L2, and the L2 -> SM fabric (about 10 TB/s on
// B200) is the bound: a 128 x 256 tile moves 48 KiB per 128-K step. This kernel pairs two
// 128-token operand tiles with one weight tile (two MMAs per K-step share the B operand in
// shared memory), which cuts the bytes per MAC by 1.4x, and it is persistent so the TMA
// producer runs ahead into the next tile while the epilogue drains TMEM.
//
//   warp 0      TMA producer (no multicast)
//   warp 1      TMEM owner + MMA issuer
//   warps 2..9  epilogue: two warps per TMEM lane quadrant, alternating 32-column chunks
//
// TMEM plan (BN = 192): [acc tokens 0..127 : BN][acc tokens 128..255 : BN][SFA x2 : 8]
// [SFB : 12]. Weight scale atoms are 128 rows; a tile copies every atom it touches and points
// the MMA at column (n0 % 128) / 32 of the first. That column must be even (an odd column
// raises a misaligned-address fault), hence tiles start on multiples of 64 rows.
//
// Epilogues: BF16 store, or SwiGLU + MXFP8 requant for gate_up weights whose rows are
// interleaved in groups of 32 ([32 gate | 32 up | 32 gate | ...], see
// mach_mx_interleave_gate_up): every 64 accumulator columns hold the gate and up values of
// the same 32 features.
#include <cuda.h>
#include <cuda_bf16.h>
#include "gemm_mx_tm.h"
#include "host_util.h"
#include "ptx.cuh"
#include "quant_math.cuh"

namespace mach {

int make_operand_map(CUtensorMap* map, const void* base, int64_t rows, int64_t k, int format,
                     int box_rows);

namespace {

constexpr int kHalfRows = 128;
constexpr int kTileK = 128;
constexpr int kHalfBytes = kHalfRows * kTileK;
constexpr int kSfAtom = 512;
constexpr int kThreads = 320;
constexpr int kEpiWarps = 8;
constexpr int kMaxStages = 8;
constexpr int kMaxBAtoms = 3;

enum { kWaitEmpty = 301, kWaitFull = 302, kWaitAccFull = 303, kWaitAccEmpty = 304 };

struct TmParams {
  const uint8_t* sf_a;
  const uint8_t* sf_b;
  void* out;
  uint8_t* out_sf;
  int* status;
  int m, n_rows;       // tokens; physical weight rows (plain: N, SwiGLU: 2I)
  int n_out;           // row length of the output (plain: N, SwiGLU: I)
  int k, k_tiles, out_k_tiles;
  int bn, stages;
  int tiles_m, tiles_n, panel_m;
  int b_atoms_total;   // ceil(n_rows / 128)
  int interleaved;     // plain epilogue: weight rows are gate/up interleaved by 32
  int b_tx_bytes;      // transaction bytes of one weight box (packed 6-bit rows count 96 B)
  int tmem_cols;
  uint32_t idesc;
};

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

struct TileCoord {
  int m0, n0;
};
__device__ __forceinline__ TileCoord tile_coord(const TmParams& p, int t) {
  const int per_panel = p.panel_m * p.tiles_n;
  const int panel = t / per_panel;
  const int in_panel = t - panel * per_panel;
  const int rows_here = min(p.panel_m, p.tiles_m - panel * p.panel_m);
  TileCoord c;
  c.m0 = (panel * p.panel_m + in_panel % rows_here) * 2 * kHalfRows;
  c.n0 = (in_panel / rows_here) * p.bn;
  return c;
}

template <bool kSwiglu>
__global__ void __launch_bounds__(kThreads, 1)
mx_gemm_tm_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                  const TmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int bn = p.bn;
  const int b_bytes = bn * kTileK;
  const int sf_off = 2 * kHalfBytes + b_bytes;
  const int stage_bytes = (sf_off + (2 + kMaxBAtoms) * kSfAtom + 1023) & ~1023;
  const int stages = p.stages;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)stages * stage_bytes);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kMaxStages + 2);
  const uint32_t full0 = smem_u32(bars);
  const uint32_t empty0 = smem_u32(bars + kMaxStages);
  const uint32_t acc_full = smem_u32(bars + 2 * kMaxStages);
  const uint32_t acc_empty = smem_u32(bars + 2 * kMaxStages + 1);
  const int num_tiles = p.tiles_m * p.tiles_n;
  const int sfa_col = 2 * bn;
  const int sfb_col = 2 * bn + 8;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    mbar_init(acc_full, 1);
    mbar_init(acc_empty, kEpiWarps);
    fence_mbar_init();
    prefetch_tensormap(&tm_a);
    prefetch_tensormap(&tm_b);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), (uint32_t)p.tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (threadIdx.x == 0) pdl_launch_dependents();

  if (warp == 0) {
    // =============================== TMA producer
    if (lane == 0) {
      pdl_wait();  // the activations come from the preceding kernel
      const uint64_t pol = policy_evict_normal();
      int it = 0;
      for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
        const TileCoord c = tile_coord(p, t);
        const int halves = (c.m0 + kHalfRows < p.m) ? 2 : 1;
        const int atom0 = c.n0 >> 7;
        const int atoms = min(((c.n0 + bn - 1) >> 7), p.b_atoms_total - 1) - atom0 + 1;
        const uint32_t tx =
            (uint32_t)(halves * (kHalfBytes + kSfAtom) + p.b_tx_bytes + atoms * kSfAtom);
        bool ok = true;
        for (int kb = 0; kb < p.k_tiles && ok; ++kb, ++it) {
          const int s = it % stages;
          const uint32_t ph = (uint32_t)(it / stages) & 1u;
          ok = mbar_wait(empty0 + 8 * s, ph ^ 1u, p.status, kWaitEmpty);
          if (!ok) break;
          const uint32_t full = full0 + 8 * s;
          mbar_expect_tx(full, tx);
          const uint32_t base = smem_u32(smem + (size_t)s * stage_bytes);
          const int k0 = kb * kTileK;
          for (int h = 0; h < halves; ++h) {
            tma_load_2d(base + h * kHalfBytes, &tm_a, full, k0, c.m0 + h * kHalfRows, pol);
            bulk_load_1d(base + sf_off + h * kSfAtom,
                         p.sf_a + ((size_t)((c.m0 >> 7) + h) * p.k_tiles + kb) * kSfAtom, kSfAtom,
                         full);
          }
          tma_load_2d(base + 2 * kHalfBytes, &tm_b, full, k0, c.n0, pol);
          for (int j = 0; j < atoms; ++j)
            bulk_load_1d(base + sf_off + (2 + j) * kSfAtom,
                         p.sf_b + ((size_t)(atom0 + j) * p.k_tiles + kb) * kSfAtom, kSfAtom, full);
        }
        if (!ok) break;
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // =============================== MMA issuer
    if (lane == 0) {
      const int k_rem = p.k - (p.k_tiles - 1) * kTileK;
      int it = 0, tile_i = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++tile_i) {
        const TileCoord c = tile_coord(p, t);
        const int halves = (c.m0 + kHalfRows < p.m) ? 2 : 1;
        const int atom0 = c.n0 >> 7;
        const int atoms = min(((c.n0 + bn - 1) >> 7), p.b_atoms_total - 1) - atom0 + 1;
        const uint32_t sfb_tmem = tmem_base + sfb_col + ((c.n0 & 127) >> 5);
        ok = mbar_wait(acc_empty, ((uint32_t)tile_i & 1u) ^ 1u, p.status, kWaitAccEmpty);
        if (!ok) break;
        tc_fence_after();
        for (int kb = 0; kb < p.k_tiles; ++kb, ++it) {
          const int s = it % stages;
          const uint32_t ph = (uint32_t)(it / stages) & 1u;
          ok = mbar_wait(full0 + 8 * s, ph, p.status, kWaitFull);
          if (!ok) break;
          tc_fence_after();
          const uint32_t base = smem_u32(smem + (size_t)s * stage_bytes);
          for (int h = 0; h < halves; ++h)
            tc_cp_32x128b_warpx4(tmem_base + sfa_col + 4 * h,
                                 smem_desc_sf(base + sf_off + h * kSfAtom));
          for (int j = 0; j < atoms; ++j)
            tc_cp_32x128b_warpx4(tmem_base + sfb_col + 4 * j,
                                 smem_desc_sf(base + sf_off + (2 + j) * kSfAtom));
          const int nsub = (kb == p.k_tiles - 1) ? (k_rem >> 5) : 4;
          const uint64_t bdesc = smem_desc_k_sw128(base + 2 * kHalfBytes);
          for (int sub = 0; sub < nsub; ++sub) {
            const uint32_t idesc = idesc_mx_sf(p.idesc, (uint32_t)sub, (uint32_t)sub);
            for (int h = 0; h < halves; ++h)
              tc_mma_mx(tmem_base + h * bn, smem_desc_k_sw128(base + h * kHalfBytes) + 2 * sub,
                        bdesc + 2 * sub, idesc, (kb > 0 || sub > 0) ? 1u : 0u,
                        tmem_base + sfa_col + 4 * h, sfb_tmem);
          }
          tc_commit(empty0 + 8 * s);
        }
        if (ok) tc_commit(acc_full);
      }
    }
    __syncwarp();
  } else {
    // =============================== epilogue warps
    const int ew = warp - 2;      // 0..7
    const int quad = warp & 3;    // TMEM lane quadrant this warp may read
    const int part = ew >> 2;     // which of the two warps sharing the quadrant
    const uint32_t t_lane = tmem_base + ((uint32_t)(quad * 32) << 16);
    int tile_i = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++tile_i) {
      const TileCoord c = tile_coord(p, t);
      const int halves = (c.m0 + kHalfRows < p.m) ? 2 : 1;
      ok = mbar_wait(acc_full, (uint32_t)tile_i & 1u, p.status, kWaitAccFull);
      tc_fence_after();
      if (!ok) break;
      for (int h = 0; h < halves; ++h) {
        const int row = c.m0 + h * kHalfRows + quad * 32 + lane;
        if (!kSwiglu) {
          __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.out);
          for (int ch = part; ch * 32 < bn; ch += 2) {
            uint32_t r[32];
            tmem_ld_x32(t_lane + h * bn + ch * 32, r);
            tmem_ld_wait();
            const int n_phys = c.n0 + ch * 32;
            if (row < p.m && n_phys < p.n_rows) {
              // Interleaved gate_up rows: physical 32-row group g holds gate (g even) or up
              // (g odd) of features (g/2)*32..; logical column = is_up * I + feature.
              int n = n_phys;
              if (p.interleaved) n = ((n_phys >> 5) & 1) * (p.n_rows >> 1) + ((n_phys >> 6) << 5);
              uint32_t w[16];
#pragma unroll
              for (int i = 0; i < 16; ++i)
                w[i] = pack_bf16x2(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
              uint4* dst = reinterpret_cast<uint4*>(out + (size_t)row * p.n_out + n);
              dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
              dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
              if (n_phys + 32 <= p.n_rows) {
                dst[2] = make_uint4(w[8], w[9], w[10], w[11]);
                dst[3] = make_uint4(w[12], w[13], w[14], w[15]);
              }
            }
          }
        } else {
          uint8_t* codes = reinterpret_cast<uint8_t*>(p.out);
          for (int g = part; g * 64 < bn; g += 2) {
            uint32_t gr[32], ur[32];
            tmem_ld_x32(t_lane + h * bn + g * 64, gr);
            tmem_ld_x32(t_lane + h * bn + g * 64 + 32, ur);
            tmem_ld_wait();
            const int feat = ((c.n0 + g * 64) >> 1);  // first of 32 features
            if (row < p.m && feat < p.n_out) {
              float v[32];
              float amax = 0.0f;
#pragma unroll
              for (int i = 0; i < 32; ++i) {
                v[i] = swiglu_bf16(bf16_round(__uint_as_float(gr[i])),
                                   bf16_round(__uint_as_float(ur[i])));
                amax = fmaxf(amax, fabsf(v[i]));
              }
              const uint32_t bits = mx_scale_bits(amax);
              const float inv = mx_inverse(bits);
              uint32_t w[8];
#pragma unroll
              for (int i = 0; i < 8; ++i)
                w[i] = e4m3x4(__fmul_rn(v[4 * i], inv), __fmul_rn(v[4 * i + 1], inv),
                              __fmul_rn(v[4 * i + 2], inv), __fmul_rn(v[4 * i + 3], inv));
              uint4* dst = reinterpret_cast<uint4*>(codes + (size_t)row * p.n_out + feat);
              dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
              dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
              p.out_sf[sf_offset(row, feat >> 5, p.out_k_tiles)] = (uint8_t)(bits >> 23);
            }
          }
        }
      }
      // Every TMEM read of this warp has completed (tmem_ld_wait): hand the accumulator back.
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, (uint32_t)p.tmem_cols);
  }
}

template <bool kSwiglu>
int launch(const CUtensorMap& tm_a, const CUtensorMap& tm_b, const TmParams& prm, int grid,
           int smem_bytes, cudaStream_t stream) {
  auto kernel = mx_gemm_tm_kernel<kSwiglu>;
  static int configured_smem_dev[kMaxDeviceSlots] = {};  // the attribute is per device
  int& configured_smem = configured_smem_dev[device_slot()];
  if (smem_bytes > configured_smem) {
    const cudaError_t e =
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
    if (e != cudaSuccess)
      return fail(MACH_ERR_CUDA, "mx_gemm_tm: shared memory opt-in failed: %s",
                  cudaGetErrorString(e));
    configured_smem = smem_bytes;
  }
  const cudaError_t e = launch_ex(kernel, dim3((unsigned)grid), dim3(kThreads), (size_t)smem_bytes,
                                  stream, dim3(1, 1, 1), pdl_enabled(), tm_a, tm_b, prm);
  if (e != cudaSuccess) return fail(MACH_ERR_CUDA, "mx_gemm_tm launch: %s", cudaGetErrorString(e));
  return MACH_OK;
}

}  // namespace

int run_mx_gemm_tm(const TmGemmArgs& a, cudaStream_t stream) {
  TmParams prm = {};
  prm.sf_a = reinterpret_cast<const uint8_t*>(a.a_sf);
  prm.sf_b = reinterpret_cast<const uint8_t*>(a.w_sf);
  prm.out = a.out;
  prm.out_sf = reinterpret_cast<uint8_t*>(a.out_sf);
  prm.status = device_status_ptr();
  if (!prm.status) return fail(MACH_ERR_CUDA, "mx_gemm_tm: cannot resolve the device status word");
  prm.m = (int)a.m;
  prm.n_rows = (int)a.w_rows;
  prm.n_out = a.swiglu ? (int)(a.w_rows / 2) : (int)a.w_rows;
  prm.k = (int)a.k;
  prm.k_tiles = (int)((a.k + 127) / 128);
  prm.out_k_tiles = (prm.n_out + 127) / 128;
  prm.bn = a.bn;
  prm.interleaved = a.interleaved ? 1 : 0;
  prm.tiles_m = (int)((a.m + 255) / 256);
  prm.tiles_n = (int)((a.w_rows + a.bn - 1) / a.bn);
  prm.panel_m = a.panel_m > 0 ? a.panel_m : 8;
  prm.b_atoms_total = (int)((a.w_rows + 127) / 128);
  int cols = 32;
  while (cols < 2 * a.bn + 8 + 4 * kMaxBAtoms) cols <<= 1;
  // The MMA takes its B scale factors from an even TMEM column, so tiles start on 64 rows.
  if (cols > 512 || a.bn % 64 || a.bn < 64)
    return fail(MACH_ERR_UNSUPPORTED, "mx_gemm_tm: unsupported tile width %d", a.bn);
  prm.tmem_cols = cols;
  prm.idesc = idesc_mx(kFmtE4M3, (uint32_t)a.w_format, (uint32_t)a.bn);
  prm.b_tx_bytes = a.bn * (a.w_format == MACH_FMT_E4M3 ? 128 : 96);
  const int stage_bytes =
      (2 * kHalfBytes + a.bn * kTileK + (2 + kMaxBAtoms) * kSfAtom + 1023) & ~1023;
  const int fixed = (2 * kMaxStages + 2) * 8 + 16 + 1024;
  int stages = (max_smem_optin() - fixed) / stage_bytes;
  stages = std::min(stages, kMaxStages);
  if (a.stages > 0) stages = std::min(stages, a.stages);
  if (stages < 2) return fail(MACH_ERR_UNSUPPORTED, "mx_gemm_tm: tile does not fit in shared memory");
  prm.stages = stages;
  const int smem_bytes = stages * stage_bytes + fixed;
  CUtensorMap tm_a, tm_b;
  int rc = make_operand_map(&tm_a, a.a_codes, a.m, a.k, MACH_FMT_E4M3, kHalfRows);
  if (rc) return rc;
  rc = make_operand_map(&tm_b, a.w, a.w_rows, a.k, a.w_format, a.bn);
  if (rc) return rc;
  const int grid = std::min(prm.tiles_m * prm.tiles_n, sm_count());
  return a.swiglu ? launch<true>(tm_a, tm_b, prm, grid, smem_bytes, stream)
                  : launch<false>(tm_a, tm_b, prm, grid, smem_bytes, stream);
}

}  // namespace mach
