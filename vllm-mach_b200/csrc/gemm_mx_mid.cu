// Token-major block-scaled GEMM for one token tile (M <= 128) and a wide weight matrix:
// one CTA per SM, every CTA one tile of 128 tokens x a BALANCED share of the weight rows.
//
// Between the decode batches (feature-major kernel, tokens on the MMA N side) and the 256-token
// persistent kernels there is a range where the weights are still read once and the batch fills
// one 128-row MMA. There the time is the weight stream plus one tile's MMAs, and what decides
// it is how evenly the weight rows spread over the SMs: uniform tiles of 192 or 256 rows of a
// 38912-row gate_up matrix give 203 or 152 tiles for 148 SMs - two rounds. This kernel cuts the
// weight rows into groups of 64 (one gate/up group of the interleaved layout, and the even
// scale-column rule of the MMA) and gives CTA i the groups [i * G / C, (i + 1) * G / C): every
// SM gets 4 or 5 groups and there is one round.
//
//   warp 0      TMA producer (no multicast): activations 128 x 128 B, weights as 64-row boxes
//   warp 1      TMEM owner + MMA issuer: one or two tcgen05.mma per 32-K sub-step (N <= 256 each)
//   warps 2..17 epilogue, four per TMEM lane quadrant: BF16 rows, or SwiGLU + MXFP8 requant
//
// The weights do not depend on the preceding kernel, so with programmatic dependent launch the
// ring is filled with weight boxes before griddepcontrol.wait.
#include <cuda.h>
#include <cuda_bf16.h>
#include <algorithm>
#include "gemm_mx_tm.h"
#include "host_util.h"
#include "ptx.cuh"
#include "quant_math.cuh"

namespace mach {

int make_operand_map(CUtensorMap* map, const void* base, int64_t rows, int64_t k, int format,
                     int box_rows);

namespace {

constexpr int kRows = 128;            // tokens per tile
constexpr int kTileK = 128;
constexpr int kABytes = kRows * kTileK;
constexpr int kGroupRows = 64;        // weight rows per group
constexpr int kGroupBytes = kGroupRows * kTileK;
constexpr int kMaxGroups = 7;         // 448 accumulator columns + scale columns <= 512
constexpr int kSfAtom = 512;
constexpr int kMaxBAtoms = 4;
constexpr int kEpiWarps = 16;
constexpr int kThreads = (2 + kEpiWarps) * 32;
constexpr int kMaxStages = 8;
constexpr int kSfCols = 4 + 4 * kMaxBAtoms;      // TMEM columns of the scale factors

enum { kWaitEmpty = 801, kWaitFull = 802, kWaitAccum = 803 };

struct MidParams {
  const uint8_t* sf_a;
  const uint8_t* sf_b;
  void* out;
  uint8_t* out_sf;
  int* status;
  int m, n_rows, n_out;      // tokens; physical weight rows; row length of the output
  int k, k_tiles, out_k_tiles;
  int groups;                // ceil(n_rows / 64)
  int max_groups;            // most groups any CTA owns (sizes the stage)
  int stages;
  int tmem_cols;             // power of two >= 64 * max_groups + scale columns
  int b_atoms_total;
  int interleaved;           // plain epilogue: weight rows are gate/up interleaved by 32
  int w_row_tx;              // transaction bytes per weight row and K step (128; packed 6-bit: 96)
  uint32_t idesc_base;       // instruction descriptor with N = 0
};

__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}
__device__ __forceinline__ uint32_t with_n(uint32_t idesc, int n) {
  return idesc | ((uint32_t)(n >> 3) << 17);
}

template <bool kSwiglu>
__global__ void __launch_bounds__(kThreads, 1)
mx_gemm_mid_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                   const MidParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // ---- this CTA's share of the weight rows
  const int g_begin = (int)(((long long)blockIdx.x * p.groups) / gridDim.x);
  const int g_end = (int)(((long long)(blockIdx.x + 1) * p.groups) / gridDim.x);
  const int my_groups = g_end - g_begin;
  const int n0 = g_begin * kGroupRows;
  const int bn = my_groups * kGroupRows;
  const int bn_a = min(bn, 256);
  const int bn_b = bn - bn_a;
  const int atom0 = n0 >> 7;
  const int atoms = min((n0 + bn - 1) >> 7, p.b_atoms_total - 1) - atom0 + 1;

  const int sf_off = kABytes + p.max_groups * kGroupBytes;
  const int stage_bytes = (sf_off + (1 + kMaxBAtoms) * kSfAtom + 1023) & ~1023;
  const int stages = p.stages;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)stages * stage_bytes);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kMaxStages + 1);
  const uint32_t full0 = smem_u32(bars);
  const uint32_t empty0 = smem_u32(bars + kMaxStages);
  const uint32_t accum_bar = smem_u32(bars + 2 * kMaxStages);

  // TMEM plan: [accumulator : 64 * max_groups][SFA : 4][SFB : 16]
  const int sfa_col = p.max_groups * kGroupRows;
  const int sfb_col = sfa_col + 4;

  // Warp 0 initialises the barriers and starts streaming weights at once: neither needs the
  // TMEM allocation, and a CTA that became resident under the tail of the preceding kernel
  // (programmatic dependent launch) uses that time to fill its ring.
  const uint32_t base0 = smem_u32(smem);
  const uint32_t tx = (uint32_t)(kABytes + bn * p.w_row_tx + (1 + atoms) * kSfAtom);
  const int pre = min(stages, p.k_tiles);
  uint64_t pol_w = 0;
  if (warp == 0) {
    pol_w = policy_evict_first();
    if (lane == 0) {
      for (int s = 0; s < stages; ++s) {
        mbar_init(full0 + 8 * s, 1);
        mbar_init(empty0 + 8 * s, 1);
      }
      mbar_init(accum_bar, 1);
      fence_mbar_init();
      prefetch_tensormap(&tm_a);
      prefetch_tensormap(&tm_b);
      for (int it = 0; it < pre; ++it) {
        const uint32_t full = full0 + 8 * it;
        const uint32_t base = base0 + (uint32_t)(it * stage_bytes);
        mbar_expect_tx(full, tx);
        for (int g = 0; g < my_groups; ++g)
          tma_load_2d(base + kABytes + g * kGroupBytes, &tm_b, full, it * kTileK,
                      n0 + g * kGroupRows, pol_w);
        for (int j = 0; j < atoms; ++j)
          bulk_load_1d(base + sf_off + (1 + j) * kSfAtom,
                       p.sf_b + ((size_t)(atom0 + j) * p.k_tiles + it) * kSfAtom, kSfAtom, full);
      }
    }
    __syncwarp();
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
    const uint64_t pol_a = policy_evict_last();
    auto load_w = [&](int kb, uint32_t base, uint32_t full) {
      for (int g = 0; g < my_groups; ++g)
        tma_load_2d(base + kABytes + g * kGroupBytes, &tm_b, full, kb * kTileK,
                    n0 + g * kGroupRows, pol_w);
      for (int j = 0; j < atoms; ++j)
        bulk_load_1d(base + sf_off + (1 + j) * kSfAtom,
                     p.sf_b + ((size_t)(atom0 + j) * p.k_tiles + kb) * kSfAtom, kSfAtom, full);
    };
    auto load_a = [&](int kb, uint32_t base, uint32_t full) {
      tma_load_2d(base, &tm_a, full, kb * kTileK, 0, pol_a);
      bulk_load_1d(base + sf_off, p.sf_a + (size_t)kb * kSfAtom, kSfAtom, full);
    };
    if (elect_one()) {
      pdl_wait();  // the activations come from the preceding kernel
      for (int it = 0; it < pre; ++it)
        load_a(it, base0 + (uint32_t)(it * stage_bytes), full0 + 8 * it);
    }
    __syncwarp();
    int s = pre % stages;
    uint32_t ph = (pre == stages) ? 1u : 0u;
    for (int kb = pre; kb < p.k_tiles; ++kb) {
      if (!mbar_wait(empty0 + 8 * s, ph ^ 1u, p.status, kWaitEmpty)) break;
      if (elect_one()) {
        const uint32_t full = full0 + 8 * s;
        mbar_expect_tx(full, tx);
        const uint32_t base = base0 + (uint32_t)(s * stage_bytes);
        load_a(kb, base, full);
        load_w(kb, base, full);
      }
      __syncwarp();
      if (++s == stages) { s = 0; ph ^= 1u; }
    }
  } else if (warp == 1) {
    // =============================== MMA issuer (warp-uniform loop, one elected lane issues)
    const int k_rem = p.k - (p.k_tiles - 1) * kTileK;
    const int last_subs = k_rem >> 5;
    uint32_t idesc_a[4], idesc_b[4];
#pragma unroll
    for (int sub = 0; sub < 4; ++sub) {
      idesc_a[sub] = idesc_mx_sf(with_n(p.idesc_base, bn_a), (uint32_t)sub, (uint32_t)sub);
      idesc_b[sub] = idesc_mx_sf(with_n(p.idesc_base, max(bn_b, 16)), (uint32_t)sub, (uint32_t)sub);
    }
    const uint32_t lo_stage0 = desc_lo(smem_u32(smem));
    const uint32_t lo_step = (uint32_t)stage_bytes >> 4;
    const uint32_t lo_b = (uint32_t)kABytes >> 4;
    const uint32_t lo_b2 = (uint32_t)(kABytes + 256 * kTileK) >> 4;
    const uint32_t lo_sf = (uint32_t)sf_off >> 4;
    const uint32_t sfa_tmem = tmem_base + sfa_col;
    const uint32_t sfb_tmem = tmem_base + sfb_col + ((n0 & 127) >> 5);
    const uint32_t sfb_tmem2 = sfb_tmem + (256 >> 5);
    const bool two = bn_b > 0;
    int s = 0;
    uint32_t ph = 0;
    for (int kb = 0; kb < p.k_tiles; ++kb) {
      if (!mbar_wait(full0 + 8 * s, ph, p.status, kWaitFull)) break;
      tc_fence_after();
      if (elect_one()) {
        const uint32_t lo = lo_stage0 + (uint32_t)s * lo_step;
        tc_cp_sf_lo(sfa_tmem, lo + lo_sf);
        for (int j = 0; j < atoms; ++j)
          tc_cp_sf_lo(tmem_base + sfb_col + 4 * j, lo + lo_sf + 32u * (uint32_t)(1 + j));
        uint32_t acc = kb > 0 ? 1u : 0u;
        const int subs = (kb + 1 < p.k_tiles) ? 4 : last_subs;
        if (subs == 4) {
#pragma unroll
          for (int sub = 0; sub < 4; ++sub) {
            tc_mma_mx_lo(tmem_base, lo + 2 * sub, lo + lo_b + 2 * sub, idesc_a[sub], acc, sfa_tmem,
                         sfb_tmem);
            if (two)
              tc_mma_mx_lo(tmem_base + 256, lo + 2 * sub, lo + lo_b2 + 2 * sub, idesc_b[sub], acc,
                           sfa_tmem, sfb_tmem2);
            acc = 1;
          }
        } else {
          for (int sub = 0; sub < subs; ++sub) {
            tc_mma_mx_lo(tmem_base, lo + 2 * sub, lo + lo_b + 2 * sub, idesc_a[sub], acc, sfa_tmem,
                         sfb_tmem);
            if (two)
              tc_mma_mx_lo(tmem_base + 256, lo + 2 * sub, lo + lo_b2 + 2 * sub, idesc_b[sub], acc,
                           sfa_tmem, sfb_tmem2);
            acc = 1;
          }
        }
        tc_commit(empty0 + 8 * s);
      }
      __syncwarp();
      if (++s == stages) { s = 0; ph ^= 1u; }
    }
    if (elect_one()) tc_commit(accum_bar);
    __syncwarp();
  } else {
    // =============================== epilogue warps
    const int quad = warp & 3;
    const int part = (warp - 2) >> 2;  // which of the warps sharing the lane quadrant
    constexpr int kParts = kEpiWarps / 4;
    const uint32_t t_lane = tmem_base + ((uint32_t)(quad * 32) << 16);
    const bool ready = mbar_wait(accum_bar, 0, p.status, kWaitAccum);
    tc_fence_after();
    const int row = quad * 32 + lane;
    if (!kSwiglu) {
      __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.out);
      for (int ch = part; ch * 32 < bn; ch += kParts) {
        uint32_t r[32];
        tmem_ld_x32(t_lane + ch * 32, r);
        tmem_ld_wait();
        const int n_phys = n0 + ch * 32;
        int n = n_phys;
        if (p.interleaved)
          n = ((n_phys >> 5) & 1) * (p.n_rows >> 1) + ((n_phys >> 6) << 5);
        if (ready && row < p.m && n_phys < p.n_rows) {
          uint32_t w[16];
#pragma unroll
          for (int i = 0; i < 16; ++i)
            w[i] = pack2(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
          uint4* dst = reinterpret_cast<uint4*>(out + (size_t)row * p.n_out + n);
          dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
          dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
          if (n_phys + 16 < p.n_rows) {  // N % 16 == 0: the second half is all in or all out
            dst[2] = make_uint4(w[8], w[9], w[10], w[11]);
            dst[3] = make_uint4(w[12], w[13], w[14], w[15]);
          }
        }
      }
    } else {
      uint8_t* codes = reinterpret_cast<uint8_t*>(p.out);
      for (int g = part; g < my_groups; g += kParts) {
        uint32_t gr[32], ur[32];
        tmem_ld_x32(t_lane + g * 64, gr);
        tmem_ld_x32(t_lane + g * 64 + 32, ur);
        tmem_ld_wait();
        const int feat = (n0 + g * 64) >> 1;
        if (ready && row < p.m && feat < p.n_out) {
          float v[32];
          float amax = 0.0f;
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            v[i] = swiglu_bf16(bf16_round(__uint_as_float(gr[i])), bf16_round(__uint_as_float(ur[i])));
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
    tc_fence_before();
  }

  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, (uint32_t)p.tmem_cols);
  }
}

template <bool kSwiglu>
int launch(const CUtensorMap& tm_a, const CUtensorMap& tm_b, const MidParams& prm, int grid,
           int smem_bytes, cudaStream_t stream) {
  auto kernel = mx_gemm_mid_kernel<kSwiglu>;
  static int configured_smem_dev[kMaxDeviceSlots] = {};  // the attribute is per device
  int& configured_smem = configured_smem_dev[device_slot()];
  if (smem_bytes > configured_smem) {
    const cudaError_t e =
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
    if (e != cudaSuccess)
      return fail(MACH_ERR_CUDA, "mx_gemm_mid: shared memory opt-in failed: %s", cudaGetErrorString(e));
    configured_smem = smem_bytes;
  }
  const cudaError_t e = launch_ex(kernel, dim3((unsigned)grid), dim3(kThreads), (size_t)smem_bytes,
                                  stream, dim3(1, 1, 1), pdl_enabled(), tm_a, tm_b, prm);
  if (e != cudaSuccess) return fail(MACH_ERR_CUDA, "mx_gemm_mid launch: %s", cudaGetErrorString(e));
  return MACH_OK;
}

}  // namespace

// Whether the one-token-tile kernel takes this shape: at most 128 tokens, and enough 64-row
// groups that every SM gets at least one (narrower matrices split K over a cluster instead).
bool mx_gemm_mid_fits(int64_t m, int64_t w_rows) {
  return m >= 1 && m <= kRows && (w_rows + kGroupRows - 1) / kGroupRows >= (int64_t)sm_count();
}

int run_mx_gemm_mid(const TmGemmArgs& a, cudaStream_t stream) {
  MidParams prm = {};
  prm.sf_a = reinterpret_cast<const uint8_t*>(a.a_sf);
  prm.sf_b = reinterpret_cast<const uint8_t*>(a.w_sf);
  prm.out = a.out;
  prm.out_sf = reinterpret_cast<uint8_t*>(a.out_sf);
  prm.status = device_status_ptr();
  if (!prm.status) return fail(MACH_ERR_CUDA, "mx_gemm_mid: cannot resolve the device status word");
  if (a.m > kRows) return fail(MACH_ERR_UNSUPPORTED, "mx_gemm_mid: at most 128 tokens");
  if (a.swiglu && !a.interleaved)
    return fail(MACH_ERR_UNSUPPORTED, "mx_gemm_mid: SwiGLU needs interleaved gate_up rows");
  prm.m = (int)a.m;
  prm.n_rows = (int)a.w_rows;
  prm.n_out = a.swiglu ? (int)(a.w_rows / 2) : (int)a.w_rows;
  prm.k = (int)a.k;
  prm.k_tiles = (int)((a.k + 127) / 128);
  prm.out_k_tiles = (prm.n_out + 127) / 128;
  prm.groups = (int)((a.w_rows + kGroupRows - 1) / kGroupRows);
  prm.b_atoms_total = (int)((a.w_rows + 127) / 128);
  prm.interleaved = a.interleaved ? 1 : 0;
  prm.w_row_tx = a.w_format == MACH_FMT_E4M3 ? 128 : 96;
  prm.idesc_base = idesc_mx(kFmtE4M3, (uint32_t)a.w_format, 0);
  // One round when the groups fit (at most 7 per CTA); otherwise whole rounds of the SM count.
  const int sms = sm_count();
  const int rounds = (prm.groups + kMaxGroups * sms - 1) / (kMaxGroups * sms);
  const int grid = std::min(prm.groups, sms * rounds);
  prm.max_groups = (prm.groups + grid - 1) / grid;
  const int stage_bytes =
      (kABytes + prm.max_groups * kGroupBytes + (1 + kMaxBAtoms) * kSfAtom + 1023) & ~1023;
  const int fixed = (2 * kMaxStages + 1) * 8 + 16 + 1024;
  int cols = 32;
  while (cols < prm.max_groups * kGroupRows + kSfCols) cols <<= 1;
  prm.tmem_cols = cols;
  // The ring takes all of the SM's shared memory. Measured on B200 (19456 x 2560, M = 64..128,
  // graph replay): 20.4 us with five stages against 25.2 us with CTAs of half an SM (two
  // stages), which would let the next kernel's CTAs prefetch beside these.
  int budget = max_smem_optin();
  if (a.smem_cap_kb > 0) budget = std::min(max_smem_optin(), a.smem_cap_kb * 1024);
  int stages = std::min((budget - fixed) / stage_bytes, kMaxStages);
  if (a.stages > 0) stages = std::min(stages, a.stages);
  stages = std::min(stages, prm.k_tiles);
  if (stages < 1) return fail(MACH_ERR_UNSUPPORTED, "mx_gemm_mid: tile does not fit in shared memory");
  prm.stages = stages;
  const int smem_bytes = stages * stage_bytes + fixed;
  CUtensorMap tm_a, tm_b;
  int rc = make_operand_map(&tm_a, a.a_codes, a.m, a.k, MACH_FMT_E4M3, kRows);
  if (rc) return rc;
  rc = make_operand_map(&tm_b, a.w, a.w_rows, a.k, a.w_format, kGroupRows);
  if (rc) return rc;
  return a.swiglu ? launch<true>(tm_a, tm_b, prm, grid, smem_bytes, stream)
                  : launch<false>(tm_a, tm_b, prm, grid, smem_bytes, stream);
}

}  // namespace mach
