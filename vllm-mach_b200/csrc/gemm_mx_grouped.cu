// Grouped (MoE expert) block-scaled GEMM: for every work item (expert, first routed row,
// rows) and every 128-feature tile of that expert's weight,
//     out[row, feature] = dq(A[row, :]) . dq(W_expert[feature, :])
// over expert-major permuted activations. Feature-major orientation: the expert's weight
// rows are the 128-row MMA operand (streamed once from HBM, the dominant traffic of MoE
// layers up to thousands of tokens), the routed rows are the MMA N operand (runtime N =
// rows rounded up to 16). The work list comes from mach_moe_route on the device, so CTAs
// beyond the live count leave immediately and the host never synchronises.
//
// Epilogues: BF16 rows (W2 / down), or SwiGLU + MXFP8 requant for W1 whose gate/up rows are
// interleaved in groups of 32 (codes and swizzled scales in permuted row order, ready to be
// the next grouped GEMM's A operand). Replaces grouped_gemm_w6a8_out and
// silu_and_mul_mxfp8_grouped (src/vllm_mach/mxfp6/moe_utils.py:205-282, 392-394).
#include <cuda.h>
#include <cuda_bf16.h>
#include "host_util.h"
#include "ptx.cuh"
#include "quant_math.cuh"

namespace mach {

int make_operand_map(CUtensorMap* map, const void* base, int64_t rows, int64_t k, int format,
                     int box_rows);
int tuned_moe_ctas_per_sm();
int tuned_moe_token_major();
int tuned_moe_tm_min_rows();

namespace {

constexpr int kTileRows = 128;
constexpr int kTileK = 128;
constexpr int kTileBytes = kTileRows * kTileK;
constexpr int kSfAtom = 512;
constexpr int kThreads = 192;
constexpr int kMaxStages = 12;
constexpr int kXchCols = 32;
constexpr int kXchBytes = kTileRows * kXchCols * 4;

enum { kWaitEmpty = 501, kWaitFull = 502, kWaitAccFull = 503, kWaitAccEmpty = 504 };

struct GroupedParams {
  const uint8_t* sf_w;
  const uint8_t* sf_a;
  void* out;
  uint8_t* out_sf;
  const int* work;
  const int* num_work;
  int* status;
  int w_rows;        // weight rows per expert (N, or 2I for gate_up)
  int n_out;         // output row length (N, or I with SwiGLU)
  int k, k_tiles, out_k_tiles;
  int tiles_n;       // w_rows / 128
  int box_rows;      // rows of one activation TMA box = rows per work item at most
  int stages, tmem_cols;
  int bufs;          // accumulator buffers in TMEM (2 when 2 * box_rows + scale columns fit)
  int w_atoms_total; // scale atoms of the stacked weight matrix
  int work_cap, rows_cap, experts;  // bounds the device-side work list is checked against
  int rows_min, rows_max;  // this launch handles the work items with rows_min <= rows <= rows_max
  uint32_t w_fmt;
  int w_row_tx;      // transaction bytes per weight row per K step (128, packed 6-bit: 96)
};

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}
__device__ __forceinline__ void named_barrier_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// Decoded work unit: one (expert, row chunk) item x one 128-feature tile of the expert.
struct Unit {
  int nt, row0, rows, n_mma, w_row, a_atom0, a_atoms;
};
__device__ __forceinline__ Unit decode_unit(const GroupedParams& p, int u) {
  Unit x;
  const int item = u / p.tiles_n;
  x.nt = u - item * p.tiles_n;
  const int expert = __ldg(p.work + 3 * item);
  x.row0 = __ldg(p.work + 3 * item + 1);
  x.rows = __ldg(p.work + 3 * item + 2);
  x.n_mma = (x.rows + 15) & ~15;
  x.w_row = expert * p.w_rows + x.nt * kTileRows;  // row in the stacked weight matrix
  x.a_atom0 = x.row0 >> 7;
  x.a_atoms = ((x.row0 + x.n_mma - 1) >> 7) - x.a_atom0 + 1;  // 1 or 2
  // A work list that did not come from mach_moe_route (or was never written) must not steer
  // loads or stores out of bounds: such items read as "not mine" everywhere.
  if (expert < 0 || expert >= p.experts || x.row0 < 0 || x.rows < 1 || x.rows > p.box_rows ||
      x.row0 + x.rows > p.rows_cap)
    x.rows = -1;
  return x;
}

// Persistent: each CTA walks units u = blockIdx.x, blockIdx.x + gridDim.x, ... of the device-side
// work list. The accumulator is double-buffered in TMEM (when 2 * box_rows columns fit), so the
// epilogue of one unit overlaps the weight stream of the next, and the operand ring keeps
// running across unit boundaries.
template <bool kSwiglu>
__global__ void __launch_bounds__(kThreads, 1)
mx_grouped_gemm_kernel(const __grid_constant__ CUtensorMap tm_w,
                       const __grid_constant__ CUtensorMap tm_a, const GroupedParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int a_bytes = p.box_rows * kTileK;
  const int sf_off = kTileBytes + a_bytes;
  const int stage_bytes = (sf_off + 3 * kSfAtom + 1023) & ~1023;
  const int stages = p.stages;
  float* xch = reinterpret_cast<float*>(smem + (size_t)stages * stage_bytes);
  uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(xch) + kXchBytes);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kMaxStages + 4);
  const uint32_t full0 = smem_u32(bars);
  const uint32_t empty0 = smem_u32(bars + kMaxStages);
  const uint32_t acc_full0 = smem_u32(bars + 2 * kMaxStages);
  const uint32_t acc_empty0 = smem_u32(bars + 2 * kMaxStages + 2);
  const int acc_cols = p.box_rows;
  const int bufs = p.bufs;
  const int sfw_col = bufs * acc_cols;
  const int sfa_col = sfw_col + 4;

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
    prefetch_tensormap(&tm_w);
    prefetch_tensormap(&tm_a);
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
  // The work list, the activations and the output buffers all belong to preceding kernels.
  pdl_wait();
  const int num_units = max(0, min(__ldg(p.num_work), p.work_cap)) * p.tiles_n;

  if (warp == 0) {
    // TMA producer: warp-uniform loop, one elected lane issues.
    const uint64_t pol_w = policy_evict_first();
    const uint64_t pol_a = policy_evict_last();
    const uint32_t base0 = smem_u32(smem);
    int s = 0;
    uint32_t ph = 0;
    bool ok = true;
    for (int u = blockIdx.x; u < num_units && ok; u += gridDim.x) {
      const Unit x = decode_unit(p, u);
      if (x.rows < p.rows_min || x.rows > p.rows_max) continue;
      const uint32_t tx_bytes =
          (uint32_t)(kTileRows * p.w_row_tx + a_bytes + (1 + x.a_atoms) * kSfAtom);
      for (int kb = 0; kb < p.k_tiles; ++kb) {
        ok = mbar_wait(empty0 + 8 * s, ph ^ 1u, p.status, kWaitEmpty);
        if (!ok) break;
        if (elect_one()) {
          const uint32_t full = full0 + 8 * s;
          mbar_expect_tx(full, tx_bytes);
          const uint32_t base = base0 + (uint32_t)(s * stage_bytes);
          const int k0 = kb * kTileK;
          tma_load_2d(base, &tm_w, full, k0, x.w_row, pol_w);
          tma_load_2d(base + kTileBytes, &tm_a, full, k0, x.row0, pol_a);
          bulk_load_1d(base + sf_off, p.sf_w + ((size_t)(x.w_row >> 7) * p.k_tiles + kb) * kSfAtom,
                       kSfAtom, full);
          for (int j = 0; j < x.a_atoms; ++j)
            bulk_load_1d(base + sf_off + (1 + j) * kSfAtom,
                         p.sf_a + ((size_t)(x.a_atom0 + j) * p.k_tiles + kb) * kSfAtom, kSfAtom,
                         full);
        }
        __syncwarp();
        if (++s == stages) { s = 0; ph ^= 1u; }
      }
    }
  } else if (warp == 1) {
    // MMA issuer: warp-uniform loop, one elected lane issues.
    const int k_rem = p.k - (p.k_tiles - 1) * kTileK;
    const int last_subs = k_rem >> 5;
    const uint32_t lo_stage0 = desc_lo(smem_u32(smem));
    const uint32_t lo_step = (uint32_t)stage_bytes >> 4;
    const uint32_t lo_a = (uint32_t)kTileBytes >> 4;
    const uint32_t lo_sf = (uint32_t)sf_off >> 4;
    int s = 0;
    uint32_t ph = 0;
    uint32_t ui_next = 0;
    bool ok = true;
    for (int u = blockIdx.x; u < num_units && ok; u += gridDim.x) {
      const Unit x = decode_unit(p, u);
      if (x.rows < p.rows_min || x.rows > p.rows_max) continue;
      const uint32_t ui = ui_next++;
      const uint32_t idesc0 = idesc_mx(p.w_fmt, kFmtE4M3, (uint32_t)x.n_mma);
      uint32_t idesc[4];
#pragma unroll
      for (int sub = 0; sub < 4; ++sub)
        idesc[sub] = idesc_mx_sf(idesc0, (uint32_t)sub, (uint32_t)sub);
      const uint32_t sfa_tmem = tmem_base + sfa_col + ((x.row0 & 127) >> 5);
      const uint32_t buf = bufs == 2 ? (ui & 1u) : 0u;
      const uint32_t use = bufs == 2 ? (ui >> 1) : ui;
      const uint32_t d_tmem = tmem_base + buf * (uint32_t)acc_cols;
      ok = mbar_wait(acc_empty0 + 8 * buf, (use & 1u) ^ 1u, p.status, kWaitAccEmpty);
      if (!ok) break;
      tc_fence_after();
      for (int kb = 0; kb < p.k_tiles; ++kb) {
        ok = mbar_wait(full0 + 8 * s, ph, p.status, kWaitFull);
        if (!ok) break;
        tc_fence_after();
        if (elect_one()) {
          const uint32_t lo = lo_stage0 + (uint32_t)s * lo_step;
          tc_cp_sf_lo(tmem_base + sfw_col, lo + lo_sf);
          for (int j = 0; j < x.a_atoms; ++j)
            tc_cp_sf_lo(tmem_base + sfa_col + 4 * j, lo + lo_sf + 32u * (uint32_t)(1 + j));
          uint32_t acc = kb > 0 ? 1u : 0u;
#pragma unroll
          for (int sub = 0; sub < 4; ++sub) {
            if (kb + 1 < p.k_tiles || sub < last_subs) {
              tc_mma_mx_lo(d_tmem, lo + 2 * sub, lo + lo_a + 2 * sub, idesc[sub], acc,
                           tmem_base + sfw_col, sfa_tmem);
              acc = 1;
            }
          }
          tc_commit(empty0 + 8 * s);
        }
        __syncwarp();
        if (++s == stages) { s = 0; ph ^= 1u; }
      }
      if (ok && elect_one()) tc_commit(acc_full0 + 8 * buf);
      __syncwarp();
    }
  } else {
    const int quad = warp & 3;
    const int trow = quad * 32 + lane;  // weight row inside the tile
    const uint32_t t_lane = tmem_base + ((uint32_t)(quad * 32) << 16);
    uint32_t ui_next = 0;
    bool ok = true;
    for (int u = blockIdx.x; u < num_units && ok; u += gridDim.x) {
      const Unit x = decode_unit(p, u);
      if (x.rows < p.rows_min || x.rows > p.rows_max) continue;
      const uint32_t ui = ui_next++;
      const uint32_t buf = bufs == 2 ? (ui & 1u) : 0u;
      const uint32_t use = bufs == 2 ? (ui >> 1) : ui;
      const uint32_t t_acc = t_lane + buf * (uint32_t)acc_cols;
      ok = mbar_wait(acc_full0 + 8 * buf, use & 1u, p.status, kWaitAccFull);
      tc_fence_after();
      if (!ok) break;
      if (!kSwiglu) {
        __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.out);
        const int n = x.nt * kTileRows + trow;
        for (int c = 0; c < x.n_mma; c += 16) {
          uint32_t r[16];
          tmem_ld_x16(t_acc + c, r);
          tmem_ld_wait();
          if (c + 16 >= x.n_mma) {  // last read of this buffer: hand it back
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty0 + 8 * buf);
          }
#pragma unroll
          for (int i = 0; i < 16; ++i)
            if (c + i < x.rows && n < p.n_out)
              out[(size_t)(x.row0 + c + i) * p.n_out + n] =
                  __float2bfloat16_rn(__uint_as_float(r[i]));
        }
      } else {
        uint8_t* codes = reinterpret_cast<uint8_t*>(p.out);
        for (int cc = 0; cc < x.n_mma; cc += kXchCols) {
          // (a) this thread's weight row, 32 routed rows -> exchange buffer [col][row]
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            if (cc + half * 16 < x.n_mma) {
              uint32_t r[16];
              tmem_ld_x16(t_acc + cc + half * 16, r);
              tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 16; ++i)
                xch[(half * 16 + i) * kTileRows + trow] = __uint_as_float(r[i]);
            }
          }
          if (cc + kXchCols >= x.n_mma) {  // last read of this buffer: hand it back
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty0 + 8 * buf);
          }
          named_barrier_sync(1, 128);
          // (b) one warp per (routed row, 32-feature block): gate rows 64g.., up rows 64g+32..
          for (int unit = warp - 2; unit < kXchCols * 2; unit += 4) {
            const int c = unit >> 1;
            const int g = unit & 1;
            const int col = cc + c;
            float gate = xch[c * kTileRows + 64 * g + lane];
            float up = xch[c * kTileRows + 64 * g + 32 + lane];
            if (col >= x.rows) gate = up = 0.0f;
            const float v = swiglu_bf16(bf16_round(gate), bf16_round(up));
            float amax = fabsf(v);
#pragma unroll
            for (int d = 16; d > 0; d >>= 1)
              amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, d));
            const uint32_t bits = mx_scale_bits(amax);
            const float q = __fmul_rn(v, mx_inverse(bits));
            const int feat = x.nt * 64 + 32 * g + lane;
            if (col < x.rows && feat < p.n_out) {
              const int orow = x.row0 + col;
              codes[(size_t)orow * p.n_out + feat] = (uint8_t)(e4m3x2(q, 0.0f) & 0xFFu);
              if (lane == 0)
                p.out_sf[sf_offset(orow, feat >> 5, p.out_k_tiles)] = (uint8_t)(bits >> 23);
            }
          }
          named_barrier_sync(1, 128);
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

// ---------------------------------------------------------------------------------------------
// Token-major form for work items with many rows (prefill): the item's routed rows (at most
// 128, starting on a multiple of 128 because segments are padded) are the 128-lane MMA
// operand and 256 weight rows of the expert are the MMA N operand, so every thread of the
// epilogue owns one token row and 128 consecutive features: the SwiGLU pairs (gate/up
// interleaved by 32) sit in its own registers and no exchange through shared memory is needed.
// Persistent, one CTA per SM, eight epilogue warps; the operand ring keeps filling while the
// (single) accumulator is drained.
constexpr int kTmThreads = 320;
constexpr int kTmBn = 256;
constexpr int kTmMaxStages = 6;

template <bool kSwiglu>
__global__ void __launch_bounds__(kTmThreads, 1)
mx_grouped_tm_kernel(const __grid_constant__ CUtensorMap tm_a,
                     const __grid_constant__ CUtensorMap tm_w, const GroupedParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  constexpr int kWBytes = kTmBn * kTileK;
  constexpr int kSfOff = kTileBytes + kWBytes;
  constexpr int kStageBytes = kSfOff + 3 * kSfAtom + 512;  // multiple of 1024
  const int stages = p.stages;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)stages * kStageBytes);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kTmMaxStages + 2);
  const uint32_t full0 = smem_u32(bars);
  const uint32_t empty0 = smem_u32(bars + kTmMaxStages);
  const uint32_t acc_full = smem_u32(bars + 2 * kTmMaxStages);
  const uint32_t acc_empty = smem_u32(bars + 2 * kTmMaxStages + 1);
  constexpr int kSfaCol = kTmBn;
  constexpr int kSfbCol = kTmBn + 4;
  const int tiles_n = (p.w_rows + kTmBn - 1) / kTmBn;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    mbar_init(acc_full, 1);
    mbar_init(acc_empty, 8);  // one arrival per epilogue warp
    fence_mbar_init();
    prefetch_tensormap(&tm_a);
    prefetch_tensormap(&tm_w);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), 512u);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (threadIdx.x == 0) pdl_launch_dependents();
  pdl_wait();  // work list, activations and output buffers belong to preceding kernels
  const int num_units = max(0, min(__ldg(p.num_work), p.work_cap)) * tiles_n;

  // Unit u -> (work item, 256-row weight tile); items outside [rows_min, rows_max] are skipped.
  auto decode = [&](int u, int& row0, int& rows, int& n0, int& w_row) {
    const int item = u / tiles_n;
    const int nt = u - item * tiles_n;
    const int expert = __ldg(p.work + 3 * item);
    row0 = __ldg(p.work + 3 * item + 1);
    rows = __ldg(p.work + 3 * item + 2);
    n0 = nt * kTmBn;
    w_row = expert * p.w_rows + n0;
    // Items that cannot have come from mach_moe_route are skipped (see decode_unit).
    if (expert < 0 || expert >= p.experts || row0 < 0 || (row0 & 127) || row0 + rows > p.rows_cap)
      return false;
    return rows >= p.rows_min && rows <= p.rows_max;
  };

  if (warp == 0) {
    const uint64_t pol_w = policy_evict_normal();  // a weight tile is shared by the expert's items
    const uint64_t pol_a = policy_evict_last();
    const uint32_t base0 = smem_u32(smem);
    const uint32_t tx_bytes = (uint32_t)(kTileBytes + kTmBn * p.w_row_tx + 3 * kSfAtom);
    int s = 0;
    uint32_t ph = 0;
    bool ok = true;
    for (int u = blockIdx.x; u < num_units && ok; u += gridDim.x) {
      int row0, rows, n0, w_row;
      if (!decode(u, row0, rows, n0, w_row)) continue;
      for (int kb = 0; kb < p.k_tiles; ++kb) {
        ok = mbar_wait(empty0 + 8 * s, ph ^ 1u, p.status, kWaitEmpty);
        if (!ok) break;
        if (elect_one()) {
          const uint32_t full = full0 + 8 * s;
          mbar_expect_tx(full, tx_bytes);
          const uint32_t base = base0 + (uint32_t)(s * kStageBytes);
          const int k0 = kb * kTileK;
          tma_load_2d(base, &tm_a, full, k0, row0, pol_a);
          tma_load_2d(base + kTileBytes, &tm_w, full, k0, w_row, pol_w);
          bulk_load_1d(base + kSfOff, p.sf_a + ((size_t)(row0 >> 7) * p.k_tiles + kb) * kSfAtom,
                       kSfAtom, full);
          for (int j = 0; j < 2; ++j)
            bulk_load_1d(base + kSfOff + (1 + j) * kSfAtom,
                         p.sf_w + ((size_t)min((w_row >> 7) + j, p.w_atoms_total - 1) * p.k_tiles + kb) * kSfAtom,
                         kSfAtom, full);
        }
        __syncwarp();
        if (++s == stages) { s = 0; ph ^= 1u; }
      }
    }
  } else if (warp == 1) {
    const int k_rem = p.k - (p.k_tiles - 1) * kTileK;
    const int last_subs = k_rem >> 5;
    const uint32_t idesc0 = idesc_mx(kFmtE4M3, p.w_fmt, (uint32_t)kTmBn);
    uint32_t idesc[4];
#pragma unroll
    for (int sub = 0; sub < 4; ++sub) idesc[sub] = idesc_mx_sf(idesc0, (uint32_t)sub, (uint32_t)sub);
    const uint32_t lo_stage0 = desc_lo(smem_u32(smem));
    const uint32_t lo_step = (uint32_t)kStageBytes >> 4;
    const uint32_t lo_w = (uint32_t)kTileBytes >> 4;
    const uint32_t lo_sf = (uint32_t)kSfOff >> 4;
    int s = 0;
    uint32_t ph = 0;
    uint32_t ui = 0;
    bool ok = true;
    for (int u = blockIdx.x; u < num_units && ok; u += gridDim.x) {
      int row0, rows, n0, w_row;
      if (!decode(u, row0, rows, n0, w_row)) continue;
      ok = mbar_wait(acc_empty, (ui & 1u) ^ 1u, p.status, kWaitAccEmpty);
      if (!ok) break;
      tc_fence_after();
      for (int kb = 0; kb < p.k_tiles; ++kb) {
        ok = mbar_wait(full0 + 8 * s, ph, p.status, kWaitFull);
        if (!ok) break;
        tc_fence_after();
        if (elect_one()) {
          const uint32_t lo = lo_stage0 + (uint32_t)s * lo_step;
          tc_cp_sf_lo(tmem_base + kSfaCol, lo + lo_sf);
          tc_cp_sf_lo(tmem_base + kSfbCol, lo + lo_sf + 32u);
          tc_cp_sf_lo(tmem_base + kSfbCol + 4, lo + lo_sf + 64u);
          uint32_t acc = kb > 0 ? 1u : 0u;
#pragma unroll
          for (int sub = 0; sub < 4; ++sub) {
            if (kb + 1 < p.k_tiles || sub < last_subs) {
              tc_mma_mx_lo(tmem_base, lo + 2 * sub, lo + lo_w + 2 * sub, idesc[sub], acc,
                           tmem_base + kSfaCol, tmem_base + kSfbCol);
              acc = 1;
            }
          }
          tc_commit(empty0 + 8 * s);
        }
        __syncwarp();
        if (++s == stages) { s = 0; ph ^= 1u; }
      }
      if (ok && elect_one()) tc_commit(acc_full);
      __syncwarp();
      ++ui;
    }
  } else {
    const int quad = warp & 3;
    const int part = (warp - 2) >> 2;  // which 128 of the 256 columns
    const int trow = quad * 32 + lane;
    const uint32_t t_acc = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(part * 128);
    uint32_t ui = 0;
    bool ok = true;
    for (int u = blockIdx.x; u < num_units && ok; u += gridDim.x) {
      int row0, rows, n0, w_row;
      if (!decode(u, row0, rows, n0, w_row)) continue;
      ok = mbar_wait(acc_full, ui & 1u, p.status, kWaitAccFull);
      tc_fence_after();
      if (!ok) break;
      ++ui;
      const bool live = trow < rows;
      const int orow = row0 + trow;
      const int c0 = n0 + part * 128;  // first weight row (output column) of this warp
      if (!kSwiglu) {
        __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.out);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          uint32_t ra[32], rb[32];
          tmem_ld_x32(t_acc + h * 64, ra);
          tmem_ld_x32(t_acc + h * 64 + 32, rb);
          tmem_ld_wait();
          if (h == 1) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty);
          }
          const int n = c0 + h * 64;
          if (live && n < p.w_rows) {  // w_rows % 128 == 0: a 64-column group is all in or out
            uint4* dst = reinterpret_cast<uint4*>(out + (size_t)orow * p.n_out + n);
#pragma unroll
            for (int i = 0; i < 4; ++i)
              dst[i] = make_uint4(
                  pack_bf16x2(__uint_as_float(ra[8 * i]), __uint_as_float(ra[8 * i + 1])),
                  pack_bf16x2(__uint_as_float(ra[8 * i + 2]), __uint_as_float(ra[8 * i + 3])),
                  pack_bf16x2(__uint_as_float(ra[8 * i + 4]), __uint_as_float(ra[8 * i + 5])),
                  pack_bf16x2(__uint_as_float(ra[8 * i + 6]), __uint_as_float(ra[8 * i + 7])));
#pragma unroll
            for (int i = 0; i < 4; ++i)
              dst[4 + i] = make_uint4(
                  pack_bf16x2(__uint_as_float(rb[8 * i]), __uint_as_float(rb[8 * i + 1])),
                  pack_bf16x2(__uint_as_float(rb[8 * i + 2]), __uint_as_float(rb[8 * i + 3])),
                  pack_bf16x2(__uint_as_float(rb[8 * i + 4]), __uint_as_float(rb[8 * i + 5])),
                  pack_bf16x2(__uint_as_float(rb[8 * i + 6]), __uint_as_float(rb[8 * i + 7])));
          }
        }
      } else {
        uint8_t* codes = reinterpret_cast<uint8_t*>(p.out);
#pragma unroll
        for (int g = 0; g < 2; ++g) {
          uint32_t gr[32], ur[32];
          tmem_ld_x32(t_acc + g * 64, gr);
          tmem_ld_x32(t_acc + g * 64 + 32, ur);
          tmem_ld_wait();
          if (g == 1) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty);
          }
          const int feat = (c0 + g * 64) >> 1;
          if (live && feat < p.n_out) {
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
            uint4* dst = reinterpret_cast<uint4*>(codes + (size_t)orow * p.n_out + feat);
            dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
            dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
            p.out_sf[sf_offset(orow, feat >> 5, p.out_k_tiles)] = (uint8_t)(bits >> 23);
          }
        }
      }
    }
    tc_fence_before();
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512u);
  }
}

template <bool kSwiglu>
int launch_tm(const CUtensorMap& tm_a, const CUtensorMap& tm_w, const GroupedParams& prm, int grid,
              int smem_bytes, cudaStream_t stream) {
  auto kernel = mx_grouped_tm_kernel<kSwiglu>;
  static int configured_smem_dev[kMaxDeviceSlots] = {};  // the attribute is per device
  int& configured_smem = configured_smem_dev[device_slot()];
  if (smem_bytes > configured_smem) {
    const cudaError_t e =
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
    if (e != cudaSuccess)
      return fail(MACH_ERR_CUDA, "moe_grouped_gemm: shared memory opt-in failed: %s",
                  cudaGetErrorString(e));
    configured_smem = smem_bytes;
  }
  const cudaError_t e = launch_ex(kernel, dim3((unsigned)grid), dim3(kTmThreads), (size_t)smem_bytes,
                                  stream, dim3(1, 1, 1), pdl_enabled(), tm_a, tm_w, prm);
  if (e != cudaSuccess) return fail(MACH_ERR_CUDA, "moe_grouped_gemm launch: %s", cudaGetErrorString(e));
  return MACH_OK;
}

template <bool kSwiglu>
int launch(const CUtensorMap& tm_w, const CUtensorMap& tm_a, const GroupedParams& prm, int grid,
           int smem_bytes, cudaStream_t stream) {
  auto kernel = mx_grouped_gemm_kernel<kSwiglu>;
  static int configured_smem_dev[kMaxDeviceSlots] = {};  // the attribute is per device
  int& configured_smem = configured_smem_dev[device_slot()];
  if (smem_bytes > configured_smem) {
    const cudaError_t e =
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
    if (e != cudaSuccess)
      return fail(MACH_ERR_CUDA, "moe_grouped_gemm: shared memory opt-in failed: %s",
                  cudaGetErrorString(e));
    configured_smem = smem_bytes;
  }
  const cudaError_t e = launch_ex(kernel, dim3((unsigned)grid), dim3(kThreads), (size_t)smem_bytes,
                                  stream, dim3(1, 1, 1), pdl_enabled(), tm_w, tm_a, prm);
  if (e != cudaSuccess) return fail(MACH_ERR_CUDA, "moe_grouped_gemm launch: %s", cudaGetErrorString(e));
  return MACH_OK;
}

}  // namespace
}  // namespace mach

using namespace mach;

extern "C" int mach_moe_grouped_gemm(const void* a_codes, const void* a_scales, const void* w,
                                     const void* w_scales, void* out, void* out_scales,
                                     const void* work, const void* num_work, int64_t work_cap,
                                     int64_t rows_cap, int64_t experts, int64_t w_rows,
                                     int64_t k, int64_t chunk_rows, int w_format, int swiglu,
                                     void* stream) {
  if (rows_cap < 0 || work_cap < 0 || experts < 1 || w_rows < 1 || k < 1)
    return fail(MACH_ERR_INVALID, "moe_grouped_gemm: bad sizes");
  if (rows_cap == 0 || work_cap == 0) return MACH_OK;
  if (!a_codes || !a_scales || !w || !w_scales || !out || !work || !num_work ||
      (swiglu && !out_scales))
    return fail(MACH_ERR_INVALID, "moe_grouped_gemm: null pointer");
  if (w_format != MACH_FMT_E4M3 && w_format != MACH_FMT_E2M3 && w_format != MACH_FMT_E3M2)
    return fail(MACH_ERR_INVALID, "moe_grouped_gemm: unknown weight format %d", w_format);
  const bool six = w_format != MACH_FMT_E4M3;
  if (w_rows % 128 || k % 32 || (six && k % 128) ||
      (chunk_rows != 16 && chunk_rows != 64 && chunk_rows != 128 && chunk_rows != 256))
    return fail(MACH_ERR_UNSUPPORTED,
                "moe_grouped_gemm: rows per expert %% 128, K %% 32 (128 for 6-bit), chunk in "
                "{16, 64, 128, 256} required");
  if (!aligned16(a_codes) || !aligned16(a_scales) || !aligned16(w_scales) || !aligned16(out) ||
      (reinterpret_cast<uintptr_t>(w) & (six ? 31 : 15)))
    return fail(MACH_ERR_UNSUPPORTED, "moe_grouped_gemm: 16-byte aligned operands (32 for 6-bit)");
  GroupedParams prm = {};
  prm.sf_w = (const uint8_t*)w_scales;
  prm.sf_a = (const uint8_t*)a_scales;
  prm.out = out;
  prm.out_sf = (uint8_t*)out_scales;
  prm.work = (const int*)work;
  prm.num_work = (const int*)num_work;
  prm.status = device_status_ptr();
  if (!prm.status) return fail(MACH_ERR_CUDA, "moe_grouped_gemm: cannot resolve the status word");
  prm.w_rows = (int)w_rows;
  prm.n_out = swiglu ? (int)(w_rows / 2) : (int)w_rows;
  prm.k = (int)k;
  prm.k_tiles = (int)((k + 127) / 128);
  prm.out_k_tiles = (prm.n_out + 127) / 128;
  prm.tiles_n = (int)(w_rows / 128);
  prm.w_fmt = (uint32_t)w_format;
  prm.w_row_tx = six ? 96 : 128;
  prm.w_atoms_total = (int)(experts * w_rows / 128);
  prm.work_cap = (int)std::min<int64_t>(work_cap, INT32_MAX);
  prm.rows_cap = (int)std::min<int64_t>(rows_cap, INT32_MAX);
  prm.experts = (int)experts;
  if (work_cap * prm.tiles_n > INT32_MAX)
    return fail(MACH_ERR_UNSUPPORTED, "moe_grouped_gemm: work list too large");

  // Feature-major pass over the items with rows_min <= rows <= rows_max (activation box = box_rows).
  auto run_feature_major = [&](int box_rows, int rows_min, int rows_max) -> int {
    GroupedParams q = prm;
    q.box_rows = box_rows;
    q.rows_min = rows_min;
    q.rows_max = rows_max;
    q.bufs = 2 * box_rows + 12 <= 512 ? 2 : 1;
    int cols = 32;
    while (cols < q.bufs * box_rows + 4 + 8) cols <<= 1;
    q.tmem_cols = cols;
    // CTAs per SM: two when their TMEM and a useful ring both fit (their set-up, ramp and
    // epilogue phases then overlap each other's weight streams), else one.
    const int stage_bytes = (kTileBytes + box_rows * kTileK + 3 * kSfAtom + 1023) & ~1023;
    const int fixed = kXchBytes + (2 * kMaxStages + 4) * 8 + 16 + 1024;
    int per_sm = tuned_moe_ctas_per_sm();
    if (per_sm <= 0) per_sm = 2;
    per_sm = std::max(1, std::min(per_sm, 512 / q.tmem_cols));
    while (per_sm > 1 && ((228 * 1024) / per_sm - 1024 - fixed) / stage_bytes < 3) --per_sm;
    const int budget = std::min(max_smem_optin(), (228 * 1024) / per_sm - 1024);
    const int stages = std::min((budget - fixed) / stage_bytes, kMaxStages);
    if (stages < 1) return fail(MACH_ERR_UNSUPPORTED, "moe_grouped_gemm: tile does not fit in shared memory");
    q.stages = stages;
    // Pad so that exactly per_sm CTAs share an SM (TMEM is never over-subscribed).
    int smem_bytes = std::max(stages * stage_bytes + fixed, (228 * 1024) / (per_sm + 1) + 1);
    smem_bytes = std::min(smem_bytes, max_smem_optin());
    CUtensorMap tm_w, tm_a;
    int rc = make_operand_map(&tm_w, w, experts * w_rows, k, w_format, kTileRows);
    if (rc) return rc;
    rc = make_operand_map(&tm_a, a_codes, rows_cap, k, MACH_FMT_E4M3, box_rows);
    if (rc) return rc;
    const int64_t grid = std::min<int64_t>(work_cap * q.tiles_n, (int64_t)per_sm * sm_count());
    return swiglu ? launch<true>(tm_w, tm_a, q, (int)grid, smem_bytes, (cudaStream_t)stream)
                  : launch<false>(tm_w, tm_a, q, (int)grid, smem_bytes, (cudaStream_t)stream);
  };
  // Token-major pass (128-row activation tiles x 256 weight rows).
  auto run_token_major = [&](int rows_min, int rows_max) -> int {
    GroupedParams q = prm;
    q.box_rows = kTileRows;
    q.rows_min = rows_min;
    q.rows_max = rows_max;
    const int stage_bytes = kTileBytes + kTmBn * kTileK + 3 * kSfAtom + 512;
    const int fixed = (2 * kTmMaxStages + 2) * 8 + 16 + 1024;
    const int stages = std::min((max_smem_optin() - fixed) / stage_bytes, kTmMaxStages);
    if (stages < 2) return fail(MACH_ERR_UNSUPPORTED, "moe_grouped_gemm: tile does not fit in shared memory");
    q.stages = stages;
    const int smem_bytes = stages * stage_bytes + fixed;
    CUtensorMap tm_w, tm_a;
    int rc = make_operand_map(&tm_w, w, experts * w_rows, k, w_format, kTmBn);
    if (rc) return rc;
    rc = make_operand_map(&tm_a, a_codes, rows_cap, k, MACH_FMT_E4M3, kTileRows);
    if (rc) return rc;
    const int64_t tiles_n = (w_rows + kTmBn - 1) / kTmBn;
    const int64_t grid = std::min<int64_t>(work_cap * tiles_n, (int64_t)sm_count());
    return swiglu ? launch_tm<true>(tm_a, tm_w, q, (int)grid, smem_bytes, (cudaStream_t)stream)
                  : launch_tm<false>(tm_a, tm_w, q, (int)grid, smem_bytes, (cudaStream_t)stream);
  };

  // Items of a 128-row chunking start on multiples of 128 rows and go token-major, whatever
  // their row count: measured on B200 (256 experts, top-8), one token-major pass beats a
  // token-major pass for the long items plus a feature-major pass for the short ones, which
  // streams those experts' weights a second time. The host picks 128-row chunks once experts
  // average more than about 20 rows, and 64-row (feature-major) chunks below that.
  // "moe_tm_min_rows" > 1 restores the split (experiments).
  if (chunk_rows == 128 && tuned_moe_token_major() != 0) {
    const int cut = std::max(1, std::min(tuned_moe_tm_min_rows(), 65));
    if (cut > 1) {
      const int rc = run_feature_major(cut <= 17 ? 16 : 64, 1, cut - 1);
      if (rc) return rc;
    }
    return run_token_major(cut, 128);
  }
  return run_feature_major((int)chunk_rows, 1, (int)chunk_rows);
}
