// Token-major block-scaled GEMM on CTA pairs (tcgen05 cta_group::2), persistent, with a
// double-buffered TMEM accumulator so the epilogue of tile i overlaps the MMAs of tile i+1.
//
// A pair of CTAs (a 2-CTA cluster on adjacent SMs) owns a 256-token x BN-feature tile. Each
// CTA stages its own 128 tokens of A and HALF of the weight tile (BN/2 rows) per K step;
// one tcgen05.mma.cta_group::2 issued by the even CTA drives both tensor cores, each of which
// reads the other half of B from its partner's shared memory. Per CTA and K step that is
// 16 KiB + BN/2 * 128 B from L2 for 128 x BN outputs, and the accumulator needs only BN TMEM
// columns per CTA, which leaves room for two accumulator buffers (2 * 192 + scale factors).
//
// Synchronisation (no TMA multicast anywhere):
//   * every TMA load of either CTA carries .cta_group::2 and completes its bytes on the EVEN
//     CTA's `full` barrier of the stage (the barrier address is mapped with mapa);
//   * the MMA thread frees a stage in BOTH CTAs with one multicast tcgen05.commit, and
//     announces a finished accumulator to both epilogues the same way;
//   * the odd CTA's epilogue warps hand an accumulator buffer back with a remote mbarrier
//     arrive on the even CTA.
//
// Scale factors: each CTA copies its own A atom and all B atoms of the tile into its own
// TMEM (tcgen05.cp.cta_group::2 performs the copy in both CTAs from the same smem offsets).
#include <cuda.h>
#include <cuda_bf16.h>
#include "gemm_mx_tm.h"
#include "host_util.h"
#include "ptx.cuh"
#include "quant_math.cuh"

namespace mach {

int make_operand_map(CUtensorMap* map, const void* base, int64_t rows, int64_t k, int format,
                     int box_rows);
int make_sf_map(CUtensorMap* map, const void* base, int64_t atoms);

namespace {

constexpr int kHalfRows = 128;
constexpr int kTileK = 128;
constexpr int kABytes = kHalfRows * kTileK;
constexpr int kSfAtom = 512;
constexpr int kEpiWarps = 12;  // three per TMEM lane quadrant
constexpr int kThreads = (2 + kEpiWarps) * 32;
constexpr int kMaxStages = 10;
constexpr int kMaxBAtoms = 4;
constexpr int kEpiStageBytes = 32 * 128;  // per epilogue warp: 32 rows x 64 BF16 (BF16 epilogue only)

enum { kWaitEmpty = 601, kWaitFull = 602, kWaitAccFull = 603, kWaitAccEmpty = 604 };

struct PairParams {
  void* out;
  uint8_t* out_sf;
  int* status;
  int m, n_rows, n_out, k, k_tiles, out_k_tiles;
  int bn, stages;      // bn = bn_a + bn_b: tile width in weight rows
  int bn_a, bn_b;      // N of the first MMA (<= 256) and of the optional second one
  int bufs;            // accumulator buffers in TMEM (2 when 2 * bn + scale columns fit)
  int b_atom_slots;    // scale atoms of B staged per K step (tile rows / 128, rounded up, + 1)
  int tiles_m, tiles_n, panel_m;
  int b_atoms_total;
  int interleaved;
  int tmem_cols;
  uint32_t idesc_a, idesc_b;
  int w_row_tx;    // transaction bytes per weight row and K step (128, packed 6-bit: 96)
  int debug;       // experiment bits: 1 skip scale copies, 2 skip MMAs, 4 copy scales once per tile
  ScatterTarget scatter;  // world == 0: plain output
};

// ---- cta_group::2 forms of the tcgen05 / TMA instructions
__device__ __forceinline__ void tmem_alloc2(uint32_t smem_result, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result),
               "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tc_cp2_32x128b_warpx4(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc)
               : "memory");
}
__device__ __forceinline__ void tc_mma2_mx(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc,
                                           uint32_t idesc, uint32_t accumulate, uint32_t sfa,
                                           uint32_t sfb) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale.scale_vec::1X [%0], %1, %2, %3, [%5], "
      "[%6], p;\n\t}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
      : "memory");
}
// Same instructions with the shared-memory descriptors given as their low words (start address
// >> 4); the high word is fixed: K-major, 128-byte swizzle, 8-row groups 1024 B apart, sm_100
// descriptor version (operands), or unswizzled 8-row groups 128 B apart (scale atoms).
constexpr uint32_t kDescHiSw128 = (1024u >> 4) | (1u << 14) | (2u << 29);
constexpr uint32_t kDescHiSf = (128u >> 4) | (1u << 14);
__device__ __forceinline__ void tc_mma2_lo(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo,
                                           uint32_t idesc, uint32_t accumulate, uint32_t sfa,
                                           uint32_t sfb) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
      "mov.b64 da, {%1, %7};\n\t"
      "mov.b64 db, {%2, %7};\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale.scale_vec::1X [%0], da, db, %3, [%5], "
      "[%6], p;\n\t}" ::"r"(d_tmem),
      "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb), "r"(kDescHiSw128));
}
__device__ __forceinline__ void tc_cp2_sf(uint32_t taddr, uint32_t s_lo) {
  asm volatile(
      "{\n\t.reg .b64 ds;\n\t"
      "mov.b64 ds, {%1, %2};\n\t"
      "tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], ds;\n\t}" ::"r"(taddr),
      "r"(s_lo), "r"(kDescHiSf));
}
// Arrive on the barrier at this shared-memory offset in both CTAs of the pair once every
// tcgen05 operation issued so far by this thread has completed.
__device__ __forceinline__ void tc_commit2_both(uint32_t bar) {
  const uint16_t mask = 3;
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 "
      "[%0], %1;" ::"r"(bar),
      "h"(mask)
      : "memory");
}
// 2-D tiled load into this CTA's shared memory; the bytes complete on `bar`, a shared::cluster
// address that may belong to the partner CTA.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const void* desc, uint32_t bar,
                                                 int c0, int c1, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      ".L2::cache_hint [%0], [%1, {%3, %4}], [%2], %5;" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(desc)), "r"(bar), "r"(c0), "r"(c1), "l"(policy)
      : "memory");
}
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr)
               : "memory");
}
// Instruction descriptor for cta_group::2: the pair computes M = 256.
__host__ __device__ __forceinline__ uint32_t idesc_mx_pair(uint32_t a_fmt, uint32_t b_fmt,
                                                           uint32_t n) {
  return (a_fmt << 7) | (b_fmt << 10) | ((n >> 3) << 17) | (1u << 23) | ((256u >> 4) << 24);
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

struct TileCoord {
  int m0, n0;
};
__device__ __forceinline__ TileCoord tile_coord(const PairParams& p, int t) {
  const int per_panel = p.panel_m * p.tiles_n;
  const int panel = t / per_panel;
  const int in_panel = t - panel * per_panel;
  const int rows_here = min(p.panel_m, p.tiles_m - panel * p.panel_m);
  TileCoord c;
  c.m0 = (panel * p.panel_m + in_panel % rows_here) * 2 * kHalfRows;
  c.n0 = (in_panel / rows_here) * p.bn;
  return c;
}

// kTwo: the tile is wider than one MMA (256 < bn <= 448) and takes a second weight box and a
// second MMA per K step.
template <bool kSwiglu, bool kTwo>
__global__ void __launch_bounds__(kThreads, 1)
mx_gemm_pair_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                    const __grid_constant__ CUtensorMap tm_b2,
                    const __grid_constant__ CUtensorMap tm_sfa,
                    const __grid_constant__ CUtensorMap tm_sfb, const PairParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta = cluster_ctarank();  // 0 = even CTA (issues the MMAs), 1 = odd
  const int bn = p.bn;
  const int b_half_bytes = (bn / 2) * kTileK;
  const int sf_off = kABytes + b_half_bytes;
  const int stage_bytes = (sf_off + (1 + p.b_atom_slots) * kSfAtom + 1023) & ~1023;
  const int stages = p.stages;
  uint8_t* epi_stage = smem + (size_t)stages * stage_bytes;
  uint64_t* bars =
      reinterpret_cast<uint64_t*>(epi_stage + (kSwiglu ? 0 : kEpiWarps * kEpiStageBytes));
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kMaxStages + 4);
  const uint32_t full0 = smem_u32(bars);
  const uint32_t empty0 = smem_u32(bars + kMaxStages);
  const uint32_t acc_full0 = smem_u32(bars + 2 * kMaxStages);       // [2]
  const uint32_t acc_empty0 = smem_u32(bars + 2 * kMaxStages + 2);  // [2], used on the even CTA
  const int num_tiles = p.tiles_m * p.tiles_n;
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  const int sfa_col = p.bufs * bn;
  const int sfb_col = p.bufs * bn + 4;
  const int b2_off = (p.bn_a / 2) * kTileK;  // second weight box inside the B region

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full0 + 8 * b, 1);
      mbar_init(acc_empty0 + 8 * b, 2 * kEpiWarps);  // the epilogue warps of both CTAs
    }
    fence_mbar_init();
    prefetch_tensormap(&tm_a);
    prefetch_tensormap(&tm_b);
    if (kTwo) prefetch_tensormap(&tm_b2);
    prefetch_tensormap(&tm_sfa);
    prefetch_tensormap(&tm_sfb);
  }
  if (warp == 1) {
    tmem_alloc2(smem_u32(tmem_slot), (uint32_t)p.tmem_cols);
    tmem_relinquish2();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers are initialised before any remote signal
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (threadIdx.x == 0) pdl_launch_dependents();

  if (warp == 0) {
    // =============================== TMA producer (both CTAs); warp-uniform loop, one lane issues
    {
      if (elect_one()) pdl_wait();  // the activations come from the preceding kernel
      __syncwarp();
      const uint64_t pol = policy_evict_normal();
      const uint32_t base0 = smem_u32(smem);
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int t = pair; t < num_tiles && ok; t += num_pairs) {
        const TileCoord c = tile_coord(p, t);
        const int atom0 = c.n0 >> 7;
        const int atoms = min(((c.n0 + bn - 1) >> 7), p.b_atoms_total - 1) - atom0 + 1;
        // bytes both CTAs deliver per stage: 2 x (A + half B + own A atom + all B atoms)
        const bool two = kTwo && c.n0 + p.bn_a < p.n_rows;  // second MMA has live rows
        const uint32_t tx = 2u * (uint32_t)(kABytes + ((p.bn_a + (two ? p.bn_b : 0)) / 2) * p.w_row_tx +
                                            (1 + atoms) * kSfAtom);
        const int a_row = c.m0 + (int)cta * kHalfRows;
        const int b_row = c.n0 + (int)cta * (p.bn_a / 2);
        const int b2_row = c.n0 + p.bn_a + (int)cta * (p.bn_b / 2);
        const int sfa_row = ((c.m0 >> 7) + (int)cta) * p.k_tiles;
        const int sfb_row = atom0 * p.k_tiles;
        for (int kb = 0; kb < p.k_tiles; ++kb) {
          ok = mbar_wait(empty0 + 8 * s, ph ^ 1u, p.status, kWaitEmpty);
          if (!ok) break;
          if (elect_one()) {
            const uint32_t full_even = map_to_cta(full0 + 8 * s, 0);
            if (cta == 0) mbar_expect_tx(full0 + 8 * s, tx);
            const uint32_t base = base0 + (uint32_t)s * (uint32_t)stage_bytes;
            const int k0 = kb * kTileK;
            tma_load_2d_pair(base, &tm_a, full_even, k0, a_row, pol);
            tma_load_2d_pair(base + kABytes, &tm_b, full_even, k0, b_row, pol);
            if (two) tma_load_2d_pair(base + kABytes + b2_off, &tm_b2, full_even, k0, b2_row, pol);
            tma_load_2d_pair(base + sf_off, &tm_sfa, full_even, 0, sfa_row + kb, pol);
            for (int j = 0; j < atoms; ++j)
              tma_load_2d_pair(base + sf_off + (1 + j) * kSfAtom, &tm_sfb, full_even, 0,
                               sfb_row + j * p.k_tiles + kb, pol);
          }
          __syncwarp();
          if (++s == stages) { s = 0; ph ^= 1u; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // =============================== MMA issuer (even CTA only)
    // One thread issues every tcgen05 instruction of the pair, so its instruction count per K
    // step bounds the whole kernel: descriptors are kept as 32-bit halves that only need an
    // add, the four instruction descriptors are precomputed, and the K sub-steps are unrolled.
    if (cta == 0) {  // warp-uniform loop; only the issue itself is done by one elected lane
      const int k_rem = p.k - (p.k_tiles - 1) * kTileK;
      const int last_subs = k_rem >> 5;
      uint32_t idesc_a[4], idesc_b[4];
#pragma unroll
      for (int sub = 0; sub < 4; ++sub) {
        idesc_a[sub] = idesc_mx_sf(p.idesc_a, (uint32_t)sub, (uint32_t)sub);
        idesc_b[sub] = idesc_mx_sf(p.idesc_b, (uint32_t)sub, (uint32_t)sub);
      }
      const uint32_t lo_stage0 = (smem_u32(smem) & 0x3FFFF) >> 4;
      const uint32_t lo_step = (uint32_t)stage_bytes >> 4;
      const uint32_t lo_b = (uint32_t)kABytes >> 4;
      const uint32_t lo_b2 = (uint32_t)(kABytes + b2_off) >> 4;
      const uint32_t lo_sf = (uint32_t)sf_off >> 4;
      const uint32_t sfa_tmem = tmem_base + sfa_col;
#ifdef MACH_EXPERIMENTS
      const bool skip_mma = (p.debug & 2) != 0;
      const bool skip_cp = (p.debug & 1) != 0;
#else
      constexpr bool skip_mma = false, skip_cp = false;
#endif
      int s = 0;
      uint32_t ph = 0;
      int tile_i = 0;
      bool ok = true;
      for (int t = pair; t < num_tiles && ok; t += num_pairs, ++tile_i) {
        const TileCoord c = tile_coord(p, t);
        const int atom0 = c.n0 >> 7;
        const int atoms = min(((c.n0 + bn - 1) >> 7), p.b_atoms_total - 1) - atom0 + 1;
        const bool two = kTwo && c.n0 + p.bn_a < p.n_rows;
        const int buf = p.bufs == 2 ? (tile_i & 1) : 0;
        const uint32_t use = p.bufs == 2 ? ((uint32_t)tile_i >> 1) : (uint32_t)tile_i;
        const uint32_t d_tmem = tmem_base + buf * bn;
        const uint32_t d_tmem2 = d_tmem + p.bn_a;
        const uint32_t sfb_tmem = tmem_base + sfb_col + ((c.n0 & 127) >> 5);
        const uint32_t sfb_tmem2 = sfb_tmem + (p.bn_a >> 5);
        // the epilogues of both CTAs have drained this buffer
        ok = mbar_wait(acc_empty0 + 8 * buf, (use & 1u) ^ 1u, p.status, kWaitAccEmpty);
        if (!ok) break;
        tc_fence_after();
        for (int kb = 0; kb < p.k_tiles; ++kb) {
          uint32_t acc = kb > 0 ? 1u : 0u;
          ok = mbar_wait(full0 + 8 * s, ph, p.status, kWaitFull);
          if (!ok) break;
          tc_fence_after();
          const uint32_t lo = lo_stage0 + (uint32_t)s * lo_step;
          if (elect_one()) {
          if (!skip_cp) {
            tc_cp2_sf(sfa_tmem, lo + lo_sf);
            for (int j = 0; j < atoms; ++j)
              tc_cp2_sf(tmem_base + sfb_col + 4 * j, lo + lo_sf + 32u * (uint32_t)(1 + j));
          }
          if (!skip_mma) {
            if (kb + 1 < p.k_tiles || last_subs == 4) {
#pragma unroll
              for (int sub = 0; sub < 4; ++sub) {
                tc_mma2_lo(d_tmem, lo + 2 * sub, lo + lo_b + 2 * sub, idesc_a[sub], acc, sfa_tmem,
                           sfb_tmem);
                if (kTwo && two)
                  tc_mma2_lo(d_tmem2, lo + 2 * sub, lo + lo_b2 + 2 * sub, idesc_b[sub], acc,
                             sfa_tmem, sfb_tmem2);
                acc = 1;
              }
            } else {
              for (int sub = 0; sub < last_subs; ++sub) {
                tc_mma2_lo(d_tmem, lo + 2 * sub, lo + lo_b + 2 * sub, idesc_a[sub], acc, sfa_tmem,
                           sfb_tmem);
                if (kTwo && two)
                  tc_mma2_lo(d_tmem2, lo + 2 * sub, lo + lo_b2 + 2 * sub, idesc_b[sub], acc,
                             sfa_tmem, sfb_tmem2);
                acc = 1;
              }
            }
          }
          tc_commit2_both(empty0 + 8 * s);
          }
          __syncwarp();
          if (++s == stages) { s = 0; ph ^= 1u; }
        }
        if (ok && elect_one()) tc_commit2_both(acc_full0 + 8 * buf);
        __syncwarp();
      }
    }
    __syncwarp();
  } else {
    // =============================== epilogue warps (both CTAs, own 128 tokens)
    const int ew = warp - 2;
    const int quad = warp & 3;
    const int part = ew >> 2;  // which of the warps sharing the lane quadrant
    constexpr int kParts = kEpiWarps / 4;
    const uint32_t t_lane = tmem_base + ((uint32_t)(quad * 32) << 16);
    const uint32_t acc_empty_even0 = map_to_cta(acc_empty0, 0);
    // Reduce-scatter: the parity half of the all-reduce buffers follows the epoch word, which
    // the previous fused all-reduce of this rank advanced before this kernel could start.
    size_t scatter_off = 0;
    if (!kSwiglu && p.scatter.world > 0) {
      pdl_wait();
      const uint32_t epoch = *reinterpret_cast<const volatile uint32_t*>(p.scatter.epoch);
      scatter_off = p.scatter.header_bytes + (size_t)(epoch & 1u) * p.scatter.parity_bytes;
    }
    int tile_i = 0;
    bool ok = true;
    for (int t = pair; t < num_tiles && ok; t += num_pairs, ++tile_i) {
      const TileCoord c = tile_coord(p, t);
      const int buf = p.bufs == 2 ? (tile_i & 1) : 0;
      const uint32_t use = p.bufs == 2 ? ((uint32_t)tile_i >> 1) : (uint32_t)tile_i;
      ok = mbar_wait(acc_full0 + 8 * buf, use & 1u, p.status, kWaitAccFull);
      tc_fence_after();
      if (!ok) break;
      const int row = c.m0 + (int)cta * kHalfRows + quad * 32 + lane;
      const uint32_t t_acc = t_lane + buf * bn;
      if (!kSwiglu) {
        // BF16 rows leave through a per-warp transpose in shared memory, so that every store
        // instruction writes whole 128-byte row segments (4 rows x 128 B) instead of 32
        // scattered 16-byte pieces: the form NVLink peer stores need, and cheaper locally too.
        // Destination row: the caller's matrix, or (reduce-scatter) this rank's slot in the
        // all-reduce buffer of the rank that owns the row.
        const int row_base = c.m0 + (int)cta * kHalfRows + quad * 32;
        const bool to_all = p.scatter.world > 0 && p.scatter.one_shot != 0;
        __nv_bfloat16* row_ptr[8];  // to_all: offset from a buffer base instead of a pointer
#pragma unroll
        for (int it = 0; it < 8; ++it) {
          const int rr = row_base + it * 4 + (lane >> 3);
          row_ptr[it] = nullptr;
          if (rr < p.m) {
            if (to_all) {
              row_ptr[it] = reinterpret_cast<__nv_bfloat16*>(scatter_off) +
                            ((size_t)p.scatter.rank * p.scatter.m + rr) * p.n_out + 1;  // +1: non-null
            } else if (p.scatter.world > 0) {
              const int owner = min(rr / p.scatter.rows_per_owner, p.scatter.world - 1);
              const int local = rr - owner * p.scatter.rows_per_owner;
              row_ptr[it] = reinterpret_cast<__nv_bfloat16*>(p.scatter.peers[owner] + scatter_off) +
                            ((size_t)p.scatter.rank * p.scatter.rows_per_owner + local) * p.n_out;
            } else {
              row_ptr[it] = reinterpret_cast<__nv_bfloat16*>(p.out) + (size_t)rr * p.n_out;
            }
          }
        }
        uint4* stage = reinterpret_cast<uint4*>(epi_stage + ew * kEpiStageBytes);  // [32][8]
        const int piece = lane & 7;
        for (int ch = part; ch * 64 < bn; ch += kParts) {
          uint32_t ra[32], rb[32];
          tmem_ld_x32(t_acc + ch * 64, ra);
          tmem_ld_x32(t_acc + ch * 64 + 32, rb);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            stage[lane * 8 + (j ^ (lane & 7))] = make_uint4(
                pack_bf16x2(__uint_as_float(ra[8 * j]), __uint_as_float(ra[8 * j + 1])),
                pack_bf16x2(__uint_as_float(ra[8 * j + 2]), __uint_as_float(ra[8 * j + 3])),
                pack_bf16x2(__uint_as_float(ra[8 * j + 4]), __uint_as_float(ra[8 * j + 5])),
                pack_bf16x2(__uint_as_float(ra[8 * j + 6]), __uint_as_float(ra[8 * j + 7])));
            stage[lane * 8 + ((4 + j) ^ (lane & 7))] = make_uint4(
                pack_bf16x2(__uint_as_float(rb[8 * j]), __uint_as_float(rb[8 * j + 1])),
                pack_bf16x2(__uint_as_float(rb[8 * j + 2]), __uint_as_float(rb[8 * j + 3])),
                pack_bf16x2(__uint_as_float(rb[8 * j + 4]), __uint_as_float(rb[8 * j + 5])),
                pack_bf16x2(__uint_as_float(rb[8 * j + 6]), __uint_as_float(rb[8 * j + 7])));
          }
          __syncwarp();
          const int n_phys = c.n0 + ch * 64 + piece * 8;
          int n = n_phys;
          if (p.interleaved)
            n = ((n_phys >> 5) & 1) * (p.n_rows >> 1) + ((n_phys >> 6) << 5) + (n_phys & 31);
          const bool col_ok = n_phys < p.n_rows;  // N % 8 == 0: a piece is all in or all out
#pragma unroll
          for (int it = 0; it < 8; ++it) {
            const int rl = it * 4 + (lane >> 3);
            const uint4 v = stage[rl * 8 + (piece ^ (rl & 7))];
            if (col_ok && row_ptr[it]) {
              if (to_all) {
                const size_t off = reinterpret_cast<size_t>(row_ptr[it] + n - 1);
                for (int d = 0; d < p.scatter.world; ++d)
                  *reinterpret_cast<uint4*>(p.scatter.peers[d] + off) = v;
              } else {
                *reinterpret_cast<uint4*>(row_ptr[it] + n) = v;
              }
            }
          }
          __syncwarp();
        }
      } else {
        uint8_t* codes = reinterpret_cast<uint8_t*>(p.out);
        for (int g = part; g * 64 < bn; g += kParts) {
          uint32_t gr[32], ur[32];
          tmem_ld_x32(t_acc + g * 64, gr);
          tmem_ld_x32(t_acc + g * 64 + 32, ur);
          tmem_ld_wait();
          const int feat = (c.n0 + g * 64) >> 1;
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
      // all TMEM reads of this warp for this buffer are complete: return it to the MMA thread
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_remote(acc_empty_even0 + 8 * buf);
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // no CTA frees TMEM or exits while its partner may still signal it
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc2(tmem_base, (uint32_t)p.tmem_cols);
  }
}

int g_last_pairs = 0;  // diagnostics: CTA pairs of the most recent launch

template <bool kSwiglu, bool kTwo>
int launch(const CUtensorMap& tm_a, const CUtensorMap& tm_b, const CUtensorMap& tm_b2,
           const CUtensorMap& tm_sfa, const CUtensorMap& tm_sfb, const PairParams& prm, int grid, int smem_bytes,
           cudaStream_t stream) {
  auto kernel = mx_gemm_pair_kernel<kSwiglu, kTwo>;
  static int configured_smem_dev[kMaxDeviceSlots] = {};  // the attribute is per device
  int& configured_smem = configured_smem_dev[device_slot()];
  if (smem_bytes > configured_smem) {
    const cudaError_t e =
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
    if (e != cudaSuccess)
      return fail(MACH_ERR_CUDA, "mx_gemm_pair: shared memory opt-in failed: %s",
                  cudaGetErrorString(e));
    configured_smem = smem_bytes;
  }
  // A persistent grid must be resident as a whole: floor-swept GPCs can hold fewer 2-CTA
  // clusters than SMs / 2, and a cluster that starts late would serialise its whole tile list.
  static int max_clusters_dev[kMaxDeviceSlots] = {};
  static int max_clusters_smem_dev[kMaxDeviceSlots] = {};   // shared memory size + 1 of the cached query
  int& max_clusters = max_clusters_dev[device_slot()];
  int& max_clusters_smem_plus1 = max_clusters_smem_dev[device_slot()];
  if (max_clusters_smem_plus1 != smem_bytes + 1) {
    cudaLaunchConfig_t q = {};
    q.gridDim = dim3((unsigned)grid);
    q.blockDim = dim3(kThreads);
    q.dynamicSmemBytes = (size_t)smem_bytes;
    cudaLaunchAttribute qa[1];
    qa[0].id = cudaLaunchAttributeClusterDimension;
    qa[0].val.clusterDim.x = 2;
    qa[0].val.clusterDim.y = 1;
    qa[0].val.clusterDim.z = 1;
    q.attrs = qa;
    q.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kernel, &q) == cudaSuccess && n > 0) max_clusters = n;
    else max_clusters = sm_count() / 2;
    max_clusters_smem_plus1 = smem_bytes + 1;
  }
  grid = 2 * std::max(1, std::min(grid / 2, max_clusters));
  g_last_pairs = grid / 2;
  const cudaError_t e =
      launch_ex(kernel, dim3((unsigned)grid), dim3(kThreads), (size_t)smem_bytes, stream,
                dim3(2, 1, 1), pdl_enabled(), tm_a, tm_b, tm_b2, tm_sfa, tm_sfb, prm);
  if (e != cudaSuccess) return fail(MACH_ERR_CUDA, "mx_gemm_pair launch: %s", cudaGetErrorString(e));
  return MACH_OK;
}

}  // namespace

int last_pair_count() { return g_last_pairs; }

int run_mx_gemm_pair(const TmGemmArgs& a, cudaStream_t stream) {
  PairParams prm = {};
  prm.out = a.out;
  prm.out_sf = reinterpret_cast<uint8_t*>(a.out_sf);
  prm.status = device_status_ptr();
  if (!prm.status) return fail(MACH_ERR_CUDA, "mx_gemm_pair: cannot resolve the device status word");
  prm.m = (int)a.m;
  prm.n_rows = (int)a.w_rows;
  prm.n_out = a.swiglu ? (int)(a.w_rows / 2) : (int)a.w_rows;
  prm.k = (int)a.k;
  prm.k_tiles = (int)((a.k + 127) / 128);
  prm.out_k_tiles = (prm.n_out + 127) / 128;
  prm.bn = a.bn;
  prm.bn_a = a.bn <= 256 ? a.bn : 256;
  prm.bn_b = a.bn - prm.bn_a;
  prm.interleaved = a.interleaved ? 1 : 0;
  prm.tiles_m = (int)((a.m + 255) / 256);
  prm.tiles_n = (int)((a.w_rows + a.bn - 1) / a.bn);
  prm.panel_m = a.panel_m > 0 ? a.panel_m : 8;
  prm.b_atoms_total = (int)((a.w_rows + 127) / 128);
  // Tiles start on multiples of 64 weight rows (even scale column); up to 4 scale atoms.
  if (a.bn % 64 || a.bn < 64 || a.bn > 448)
    return fail(MACH_ERR_UNSUPPORTED, "mx_gemm_pair: unsupported tile width %d", a.bn);
  prm.b_atom_slots = std::min(kMaxBAtoms, (a.bn + 63) / 128 + 1);
  const int sf_cols = 4 + 4 * prm.b_atom_slots;
  prm.bufs = (2 * a.bn + sf_cols <= 512) ? 2 : 1;
  if (prm.bufs * a.bn + sf_cols > 512)
    return fail(MACH_ERR_UNSUPPORTED, "mx_gemm_pair: TMEM plan exceeds 512 columns");
  int cols = 32;
  while (cols < prm.bufs * a.bn + sf_cols) cols <<= 1;
  prm.tmem_cols = cols;
  prm.idesc_a = idesc_mx_pair(kFmtE4M3, (uint32_t)a.w_format, (uint32_t)prm.bn_a);
  prm.idesc_b = idesc_mx_pair(kFmtE4M3, (uint32_t)a.w_format, (uint32_t)std::max(prm.bn_b, 16));
  prm.debug = a.debug;
  if (a.scatter) {
    if (a.swiglu) return fail(MACH_ERR_UNSUPPORTED, "mx_gemm_pair: reduce-scatter needs the BF16 epilogue");
    prm.scatter = *a.scatter;
  }
  prm.w_row_tx = a.w_format == MACH_FMT_E4M3 ? 128 : 96;
  const int stage_bytes =
      (kABytes + (a.bn / 2) * kTileK + (1 + prm.b_atom_slots) * kSfAtom + 1023) & ~1023;
  const int fixed =
      (2 * kMaxStages + 4) * 8 + 16 + 1024 + (a.swiglu ? 0 : kEpiWarps * kEpiStageBytes);
  int stages = std::min((max_smem_optin() - fixed) / stage_bytes, kMaxStages);
  if (a.stages > 0) stages = std::min(stages, a.stages);
  if (stages < 2) return fail(MACH_ERR_UNSUPPORTED, "mx_gemm_pair: tile does not fit in shared memory");
  prm.stages = stages;
  const int smem_bytes = stages * stage_bytes + fixed;
  CUtensorMap tm_a, tm_b, tm_b2, tm_sfa, tm_sfb;
  int rc = make_operand_map(&tm_a, a.a_codes, a.m, a.k, MACH_FMT_E4M3, kHalfRows);
  if (rc) return rc;
  rc = make_operand_map(&tm_b, a.w, a.w_rows, a.k, a.w_format, prm.bn_a / 2);
  if (rc) return rc;
  rc = make_operand_map(&tm_b2, a.w, a.w_rows, a.k, a.w_format, std::max(prm.bn_b, 16) / 2);
  if (rc) return rc;
  rc = make_sf_map(&tm_sfa, a.a_sf, ((a.m + 127) / 128) * (int64_t)prm.k_tiles);
  if (rc) return rc;
  rc = make_sf_map(&tm_sfb, a.w_sf, (int64_t)prm.b_atoms_total * prm.k_tiles);
  if (rc) return rc;
  const int pairs = std::max(1, std::min(prm.tiles_m * prm.tiles_n, sm_count() / 2));
  if (prm.bn_b > 0)
    return a.swiglu
               ? launch<true, true>(tm_a, tm_b, tm_b2, tm_sfa, tm_sfb, prm, 2 * pairs, smem_bytes, stream)
               : launch<false, true>(tm_a, tm_b, tm_b2, tm_sfa, tm_sfb, prm, 2 * pairs, smem_bytes, stream);
  return a.swiglu
             ? launch<true, false>(tm_a, tm_b, tm_b2, tm_sfa, tm_sfb, prm, 2 * pairs, smem_bytes, stream)
             : launch<false, false>(tm_a, tm_b, tm_b2, tm_sfa, tm_sfb, prm, 2 * pairs, smem_bytes, stream);
}

}  // namespace mach
