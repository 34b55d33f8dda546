// Block-scaled MXFP8 / MXFP6 GEMM for sm_100a:  out = dq(A) * dq(W)^T.
//
//   tcgen05.mma kind::mxf8f6f4.block_scale (UE8M0 scale per 32 K), M = 128 per instruction,
//   operands staged by TMA (128B swizzle, no multicast) through an mbarrier ring,
//   scale factors moved smem -> TMEM with tcgen05.cp, FP32 accumulators in TMEM.
//
// Two tile orientations share one kernel:
//   * token-major (kSwap = false, M > 64): activations are the 128-row MMA "A" operand
//     (TMEM lanes = tokens), weights the "B" operand (TMEM columns = output features).
//   * feature-major (kSwap = true, M <= 64): weights are the 128-row operand so a decode
//     batch does not waste the 128-row MMA; the batch (padded to 16) is the N operand.
//     K is split over a thread-block cluster; partial tiles are exchanged through
//     distributed shared memory and summed in rank order (deterministic).
//
// Epilogues: BF16 store, or SwiGLU + MXFP8 requantisation (gate and up rows of the fused
// gate_up weight land in the same tile, so the BF16 [M, 2I] intermediate never exists).
//
// Warp roles (192 threads): warp 0 = TMA producer, warp 1 = TMEM owner + MMA issuer,
// warps 2..5 = epilogue (each owns the TMEM lane quadrant warp_id % 4).
#include <cuda.h>
#include <cuda_bf16.h>
#include <cstring>
#include <mutex>
#include "gemm_mx_tm.h"
#include "host_util.h"
#include "ptx.cuh"
#include "quant_math.cuh"

namespace mach {

namespace {

constexpr int kTileRows = 128;       // rows of the lane-side operand per tile
constexpr int kTileK = 128;          // K elements (= smem bytes per row) per pipeline stage
constexpr int kTileBytes = kTileRows * kTileK;  // 16 KiB
constexpr int kSfAtom = 512;         // bytes of one 128-row x 4-group scale atom
constexpr int kThreads = 192;
constexpr int kMaxStages = 12;

// Wait codes written to the device status word.
enum { kWaitEmpty = 101, kWaitFull = 102, kWaitAccum = 103 };

struct MxGemmParams {
  const uint8_t* sf_p;   // swizzled scales of the lane-side operand
  const uint8_t* sf_q;   // swizzled scales of the column-side operand
  void* out;             // BF16 [M, N]   or   E4M3 codes [M, I] (SwiGLU)
  uint8_t* out_sf;       // SwiGLU: swizzled scales of the codes
  int* status;
  int m;                 // tokens
  int n;                 // output features (SwiGLU: I, the weight has 2I rows)
  int k;
  int k_tiles;           // ceil(k / 128)
  int out_k_tiles;       // SwiGLU: ceil(I / 128)
  int bn;                // MMA N (columns of the accumulator)
  int stages;
  int split;             // CTAs per cluster along K (feature-major only)
  int tmem_cols;         // power of two >= 32
  uint32_t idesc;
  int stream_weights;    // 1: weights are read once (evict-first)
  int panel_m;           // token-major raster: m-tiles per panel (tiles run n-fastest inside)
  int debug;             // experiment bits: 1 skip scale copies, 2 skip MMAs, 8 alternate SF columns
  int interleaved;       // weight rows are gate/up interleaved by 32 (plain epilogue remaps)
  int tx_discount;       // bytes per stage TMA does not count: packed 6-bit rows report 96 of 128
  int recv_off;          // feature-major: byte offset of the receive slots (0: they reuse the ring)
  int bars_off;          // byte offset of the barriers
};

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

template <bool kSwap, bool kSwiglu, bool kIl>
__global__ void __launch_bounds__(kThreads, 1)
mx_gemm_kernel(const __grid_constant__ CUtensorMap tm_p, const __grid_constant__ CUtensorMap tm_q,
               const MxGemmParams p) {
  // kIl: gate_up rows interleaved in groups of 32 (feature-major SwiGLU then needs one tile).
  constexpr int kNumP = (kSwap && kSwiglu && !kIl) ? 2 : 1;  // lane-side tiles per stage
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int bn = p.bn;
  const int num_q_sf = kSwap ? (bn + 127) / 128 : bn / 128;  // scale atoms cover 128 rows
  const int q_bytes = bn * kTileK;
  const int sf_off = kNumP * kTileBytes + q_bytes;
  const int tx_bytes = sf_off + (kNumP + num_q_sf) * kSfAtom - p.tx_discount;
  const int stage_bytes = (sf_off + (kNumP + num_q_sf) * kSfAtom + 1023) & ~1023;
  const int stages = p.stages;
  const int split = kSwap ? p.split : 1;
  // token columns of the tile this CTA finalises (the last CTAs of an odd-sized cluster own
  // fewer, possibly none)
  const int cols_owned = (bn + split - 1) / split;

  // Receive slots of the K-split exchange. Wide batches have no room for them beside the ring:
  // they then reuse it (recv_off == 0), and one more cluster barrier keeps every CTA's partial
  // sums out of a ring that its owner's MMAs still read.
  float* recv = reinterpret_cast<float*>(smem + p.recv_off);
  const bool recv_in_ring = kSwap && p.recv_off == 0 && split > 1;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + p.bars_off);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kMaxStages + 1);
  const uint32_t full0 = smem_u32(bars);
  const uint32_t empty0 = smem_u32(bars + kMaxStages);
  const uint32_t accum_bar = smem_u32(bars + 2 * kMaxStages);

  // ---- tile coordinates
  int p_row[kNumP];       // first row of each lane-side tile in its tensor
  int q_row[2];           // first row of each column-side TMA box
  int num_q_box = 1;
  int q_box_bytes = q_bytes;
  int m0 = 0, n0 = 0;
  int rank = 0;
  if (kSwap) {
    n0 = blockIdx.x * kTileRows;
    rank = blockIdx.y;
    p_row[0] = n0;
    if (kNumP == 2) p_row[kNumP - 1] = p.n + n0;  // up rows follow the I gate rows
    q_row[0] = 0;
  } else {
    // Raster: panels of panel_m token tiles; inside a panel the token tile varies fastest, so
    // the CTAs resident at one time cover a panel_m x (SMs / panel_m) patch of the output and
    // every operand tile is shared through L2 by a bounded number of CTAs.
    const int tiles_m = (p.m + kTileRows - 1) / kTileRows;
    const int tiles_n = gridDim.x / tiles_m;
    const int per_panel = p.panel_m * tiles_n;
    const int panel = blockIdx.x / per_panel;
    const int in_panel = blockIdx.x - panel * per_panel;
    const int rows_here = min(p.panel_m, tiles_m - panel * p.panel_m);
    const int mt = panel * p.panel_m + in_panel % rows_here;
    const int nt = in_panel / rows_here;
    m0 = mt * kTileRows;
    p_row[0] = m0;
    if (kSwiglu) {
      n0 = nt * 128;  // 128 gate + 128 up rows per tile
      q_row[0] = n0;
      q_row[1] = p.n + n0;
      num_q_box = 2;
      q_box_bytes = kTileBytes;
    } else {
      n0 = nt * bn;
      q_row[0] = n0;
    }
  }
  const int kb_begin = (int)(((long long)rank * p.k_tiles) / split);
  const int kb_end = (int)(((long long)(rank + 1) * p.k_tiles) / split);
  const bool has_k = kb_end > kb_begin;

  // ---- TMEM column plan
  const int acc_cols = kNumP * bn;
  const int sfp_col = acc_cols;
  const int sfq_col = acc_cols + 4 * kNumP;

  // ---- one-time setup
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    mbar_init(accum_bar, 1);
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
  if (kSwap && split > 1) cluster_sync_all();  // every CTA of the cluster is resident
  if (threadIdx.x == 0) pdl_launch_dependents();

  if (warp == 0) {
    // =============================== TMA producer (warp-uniform loop, one elected lane issues)
    const uint64_t pol_w = p.stream_weights ? policy_evict_first() : policy_evict_normal();
    const uint64_t pol_a = policy_evict_last();
    const uint64_t pol_p = kSwap ? pol_w : pol_a;
    const uint64_t pol_q = kSwap ? pol_a : pol_w;
    const uint32_t base0 = smem_u32(smem);
    // Loads of the lane-side operand (P) and of the column-side operand (Q) of one stage.
    auto load_p = [&](int kb, uint32_t base, uint32_t full) {
#pragma unroll
      for (int a = 0; a < kNumP; ++a) {
        tma_load_2d(base + a * kTileBytes, &tm_p, full, kb * kTileK, p_row[a], pol_p);
        bulk_load_1d(base + sf_off + a * kSfAtom,
                     p.sf_p + ((size_t)(p_row[a] >> 7) * p.k_tiles + kb) * kSfAtom, kSfAtom, full);
      }
    };
    auto load_q = [&](int kb, uint32_t base, uint32_t full) {
      for (int j = 0; j < num_q_box; ++j)
        tma_load_2d(base + kNumP * kTileBytes + j * q_box_bytes, &tm_q, full, kb * kTileK, q_row[j],
                    pol_q);
      for (int j = 0; j < num_q_sf; ++j) {
        const int qr = (!kSwap && kSwiglu) ? q_row[j] : q_row[0] + j * 128;
        bulk_load_1d(base + sf_off + (kNumP + j) * kSfAtom,
                     p.sf_q + ((size_t)(qr >> 7) * p.k_tiles + kb) * kSfAtom, kSfAtom, full);
      }
    };
    // The weights do not depend on the preceding kernel: fill the ring with them first, then
    // wait for the predecessor (programmatic dependent launch) and add the activations.
    const int my_kb = kb_end - kb_begin;
    const int pre = min(stages, my_kb);
    if (elect_one()) {
      for (int it = 0; it < pre; ++it) {
        const uint32_t full = full0 + 8 * it;
        mbar_expect_tx(full, (uint32_t)tx_bytes);
        const uint32_t base = base0 + (uint32_t)(it * stage_bytes);
        if (kSwap) load_p(kb_begin + it, base, full); else load_q(kb_begin + it, base, full);
      }
      pdl_wait();
      for (int it = 0; it < pre; ++it) {
        const uint32_t full = full0 + 8 * it;
        const uint32_t base = base0 + (uint32_t)(it * stage_bytes);
        if (kSwap) load_q(kb_begin + it, base, full); else load_p(kb_begin + it, base, full);
      }
    }
    __syncwarp();
    int s = pre % stages;
    uint32_t ph = (pre == stages) ? 1u : 0u;
    for (int it = pre; it < my_kb; ++it) {
      if (!mbar_wait(empty0 + 8 * s, ph ^ 1u, p.status, kWaitEmpty)) break;
      if (elect_one()) {
        const uint32_t full = full0 + 8 * s;
        mbar_expect_tx(full, (uint32_t)tx_bytes);
        const uint32_t base = base0 + (uint32_t)(s * stage_bytes);
        load_p(kb_begin + it, base, full);
        load_q(kb_begin + it, base, full);
      }
      __syncwarp();
      if (++s == stages) { s = 0; ph ^= 1u; }
    }
    if (recv_in_ring) cluster_sync_all();
  } else if (warp == 1) {
    // =============================== MMA issuer (warp-uniform loop, one elected lane issues)
    // The issuing thread bounds the kernel: descriptors are 32-bit low words that only need an
    // add, the instruction descriptors are precomputed and the K sub-steps are unrolled.
    const int k_rem = p.k - (p.k_tiles - 1) * kTileK;
    const int last_subs = k_rem >> 5;
    uint32_t idesc[4];
#pragma unroll
    for (int sub = 0; sub < 4; ++sub) idesc[sub] = idesc_mx_sf(p.idesc, (uint32_t)sub, (uint32_t)sub);
    const uint32_t lo_stage0 = desc_lo(smem_u32(smem));
    const uint32_t lo_step = (uint32_t)stage_bytes >> 4;
    const uint32_t lo_q = (uint32_t)(kNumP * kTileBytes) >> 4;
    const uint32_t lo_sf = (uint32_t)sf_off >> 4;
#ifdef MACH_EXPERIMENTS
    const bool skip_cp = (p.debug & 1) != 0, skip_mma = (p.debug & 2) != 0;
#else
    constexpr bool skip_cp = false, skip_mma = false;
#endif
    int s = 0;
    uint32_t ph = 0;
    for (int kb = kb_begin; kb < kb_end; ++kb) {
      if (!mbar_wait(full0 + 8 * s, ph, p.status, kWaitFull)) break;
      tc_fence_after();
      if (elect_one()) {
        const uint32_t lo = lo_stage0 + (uint32_t)s * lo_step;
        if (!skip_cp) {
#pragma unroll
          for (int a = 0; a < kNumP; ++a)
            tc_cp_sf_lo(tmem_base + sfp_col + 4 * a, lo + lo_sf + 32u * (uint32_t)a);
          for (int j = 0; j < num_q_sf; ++j)
            tc_cp_sf_lo(tmem_base + sfq_col + 4 * j, lo + lo_sf + 32u * (uint32_t)(kNumP + j));
        }
        uint32_t acc = kb > kb_begin ? 1u : 0u;
        if (!skip_mma) {
          if (kb + 1 < p.k_tiles || last_subs == 4) {
#pragma unroll
            for (int sub = 0; sub < 4; ++sub) {
#pragma unroll
              for (int a = 0; a < kNumP; ++a)
                tc_mma_mx_lo(tmem_base + a * bn, lo + (uint32_t)(a * (kTileBytes >> 4)) + 2 * sub,
                             lo + lo_q + 2 * sub, idesc[sub], acc, tmem_base + sfp_col + 4 * a,
                             tmem_base + sfq_col);
              acc = 1;
            }
          } else {
            for (int sub = 0; sub < last_subs; ++sub) {
#pragma unroll
              for (int a = 0; a < kNumP; ++a)
                tc_mma_mx_lo(tmem_base + a * bn, lo + (uint32_t)(a * (kTileBytes >> 4)) + 2 * sub,
                             lo + lo_q + 2 * sub, idesc[sub], acc, tmem_base + sfp_col + 4 * a,
                             tmem_base + sfq_col);
              acc = 1;
            }
          }
        }
        tc_commit(empty0 + 8 * s);  // frees the stage once these MMAs have read it
      }
      __syncwarp();
      if (++s == stages) { s = 0; ph ^= 1u; }
    }
    if (elect_one()) tc_commit(accum_bar);
    __syncwarp();
    if (recv_in_ring) cluster_sync_all();
  } else {
    // =============================== epilogue warps
    const int quad = warp & 3;
    const uint32_t t_lane = tmem_base + ((uint32_t)(quad * 32) << 16);
    const bool ready = mbar_wait(accum_bar, 0, p.status, kWaitAccum);
    tc_fence_after();
    // every CTA of the cluster has finished reading its ring (its accumulator is complete)
    if (recv_in_ring) cluster_sync_all();
    if (!kSwap) {
      const int row = m0 + quad * 32 + lane;
      if (!kSwiglu) {
        __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.out);
        for (int c = 0; c < bn; c += 32) {
          uint32_t r[32];
          tmem_ld_x32(t_lane + c, r);
          tmem_ld_wait();
          const int n = n0 + c;
          if (ready && row < p.m && n < p.n) {
            uint32_t w[16];
#pragma unroll
            for (int i = 0; i < 16; ++i)
              w[i] = pack_bf16x2(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
            uint4* dst = reinterpret_cast<uint4*>(out + (size_t)row * p.n + n);
            dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
            dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
            if (n + 32 <= p.n) {
              dst[2] = make_uint4(w[8], w[9], w[10], w[11]);
              dst[3] = make_uint4(w[12], w[13], w[14], w[15]);
            }
          }
        }
      } else {
        uint8_t* codes = reinterpret_cast<uint8_t*>(p.out);
        for (int c = 0; c < 128; c += 32) {
          uint32_t g[32], u[32];
          tmem_ld_x32(t_lane + c, g);
          tmem_ld_x32(t_lane + 128 + c, u);
          tmem_ld_wait();
          const int col = n0 + c;  // index into I
          if (ready && row < p.m && col < p.n) {
            float v[32];
            float amax = 0.0f;
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              v[i] = swiglu_bf16(bf16_round(__uint_as_float(g[i])),
                                 bf16_round(__uint_as_float(u[i])));
              amax = fmaxf(amax, fabsf(v[i]));
            }
            const uint32_t bits = mx_scale_bits(amax);
            const float inv = mx_inverse(bits);
            uint32_t w[8];
#pragma unroll
            for (int i = 0; i < 8; ++i)
              w[i] = e4m3x4(__fmul_rn(v[4 * i], inv), __fmul_rn(v[4 * i + 1], inv),
                            __fmul_rn(v[4 * i + 2], inv), __fmul_rn(v[4 * i + 3], inv));
            uint4* dst = reinterpret_cast<uint4*>(codes + (size_t)row * p.n + col);
            dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
            dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
            p.out_sf[sf_offset(row, col >> 5, p.out_k_tiles)] = (uint8_t)(bits >> 23);
          }
        }
      }
    } else {
      // Feature-major: every CTA of the cluster owns bn / split token columns of the tile and
      // receives, from each CTA, that CTA's partial sums for them
      // (recv[tile][source rank][owned column][128 rows], row fastest).
      const int row = quad * 32 + lane;  // row inside the 128-row tile
      const uint32_t recv_local = smem_u32(recv);
#pragma unroll
      for (int a = 0; a < kNumP; ++a) {
        for (int c = 0; c < bn; c += 16) {
          uint32_t r[16];
          if (has_k) {
            tmem_ld_x16(t_lane + a * bn + c, r);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) r[i] = 0u;
          }
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const int col = c + i;
            const int owner = col / cols_owned;
            const int cl = col - owner * cols_owned;
            const uint32_t off =
                (uint32_t)((((a * split + rank) * cols_owned + cl) * kTileRows + row) * 4);
            const uint32_t dst =
                split > 1 ? map_to_cta(recv_local + off, (uint32_t)owner) : recv_local + off;
            st_cluster_f32(dst, __uint_as_float(r[i]));
          }
        }
      }
    }
    tc_fence_before();
  }

  if (kSwap) {
    // All partials of every CTA are in place after this barrier.
    if (split > 1) cluster_sync_all(); else __syncthreads();
    if (warp >= 2) {
      const int et = threadIdx.x - 64;  // 0..127
      if (!kSwiglu) {
        __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.out);
        // Logical output column of physical weight row n0 + et.
        const int r_phys = n0 + et;
        int n = r_phys;
        if (p.interleaved)
          n = ((r_phys >> 5) & 1) * (p.n >> 1) + ((r_phys >> 6) << 5) + (r_phys & 31);
        for (int cl = 0; cl < cols_owned; ++cl) {
          float acc = 0.0f;
          for (int c = 0; c < split; ++c)
            acc = __fadd_rn(acc, recv[((size_t)c * cols_owned + cl) * kTileRows + et]);
          const int col = rank * cols_owned + cl;
          if (col < p.m && r_phys < p.n) out[(size_t)col * p.n + n] = __float2bfloat16_rn(acc);
        }
      } else {
        uint8_t* codes = reinterpret_cast<uint8_t*>(p.out);
        // Rows layout: two tiles (gate, up) of 128 features -> 4 blocks of 32 per token.
        // Interleaved layout: one tile of 64 features -> 2 blocks; gate rows 64g.., up 64g+32..
        constexpr int kGroups = kIl ? 2 : 4;
        const int units = kGroups * cols_owned;
        for (int unit = (warp - 2); unit < units; unit += 4) {
          const int cl = unit / kGroups;
          const int g = unit - cl * kGroups;
          const int g_row = kIl ? 64 * g + lane : 32 * g + lane;
          const int u_row = kIl ? g_row + 32 : g_row;
          float gate = 0.0f, up = 0.0f;
          for (int c = 0; c < split; ++c) {
            gate = __fadd_rn(gate, recv[((size_t)c * cols_owned + cl) * kTileRows + g_row]);
            up = __fadd_rn(up, recv[((size_t)((kIl ? 0 : split) + c) * cols_owned + cl) * kTileRows +
                                    u_row]);
          }
          const float v = swiglu_bf16(bf16_round(gate), bf16_round(up));
          float amax = fabsf(v);
#pragma unroll
          for (int d = 16; d > 0; d >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, d));
          const uint32_t bits = mx_scale_bits(amax);
          const float q = __fmul_rn(v, mx_inverse(bits));
          const int feat = (kIl ? (n0 >> 1) : n0) + 32 * g + lane;
          const int col = rank * cols_owned + cl;
          if (col < p.m && feat < p.n) {
            codes[(size_t)col * p.n + feat] = (uint8_t)(e4m3x2(q, 0.0f) & 0xFFu);
            if (lane == 0) p.out_sf[sf_offset(col, feat >> 5, p.out_k_tiles)] = (uint8_t)(bits >> 23);
          }
        }
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

}  // namespace

// ------------------------------------------------------------------ host side

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) ==
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  });
  return fn;
}

// K-major operand [rows, K] of 8-bit codes, or packed 6-bit codes (4 per 3 bytes).
int make_operand_map(CUtensorMap* map, const void* base, int64_t rows, int64_t k, int format,
                     int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(MACH_ERR_CUDA, "cuTensorMapEncodeTiled is not available");
  const bool six = format == MACH_FMT_E2M3 || format == MACH_FMT_E3M2;
  const cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)(six ? k * 3 / 4 : k)};
  const cuuint32_t box[2] = {(cuuint32_t)kTileK, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = fn(map, six ? CU_TENSOR_MAP_DATA_TYPE_16U6_ALIGN16B : CU_TENSOR_MAP_DATA_TYPE_UINT8,
                        2, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(MACH_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d)", (int)r);
  return MACH_OK;
}

// Swizzled scale buffer as a 2-D tensor [atoms, 128 x u32]: one 512-byte atom per row.
int make_sf_map(CUtensorMap* map, const void* base, int64_t atoms) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(MACH_ERR_CUDA, "cuTensorMapEncodeTiled is not available");
  const cuuint64_t dims[2] = {128, (cuuint64_t)atoms};
  const cuuint64_t strides[1] = {512};
  const cuuint32_t box[2] = {128, 1};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(base), dims,
                        strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(MACH_ERR_CUDA, "cuTensorMapEncodeTiled(sf) failed (%d)", (int)r);
  return MACH_OK;
}

// Row-major BF16 matrix [rows, cols] as the destination of TMA stores: boxes of 64 columns
// (128 bytes, 128-byte swizzle) x box_rows rows.
int make_bf16_store_map(CUtensorMap* map, const void* base, int64_t rows, int64_t cols,
                        int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(MACH_ERR_CUDA, "cuTensorMapEncodeTiled is not available");
  const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
  const cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims,
                        strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(MACH_ERR_CUDA, "cuTensorMapEncodeTiled(store) failed (%d)", (int)r);
  return MACH_OK;
}

int run_mx_gemm_pair(const TmGemmArgs& args, cudaStream_t stream);
int run_mx_gemm_mid(const TmGemmArgs& args, cudaStream_t stream);
bool mx_gemm_mid_fits(int64_t m, int64_t w_rows);
int last_pair_count();

namespace {

struct Tuning {
  int force_split = 0;     // feature-major cluster size (0 = heuristic)
  int split_fill_pct = 0;  // heuristic: grow the cluster until CTAs >= this % of the SM count (0 = choose)
  int force_stages = 0;    // pipeline depth (0 = fill shared memory)
  int force_bn = 0;        // token-major N tile (0 = heuristic)
  int swap_max_m = 256;    // largest batch handled feature-major (further limited by shape)
  int smem_cap_kb = 0;     // cap on dynamic smem per CTA in KiB (0 = device limit)
  int panel_m = 0;         // token-major raster panel height in tiles (0 = heuristic)
  int debug = 0;           // experiment bits (see MxGemmParams::debug)
  int moe_ctas_per_sm = 0; // grouped GEMM residency (0 = heuristic)
  int moe_token_major = 1; // 0: every MoE work item takes the feature-major kernel
  int moe_tm_min_rows = 0; // fewest rows of a token-major work item (0 or 1 = all of them)
  int tm_min_m = 65;       // smallest batch routed to the persistent 256-token kernels
  int tm_bn = 0;           // its tile width in weight rows (0 = 192)
  int pair = -1;           // large batches: 1 or -1 (default) = cta_group::2 kernel,
                           // 0 = single-CTA persistent kernel
  int mid = 1;             // 0: batches of 49..128 tokens skip the one-token-tile kernel
  int narrow_max_m = 256;  // largest batch a narrow plain GEMM runs feature-major
  int wide_max_m = 0;      // largest batch a wide GEMM runs feature-major (0 = heuristic)
};
Tuning g_tune;

}  // namespace

int tuned_split() { return g_tune.force_split; }
int tuned_stages() { return g_tune.force_stages; }
int tuned_pair() { return g_tune.pair; }
int tuned_debug() { return g_tune.debug; }
int tuned_moe_ctas_per_sm() { return g_tune.moe_ctas_per_sm; }
int tuned_moe_token_major() { return g_tune.moe_token_major; }
int tuned_moe_tm_min_rows() { return g_tune.moe_tm_min_rows; }
int tuned_tile_width() { return g_tune.tm_bn; }

namespace {

int next_pow2_cols(int cols) {
  int c = 32;
  while (c < cols) c <<= 1;
  return c;
}

template <bool kSwap, bool kSwiglu, bool kIl>
int launch(const CUtensorMap& tm_p, const CUtensorMap& tm_q, MxGemmParams& prm, dim3 grid,
           int smem_bytes, cudaStream_t stream) {
  auto kernel = mx_gemm_kernel<kSwap, kSwiglu, kIl>;
  if (!ensure_smem_optin(reinterpret_cast<const void*>(kernel)))
    return fail(MACH_ERR_CUDA, "mx_gemm: cannot opt in to %d B of shared memory", max_smem_optin());
  const cudaError_t e =
      launch_ex(kernel, grid, dim3(kThreads), (size_t)smem_bytes, stream,
                dim3(1, (kSwap && prm.split > 1) ? (unsigned)prm.split : 1u, 1), pdl_enabled(), tm_p,
                tm_q, prm);
  if (e != cudaSuccess) return fail(MACH_ERR_CUDA, "mx_gemm launch: %s", cudaGetErrorString(e));
  return MACH_OK;
}

// Tile width of the cta_group::2 kernel. Model fitted to CUDA-event timings on B200
// (M = 128..4096, N = 2560 / 19456, K = 2560 / 9728): a K step of a 256 x bn pair tile costs
// about 0.22 + 0.00105 * bn microseconds (operand delivery from L2 and instruction issue), and
// tiles wider than 192 have a single TMEM buffer, so their epilogue (about 0.0155 * bn us) is
// exposed once per tile. The grid is persistent, so time = rounds * tile time.
int pick_pair_bn(int64_t m, int64_t w_rows, int64_t k, bool swiglu) {
  if (swiglu) return 192;  // the SwiGLU epilogue needs the double buffer to stay hidden
  const int64_t pairs = std::max(1, sm_count() / 2);
  const int64_t tiles_m = (m + 255) / 256;
  const double k_steps = (double)((k + 127) / 128);
  int best = 192;
  double best_t = 1e30;
  for (int bn : {128, 192, 256, 320, 384, 448}) {
    const int64_t tiles = tiles_m * ((w_rows + bn - 1) / bn);
    const double rounds = (double)((tiles + pairs - 1) / pairs);
    const double t = rounds * (k_steps * (0.22 + 0.00105 * bn) + (bn > 192 ? 0.0155 * bn : 0.0));
    if (t < best_t - 1e-9) { best_t = t; best = bn; }
  }
  return best;
}

// Shared launcher. `n` is N (plain) or I (SwiGLU; the weight then has 2I rows).
int run_mx_gemm(const void* a_codes, const void* a_sf, const void* w, const void* w_sf, void* out,
                void* out_sf, int64_t m, int64_t n, int64_t k, int w_format, bool swiglu,
                int w_layout, cudaStream_t stream, const ScatterTarget* scatter = nullptr) {
  const char* what = swiglu ? "mx_gemm_swiglu" : (scatter ? "mx_gemm_reduce_scatter" : "mx_gemm");
  if (m < 0 || n < 0 || k < 0) return fail(MACH_ERR_INVALID, "%s: negative size", what);
  if (m == 0 || n == 0) return MACH_OK;
  if (!a_codes || !a_sf || !w || !w_sf || (!out && !scatter) || (swiglu && !out_sf))
    return fail(MACH_ERR_INVALID, "%s: null pointer", what);
  if (w_format != MACH_FMT_E4M3 && w_format != MACH_FMT_E2M3 && w_format != MACH_FMT_E3M2)
    return fail(MACH_ERR_INVALID, "%s: unknown weight format %d", what, w_format);
  const bool six = w_format != MACH_FMT_E4M3;
  if (k < 32 || k % 32 || (six && k % 128))
    return fail(MACH_ERR_UNSUPPORTED, "%s: K must be a positive multiple of 32 (128 for 6-bit)", what);
  if (swiglu ? (n % (w_layout == MACH_LAYOUT_GATE_UP_32 ? 32 : 128) != 0) : (n % 16 != 0))
    return fail(MACH_ERR_UNSUPPORTED,
                "%s: N %% 16 (SwiGLU: I %% 128, or I %% 32 with interleaved rows) required", what);
  if (k % 16 || !aligned16(a_codes) || !aligned16(a_sf) || !aligned16(w_sf) || !aligned16(out) ||
      (reinterpret_cast<uintptr_t>(w) & (six ? 31 : 15)))
    return fail(MACH_ERR_UNSUPPORTED, "%s: 16-byte aligned operands required (32 for 6-bit)", what);
  if (m > (1 << 24) || n > (1 << 24) || k > (1 << 24))
    return fail(MACH_ERR_UNSUPPORTED, "%s: dimension too large", what);

  if (w_layout != MACH_LAYOUT_ROWS && w_layout != MACH_LAYOUT_GATE_UP_32)
    return fail(MACH_ERR_INVALID, "%s: unknown weight layout %d", what, w_layout);
  const bool interleaved = w_layout == MACH_LAYOUT_GATE_UP_32;
  if (interleaved && (swiglu ? n % 32 : n % 64))
    return fail(MACH_ERR_UNSUPPORTED, "%s: interleaved gate_up needs I %% 32 == 0", what);
  const int64_t w_rows = swiglu ? 2 * n : n;
  // Which orientation. Feature-major (weights on the 128-row side, cluster split-K) wins while
  // the batch is a small MMA-N; measured on B200 (graph replay, us):
  //   19456 x 2560 interleaved gate_up + SwiGLU   M = 32: 17.2 feature-major / 20.3 one token tile
  //                                               M = 40: 20.3 / 20.0      M = 48: 20.3 / 19.1
  //                                               M = 64: 22.7 / 17.5
  //   19456 x 2560 plain rows, BF16 out           M = 32: 15.0 / 15.6      M = 48: 17.3 / 15.3
  //                                               M = 64: 22.9 / 13.9
  //   2560 x 9728 (narrow: too few tiles for the token-major kernels)
  //                                               M = 192: 20.3 / 29 (pair)   M = 256: 24.9 / 28.1
  const bool narrow = !swiglu && (n + 127) / 128 * 4 <= sm_count();
  const bool mid_layout = interleaved || !swiglu;   // layouts the one-token-tile kernel takes
  const bool mid_shape = g_tune.mid != 0 && !scatter && mid_layout && mx_gemm_mid_fits(128, w_rows);
  const int64_t wide_max = g_tune.wide_max_m > 0 ? g_tune.wide_max_m
                           : mid_shape ? 32
                           : (swiglu && interleaved) ? 48 : 64;
  const bool swap =
      m <= g_tune.swap_max_m && (m <= wide_max || (narrow && m <= g_tune.narrow_max_m));
  const bool token_major_pair =
      ((!swap && m >= g_tune.tm_min_m && (!swiglu || interleaved)) || (interleaved && !swap));
  if (scatter && (!token_major_pair || g_tune.pair == 0))
    return fail(MACH_ERR_UNSUPPORTED,
                "%s: this shape does not take the CTA-pair kernel; run the plain GEMM and the "
                "all-reduce separately", what);
  // One token tile and a weight matrix wide enough to give every SM its own rows: balanced
  // variable-width tiles in one round (measured on B200 against the 256-token pair tiles).
  const bool one_tile = !swap && mid_shape && mx_gemm_mid_fits(m, w_rows);
  if (token_major_pair || one_tile) {
    TmGemmArgs args = {};
    args.scatter = scatter;
    args.a_codes = a_codes; args.a_sf = a_sf; args.w = w; args.w_sf = w_sf;
    args.out = out; args.out_sf = out_sf;
    args.m = m; args.w_rows = w_rows; args.k = k; args.w_format = w_format;
    args.swiglu = swiglu; args.interleaved = interleaved;
    args.bn = g_tune.tm_bn > 0 ? g_tune.tm_bn : (g_tune.pair != 0 ? pick_pair_bn(m, w_rows, k, swiglu) : 192);
    // Peer stores from the epilogue must overlap the next tile's MMAs: keep the double buffer.
    if (scatter && g_tune.tm_bn == 0) args.bn = std::min(args.bn, 192);
    args.stages = g_tune.force_stages; args.panel_m = g_tune.panel_m;
    args.debug = g_tune.debug;
    args.smem_cap_kb = g_tune.smem_cap_kb;
    if (one_tile) return run_mx_gemm_mid(args, stream);
    const bool pair = g_tune.pair != 0;
    return pair ? run_mx_gemm_pair(args, stream) : run_mx_gemm_tm(args, stream);
  }

  MxGemmParams prm = {};
  prm.out = out;
  prm.out_sf = reinterpret_cast<uint8_t*>(out_sf);
  prm.status = device_status_ptr();
  if (!prm.status) return fail(MACH_ERR_CUDA, "%s: cannot resolve the device status word", what);
  prm.m = (int)m;
  prm.n = (int)n;
  prm.k = (int)k;
  prm.k_tiles = (int)((k + 127) / 128);
  prm.out_k_tiles = (int)((n + 127) / 128);

  const int num_p = (swap && swiglu && !interleaved) ? 2 : 1;
  prm.interleaved = interleaved ? 1 : 0;
  int bn;
  dim3 grid;
  int64_t tiles;
  if (swap) {
    bn = (int)((m + 15) / 16) * 16;
    tiles = ((swiglu && interleaved ? 2 * n : n) + 127) / 128;
    // Cluster split along K: enough CTAs to cover every SM, at most 8, never more than the
    // K tiles; each CTA of the cluster finalises bn / split token columns.
    const int max_split = 8;
    int split = 1;
    if (g_tune.force_split > 0) {
      split = g_tune.force_split;
    } else {
      // Measured on B200: about two CTAs per SM (each with a short ring) stream weights faster
      // than one CTA per SM with a deep ring, and finer pieces balance better over 148 SMs.
      // Fewer tiles than SMs (narrow N): stop at 1.25 CTAs per SM. Measured on B200, 6144 x 2048
      // at M = 16: 5.3 us with 4 CTAs per cluster (192 CTAs) against 6.3 us with 8 (384); with
      // at least one tile per SM the second CTA per SM pays (34816 x 5120: 25.7 us against 29).
      const int fill_pct = g_tune.split_fill_pct > 0 ? g_tune.split_fill_pct
                                                     : (tiles >= sm_count() ? 200 : 125);
      while (split < max_split && tiles * split * 100 < (int64_t)fill_pct * sm_count()) split <<= 1;
    }
    split = std::min(split, max_split);
    while (split > 1 && split > prm.k_tiles) split >>= 1;
    if (split < 1 || split > max_split)
      return fail(MACH_ERR_INVALID, "%s: cluster split must be 1..8", what);
    prm.split = split;
    grid = dim3((unsigned)tiles, (unsigned)split, 1);
    prm.stream_weights = 1;
  } else {
    if (swiglu) {
      bn = 256;
      tiles = ((m + 127) / 128) * (n / 128);
    } else {
      bn = g_tune.force_bn > 0 ? g_tune.force_bn : 256;
      if (bn != 128 && bn != 256) return fail(MACH_ERR_INVALID, "%s: bn must be 128 or 256", what);
      if (g_tune.force_bn == 0 && ((m + 127) / 128) * ((n + 255) / 256) < sm_count()) bn = 128;
      tiles = ((m + 127) / 128) * ((n + bn - 1) / bn);
    }
    prm.split = 1;
    prm.panel_m = g_tune.panel_m > 0 ? g_tune.panel_m : 16;
    grid = dim3((unsigned)tiles, 1, 1);
    prm.stream_weights = (m <= 128) ? 1 : 0;
  }
  prm.bn = bn;
  const int num_q_sf = swap ? (bn + 127) / 128 : bn / 128;
  const int acc_cols = num_p * bn;
  prm.debug = g_tune.debug;
  prm.tmem_cols = next_pow2_cols(acc_cols + 2 * (4 * num_p + 4 * num_q_sf));
  if (prm.tmem_cols > 512) return fail(MACH_ERR_UNSUPPORTED, "%s: TMEM plan exceeds 512 columns", what);

  // A packed 6-bit box completes 96 transaction bytes per 128-element row (the bytes read
  // from global memory), although it occupies 128 bytes of shared memory.
  prm.tx_discount = six ? (swap ? num_p * kTileRows : bn) * 32 : 0;
  const uint32_t w_fmt = (uint32_t)w_format;
  prm.idesc = swap ? idesc_mx(w_fmt, kFmtE4M3, (uint32_t)bn) : idesc_mx(kFmtE4M3, w_fmt, (uint32_t)bn);

  // Shared memory plan: [stages][recv][barriers + TMEM slot] (+ 1 KiB alignment slack).
  const int tx = num_p * kTileBytes + bn * kTileK + (num_p + num_q_sf) * kSfAtom;
  const int stage_bytes = (tx + 1023) & ~1023;
  // receive slots: [tile][source rank][owned column][128 rows]; sized for the largest cluster
  // the heuristic below may still shrink to, so the plan does not depend on that choice
  const int recv_bytes = swap ? num_p * kTileRows * (bn + 7) * 4 : 0;
  const int tail = (2 * kMaxStages + 1) * 8 + 16 + 1024;
  // Wide batches: two stages and the receive slots do not fit side by side; the slots then
  // reuse the ring once every CTA of the cluster has finished its MMAs.
  const bool reuse_ring = swap && 2 * stage_bytes + recv_bytes + tail > max_smem_optin();
  auto plan_bytes = [&](int st) {
    return (reuse_ring ? std::max(st * stage_bytes, recv_bytes) : st * stage_bytes + recv_bytes) + tail;
  };
  int budget = max_smem_optin();
  // Feature-major CTAs stay small (three per SM) so that every CTA of the grid is resident at
  // once and a dependent kernel finds room to prefetch its weights.
  // Grids of at most two CTAs per SM may take half an SM each: measured on B200, 2560 x 9728 at
  // M = 16 (160 CTAs): 7.1 us with five stages in 110 KB against 7.6 us with three in 70 KB.
  const int small_cta = tiles * prm.split <= 2 * (int64_t)sm_count() ? 110 * 1024 : 70 * 1024;
  if (swap && !reuse_ring) budget = std::min(budget, std::max(small_cta, plan_bytes(3)));
  if (g_tune.smem_cap_kb > 0) budget = std::min(max_smem_optin(), g_tune.smem_cap_kb * 1024);
  int stages = std::min(kMaxStages, g_tune.force_stages > 0 ? g_tune.force_stages : kMaxStages);
  while (stages > 1 && plan_bytes(stages) > budget) --stages;
  if (plan_bytes(stages) > max_smem_optin())
    return fail(MACH_ERR_UNSUPPORTED, "%s: tile does not fit in shared memory", what);
  stages = std::max(1, std::min(stages, swap ? (prm.k_tiles + prm.split - 1) / prm.split : prm.k_tiles));
  // Co-resident CTAs must never over-subscribe TMEM: a CTA blocked in tcgen05.alloc while a
  // cluster peer waits for it could deadlock. Pad shared memory until residency is safe.
  auto padded_bytes = [&](int st) {
    const int max_resident = 512 / prm.tmem_cols;
    const int sm_smem = 228 * 1024;
    int bytes = plan_bytes(st);
    if ((sm_smem / (bytes + 1024)) > max_resident) bytes = sm_smem / (max_resident + 1) + 1;
    return bytes;
  };
  const void* kfn =
      !swap ? (swiglu ? reinterpret_cast<const void*>(mx_gemm_kernel<false, true, false>)
                      : reinterpret_cast<const void*>(mx_gemm_kernel<false, false, false>))
            : (!swiglu ? reinterpret_cast<const void*>(mx_gemm_kernel<true, false, false>)
                       : (interleaved ? reinterpret_cast<const void*>(mx_gemm_kernel<true, true, true>)
                                      : reinterpret_cast<const void*>(mx_gemm_kernel<true, true, false>)));
  if (swap && g_tune.force_split == 0) {
    // Every CTA of the grid should be resident at once (a second, nearly empty wave doubles
    // the time of a 10 us kernel). With one CTA per SM a cluster must also find its SMs inside
    // one GPC, so there the device is asked how many clusters of the size it keeps resident
    // (fewer than SMs / size). First give up ring depth (two stages per CTA still leave
    // several stages in flight per SM), only then shrink the cluster.
    auto fits = [&](int st, int sp) {
      const int bytes = padded_bytes(st);
      const int per_sm = std::max(1, std::min((228 * 1024) / (bytes + 1024), 512 / prm.tmem_cols));
      if (tiles * sp > (int64_t)per_sm * sm_count()) return false;
      if (per_sm == 1 && sp > 1) return tiles <= active_clusters(kfn, kThreads, bytes, sp);
      return true;
    };
    if (!fits(stages, prm.split) && stages > 2 && g_tune.force_stages == 0 && fits(2, prm.split))
      stages = 2;
    while (prm.split > 1 && !fits(stages, prm.split)) --prm.split;
    stages = std::max(1, std::min(stages, (prm.k_tiles + prm.split - 1) / prm.split));
    grid = dim3((unsigned)tiles, (unsigned)prm.split, 1);
  }
  prm.stages = stages;
  const int smem_bytes = padded_bytes(stages);
  prm.recv_off = reuse_ring ? 0 : stages * stage_bytes;
  prm.bars_off = plan_bytes(stages) - tail;
  if (smem_bytes > max_smem_optin())
    return fail(MACH_ERR_UNSUPPORTED, "%s: shared memory plan exceeds the device limit", what);

  CUtensorMap tm_act, tm_w;
  const int act_box = swap ? bn : kTileRows;
  const int w_box = swap ? kTileRows : (swiglu ? 128 : bn);
  int rc = make_operand_map(&tm_act, a_codes, m, k, MACH_FMT_E4M3, act_box);
  if (rc) return rc;
  rc = make_operand_map(&tm_w, w, w_rows, k, w_format, w_box);
  if (rc) return rc;
  const uint8_t* sf_act = reinterpret_cast<const uint8_t*>(a_sf);
  const uint8_t* sf_w = reinterpret_cast<const uint8_t*>(w_sf);
  prm.sf_p = swap ? sf_w : sf_act;
  prm.sf_q = swap ? sf_act : sf_w;
  const CUtensorMap& tm_p = swap ? tm_w : tm_act;
  const CUtensorMap& tm_q = swap ? tm_act : tm_w;
  if (swap) {
    if (!swiglu) return launch<true, false, false>(tm_p, tm_q, prm, grid, smem_bytes, stream);
    return interleaved ? launch<true, true, true>(tm_p, tm_q, prm, grid, smem_bytes, stream)
                       : launch<true, true, false>(tm_p, tm_q, prm, grid, smem_bytes, stream);
  }
  return swiglu ? launch<false, true, false>(tm_p, tm_q, prm, grid, smem_bytes, stream)
                : launch<false, false, false>(tm_p, tm_q, prm, grid, smem_bytes, stream);
}

}  // namespace

}  // namespace mach

extern "C" int mach_mx_gemm(const void* a_codes, const void* a_scales, const void* w,
                            const void* w_scales, void* out, int64_t m, int64_t n, int64_t k,
                            int w_format, int w_layout, void* stream) {
  return mach::run_mx_gemm(a_codes, a_scales, w, w_scales, out, nullptr, m, n, k, w_format, false,
                           w_layout, (cudaStream_t)stream);
}

namespace mach {
int ar_scatter_target(void* workspace, int64_t m, int64_t h, ScatterTarget* out);
}

extern "C" int mach_mx_gemm_reduce_scatter(void* ar_workspace, const void* a_codes,
                                           const void* a_scales, const void* w,
                                           const void* w_scales, int64_t m, int64_t n, int64_t k,
                                           int w_format, void* stream) {
  mach::ScatterTarget target;
  const int rc = mach::ar_scatter_target(ar_workspace, m, n, &target);
  if (rc) return rc;
  return mach::run_mx_gemm(a_codes, a_scales, w, w_scales, nullptr, nullptr, m, n, k, w_format,
                           false, MACH_LAYOUT_ROWS, (cudaStream_t)stream, &target);
}

extern "C" int mach_mx_gemm_swiglu(const void* a_codes, const void* a_scales, const void* w,
                                   const void* w_scales, void* out_codes, void* out_scales,
                                   int64_t m, int64_t i, int64_t k, int w_format, int w_layout,
                                   void* stream) {
  return mach::run_mx_gemm(a_codes, a_scales, w, w_scales, out_codes, out_scales, m, i, k,
                           w_format, true, w_layout, (cudaStream_t)stream);
}

extern "C" int mach_tune_get(const char* name) {
  if (name && !strcmp(name, "last_pairs")) return mach::last_pair_count();
  return -1;
}

extern "C" int mach_tune_set(const char* name, int value) {
  using mach::g_tune;
  if (!name) return mach::fail(MACH_ERR_INVALID, "tune_set: null name");
  if (!strcmp(name, "split")) g_tune.force_split = value;
  else if (!strcmp(name, "split_fill_pct")) g_tune.split_fill_pct = value;
  else if (!strcmp(name, "stages")) g_tune.force_stages = value;
  else if (!strcmp(name, "bn")) g_tune.force_bn = value;
  else if (!strcmp(name, "swap_max_m")) g_tune.swap_max_m = value;
  else if (!strcmp(name, "smem_cap_kb")) g_tune.smem_cap_kb = value;
  else if (!strcmp(name, "panel_m")) g_tune.panel_m = value;
#ifdef MACH_EXPERIMENTS
  else if (!strcmp(name, "debug")) g_tune.debug = value;
#endif
  else if (!strcmp(name, "moe_ctas_per_sm")) g_tune.moe_ctas_per_sm = value;
  else if (!strcmp(name, "moe_token_major")) g_tune.moe_token_major = value;
  else if (!strcmp(name, "moe_tm_min_rows")) g_tune.moe_tm_min_rows = value;
  else if (!strcmp(name, "tm_min_m")) g_tune.tm_min_m = value > 0 ? value : 65;
  else if (!strcmp(name, "tm_bn")) g_tune.tm_bn = value;
  else if (!strcmp(name, "pair")) g_tune.pair = value;  // pass -1 for the default
  else if (!strcmp(name, "mid")) g_tune.mid = value;
  else if (!strcmp(name, "narrow_max_m")) g_tune.narrow_max_m = value;
  else if (!strcmp(name, "wide_max_m")) g_tune.wide_max_m = value;
  else if (!strcmp(name, "pdl")) mach::set_pdl_enabled(value != 0);
  else return mach::fail(MACH_ERR_INVALID, "tune_set: unknown knob '%s'", name);
  return MACH_OK;
}
