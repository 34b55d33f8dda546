// Row-parallel all-reduce fused with residual add + RMSNorm (+ MXFP8 requant) over NVLink
// peer memory. One process per GPU; every rank owns one communication buffer that all
// ranks map (CUDA IPC). No multicast, no TMA on peer memory.
//
//   one-shot (small payloads, or 2 ranks): each rank stores its whole partial [M, H] into
//     every peer, then sums the `world` copies in rank order.
//   two-shot: rows are owned by ranks in contiguous blocks. (1) each rank stores the rows a
//     peer owns into that peer; (2) the owner sums its rows in rank order, rounds to BF16 and
//     stores the sum into every rank; (3) every rank adds the residual and normalises all
//     rows locally.
//   owner form (row ownership between norms, native/owner_prefill/owner.cu:64-160 of the
//     reference): the partial sums sit in each rank's own buffer (the producing GEMM writes
//     them there); after one flag exchange every owner PULLS its rows from all ranks with
//     plain peer loads, sums them in rank order, adds its rows of the residual, normalises
//     and quantises them; after a second flag exchange every rank pulls the other owners'
//     E4M3 codes and E8M0 scales (1.03 bytes per element instead of 2). The residual and the
//     BF16 norm stay with the owner.
//
// Rounding points follow the reference's fused kernel
// (native/ar_norm/trtllm_allreduce_fusion_mxfp8.cuh:1470-1494, 1092-1108, 1303-1342):
//   a = bf16(sum_r f32(x_r)), rank order; res = bf16(f32(a) + f32(residual));
//   norm = bf16(f32(res) * rsqrt(mean(res^2) + eps) * (weight_bias + gamma)); MXFP8 of norm.
//
// Synchronisation: flags are `epoch + 1` values written with system-scope release stores into
// the destination's buffer and polled there with acquire loads. Every wait is bounded (the
// workspace's wait limit, about one second by default). A wait that gives up records a code in
// the device status word, marks the workspace as failed (every later call on it returns
// poisoned outputs at once, without waiting, until mach_ar_reset) and the CTA writes NaN
// (BF16), 0x7F (E4M3) and 0xFF (E8M0) into the outputs it is responsible for, so that a late
// or dead peer can never yield plausible-looking activations. The epoch lives in the buffer
// and is advanced by the last CTA to finish, so a CUDA-graph replay sees fresh values. The
// push forms alternate their data area with the epoch parity: a rank can only reach epoch n+2
// after every peer has finished reading epoch n.
#include <cuda_bf16.h>
#include <cstring>
#include "gemm_mx_tm.h"
#include "host_util.h"
#include "ptx.cuh"
#include "quant_math.cuh"

namespace mach {

namespace {

constexpr int kMaxWorld = 8;
constexpr int kMaxCtas = 1024;
constexpr size_t kHeaderBytes = 256 + 2 * kMaxWorld * kMaxCtas * sizeof(uint32_t);
// Control words at the head of every buffer.
enum { kCtrlEpoch = 0, kCtrlDone = 1, kCtrlTicketA = 2, kCtrlTicketB = 3, kCtrlFailed = 4 };

enum { kWaitScatter = 401, kWaitGather = 402, kWorkspaceFailed = 403 };

struct ArWorkspace {
  int world, rank;
  int64_t tokens_cap, hidden;
  size_t parity_bytes;          // bytes of one parity half of the push-form data area
  size_t owner_partial_off;     // owner form: BF16 partial sums [tokens_cap, hidden]
  size_t owner_stage_off;       // owner form: codes of ALL rows [tokens_cap, hidden] ...
  size_t owner_scales_off;      // ... and their swizzled scales, written by the rows' owners
  long long wait_cycles;
#ifdef MACH_EXPERIMENTS
  unsigned long long* trace;
#endif
  uint8_t* peers[kMaxWorld];    // peers[rank] is this rank's own buffer
  // hand-off from mach_mx_gemm_reduce_scatter to the reduce that follows it
  int scatter_pending, scattered_one_shot;
  int64_t scattered_m;
};

struct ArParams {
  const __nv_bfloat16* partial;
  const __nv_bfloat16* residual;   // owner form: this rank's rows only
  const __nv_bfloat16* gamma;
  __nv_bfloat16* norm_out;         // owner form: this rank's rows only
  __nv_bfloat16* res_out;          // owner form: this rank's rows only
  uint8_t* codes;
  uint8_t* scales;
  uint8_t* peers[kMaxWorld];
  int* status;
  long long wait_cycles;
  float eps, weight_bias;
  int rank, world, m, h, k_tiles;
  int rows_per_owner;      // two-shot / owner form: ceil(m / world)
  int two_shot;
  int prescattered;        // two-shot: the partial rows are already in the owners' slots
  int coarse;              // two-shot: one flag per (rank, phase) instead of one per CTA
  int owner;               // owner form
  size_t parity_bytes, owner_partial_off, owner_stage_off, owner_scales_off;
#ifdef MACH_EXPERIMENTS
  unsigned long long* trace;  // phase time stamps of CTA 0: [epoch % 64][8] (globaltimer, ns)
#endif
};

#ifdef MACH_EXPERIMENTS
__device__ __forceinline__ void trace_stamp(const ArParams& p, uint32_t epoch, int slot) {
  if (p.trace != nullptr && blockIdx.x == 0 && threadIdx.x == 0) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    p.trace[(epoch & 63u) * 8 + slot] = t;
  }
}
#define MACH_TRACE(p, epoch, slot) trace_stamp(p, epoch, slot)
#else
#define MACH_TRACE(p, epoch, slot)
#endif

struct ArParamsMulti {
  ArParams r[kMaxWorld];
};

// A flag store that follows ONE system-scope fence (`__threadfence_system()`): fence + relaxed
// stores are a release pattern, and every st.release.sys would pay the fence again (measured
// on two B200s: about 2 us per system-scope fence, i.e. 2 us per destination rank).
__device__ __forceinline__ void st_relaxed_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_cg(const void* p) {
  return __ldcg(reinterpret_cast<const uint4*>(p));
}
// Loads of memory another GPU (or another rank's grid) wrote: never served from this SM's L1.
__device__ __forceinline__ uint4 ld_peer16(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ld_peer4(const void* p) {
  uint32_t v;
  asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ld_peer1(const void* p) {
  uint32_t v;
  asm volatile("ld.relaxed.sys.global.u8 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Buffer layout: control words ... 256 B | scatter flags [world][kMaxCtas] |
// gather flags [world][kMaxCtas] | data parity 0 | data parity 1 | owner partial | owner stage.
__device__ __forceinline__ uint32_t* scatter_flag(uint8_t* base, int src, int cta) {
  return reinterpret_cast<uint32_t*>(base + 256) + src * kMaxCtas + cta;
}
__device__ __forceinline__ uint32_t* gather_flag(uint8_t* base, int src, int cta) {
  return reinterpret_cast<uint32_t*>(base + 256) + (kMaxWorld + src) * kMaxCtas + cta;
}

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
  }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    w[i] = *reinterpret_cast<const uint32_t*>(&v);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

// Bounded wait of one thread for flag >= target. False when it gave up.
__device__ __forceinline__ bool wait_flag(const uint32_t* flag, uint32_t target,
                                          long long limit) {
  if ((int32_t)(ld_acquire_sys(flag) - target) >= 0) return true;
  const long long start = clock64();
  while ((int32_t)(ld_acquire_sys(flag) - target) < 0) {
    if (clock64() - start > limit) return false;
  }
  return true;
}

// Threads [0, world) of the CTA wait for the flag of the rank with their index (scatter or
// gather family, slot `cta`). Returns CTA-uniformly whether any wait gave up; the first one
// records `code` in the status word and marks the workspace as failed.
__device__ __forceinline__ bool wait_peers(const ArParams& p, uint8_t* mine, bool gather, int slot,
                                           uint32_t target, int code) {
  bool bad = false;
  if ((int)threadIdx.x < p.world && (int)threadIdx.x != p.rank) {
    const uint32_t* flag = gather ? gather_flag(mine, threadIdx.x, slot)
                                  : scatter_flag(mine, threadIdx.x, slot);
    if (!wait_flag(flag, target, p.wait_cycles)) {
      bad = true;
      report_timeout(p.status, code);
      reinterpret_cast<uint32_t*>(mine)[kCtrlFailed] = 1u;
    }
  }
  return __syncthreads_or(bad ? 1 : 0) != 0;
}

// Coarse flags: the last CTA of the grid to finish a phase publishes ONE flag per peer. Every
// CTA fences its own stores at device scope before taking a ticket; the last one fences at
// system scope, so by cumulativity all of the grid's stores precede the flag. CTAs then wait
// for the peers' flags, which the peers' last CTAs publish: the whole grid must be resident
// (cooperative launch).
__device__ __forceinline__ void publish_phase(const ArParams& p, uint32_t* counter, bool gather,
                                              uint32_t target, int ctas) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const uint32_t ticket = atomicAdd(counter, 1u);
    if (ticket == (uint32_t)ctas - 1) {
      *counter = 0;
      __threadfence_system();
      for (int d = 1; d < p.world; ++d) {
        uint8_t* peer = p.peers[(p.rank + d) % p.world];
        st_relaxed_sys(gather ? gather_flag(peer, p.rank, 0) : scatter_flag(peer, p.rank, 0), target);
      }
    }
  }
}

constexpr uint32_t kNanBf16x2 = 0x7FC07FC0u;

// Where one row's results go. Null pointers skip that output.
struct RowOut {
  __nv_bfloat16* res;      // residual_out row
  __nv_bfloat16* norm;     // norm row
  uint8_t* codes;          // E4M3 row
  uint8_t* scales;         // swizzled scale buffer (whole tensor) or null
  int scale_row;           // row index inside the swizzled buffer
  // owner form: the row's codes and scales also go to every other rank's buffer, at the same
  // place of its all-rows code matrix and swizzled scale buffer
  bool bcast;
  size_t peer_codes_off;   // byte offset of the row's codes inside a rank's buffer
  size_t peer_scales_off;  // byte offset of the swizzled scale buffer inside a rank's buffer
};

// residual add + RMSNorm (+ quant) of one row whose reduced BF16 sum is `a` (this thread's
// 8 elements at column `col`, valid when have). All threads of the CTA call it. With
// `poison` the row's outputs are written as NaN / 0x7F / 0xFF instead.
__device__ __forceinline__ void norm_row(const ArParams& p, const __nv_bfloat16* residual_row,
                                         const RowOut& out, int col, bool have, bool poison,
                                         const float (&a)[8], float* warp_sums) {
  float r[8];
  float sq = 0.0f;
  if (have) {
    float resid[8];
    unpack8(*reinterpret_cast<const uint4*>(residual_row + col), resid);
#pragma unroll
    for (int i = 0; i < 8; ++i) r[i] = bf16_round(__fadd_rn(a[i], resid[i]));
    if (out.res)
      *reinterpret_cast<uint4*>(out.res + col) =
          poison ? make_uint4(kNanBf16x2, kNanBf16x2, kNanBf16x2, kNanBf16x2) : pack8(r);
#pragma unroll
    for (int i = 0; i < 8; ++i) sq = __fadd_rn(sq, __fmul_rn(r[i], r[i]));
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) r[i] = 0.0f;
  }
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) sq = __fadd_rn(sq, __shfl_xor_sync(0xffffffffu, sq, d));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();  // warp_sums reuse across rows
  if (lane == 0) warp_sums[warp] = sq;
  __syncthreads();
  if (warp == 0) {
    float t = lane < (int)(blockDim.x >> 5) ? warp_sums[lane] : 0.0f;
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) t = __fadd_rn(t, __shfl_xor_sync(0xffffffffu, t, d));
    if (lane == 0) warp_sums[32] = t;
  }
  __syncthreads();
  const float var = __fdiv_rn(warp_sums[32], (float)p.h);
  const float rs = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(var, p.eps)));
  float y[8];
  if (have) {
    float g[8];
    unpack8(__ldg(reinterpret_cast<const uint4*>(p.gamma + col)), g);
#pragma unroll
    for (int i = 0; i < 8; ++i)
      y[i] = bf16_round(__fmul_rn(__fmul_rn(r[i], rs), __fadd_rn(p.weight_bias, g[i])));
    if (out.norm)
      *reinterpret_cast<uint4*>(out.norm + col) =
          poison ? make_uint4(kNanBf16x2, kNanBf16x2, kNanBf16x2, kNanBf16x2) : pack8(y);
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) y[i] = 0.0f;
  }
  if (out.codes) {
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(y[i]));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    const uint32_t bits = mx_scale_bits(amax);
    const float inv = mx_inverse(bits);
    if (have) {
      uint2 q;
      q.x = e4m3x4(__fmul_rn(y[0], inv), __fmul_rn(y[1], inv), __fmul_rn(y[2], inv),
                   __fmul_rn(y[3], inv));
      q.y = e4m3x4(__fmul_rn(y[4], inv), __fmul_rn(y[5], inv), __fmul_rn(y[6], inv),
                   __fmul_rn(y[7], inv));
      if (poison) q = make_uint2(0x7F7F7F7Fu, 0x7F7F7F7Fu);
      *reinterpret_cast<uint2*>(out.codes + col) = q;
      if (out.bcast && !poison) {
        for (int d = 1; d < p.world; ++d)
          *reinterpret_cast<uint2*>(p.peers[(p.rank + d) % p.world] + out.peer_codes_off + col) = q;
      }
      if ((threadIdx.x & 3) == 0) {
        const uint8_t sb = poison ? (uint8_t)0xFF : (uint8_t)(bits >> 23);
        if (out.scales) out.scales[sf_offset(out.scale_row, col >> 5, p.k_tiles)] = sb;
      }
    }
    if (out.bcast && !poison) {
      // Four consecutive scale bytes of a row are one aligned word of the swizzled layout:
      // lane 16j collects the bytes its 16 threads produced (lanes 16j, +4, +8, +12; threads
      // past the row contribute 0, which lands in the layout's padding).
      uint32_t w = have ? (bits >> 23) & 0xFFu : 0u;
      w |= __shfl_down_sync(0xffffffffu, w, 4) << 8;
      w |= __shfl_down_sync(0xffffffffu, w, 8) << 16;
      if ((threadIdx.x & 15) == 0 && have) {
        const size_t off = out.peer_scales_off + sf_offset(out.scale_row, col >> 5, p.k_tiles);
        for (int d = 1; d < p.world; ++d)
          *reinterpret_cast<uint32_t*>(p.peers[(p.rank + d) % p.world] + off) = w;
      }
    }
  }
}

__device__ __forceinline__ RowOut full_row_out(const ArParams& p, int row) {
  RowOut o;
  o.res = p.res_out ? p.res_out + (size_t)row * p.h : nullptr;
  o.norm = p.norm_out ? p.norm_out + (size_t)row * p.h : nullptr;
  o.codes = p.codes ? p.codes + (size_t)row * p.h : nullptr;
  o.scales = p.scales;
  o.scale_row = row;
  o.bcast = false;
  o.peer_codes_off = 0;
  o.peer_scales_off = 0;
  return o;
}

// ------------------------------------------------------------------ owner form
template <bool kPrefetch>
__device__ __forceinline__ void owner_body(const ArParams& p, uint8_t* mine, uint32_t* ctrl,
                                           uint32_t target, bool failed_before, float* warp_sums) {
  const int cta = blockIdx.x, ctas = gridDim.x;
  const int col = threadIdx.x * 8;
  const bool have = col < p.h;
  const size_t row_bytes = (size_t)p.h * 2;
  const int rpo = p.rows_per_owner;
  const int first = min(p.rank * rpo, p.m);
  const int count = min(rpo, p.m - first);
  const int groups = p.h >> 5;
  bool poison = failed_before;

  // ---- (0) a partial tensor outside the buffer: expose the rows other ranks own
  if (p.partial && !poison) {
    for (int row = cta; row < p.m; row += ctas) {
      if (row >= first && row < first + count) continue;
      if (have)
        *reinterpret_cast<uint4*>(mine + p.owner_partial_off + (size_t)row * row_bytes +
                                  (size_t)col * 2) =
            *reinterpret_cast<const uint4*>(p.partial + (size_t)row * p.h + col);
    }
    publish_phase(p, ctrl + kCtrlTicketA, false, target, ctas);
  } else if (!poison) {
    // the producing GEMM wrote the rows; its grid has completed (stream order)
    if (cta == 0 && threadIdx.x == 0) {
      __threadfence_system();
      for (int d = 1; d < p.world; ++d)
        st_relaxed_sys(scatter_flag(p.peers[(p.rank + d) % p.world], p.rank, 0), target);
    }
  }
  MACH_TRACE(p, target - 1, 1);
  if (!poison) poison = wait_peers(p, mine, false, 0, target, kWaitScatter);
  MACH_TRACE(p, target - 1, 2);

  // ---- (1) my rows: pull from every rank, sum in rank order, residual + norm + quant.
  // With kPrefetch the loads of the CTA's NEXT row are issued before the current row is
  // reduced and normalised, so the NVLink round trip of one row hides behind the arithmetic
  // (and the block barriers) of another; rows of one CTA are otherwise strictly sequential.
  // The caller's code and scale tensors may BE this rank's all-rows buffers (zero copy).
  uint8_t* local_codes = mine + p.owner_stage_off;
  uint8_t* local_scales = mine + p.owner_scales_off;
  const bool in_place = p.codes == local_codes && p.scales == local_scales;
  auto issue = [&](int j, uint4 (&v)[kMaxWorld]) {
    const int row = first + j;
#pragma unroll
    for (int src = 0; src < kMaxWorld; ++src) {
      if (src < p.world) {
        if (src == p.rank && p.partial)
          v[src] = *reinterpret_cast<const uint4*>(p.partial + (size_t)row * p.h + col);
        else
          v[src] = ld_peer16(p.peers[src] + p.owner_partial_off + (size_t)row * row_bytes +
                             (size_t)col * 2);
      }
    }
  };
  const bool loads = have && !poison;
  uint4 cur[kMaxWorld], nxt[kMaxWorld];
  if (kPrefetch && loads && cta < count) issue(cta, cur);
  for (int j = cta; j < count; j += ctas) {
    const int row = first + j;
    if (loads) {
      if (kPrefetch) {
        if (j + ctas < count) issue(j + ctas, nxt);
      } else {
        issue(j, cur);
      }
    }
    float a[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) a[i] = 0.0f;
    if (loads) {
#pragma unroll
      for (int src = 0; src < kMaxWorld; ++src) {
        if (src < p.world) {
          float f[8];
          unpack8(cur[src], f);
#pragma unroll
          for (int i = 0; i < 8; ++i) a[i] = __fadd_rn(a[i], f[i]);
        }
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) a[i] = bf16_round(a[i]);
    }
    RowOut o;
    o.res = p.res_out ? p.res_out + (size_t)j * p.h : nullptr;
    o.norm = p.norm_out ? p.norm_out + (size_t)j * p.h : nullptr;
    o.codes = p.codes + (size_t)row * p.h;
    o.scales = p.scales;
    o.scale_row = row;
    o.bcast = true;
    o.peer_codes_off = p.owner_stage_off + (size_t)row * p.h;
    o.peer_scales_off = p.owner_scales_off;
    norm_row(p, p.residual + (size_t)j * p.h, o, col, have, poison, a, warp_sums);
    if (kPrefetch) {
#pragma unroll
      for (int src = 0; src < kMaxWorld; ++src) cur[src] = nxt[src];
    }
  }
  MACH_TRACE(p, target - 1, 3);
  if (!failed_before) {
    // also after a late scatter flag: the peers still expect this rank's gather flag
    publish_phase(p, ctrl + kCtrlTicketB, true, target, ctas);
    MACH_TRACE(p, target - 1, 4);
    const bool late = wait_peers(p, mine, true, 0, target, kWaitGather);
    poison = poison || late;
  }
  MACH_TRACE(p, target - 1, 5);

  // ---- (2) the other owners' rows are in this rank's buffer now (their owners stored them
  // there while they produced them, so the NVLink stores ran beside the pulls of phase 1).
  // A caller that reads the buffer itself is done; otherwise they are copied to its tensors.
  // After a failed wait nothing in the buffer can be trusted: every row this rank does not own
  // is poisoned.
  if (in_place && !poison) return;
  const int vpr = p.h >> 4;  // 16-byte vectors per row of codes
  const int tid = cta * blockDim.x + threadIdx.x;
  const int stride = ctas * blockDim.x;
  const uint4 bad = make_uint4(0x7F7F7F7Fu, 0x7F7F7F7Fu, 0x7F7F7F7Fu, 0x7F7F7F7Fu);
  for (int d = 1; d < p.world; ++d) {
    const int o = (p.rank + d) % p.world;
    const int ofirst = min(o * rpo, p.m);
    const int ocount = min(rpo, p.m - ofirst);
    const int total = ocount * vpr;
    const uint4* src = reinterpret_cast<const uint4*>(local_codes + (size_t)ofirst * p.h);
    uint4* dst = reinterpret_cast<uint4*>(p.codes + (size_t)ofirst * p.h);
    for (int idx = tid; idx < total; idx += stride)
      dst[idx] = poison ? bad : ld_cg(src + idx);
    // scale bytes of one row: groups consecutive bytes at four-byte granularity
    const int bytes = ocount * groups;
    for (int idx = tid; idx < bytes; idx += stride) {
      const int j = idx / groups, g = idx - j * groups;
      const size_t off = sf_offset(ofirst + j, g, p.k_tiles);
      p.scales[off] = poison ? (uint8_t)0xFF : __ldcg(local_scales + off);
    }
  }
}

// ------------------------------------------------------------------ push forms
__device__ __forceinline__ void push_body(const ArParams& p, uint8_t* mine, uint32_t* ctrl,
                                          uint32_t epoch, bool failed_before, float* warp_sums) {
  const uint32_t target = epoch + 1;
  const size_t parity_off = kHeaderBytes + (size_t)(epoch & 1) * p.parity_bytes;
  const int cta = blockIdx.x, ctas = gridDim.x;
  const int col = threadIdx.x * 8;
  const bool have = col < p.h;
  const size_t row_bytes = (size_t)p.h * 2;
  bool poison = failed_before;

  if (!p.two_shot) {
    // ---- push my partial rows to every peer: slot [src = rank][row] (already done by the
    // GEMM epilogue when prescattered, this rank's own slot included)
    for (int row = cta; row < p.m && !p.prescattered && !poison; row += ctas) {
      if (have) {
        const uint4 v = *reinterpret_cast<const uint4*>(p.partial + (size_t)row * p.h + col);
        for (int d = 1; d < p.world; ++d) {
          const int dst = (p.rank + d) % p.world;
          *reinterpret_cast<uint4*>(p.peers[dst] + parity_off +
                                    ((size_t)p.rank * p.m + row) * row_bytes + (size_t)col * 2) = v;
        }
      }
    }
    __syncthreads();
    if (threadIdx.x == 0 && !poison) {
      __threadfence_system();
      for (int d = 1; d < p.world; ++d) {
        const int dst = (p.rank + d) % p.world;
        st_relaxed_sys(scatter_flag(p.peers[dst], p.rank, cta), target);
      }
    }
    if (!poison) poison = wait_peers(p, mine, false, cta, target, kWaitScatter);
    for (int row = cta; row < p.m; row += ctas) {
      float a[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) a[i] = 0.0f;
      if (have && !poison) {
        for (int src = 0; src < p.world; ++src) {
          float v[8];
          if (src == p.rank && !p.prescattered)
            unpack8(*reinterpret_cast<const uint4*>(p.partial + (size_t)row * p.h + col), v);
          else
            unpack8(ld_cg(mine + parity_off + ((size_t)src * p.m + row) * row_bytes + (size_t)col * 2), v);
#pragma unroll
          for (int i = 0; i < 8; ++i) a[i] = __fadd_rn(a[i], v[i]);
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) a[i] = bf16_round(a[i]);
      }
      norm_row(p, p.residual + (size_t)row * p.h, full_row_out(p, row), col, have, poison, a,
               warp_sums);
    }
    return;
  }

  const int rpo = p.rows_per_owner;
  const size_t gather_off = parity_off + p.parity_bytes / 2;
  // ---- (1) scatter: rows owned by `dst` go to dst's slot [src = rank][local row]
  // (already done by the epilogue of the GEMM that produced the partial sums when
  // prescattered: that kernel has completed, so only the flags remain to be published)
  for (int d = 1; d < p.world && !p.prescattered && !poison; ++d) {
    const int dst = (p.rank + d) % p.world;
    const int first = dst * rpo;
    const int count = min(rpo, p.m - first);
    for (int j = cta; j < count; j += ctas) {
      if (have)
        *reinterpret_cast<uint4*>(p.peers[dst] + parity_off +
                                  ((size_t)p.rank * rpo + j) * row_bytes + (size_t)col * 2) =
            *reinterpret_cast<const uint4*>(p.partial + (size_t)(first + j) * p.h + col);
    }
  }
  if (poison) {
    // a workspace that failed earlier: no communication at all
  } else if (p.coarse) {
    publish_phase(p, ctrl + kCtrlTicketA, false, target, ctas);
  } else {
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence_system();
      for (int d = 1; d < p.world; ++d)
        st_relaxed_sys(scatter_flag(p.peers[(p.rank + d) % p.world], p.rank, cta), target);
    }
  }
  if (!poison) poison = wait_peers(p, mine, false, p.coarse ? 0 : cta, target, kWaitScatter);
  // ---- (2) reduce my rows in rank order, publish the BF16 sum to every rank
  if (!failed_before) {
    const int first = p.rank * rpo;
    const int count = min(rpo, p.m - first);
    for (int j = cta; j < count; j += ctas) {
      if (have) {
        float a[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) a[i] = 0.0f;
        for (int src = 0; src < p.world; ++src) {
          float v[8];
          if (src == p.rank && !p.prescattered)
            unpack8(*reinterpret_cast<const uint4*>(p.partial + (size_t)(first + j) * p.h + col), v);
          else
            unpack8(ld_cg(mine + parity_off + ((size_t)src * rpo + j) * row_bytes + (size_t)col * 2), v);
#pragma unroll
          for (int i = 0; i < 8; ++i) a[i] = __fadd_rn(a[i], v[i]);
        }
        // After a wait that gave up the sums are not trustworthy: the peers get NaN rows.
        const uint4 packed =
            poison ? make_uint4(kNanBf16x2, kNanBf16x2, kNanBf16x2, kNanBf16x2) : pack8(a);
        for (int d = 0; d < p.world; ++d) {
          const int dst = (p.rank + d) % p.world;
          *reinterpret_cast<uint4*>(p.peers[dst] + gather_off + (size_t)(first + j) * row_bytes +
                                    (size_t)col * 2) = packed;
        }
      }
    }
    if (p.coarse) {
      publish_phase(p, ctrl + kCtrlTicketB, true, target, ctas);
    } else {
      __syncthreads();
      if (threadIdx.x == 0) {
        __threadfence_system();
        for (int d = 1; d < p.world; ++d)
          st_relaxed_sys(gather_flag(p.peers[(p.rank + d) % p.world], p.rank, cta), target);
      }
    }
    const bool late = wait_peers(p, mine, true, p.coarse ? 0 : cta, target, kWaitGather);
    poison = poison || late;
  }
  // ---- (3) residual + norm of every row, from the gathered sums. With per-CTA flags a CTA
  // may only touch the rows its namesakes on the other ranks produced; with coarse flags
  // everything has arrived and the rows are dealt evenly.
  if (p.coarse) {
    for (int row = cta; row < p.m; row += ctas) {
      float a[8];
      if (have && !poison) unpack8(ld_cg(mine + gather_off + (size_t)row * row_bytes + (size_t)col * 2), a);
      else {
#pragma unroll
        for (int i = 0; i < 8; ++i) a[i] = 0.0f;
      }
      norm_row(p, p.residual + (size_t)row * p.h, full_row_out(p, row), col, have, poison, a,
               warp_sums);
    }
  } else {
    for (int owner = 0; owner < p.world; ++owner) {
      const int first = owner * rpo;
      const int count = min(rpo, p.m - first);
      for (int j = cta; j < count; j += ctas) {
        float a[8];
        if (have && !poison)
          unpack8(ld_cg(mine + gather_off + (size_t)(first + j) * row_bytes + (size_t)col * 2), a);
        else {
#pragma unroll
          for (int i = 0; i < 8; ++i) a[i] = 0.0f;
        }
        norm_row(p, p.residual + (size_t)(first + j) * p.h, full_row_out(p, first + j), col, have,
                 poison, a, warp_sums);
      }
    }
  }
}

template <bool kPrefetch>
__device__ __forceinline__ void ar_body(const ArParams& p) {
  __shared__ float warp_sums[33];
  __shared__ uint32_t s_epoch, s_failed;
  uint8_t* mine = p.peers[p.rank];
  uint32_t* ctrl = reinterpret_cast<uint32_t*>(mine);
  if (threadIdx.x == 0) {
    s_epoch = ld_acquire_sys(ctrl + kCtrlEpoch);
    s_failed = ld_acquire_sys(ctrl + kCtrlFailed);
  }
  __syncthreads();
  const uint32_t epoch = s_epoch;
  const bool failed_before = s_failed != 0;
  MACH_TRACE(p, epoch, 0);
  if (failed_before && blockIdx.x == 0 && threadIdx.x == 0) report_timeout(p.status, kWorkspaceFailed);
  if (p.owner) owner_body<kPrefetch>(p, mine, ctrl, epoch + 1, failed_before, warp_sums);
  else push_body(p, mine, ctrl, epoch, failed_before, warp_sums);

  MACH_TRACE(p, epoch, 6);
  // ---- the last CTA to finish advances the epoch for the next launch
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const uint32_t done = atomicAdd(ctrl + kCtrlDone, 1u);
    if (done == gridDim.x - 1) {
      ctrl[kCtrlDone] = 0;
      __threadfence();
      ctrl[kCtrlEpoch] = epoch + 1;   // read by this GPU's next launch only
    }
  }
}

// blockDim.x == ceil(h / 8) rounded up to a warp: one 16-byte vector per thread per row.
// Two instantiations: up to 512 threads (hidden <= 4096) leaves 128 registers per thread,
// enough to hold the next row's peer loads while the current row is processed; hidden up to
// 8192 needs 1024 threads and runs without that prefetch.
template <int kMaxThreads>
__global__ void __launch_bounds__(kMaxThreads)
allreduce_norm_kernel(const ArParams p) {
  pdl_launch_dependents();
  pdl_wait();  // the partial sums come from the preceding GEMM
  ar_body<(kMaxThreads <= 512)>(p);
}

// Every rank of a group whose buffers all live on this device, as ONE cooperative grid:
// blockIdx.y is the rank. Kernels that wait on one another must not be separate launches on
// one GPU, so this is how the multi-rank protocols run where there are fewer GPUs than ranks.
__global__ void __launch_bounds__(1024)
allreduce_norm_local_ranks_kernel(const __grid_constant__ ArParamsMulti all) {
  ar_body<false>(all.r[blockIdx.y]);
}

size_t parity_bytes_for(int world, int64_t tokens_cap, int64_t hidden) {
  // One-shot needs world full copies; two-shot needs (scatter slots + gathered sums), each at
  // most (tokens_cap + world) rows. The one-shot path is only taken while it fits.
  const size_t row = (size_t)hidden * 2;
  const size_t two_shot = 2 * (size_t)(tokens_cap + world) * row;
  return (two_shot + 255) & ~(size_t)255;
}
size_t owner_partial_bytes(int64_t tokens_cap, int64_t hidden) {
  return ((size_t)tokens_cap * hidden * 2 + 255) & ~(size_t)255;
}
// Owner form: codes of all rows [tokens_cap, hidden], then their swizzled scales (one 512-byte
// atom per 128 rows x 128 columns).
size_t owner_codes_bytes(int64_t tokens_cap, int64_t hidden) {
  return ((size_t)tokens_cap * hidden + 255) & ~(size_t)255;
}
size_t owner_stage_bytes(int64_t tokens_cap, int64_t hidden) {
  const size_t atoms = (size_t)((tokens_cap + 127) / 128) * (size_t)((hidden + 127) / 128);
  return owner_codes_bytes(tokens_cap, hidden) + atoms * 512;
}

constexpr long long kDefaultWaitCycles = kWaitCycles;

// Fills the launch parameters of one rank; returns MACH_OK or records an error.
int fill_params(ArWorkspace* ws, const void* partial, const void* residual, const void* gamma,
                float eps, float weight_bias, void* norm_out, void* residual_out, void* codes,
                void* scales, int64_t m, int64_t h, int algo, bool owner, ArParams* out) {
  if (!ws) return fail(MACH_ERR_INVALID, "allreduce_rmsnorm: null workspace");
  if (m < 0) return fail(MACH_ERR_INVALID, "allreduce_rmsnorm: negative size");
  // An owner with no rows (fewer tokens than ranks) has no residual rows either.
  const int64_t rpo_rows = (m + ws->world - 1) / ws->world;
  const bool no_rows = m == 0 || (owner && (int64_t)ws->rank * rpo_rows >= m);
  if (!gamma || (!residual && !no_rows))
    return fail(MACH_ERR_INVALID, "allreduce_rmsnorm: null pointer");
  // partial == NULL: push forms: the partial sums were written into the owners' slots by
  // mach_mx_gemm_reduce_scatter on this stream; owner form: the producing GEMM wrote them to
  // mach_ar_partial_ptr. Every rank must do the same.
  const bool no_partial = partial == nullptr;
  if (no_partial && ws->world < 2 && !owner)
    return fail(MACH_ERR_INVALID, "allreduce_rmsnorm: a partial tensor is required for one rank");
  if ((codes == nullptr) != (scales == nullptr))
    return fail(MACH_ERR_INVALID, "allreduce_rmsnorm: codes and scales go together");
  if (owner && !codes)
    return fail(MACH_ERR_INVALID, "allreduce_owner_rmsnorm: codes and scales are required");
  if (h != ws->hidden || m > ws->tokens_cap)
    return fail(MACH_ERR_INVALID, "allreduce_rmsnorm: shape [%lld, %lld] exceeds the workspace "
                "(tokens <= %lld, hidden == %lld)", (long long)m, (long long)h,
                (long long)ws->tokens_cap, (long long)ws->hidden);
  if ((partial && !aligned16(partial)) || (residual && !aligned16(residual)) || !aligned16(gamma) ||
      (norm_out && !aligned16(norm_out)) || (residual_out && !aligned16(residual_out)) ||
      (codes && !aligned16(codes)) || (scales && (reinterpret_cast<uintptr_t>(scales) & 3)))
    return fail(MACH_ERR_UNSUPPORTED, "allreduce_rmsnorm: 16-byte aligned tensors required");
  ArParams p = {};
  p.partial = (const __nv_bfloat16*)partial;
  p.residual = (const __nv_bfloat16*)residual;
  p.gamma = (const __nv_bfloat16*)gamma;
  p.norm_out = (__nv_bfloat16*)norm_out;
  p.res_out = (__nv_bfloat16*)residual_out;
  p.codes = (uint8_t*)codes;
  p.scales = (uint8_t*)scales;
  for (int i = 0; i < ws->world; ++i) p.peers[i] = ws->peers[i];
  p.status = device_status_ptr();
  if (!p.status) return fail(MACH_ERR_CUDA, "allreduce_rmsnorm: cannot resolve the status word");
  p.wait_cycles = ws->wait_cycles;
#ifdef MACH_EXPERIMENTS
  p.trace = ws->trace;
#endif
  p.eps = eps;
  p.weight_bias = weight_bias;
  p.rank = ws->rank;
  p.world = ws->world;
  p.m = (int)m;
  p.h = (int)h;
  p.k_tiles = (int)((h + 127) / 128);
  p.rows_per_owner = (int)((m + ws->world - 1) / ws->world);
  p.parity_bytes = ws->parity_bytes;
  p.owner_partial_off = ws->owner_partial_off;
  p.owner_stage_off = ws->owner_stage_off;
  p.owner_scales_off = ws->owner_scales_off;
  p.owner = owner ? 1 : 0;
  if (owner) {
    *out = p;
    return MACH_OK;
  }
  bool prescattered = false;
  if (no_partial) {
    // The hand-off must be the one mach_mx_gemm_reduce_scatter recorded for this very shape.
    if (!ws->scatter_pending || ws->scattered_m != m)
      return fail(MACH_ERR_INVALID, "allreduce_rmsnorm: partial == NULL needs a preceding "
                  "mach_mx_gemm_reduce_scatter of the same [m, h] on this workspace");
    prescattered = true;
  }
  ws->scatter_pending = 0;
  // One-shot moves (world-1) x payload per rank, two-shot 2 (world-1)/world x payload with one
  // more hop: one-shot for two ranks or small payloads that fit `world` copies.
  const size_t payload = (size_t)m * h * 2;
  const bool fits = (size_t)ws->world * payload <= ws->parity_bytes;
  bool two_shot = ws->world > 2 && payload > (256u << 10);
  if (algo == 1) two_shot = false;
  if (algo == 2 || algo == 3) two_shot = ws->world > 1;
  if (!two_shot && !fits) two_shot = true;
  if (ws->world == 1) two_shot = false;
  if (prescattered) two_shot = !ws->scattered_one_shot;
  p.two_shot = two_shot ? 1 : 0;
  p.prescattered = prescattered ? 1 : 0;
  // Two-shot defaults to coarse flags (one per rank and phase): per-CTA flags cost two
  // system-scope fences and 2 (world-1) remote flag stores per handful of rows (measured on two
  // B200s, 1.3 MB payload: 47 us per-CTA, 25 us coarse).
  bool coarse = two_shot;
  if (algo == 2) coarse = false;
  if (algo == 3) coarse = two_shot;
  p.coarse = coarse ? 1 : 0;
  *out = p;
  return MACH_OK;
}

int threads_for(int64_t h) { return (int)((h / 8 + 31) / 32) * 32; }

// CTAs that can be resident at once on the current device for this block size.
int resident_ctas(int threads, bool local_ranks) {
  int per_sm = 0;
  const cudaError_t e =
      local_ranks ? cudaOccupancyMaxActiveBlocksPerMultiprocessor(
                        &per_sm, allreduce_norm_local_ranks_kernel, threads, 0)
                  : threads <= 512
                        ? cudaOccupancyMaxActiveBlocksPerMultiprocessor(
                              &per_sm, allreduce_norm_kernel<512>, threads, 0)
                        : cudaOccupancyMaxActiveBlocksPerMultiprocessor(
                              &per_sm, allreduce_norm_kernel<1024>, threads, 0);
  if (e != cudaSuccess || per_sm < 1) return 0;
  return per_sm * sm_count();
}

// Grid of one rank. Depends only on (m, h, world) and the device, so that every rank arrives
// at the same value (the per-CTA flag forms pair CTA b of every rank).
int grid_for(const ArParams& p, int threads, int resident) {
  const int per_sm = std::max(1, std::min(4, 2048 / threads));
  int64_t want = std::max<int64_t>(p.m, 1);
  if (p.owner) want = std::max<int64_t>(p.rows_per_owner, 1);
  int ctas = (int)std::min<int64_t>(want, (int64_t)sm_count() * per_sm);
  ctas = std::min(ctas, kMaxCtas);
  if (p.coarse || p.owner) {
    // CTAs wait for flags that a grid's last CTA publishes: all of them must be resident
    ctas = std::min(ctas, resident);
    if (!p.owner) ctas = std::min(ctas, 2 * sm_count());
  }
  ctas = std::max(ctas, 1);
  if (p.owner) {
    // Every CTA the same number of rows: 512 owned rows on 444 resident CTAs would leave 376
    // CTAs idle during a second round of 68 rows.
    const int64_t rounds = (want + ctas - 1) / ctas;
    ctas = (int)((want + rounds - 1) / rounds);
  }
  return std::max(ctas, 1);
}

int launch_rank(const ArParams& p, cudaStream_t stream) {
  const int threads = threads_for(p.h);
  const bool needs_resident = p.coarse || p.owner;
  int resident = 0;
  if (needs_resident) {
    resident = resident_ctas(threads, false);
    if (resident < 1) return fail(MACH_ERR_CUDA, "allreduce_rmsnorm: occupancy query failed");
  }
  const int ctas = grid_for(p, threads, resident);
  // Forms whose CTAs wait on flags published by the grid's last CTA are launched cooperatively:
  // a grid that cannot be co-resident (another stream holds the SMs) is then held back or
  // refused by the driver instead of spinning until its waits give up.
  const bool pdl = needs_resident ? false : pdl_enabled();
  const cudaError_t e =
      threads <= 512
          ? launch_ex_attrs(allreduce_norm_kernel<512>, dim3((unsigned)ctas), dim3(threads), 0,
                            stream, dim3(1, 1, 1), pdl, needs_resident, p)
          : launch_ex_attrs(allreduce_norm_kernel<1024>, dim3((unsigned)ctas), dim3(threads), 0,
                            stream, dim3(1, 1, 1), pdl, needs_resident, p);
  if (e != cudaSuccess) return fail(MACH_ERR_CUDA, "allreduce_rmsnorm: %s", cudaGetErrorString(e));
  return MACH_OK;
}

}  // namespace

// Where a reduce-scattering GEMM of [m, h] partial sums has to put its rows.
int ar_scatter_target(void* workspace, int64_t m, int64_t h, ScatterTarget* out) {
  ArWorkspace* ws = reinterpret_cast<ArWorkspace*>(workspace);
  if (!ws || !out) return fail(MACH_ERR_INVALID, "mx_gemm_reduce_scatter: null workspace");
  if (ws->world < 2)
    return fail(MACH_ERR_INVALID, "mx_gemm_reduce_scatter: needs at least two ranks");
  if (h != ws->hidden || m > ws->tokens_cap || m < 1)
    return fail(MACH_ERR_INVALID, "mx_gemm_reduce_scatter: shape [%lld, %lld] does not fit the "
                "workspace (tokens <= %lld, hidden == %lld)", (long long)m, (long long)h,
                (long long)ws->tokens_cap, (long long)ws->hidden);
  for (int i = 0; i < kMaxWorld; ++i) out->peers[i] = i < ws->world ? ws->peers[i] : nullptr;
  out->epoch = reinterpret_cast<const uint32_t*>(ws->peers[ws->rank]);
  out->header_bytes = kHeaderBytes;
  out->parity_bytes = ws->parity_bytes;
  out->world = ws->world;
  out->rank = ws->rank;
  out->rows_per_owner = (int)((m + ws->world - 1) / ws->world);
  out->m = (int)m;
  // Two ranks: every row goes to both buffers (one-shot); more: rows go to their owners only.
  out->one_shot = ws->world == 2 && (size_t)ws->world * (size_t)m * h * 2 <= ws->parity_bytes;
  ws->scattered_one_shot = out->one_shot;
  ws->scattered_m = m;
  ws->scatter_pending = 1;
  return MACH_OK;
}

}  // namespace mach

using namespace mach;

extern "C" size_t mach_ar_buffer_bytes(int world, int64_t tokens_cap, int64_t hidden) {
  if (world < 1 || world > kMaxWorld || tokens_cap <= 0 || hidden <= 0) return 0;
  return kHeaderBytes + 2 * parity_bytes_for(world, tokens_cap, hidden) +
         owner_partial_bytes(tokens_cap, hidden) + owner_stage_bytes(tokens_cap, hidden);
}

extern "C" int mach_ar_buffer_alloc(size_t bytes, void** dev_ptr) {
  if (!dev_ptr || bytes == 0) return fail(MACH_ERR_INVALID, "ar_buffer_alloc: bad arguments");
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, bytes);
  if (e != cudaSuccess) return fail(MACH_ERR_CUDA, "ar_buffer_alloc: %s", cudaGetErrorString(e));
  e = cudaMemset(p, 0, bytes);
  if (e != cudaSuccess) {
    cudaFree(p);
    return fail(MACH_ERR_CUDA, "ar_buffer_alloc: %s", cudaGetErrorString(e));
  }
  cudaDeviceSynchronize();
  *dev_ptr = p;
  return MACH_OK;
}

extern "C" int mach_ar_buffer_free(void* dev_ptr) {
  if (!dev_ptr) return MACH_OK;
  const cudaError_t e = cudaFree(dev_ptr);
  return e == cudaSuccess ? MACH_OK : fail(MACH_ERR_CUDA, "ar_buffer_free: %s", cudaGetErrorString(e));
}

extern "C" int mach_ar_ipc_export(void* dev_ptr, void* handle_64_bytes) {
  if (!dev_ptr || !handle_64_bytes) return fail(MACH_ERR_INVALID, "ar_ipc_export: null pointer");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  cudaIpcMemHandle_t h;
  const cudaError_t e = cudaIpcGetMemHandle(&h, dev_ptr);
  if (e != cudaSuccess) return fail(MACH_ERR_CUDA, "ar_ipc_export: %s", cudaGetErrorString(e));
  memcpy(handle_64_bytes, &h, 64);
  return MACH_OK;
}

extern "C" int mach_ar_ipc_open(const void* handle_64_bytes, void** peer_ptr) {
  if (!handle_64_bytes || !peer_ptr) return fail(MACH_ERR_INVALID, "ar_ipc_open: null pointer");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle_64_bytes, 64);
  void* p = nullptr;
  const cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) return fail(MACH_ERR_CUDA, "ar_ipc_open: %s", cudaGetErrorString(e));
  *peer_ptr = p;
  return MACH_OK;
}

extern "C" int mach_ar_ipc_close(void* peer_ptr) {
  if (!peer_ptr) return MACH_OK;
  const cudaError_t e = cudaIpcCloseMemHandle(peer_ptr);
  return e == cudaSuccess ? MACH_OK : fail(MACH_ERR_CUDA, "ar_ipc_close: %s", cudaGetErrorString(e));
}

extern "C" int mach_ar_create(int world, int rank, int64_t tokens_cap, int64_t hidden,
                              void* const* buffers, void** workspace) {
  if (!buffers || !workspace || world < 1 || world > kMaxWorld || rank < 0 || rank >= world ||
      tokens_cap <= 0 || hidden <= 0)
    return fail(MACH_ERR_INVALID, "ar_create: bad arguments");
  if (hidden % 32 || hidden > 8192)
    return fail(MACH_ERR_UNSUPPORTED, "ar_create: hidden %% 32 == 0 and hidden <= 8192 required");
  ArWorkspace* ws = new ArWorkspace();
  ws->world = world;
  ws->rank = rank;
  ws->tokens_cap = tokens_cap;
  ws->hidden = hidden;
  ws->parity_bytes = parity_bytes_for(world, tokens_cap, hidden);
  ws->owner_partial_off = kHeaderBytes + 2 * ws->parity_bytes;
  ws->owner_stage_off = ws->owner_partial_off + owner_partial_bytes(tokens_cap, hidden);
  ws->owner_scales_off = ws->owner_stage_off + owner_codes_bytes(tokens_cap, hidden);
  ws->wait_cycles = kDefaultWaitCycles;
  for (int i = 0; i < world; ++i) {
    if (!buffers[i]) {
      delete ws;
      return fail(MACH_ERR_INVALID, "ar_create: null buffer for rank %d", i);
    }
    ws->peers[i] = reinterpret_cast<uint8_t*>(buffers[i]);
  }
  *workspace = ws;
  return MACH_OK;
}

extern "C" int mach_ar_destroy(void* workspace) {
  delete reinterpret_cast<ArWorkspace*>(workspace);
  return MACH_OK;
}

extern "C" int mach_ar_set_wait_limit_us(void* workspace, int64_t microseconds) {
  ArWorkspace* ws = reinterpret_cast<ArWorkspace*>(workspace);
  if (!ws || microseconds < 1)
    return fail(MACH_ERR_INVALID, "ar_set_wait_limit_us: bad arguments");
  int dev = 0, khz = 0;
  if (cudaGetDevice(&dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, dev) != cudaSuccess || khz <= 0)
    khz = 2000000;
  // SM clocks at the highest frequency the device reaches: a wait never ends early.
  ws->wait_cycles = (long long)microseconds * (long long)khz / 1000;
  return MACH_OK;
}

#ifdef MACH_EXPERIMENTS
// Experiment builds only: device buffer of 64 x 8 time stamps (ns) written by CTA 0.
extern "C" __attribute__((visibility("default"))) int mach_ar_set_trace(void* workspace, void* dev) {
  ArWorkspace* ws = reinterpret_cast<ArWorkspace*>(workspace);
  if (!ws) return fail(MACH_ERR_INVALID, "ar_set_trace: null workspace");
  ws->trace = reinterpret_cast<unsigned long long*>(dev);
  return MACH_OK;
}
#endif

extern "C" int mach_ar_reset(void* workspace, void* stream) {
  ArWorkspace* ws = reinterpret_cast<ArWorkspace*>(workspace);
  if (!ws) return fail(MACH_ERR_INVALID, "ar_reset: null workspace");
  cudaError_t e = cudaMemsetAsync(ws->peers[ws->rank], 0, kHeaderBytes, (cudaStream_t)stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize((cudaStream_t)stream);
  if (e != cudaSuccess) return fail(MACH_ERR_CUDA, "ar_reset: %s", cudaGetErrorString(e));
  ws->scatter_pending = 0;
  return MACH_OK;
}

extern "C" int mach_ar_partial_ptr(void* workspace, void** partial_bf16) {
  ArWorkspace* ws = reinterpret_cast<ArWorkspace*>(workspace);
  if (!ws || !partial_bf16) return fail(MACH_ERR_INVALID, "ar_partial_ptr: null pointer");
  *partial_bf16 = ws->peers[ws->rank] + ws->owner_partial_off;
  return MACH_OK;
}

extern "C" int mach_ar_codes_ptr(void* workspace, void** codes, void** scales) {
  ArWorkspace* ws = reinterpret_cast<ArWorkspace*>(workspace);
  if (!ws || !codes || !scales) return fail(MACH_ERR_INVALID, "ar_codes_ptr: null pointer");
  *codes = ws->peers[ws->rank] + ws->owner_stage_off;
  *scales = ws->peers[ws->rank] + ws->owner_scales_off;
  return MACH_OK;
}

extern "C" int mach_allreduce_residual_rmsnorm_mxfp8(void* workspace, const void* partial,
                                                     const void* residual, const void* gamma,
                                                     float eps, float weight_bias, void* norm_out,
                                                     void* residual_out, void* codes, void* scales,
                                                     int64_t m, int64_t h, int algo, void* stream) {
  ArWorkspace* ws = reinterpret_cast<ArWorkspace*>(workspace);
  ArParams p;
  const int rc = fill_params(ws, partial, residual, gamma, eps, weight_bias, norm_out,
                             residual_out, codes, scales, m, h, algo, false, &p);
  if (rc != MACH_OK) return rc;
  return launch_rank(p, (cudaStream_t)stream);
}

extern "C" int mach_allreduce_owner_rmsnorm_mxfp8(void* workspace, const void* partial,
                                                  const void* residual_rows, const void* gamma,
                                                  float eps, float weight_bias,
                                                  void* norm_out_rows, void* residual_out_rows,
                                                  void* codes, void* scales, int64_t m, int64_t h,
                                                  void* stream) {
  ArWorkspace* ws = reinterpret_cast<ArWorkspace*>(workspace);
  ArParams p;
  const int rc = fill_params(ws, partial, residual_rows, gamma, eps, weight_bias, norm_out_rows,
                             residual_out_rows, codes, scales, m, h, 0, true, &p);
  if (rc != MACH_OK) return rc;
  if (m == 0) return MACH_OK;
  return launch_rank(p, (cudaStream_t)stream);
}

extern "C" int mach_ar_owner_rows(int world, int rank, int64_t m, int64_t* first, int64_t* count) {
  if (world < 1 || rank < 0 || rank >= world || m < 0 || !first || !count)
    return fail(MACH_ERR_INVALID, "ar_owner_rows: bad arguments");
  const int64_t rpo = (m + world - 1) / world;
  *first = std::min<int64_t>(rank * rpo, m);
  *count = std::max<int64_t>(0, std::min<int64_t>(rpo, m - *first));
  return MACH_OK;
}

extern "C" int mach_allreduce_local_ranks(int world, void* const* workspaces,
                                          const void* const* partials,
                                          const void* const* residuals, const void* gamma,
                                          float eps, float weight_bias, void* const* norm_outs,
                                          void* const* residual_outs, void* const* codes,
                                          void* const* scales, int64_t m, int64_t h, int algo,
                                          int owner_form, void* stream) {
  if (world < 1 || world > kMaxWorld || !workspaces || !partials || !residuals || !norm_outs ||
      !residual_outs || !codes || !scales)
    return fail(MACH_ERR_INVALID, "allreduce_local_ranks: bad arguments");
  ArParamsMulti local = {};
  for (int r = 0; r < world; ++r) {
    ArWorkspace* ws = reinterpret_cast<ArWorkspace*>(workspaces[r]);
    if (!ws || ws->world != world || ws->rank != r)
      return fail(MACH_ERR_INVALID, "allreduce_local_ranks: workspace %d is not rank %d of %d", r,
                  r, world);
    const int rc = fill_params(ws, partials[r], residuals[r], gamma, eps, weight_bias,
                               norm_outs[r], residual_outs[r], codes[r], scales[r], m, h, algo,
                               owner_form != 0, &local.r[r]);
    if (rc != MACH_OK) return rc;
  }
  if (m == 0) return MACH_OK;
  const int threads = threads_for(h);
  const int resident = resident_ctas(threads, true);
  if (resident < world)
    return fail(MACH_ERR_CUDA, "allreduce_local_ranks: the device cannot hold one CTA per rank");
  int ctas = grid_for(local.r[0], threads, resident / world);
  ctas = std::min(ctas, resident / world);
  const cudaError_t e =
      launch_ex_attrs(allreduce_norm_local_ranks_kernel, dim3((unsigned)ctas, (unsigned)world),
                      dim3(threads), 0, (cudaStream_t)stream, dim3(1, 1, 1), false, true, local);
  if (e != cudaSuccess)
    return fail(MACH_ERR_CUDA, "allreduce_local_ranks: %s", cudaGetErrorString(e));
  return MACH_OK;
}
