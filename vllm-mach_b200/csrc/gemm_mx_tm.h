// Launcher interface of the persistent token-major GEMM (gemm_mx_tm.cu).
#pragma once
#include <cuda_runtime.h>
#include <cstdint>

namespace mach {

// Destination of a GEMM whose BF16 output rows go straight into the all-reduce buffers (peer
// stores from the epilogue), in the parity half selected by the epoch word.
//   two-shot form: row r belongs to rank r / rows_per_owner and lands in that rank's slot
//     [this rank][r % rows_per_owner] (reduce-scatter);
//   one-shot form: row r lands in slot [this rank][r] of EVERY rank (two ranks: the same
//     NVLink bytes as the scatter plus the gather, and the reduce needs no second exchange).
struct ScatterTarget {
  uint8_t* peers[8];        // all-reduce buffers of every rank (peers[rank] is local)
  const uint32_t* epoch;    // local epoch word: parity = epoch & 1
  uint64_t header_bytes, parity_bytes;
  int world, rank, rows_per_owner;
  int one_shot, m;
};

struct TmGemmArgs {
  const void* a_codes;   // E4M3 [M, K]
  const void* a_sf;      // swizzled E8M0
  const void* w;         // [w_rows, K] codes (E4M3 or packed 6-bit)
  const void* w_sf;      // swizzled E8M0
  void* out;             // BF16 [M, w_rows]  or  SwiGLU: E4M3 [M, w_rows / 2]
  void* out_sf;          // SwiGLU: swizzled E8M0 of the codes
  int64_t m, w_rows, k;
  int w_format;
  bool swiglu;           // requires interleaved rows
  bool interleaved;      // weight rows are gate/up interleaved in groups of 32
  int bn;                // tile width in weight rows (multiple of 32; of 64 with SwiGLU)
  int stages;            // 0 = fill shared memory
  int panel_m;           // 0 = default raster
  int debug;             // experiment bits (pair kernel)
  int smem_cap_kb;       // one-token-tile kernel: cap on dynamic shared memory (0 = heuristic)
  const ScatterTarget* scatter;  // non-null: BF16 rows go to the owners' all-reduce buffers
};

int run_mx_gemm_tm(const TmGemmArgs& args, cudaStream_t stream);

}  // namespace mach
