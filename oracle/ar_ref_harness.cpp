// TEST INFRASTRUCTURE (checker only; nothing shipped links this).
//
// Host harness around the reference's own device code for the fused all-reduce tail:
// FusedOp::operator(), rms_norm, the MXFP8 branch, vec_add, allreduce_sum and the block
// reduction it uses (native/ar_norm/trtllm_allreduce_fusion_mxfp8.cuh of the reference). The
// build recipe beside this file cuts those definitions out of the reference header where it
// lies and writes them to _ref/ar_extract.inc; this file supplies what they need to compile as
// plain C++: vec_t, the parameter struct, threadIdx/blockDim, __shfl_xor_sync and
// __syncthreads over real host threads (one per CUDA thread of a block, a C++20 barrier for
// every warp shuffle and block barrier), and the bit-cast intrinsics. BF16 and E4M3 are
// NVIDIA's own host-side types from cuda_bf16.h / cuda_fp8.h.
//
// One stand-in is not the reference's arithmetic: rsqrtf. The reference is compiled with fast
// math (rsqrt.approx); here it is 1 / sqrtf(x), which is what the oracle restates.
#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include <barrier>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <thread>
#include <type_traits>
#include <vector>

#undef __device__
#undef __forceinline__
#undef __inline__
#undef __shared__
#define __device__
#define __forceinline__ inline
#define __inline__ inline
// a __shared__ variable in a function is one object for the whole block: a function static
#define __shared__ static

namespace sim {
struct Dim { unsigned x, y, z; };
thread_local Dim tid_v{0, 0, 0};
Dim block_v{1, 1, 1};
std::barrier<>* bar = nullptr;
float xchg[2048];
inline void sync() { bar->arrive_and_wait(); }
}  // namespace sim
#define threadIdx (sim::tid_v)
#define blockDim (sim::block_v)

static inline void __syncthreads() { sim::sync(); }
static inline float __shfl_xor_sync(unsigned, float v, int lane_mask, int = 32) {
  const unsigned t = threadIdx.x;
  sim::xchg[t] = v;
  sim::sync();
  const unsigned src = (t & ~31u) | ((t ^ (unsigned)lane_mask) & 31u);
  const float r = src < blockDim.x ? sim::xchg[src] : v;
  sim::sync();
  return r;
}
static inline float __uint_as_float(uint32_t u) { float f; std::memcpy(&f, &u, 4); return f; }
static inline uint32_t __float_as_uint(float f) { uint32_t u; std::memcpy(&u, &f, 4); return u; }
static inline float rsqrtf(float x) { return 1.0f / sqrtf(x); }
static inline unsigned atomicMax(unsigned* p, unsigned v) { unsigned o = *p; if (v > o) *p = v; return o; }

namespace flashinfer {
template <typename T, size_t N>
struct vec_t {
  T data[N];
  T& operator[](size_t i) { return data[i]; }
  const T& operator[](size_t i) const { return data[i]; }
  void load(const T* p) { std::memcpy(data, p, sizeof(data)); }
  void store(T* p) const { std::memcpy(p, data, sizeof(data)); }
  void fill(T v) { for (auto& d : data) d = v; }
};
namespace trtllm_allreduce_fusion {
template <typename A, typename B>
inline int ceil_div(A a, B b) { return (int)((a + b - 1) / b); }
namespace details {
static constexpr int kBytesPerAccess = 16;
static constexpr float kFP8E4M3Max = 448.f;
static constexpr float kDynamicFP8MinScale = 1e-10f;
}  // namespace details
template <typename T>
struct AllReduceFusionParams {
  int nranks, rank, size, hidden_dim;
  void* allreduce_in; void* residual_in; void* allreduce_out; void* residual_out; void* norm_out;
  void* quant_out; void* scale_out; void* rms_gamma;
  float rms_eps, weight_bias;
  float* scale_factor;
  int layout, block_quant_group_size, tma_aligned_mn;
};
namespace utils {
template <typename T, int NUM> inline T blockReduceMaxV2(T*) { return T(0); }
}  // namespace utils

#include "_ref/ar_extract.inc"

}  // namespace trtllm_allreduce_fusion
}  // namespace flashinfer

namespace ar = flashinfer::trtllm_allreduce_fusion;
using T = __nv_bfloat16;
constexpr auto kPattern = ar::AllReduceFusionPattern::kARResidualRMSNormOutMXFP8;

template <int NRanks>
static void thread_body(const ar::AllReduceFusionParams<T>& params, const T* const* partials,
                        int token, unsigned t) {
  threadIdx.x = t;
  const int per_token = params.hidden_dim / 8;
  const int access_id = token * per_token + (int)t;
  ar::FusedOp<kPattern, T> fused_op(params, access_id, (int)t);
  flashinfer::vec_t<T, 8> vals[NRanks];
  for (int r = 0; r < NRanks; ++r) vals[r].load(partials[r] + (size_t)access_id * 8);
  flashinfer::vec_t<T, 8> sum = ar::allreduce_sum<T, 8, NRanks, true>(vals);
  fused_op(sum, token);
}

template <int NRanks>
static void run_all(const ar::AllReduceFusionParams<T>& params, const T* const* partials, int tokens) {
  const unsigned threads = (unsigned)params.hidden_dim / 8;
  sim::block_v = {threads, 1, 1};
  for (int token = 0; token < tokens; ++token) {
    std::barrier<> barrier((std::ptrdiff_t)threads);
    sim::bar = &barrier;
    std::vector<std::thread> pool;
    pool.reserve(threads);
    for (unsigned t = 0; t < threads; ++t)
      pool.emplace_back([&, t] { thread_body<NRanks>(params, partials, token, t); });
    for (auto& th : pool) th.join();
  }
}

// scale_out: the 128-row x 4-group swizzle, ceil(hidden / 128) * 512 bytes, tokens <= 128.
extern "C" int ar_ref_run(int nranks, int tokens, int hidden, const uint16_t* const* partials,
                          const uint16_t* residual, const uint16_t* gamma, float eps,
                          float weight_bias, uint16_t* residual_out, uint16_t* norm_out,
                          uint8_t* quant_out, uint8_t* scale_out) {
  if (hidden % 256 || hidden / 8 > 1024 || tokens < 1 || tokens > 128) return 1;
  ar::AllReduceFusionParams<T> p{};
  p.nranks = nranks;
  p.size = tokens * hidden;
  p.hidden_dim = hidden;
  p.residual_in = (void*)residual;
  p.residual_out = residual_out;
  p.norm_out = norm_out;
  p.quant_out = quant_out;
  p.scale_out = scale_out;
  p.rms_gamma = (void*)gamma;
  p.rms_eps = eps;
  p.weight_bias = weight_bias;
  const T* const* parts = reinterpret_cast<const T* const*>(partials);
  switch (nranks) {
    case 1: run_all<1>(p, parts, tokens); break;
    case 2: run_all<2>(p, parts, tokens); break;
    case 4: run_all<4>(p, parts, tokens); break;
    case 8: run_all<8>(p, parts, tokens); break;
    default: return 2;
  }
  return 0;
}
