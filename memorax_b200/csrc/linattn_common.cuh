// Constants and mask helpers shared by the linear-attention forward and
// backward kernels.
#pragma once

#include <cuda_bf16.h>

#include "mxk_common.cuh"
#include "umma.cuh"

namespace mxk {
namespace linattn {

constexpr int kC = 64;        // tokens per chunk
constexpr int kD = 64;        // head dimension (d_k = d_v)
constexpr int kDX = kD + 8;   // value columns + the normaliser column block
constexpr int kThreads = 128;
constexpr int kPanels = kD / 8;
constexpr int kPanelsX = kDX / 8;
constexpr uint32_t kOneBf16 = 0x3F80u;

__device__ __forceinline__ float phi(float x) { return x > 0.f ? x + 1.f : __expf(x); }

// Feature map elu(x) + 1 on packed bf16 pairs, entirely in bf16x2 arithmetic (the result is
// rounded to bf16 anyway): elu(x) + 1 = max(x, 0) + min(exp(x), 1) -- for x > 0 the second term
// is exactly 1, otherwise the first is exactly 0 -- i.e. one multiply by log2(e), one ex2, one
// min, one max, one add per pair.
__device__ __forceinline__ uint32_t phi2(uint32_t x) {
  uint32_t t, ex, pos, r;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(t) : "r"(x), "r"(0x3FB93FB9u));     // log2(e) = 1.4453 in bf16
  asm("ex2.approx.ftz.bf16x2 %0, %1;" : "=r"(ex) : "r"(t));
  asm("min.bf16x2 %0, %1, %2;" : "=r"(ex) : "r"(ex), "r"(0x3F803F80u));       // min(exp(x), 1)
  asm("max.bf16x2 %0, %1, %2;" : "=r"(pos) : "r"(x), "r"(0u));                // max(x, 0)
  asm("add.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(pos), "r"(ex));
  return r;
}
__device__ __forceinline__ uint4 phi8(uint4 x) { return make_uint4(phi2(x.x), phi2(x.y), phi2(x.z), phi2(x.w)); }

// 64 done flags of a chunk as a bit mask (bit i = token t0 + i), built in two steps so that the byte
// loads of a later chunk can be issued long
// before their values are needed.  The loaded bytes stay untouched in registers until
// done_mask_from_flags(): any arithmetic on them at load time would make the in-order
// thread wait for the loads right there.
struct DoneFlags {
  uint32_t a, b;   // raw flag bytes of tokens t0 + lane and t0 + 32 + lane (0 when out of range)
};
__device__ __forceinline__ DoneFlags load_done_flags(const uint8_t* drow, int t0, int T, int lane) {
  DoneFlags f{0u, 0u};
  if (drow && t0 >= 0) {
    const int ta = t0 + lane, tb = t0 + 32 + lane;
    if (ta < T) f.a = drow[ta];
    if (tb < T) f.b = drow[tb];
  }
  return f;
}
__device__ __forceinline__ uint64_t done_mask_from_flags(DoneFlags f) {
  const unsigned lo = __ballot_sync(0xffffffffu, f.a != 0u);
  const unsigned hi = __ballot_sync(0xffffffffu, f.b != 0u);
  return (static_cast<uint64_t>(hi) << 32) | lo;
}
__device__ __forceinline__ bool row_live(uint64_t dm, int i) { return (dm & ((2ull << i) - 1ull)) == 0ull; }
__device__ __forceinline__ bool row_keep(uint64_t dm, int j) { return j >= 63 || (dm >> (j + 1)) == 0ull; }
__device__ __forceinline__ int row_first_key(uint64_t dm, int i) {
  const uint64_t m = dm & ((2ull << i) - 1ull);
  return m ? 63 - __clzll(static_cast<long long>(m)) : 0;
}

// Vector `vid` (0..511) of a 64 x 64 bf16 tile: eight consecutive lanes take
// eight different rows (conflict-free 16-byte shared stores) while a warp still
// covers 64 contiguous bytes of every row it touches.
__device__ __forceinline__ void tile_vec(int vid, int& row, int& seg) {
  row = (vid & 7) + 8 * (vid >> 6);
  seg = (vid >> 3) & 7;
}

}  // namespace linattn
}  // namespace mxk
