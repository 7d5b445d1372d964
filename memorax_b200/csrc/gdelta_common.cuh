// Shared pieces of the gated delta-rule kernels (head dimension 128, 64-token chunks).
//
// Recurrence per head (S is d_v x d_k, a_t = done_t ? 0 : alpha_t):
//   S_t = a_t S_{t-1} (I - beta_t k_t k_t^T) + beta_t v_t k_t^T,   o_t = S_t q_t.
// Chunk form used by both kernels (rows t, j inside a chunk; cum_t = sum_{i<=t} log alpha_i):
//   G_tj  = exp(cum_t - cum_j) if no reset in (j, t] else 0           (j <= t)
//   g_t   = G from the chunk start (0 once a reset has been passed)   ("live" rows)
//   gam_j = G_{last,j}                                                  ("keep" rows)
//   L = strict_tril(G o K K^T),  (I + diag(beta) L) U = diag(beta) (V - diag(g) K S_in^T)
//   O = diag(g) Q S_in^T + tril(G o Q K^T) U,   S_out = g_last S_in + (diag(gam) U)^T K.
// Accumulators that have d_v on their rows are kept transposed ([v][t]) so that
// they fill all 128 TMEM lanes and thread v owns one value column of U.
#pragma once

#include <cuda_bf16.h>

#include "linattn_common.cuh"
#include "mxk_common.cuh"
#include "umma.cuh"

namespace mxk {
namespace gdelta {

using linattn::row_first_key;
using linattn::row_keep;
using linattn::row_live;

constexpr int kC = 64;
constexpr int kD = 128;
constexpr int kThreads = 128;
constexpr int kPanD = kD / 8;   // panels of a matrix with 128 columns
constexpr int kPanC = kC / 8;   // panels of a matrix with 64 columns
constexpr int kStateVecs = kPanD * kD;  // uint4 per bf16 state copy (32 KiB)
constexpr int kUVecs = kPanC * kD;      // uint4 per bf16 U^T of one chunk (16 KiB)
// Residual the forward call leaves per (sequence, chunk): the state entering the chunk, then U^T.
constexpr int kResidualVecs = kStateVecs + kUVecs;

// State-independent part of a chunk, written by the preparation kernel (gdelta_prep.cu) for both the
// forward and the backward kernel: T' = (I + diag(beta) L)^-1 diag(beta) as bf16, [j/8][t][8] (8 KiB).
constexpr int kAinvVecs = kPanC * kC;
// Launches the preparation kernel over all (batch, head, chunk) items; defined in gdelta_prep.cu.
int launch_prep(const void* k, const float* alpha, const float* beta, const uint8_t* done, void* ainv, int* status,
                int B, int T, int H, int d, cudaStream_t stream);

// A 64 x 128 bf16 tile as SW tiles (umma.cuh): two 64-column blocks of 64 lines x 128 bytes.
constexpr int kSwBlockVecs = kC * 8;   // uint4 per block (8 KiB)
// uint4 index of the 16-byte vector `pn` (0..15) of token row `r`
__device__ __forceinline__ int sw_slot(int r, int pn) { return (pn >> 3) * kSwBlockVecs + umma::sw_idx(r, pn & 7); }

// Element [t][c] of a 64 x 128 bf16 tile stored as SW tiles.
__device__ __forceinline__ float sw_bf16_at(const uint4* tile, int t, int c) {
  const __nv_bfloat16* p = reinterpret_cast<const __nv_bfloat16*>(tile + sw_slot(t, c >> 3));
  return __bfloat162float(p[c & 7]);
}

struct ChunkDecay {
  float alpha[kC], beta[kC], cum[kC], g[kC], gam[kC];
};

// Builds cum / g / gam from cd.alpha / cd.beta of one chunk (already in shared
// memory and visible to all threads).  Call with all threads; ends with a __syncthreads().
__device__ __forceinline__ void finish_chunk_decay(ChunkDecay& cd, uint64_t dm, int tid) {
  if (tid < 32) {
    const float l0 = __logf(cd.alpha[2 * tid]), l1 = __logf(cd.alpha[2 * tid + 1]);
    float s = l0 + l1;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const float o = __shfl_up_sync(0xffffffffu, s, off);
      if (tid >= off) s += o;
    }
    cd.cum[2 * tid] = s - l1;
    cd.cum[2 * tid + 1] = s;
  }
  __syncthreads();
  if (tid < kC) {
    cd.g[tid] = row_live(dm, tid) ? __expf(cd.cum[tid]) : 0.f;
    cd.gam[tid] = row_keep(dm, tid) ? __expf(cd.cum[kC - 1] - cd.cum[tid]) : 0.f;
  }
  __syncthreads();
}

// alpha / beta of token t0 + tid (threads 0..63) for a later chunk_decay_from_regs.
// Rows past the end of the sequence get alpha = 1, beta = 0, i.e. they leave the
// state untouched.
__device__ __forceinline__ float2 fetch_chunk_decay(const float* alpha, const float* beta, size_t bt_base, int H, int h,
                                                    int t0, int T, int tid) {
  float2 ab = make_float2(1.f, 0.f);
  if (tid < kC && t0 >= 0 && t0 + tid < T) {
    const size_t idx = (bt_base + t0 + tid) * H + h;
    ab = make_float2(__ldg(alpha + idx), __ldg(beta + idx));
  }
  return ab;
}
__device__ __forceinline__ void chunk_decay_from_regs(ChunkDecay& cd, float2 ab, uint64_t dm, int tid) {
  if (tid < kC) {
    cd.alpha[tid] = ab.x;
    cd.beta[tid] = ab.y;
  }
  __syncthreads();
  finish_chunk_decay(cd, dm, tid);
}

// Element [t][c] of a 64 x 128 bf16 tile stored row-major.
__device__ __forceinline__ float bf16_at(const uint4* plain, int t, int c) {
  const __nv_bfloat16* p = reinterpret_cast<const __nv_bfloat16*>(plain);
  return __bfloat162float(p[t * kD + c]);
}

// Unit-triangular solves, one independent column per thread, on packed fp32
// pairs (fma.rn.f32x2): r2[i] = (r[2i], r[2i+1]).
//
// forward_substitute: r holds the right-hand side on entry and the solution of
// (I + diag(beta) L) u = r on exit; nlt[j * 64 + t] = -beta_t L_tj (zero for t <= j).
// The template form eliminates columns J0 .. J1 - 1 from rows < T1 only, so that a solve
// can be blocked: rows 0..31 first (<0, 31, 32>), then -- once the 32 x 32 off-diagonal
// block times the first half has been added to rows 32..63 -- the rest (<32, 63, 64>).
template <int J0, int J1, int T1>
__device__ __forceinline__ void forward_substitute_range(float2* r2, const float* nlt) {
  const float4* lt4 = reinterpret_cast<const float4*>(nlt);
#pragma unroll
  for (int j = J0; j < J1; ++j) {
    const float uj = (j & 1) ? r2[j >> 1].y : r2[j >> 1].x;
    const float2 u2 = make_float2(uj, uj);
#pragma unroll
    for (int m = (j + 1) / 4; m < T1 / 4; ++m) {
      const float4 l = lt4[j * (kC / 4) + m];
      r2[2 * m] = __ffma2_rn(make_float2(l.x, l.y), u2, r2[2 * m]);
      r2[2 * m + 1] = __ffma2_rn(make_float2(l.z, l.w), u2, r2[2 * m + 1]);
    }
  }
}
__device__ __forceinline__ void forward_substitute(float2* r2, const float* nlt) {
  forward_substitute_range<0, kC - 1, kC>(r2, nlt);
}

// backward_substitute: r holds dU on entry and (I + diag(beta) L)^-T dU on exit;
// nl[i * kStride + t] = -beta_i L_it (zero for t >= i), kStride a multiple of 4.
// The range form eliminates rows I1 down to I0 from the entries t >= T0 only (T0 a multiple of 4),
// so that the solve can be blocked like the forward one: rows 63..33 over entries 32.. first
// (<63, 33, 32>), then -- once the off-diagonal block times the second half has been added to
// entries 0..31 -- rows 31..1 (<31, 1, 0>).
template <int kStride, int I1, int I0, int T0>
__device__ __forceinline__ void backward_substitute_range(float2* r2, const float* nl) {
  const float4* l4 = reinterpret_cast<const float4*>(nl);
#pragma unroll
  for (int i = I1; i >= I0; --i) {
    const float xi = (i & 1) ? r2[i >> 1].y : r2[i >> 1].x;
    const float2 x2 = make_float2(xi, xi);
#pragma unroll
    for (int m = T0 / 4; m <= (i - 1) / 4; ++m) {
      const float4 c = l4[i * (kStride / 4) + m];
      r2[2 * m] = __ffma2_rn(make_float2(c.x, c.y), x2, r2[2 * m]);
      r2[2 * m + 1] = __ffma2_rn(make_float2(c.z, c.w), x2, r2[2 * m + 1]);
    }
  }
}
template <int kStride>
__device__ __forceinline__ void backward_substitute(float2* r2, const float* nl) {
  backward_substitute_range<kStride, kC - 1, 1, 0>(r2, nl);
}

}  // namespace gdelta
}  // namespace mxk
