// Gate arithmetic shared by the chunked mLSTM forward and backward kernels (mlstm_tc.cu, mlstm_tc_bwd.cu):
// per 64-token chunk the chunk-local cumulative forget gates, the stabiliser of every step and the decay
// factors the tensor-core products are weighted with.
#pragma once

#include <math.h>

#include "linattn_common.cuh"

namespace mxk {
namespace mlstm_tc {

struct alignas(16) ChunkGates {
  float li[linattn::kC], lf[linattn::kC];   // log input / forget gates of the chunk's tokens (-inf / 0 past the end)
  float cum[linattn::kC];       // cumf_t = lf_0 + .. + lf_t
  float lic[linattn::kC];       // li_j - cumf_j
  alignas(16) float lic2[linattn::kC];   // the same times log2(e), for ex2
  float rowterm2[linattn::kC];  // (cumf_t - m_t) log2(e): D_tj = 2^(rowterm2_t + lic2_j)
  float m[linattn::kC];         // stabiliser after step t
  float rowterm[linattn::kC];   // cumf_t - m_t: D_tj = exp(rowterm_t + lic_j)
  float em[2][linattn::kC];     // exp(-m_t), double-buffered by chunk parity: read after the next chunk's scan has begun
  float w[linattn::kC];         // exp(m_in + cumf_t - m_t) for rows no reset precedes, else 0
  float kappa[linattn::kC];     // exp(li_j + cumf_T - cumf_j - m_T) for keys after the last reset, else 0
  float delta, m_out, f_out;    // exp(m_in + cumf_T - m_T) (0 with a reset); m_T; summed log forget gates since the last reset
};

// 2^x (one MUFU instruction; flushes denormal results to zero).
__device__ __forceinline__ float ex2_fast(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Gates of the two tokens a lane of the scanning warp owns (t0 + 2 lane, t0 + 2 lane + 1): (log_i, log_f) each;
// (-inf, 0) past the end of the sequence, so that such a token neither contributes a key nor moves the stabiliser.
struct LaneGates {
  float ia, la, ib, lb;
};
__device__ __forceinline__ LaneGates load_lane_gates(const float* log_i, const float* log_f, int b, int h, int t0, int T, int H, int lane) {
  LaneGates g{-INFINITY, 0.f, -INFINITY, 0.f};
  const int ta = t0 + 2 * lane;
  if (t0 >= 0 && ta < T) {
    const size_t idx = (static_cast<size_t>(b) * T + ta) * H + h;
    g.ia = __ldg(log_i + idx);
    g.la = __ldg(log_f + idx);
    if (ta + 1 < T) {
      g.ib = __ldg(log_i + idx + H);
      g.lb = __ldg(log_f + idx + H);
    }
  }
  return g;
}

// One warp, lane l owns tokens 2l and 2l + 1 and brings their gates; writes every field of g.  The stabiliser
//   m_t = max(m_{t-1} + lf_t, li_t)   (m_t = li_t at a reset)
// in closed form is cumf_t + max(m_in [if no reset up to t], max over the keys j of t's segment of li_j - cumf_j):
// an inclusive sum scan and a segmented running-maximum scan.
__device__ __forceinline__ void chunk_gate_scan(ChunkGates& g, const LaneGates& lg, uint64_t dm, float m_in, float f_in, int lane,
                                                int parity) {
  using linattn::row_keep;
  using linattn::row_live;
  const int a = 2 * lane, b = a + 1;
  const float la = lg.la, lb = lg.lb, ia = lg.ia, ib = lg.ib;
  g.li[a] = ia; g.li[b] = ib;
  g.lf[a] = la; g.lf[b] = lb;
  float s = la + lb;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const float o = __shfl_up_sync(0xffffffffu, s, off);
    if (lane >= off) s += o;
  }
  const float cum_b = s, cum_a = s - lb;
  const float xa = ia - cum_a, xb = ib - cum_b;
  const bool fa = (dm >> a) & 1ull, fb = (dm >> b) & 1ull;
  float v = fb ? xb : fmaxf(xa, xb);
  int f = (fa || fb) ? 1 : 0;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const float vo = __shfl_up_sync(0xffffffffu, v, off);
    const int fo = __shfl_up_sync(0xffffffffu, f, off);
    if (lane >= off) {
      v = f ? v : fmaxf(vo, v);
      f |= fo;
    }
  }
  const float ve = __shfl_up_sync(0xffffffffu, v, 1);
  const float pm_a = fa ? xa : (lane > 0 ? fmaxf(ve, xa) : xa);
  const float pm_b = v;
  const bool live_a = row_live(dm, a), live_b = row_live(dm, b);
  const float m_a = cum_a + fmaxf(live_a ? m_in : -INFINITY, pm_a);
  const float m_b = cum_b + fmaxf(live_b ? m_in : -INFINITY, pm_b);
  const float m_t = __shfl_sync(0xffffffffu, m_b, 31), cum_t = __shfl_sync(0xffffffffu, cum_b, 31);
  g.cum[a] = cum_a; g.cum[b] = cum_b;
  g.lic[a] = xa; g.lic[b] = xb;
  g.lic2[a] = xa * 1.4426950409f; g.lic2[b] = xb * 1.4426950409f;
  g.rowterm2[a] = (cum_a - m_a) * 1.4426950409f; g.rowterm2[b] = (cum_b - m_b) * 1.4426950409f;
  g.m[a] = m_a; g.m[b] = m_b;
  g.rowterm[a] = cum_a - m_a; g.rowterm[b] = cum_b - m_b;
  g.em[parity][a] = __expf(-m_a); g.em[parity][b] = __expf(-m_b);
  g.w[a] = live_a ? __expf(m_in + cum_a - m_a) : 0.f;
  g.w[b] = live_b ? __expf(m_in + cum_b - m_b) : 0.f;
  g.kappa[a] = row_keep(dm, a) ? __expf(xa + cum_t - m_t) : 0.f;
  g.kappa[b] = row_keep(dm, b) ? __expf(xb + cum_t - m_t) : 0.f;
  __syncwarp();
  if (lane == 0) {
    g.delta = dm ? 0.f : __expf(m_in + cum_t - m_t);
    g.m_out = m_t;
    if (dm) {
      const int r = 63 - __clzll(static_cast<long long>(dm));   // the chunk's last reset
      g.f_out = cum_t - g.cum[r] + g.lf[r];
    } else {
      g.f_out = f_in + cum_t;
    }
  }
  __syncwarp();
}

}  // namespace mlstm_tc
}  // namespace mxk
