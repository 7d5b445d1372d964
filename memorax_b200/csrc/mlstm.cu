// mLSTM (matrix-memory LSTM, mlstm.py:163-240) under Memoroid.scan_fn's reset rule, forward and backward.
//
// Per head, with the running-max stabiliser m (all in fp32):
//   m_t = max(m_{t-1} + log_f_t, log_i_t)
//   C_t = exp(m_{t-1} + log_f_t - m_t) C_{t-1} + exp(log_i_t - m_t) k_t v_t^T     (n_t likewise with k_t)
//   h_t = q_t^T C_t / (max(|q_t . n_t|, exp(-m_t)) + eps)
// and done_t discards (C, n, m) of the past.  The reference materialises every C_t (T x d x d per head) and
// combines them with ~2 log2(T) passes of an associative scan; here one CTA owns one (batch, head), keeps
// the d x d memory in registers and walks time once: a group of lanes holds column j of C (the read-out
// q^T C needs no exchange between threads), rows of q, k, v are staged through shared memory eight
// steps at a time, and the one scalar every thread needs per step (q . n) is a block reduction.
//
// Backward (what jax.grad derives from the scan; the reference has no hand-written rule) without storing
// any C_t: pass A walks forward again and emits dq_t = C_t dnum_t + dqn_t n_t together with five scalars
// per step; pass B walks backward carrying the cotangents dC (as columns AND as rows, so that both
// dk_t = sb_t (dC v_t + dn) and dv_t = sb_t dC^T k_t are thread-local), dn, dm and
//   G_t = <dC_t, C_t> + <dn_t, n_t>,
// which obeys G_{t-1} = G_t - sb_t k_t . (dC_t v_t + dn_t) + q_{t-1} . dq_{t-1} and yields the gate
// cotangents (sa_t d sa_t = G_t - sb_t d sb_t) without the forward states.  Both passes run in one kernel.
#include <cuda_runtime.h>
#include <math.h>

#include "mxk_common.cuh"

namespace mxk {
namespace {

constexpr int kTS = 8;        // time steps staged in shared memory at a time
constexpr int kAux = 6;       // per (b, t, h) scalars pass A leaves for pass B: den, dqn, dm_read, gq, m_t, m_prev

struct MlstmParams {
  const float* q; const float* k; const float* v;       // (B,T,H,d)
  const float* log_i; const float* log_f;               // (B,T,H)
  const float* c0; const float* n0; const float* m0; const float* f0;   // (B,H,d,d) [key][value], (B,H,d), (B,H), (B,H)
  const uint8_t* done;                                   // (B,T)
  float* h;                                              // (B,T,H,d)
  float* c_last; float* n_last; float* m_last; float* f_last;
  // backward only
  const float* dh; const float* dc_last; const float* dn_last; const float* dm_last;
  float* dq; float* dk; float* dv; float* dlog_i; float* dlog_f;
  float* dc0; float* dn0; float* dm0;
  float* aux;                                            // (B,T,H,kAux) workspace
  int B, T, H;
  float eps;
};

template <int NW>
__device__ __forceinline__ float block_sum(float x, float (*red)[NW], int slot, int warp, int lane) {
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) x += __shfl_xor_sync(0xffffffffu, x, off);
  if (NW == 1) return x;
  if (lane == 0) red[slot][warp] = x;
  __syncthreads();
  float s = red[slot][0];
#pragma unroll
  for (int w = 1; w < NW; ++w) s += red[slot][w];
  return s;
}
template <int NW>
__device__ __forceinline__ float2 block_sum2(float2 x, float2 (*red)[NW], int slot, int warp, int lane) {
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) {
    x.x += __shfl_xor_sync(0xffffffffu, x.x, off);
    x.y += __shfl_xor_sync(0xffffffffu, x.y, off);
  }
  if (NW == 1) return x;
  if (lane == 0) red[slot][warp] = x;
  __syncthreads();
  float2 s = red[slot][0];
#pragma unroll
  for (int w = 1; w < NW; ++w) { s.x += red[slot][w].x; s.y += red[slot][w].y; }
  return s;
}

// Sum over the SPLIT adjacent lanes that share one column / row index.
template <int SPLIT>
__device__ __forceinline__ float group_sum(float x) {
#pragma unroll
  for (int off = 1; off < SPLIT; off <<= 1) x += __shfl_xor_sync(0xffffffffu, x, off);
  return x;
}

// Stages rows t0 .. t0 + kTS - 1 of up to four (B,T,H,d) tensors and the step scalars of the chunk.
template <int D, int NT, int NROW>
__device__ __forceinline__ void stage_rows(const MlstmParams& p, const float* const* src, float (*dst)[kTS][D], float* sli,
                                           float* slf, uint8_t* sdone, int b, int h, int t0, int tid) {
  for (int idx = tid; idx < kTS * D; idx += NT) {
    const int tt = idx / D, c = idx % D, t = t0 + tt;
    if (t < p.T) {
      const size_t off = ((static_cast<size_t>(b) * p.T + t) * p.H + h) * D + c;
#pragma unroll
      for (int r = 0; r < NROW; ++r) dst[r][tt][c] = __ldg(src[r] + off);
    }
  }
  if (tid < kTS) {
    const int t = t0 + tid;
    if (t < p.T) {
      const size_t off = (static_cast<size_t>(b) * p.T + t) * p.H + h;
      sli[tid] = __ldg(p.log_i + off);
      slf[tid] = __ldg(p.log_f + off);
      sdone[tid] = p.done ? p.done[static_cast<size_t>(b) * p.T + t] : 0;
    }
  }
}

// One step of the stabilised gates: returns (sa, sb) and updates m.
__device__ __forceinline__ void gate_step(bool reset, float li, float lf, float& m, float& sa, float& sb) {
  const float m_dec = reset ? -INFINITY : m + lf;
  const float m_new = fmaxf(m_dec, li);
  sa = reset ? 0.f : expf(m_dec - m_new);
  sb = expf(li - m_new);
  m = m_new;
}

// ------------------------------------------------------------------ forward
// NT = D * SPLIT threads; thread (j, half) holds rows [half * L, half * L + L) of column j of C (L = D / SPLIT;
// the SPLIT threads of a column are adjacent lanes and combine through shuffles).  One thread per column is the
// fastest where the registers allow it (d <= 64; measured at d = 64: 2.0 / 2.7 / 3.6 ms backward with 1 / 2 / 4
// lanes per column): the kernel is bound by instruction throughput at low occupancy, not by per-step latency.
template <int D, int SPLIT>
__global__ void __launch_bounds__(D * SPLIT) mlstm_fwd_kernel(const MlstmParams p) {
  constexpr int L = D / SPLIT, NT = D * SPLIT, NW = NT / 32;
  __shared__ __align__(16) float rows[3][kTS][D];
  __shared__ float sli[kTS], slf[kTS];
  __shared__ uint8_t sdone[kTS];
  __shared__ float red[2][NW];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int j = tid / SPLIT, half = tid % SPLIT, i0 = half * L;
  const int bh = blockIdx.x, b = bh / p.H, h = bh % p.H;

  float cc[L];
#pragma unroll
  for (int i = 0; i < L; ++i) cc[i] = p.c0 ? p.c0[(static_cast<size_t>(bh) * D + i0 + i) * D + j] : 0.f;
  float nj = p.n0 ? p.n0[static_cast<size_t>(bh) * D + j] : 0.f;
  float m = p.m0 ? p.m0[bh] : -1e9f;
  float fsum = p.f0 ? p.f0[bh] : 0.f;
  const float* src[3] = {p.q, p.k, p.v};

  for (int t0 = 0; t0 < p.T; t0 += kTS) {
    __syncthreads();
    stage_rows<D, NT, 3>(p, src, rows, sli, slf, sdone, b, h, t0, tid);
    __syncthreads();
    const int steps = min(kTS, p.T - t0);
    for (int tt = 0; tt < steps; ++tt) {
      const bool reset = sdone[tt] != 0;
      float sa, sb;
      gate_step(reset, sli[tt], slf[tt], m, sa, sb);
      fsum = reset ? slf[tt] : fsum + slf[tt];
      const float sbv = sb * rows[2][tt][j];
      float part = 0.f;
      // broadcast reads of the staged k_t, q_t rows, four values per shared-memory access
      const float4* k4 = reinterpret_cast<const float4*>(&rows[1][tt][i0]);
      const float4* q4 = reinterpret_cast<const float4*>(&rows[0][tt][i0]);
#pragma unroll
      for (int i = 0; i < L / 4; ++i) {
        const float4 kk = k4[i], qq = q4[i];
        cc[4 * i] = fmaf(sa, cc[4 * i], kk.x * sbv);
        cc[4 * i + 1] = fmaf(sa, cc[4 * i + 1], kk.y * sbv);
        cc[4 * i + 2] = fmaf(sa, cc[4 * i + 2], kk.z * sbv);
        cc[4 * i + 3] = fmaf(sa, cc[4 * i + 3], kk.w * sbv);
        part = fmaf(qq.x, cc[4 * i], part);
        part = fmaf(qq.y, cc[4 * i + 1], part);
        part = fmaf(qq.z, cc[4 * i + 2], part);
        part = fmaf(qq.w, cc[4 * i + 3], part);
      }
      part = group_sum<SPLIT>(part);
      nj = fmaf(sa, nj, sb * rows[1][tt][j]);
      const float qn = block_sum<NW>(half == 0 ? rows[0][tt][j] * nj : 0.f, red, tt & 1, warp, lane);
      const float den = fmaxf(fabsf(qn), expf(-m)) + p.eps;
      if (half == 0) p.h[((static_cast<size_t>(b) * p.T + t0 + tt) * p.H + h) * D + j] = part / den;
    }
  }
  if (p.c_last) {
#pragma unroll
    for (int i = 0; i < L; ++i) p.c_last[(static_cast<size_t>(bh) * D + i0 + i) * D + j] = cc[i];
  }
  if (half == 0 && p.n_last) p.n_last[static_cast<size_t>(bh) * D + j] = nj;
  if (tid == 0) {
    if (p.m_last) p.m_last[bh] = m;
    if (p.f_last) p.f_last[bh] = fsum;
  }
}

// ----------------------------------------------------------------- backward
template <int D, int SPLIT>
__global__ void __launch_bounds__(D * SPLIT) mlstm_bwd_kernel(const MlstmParams p) {
  constexpr int L = D / SPLIT, NT = D * SPLIT, NW = NT / 32;
  __shared__ __align__(16) float rows[4][kTS][D];      // q, k, v, dh of the staged steps
  __shared__ float sli[kTS], slf[kTS];
  __shared__ uint8_t sdone[kTS];
  __shared__ __align__(16) float sdnum[2][D];          // dnum of the current step (double-buffered by step parity)
  __shared__ float red[2][NW];
  __shared__ float2 red2[2][NW];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int j = tid / SPLIT, half = tid % SPLIT, i0 = half * L;
  const int bh = blockIdx.x, b = bh / p.H, h = bh % p.H;
  const float* src[4] = {p.q, p.k, p.v, p.dh};
  float* aux = p.aux + static_cast<size_t>(b) * p.T * p.H * kAux;   // + (t * H + h) * kAux

  // ---- pass A: forward again; col[i] = C[i0 + i][j], row[i] = C[j][i0 + i] ----
  float g_init;
  {
    float col[L], row[L];
#pragma unroll
    for (int i = 0; i < L; ++i) {
      col[i] = p.c0 ? p.c0[(static_cast<size_t>(bh) * D + i0 + i) * D + j] : 0.f;
      row[i] = p.c0 ? p.c0[(static_cast<size_t>(bh) * D + j) * D + i0 + i] : 0.f;
    }
    float nj = p.n0 ? p.n0[static_cast<size_t>(bh) * D + j] : 0.f;
    float m = p.m0 ? p.m0[bh] : -1e9f;
    for (int t0 = 0; t0 < p.T; t0 += kTS) {
      __syncthreads();
      stage_rows<D, NT, 4>(p, src, rows, sli, slf, sdone, b, h, t0, tid);
      __syncthreads();
      const int steps = min(kTS, p.T - t0);
      for (int tt = 0; tt < steps; ++tt) {
        const bool reset = sdone[tt] != 0;
        const float m_prev = reset ? -INFINITY : m;
        float sa, sb;
        gate_step(reset, sli[tt], slf[tt], m, sa, sb);
        const float kj = rows[1][tt][j], vj = rows[2][tt][j];
        const float sbv = sb * vj, sbk = sb * kj;
        float num = 0.f;
        {
          const float4* q4 = reinterpret_cast<const float4*>(&rows[0][tt][i0]);
          const float4* k4 = reinterpret_cast<const float4*>(&rows[1][tt][i0]);
          const float4* v4 = reinterpret_cast<const float4*>(&rows[2][tt][i0]);
#pragma unroll
          for (int i = 0; i < L / 4; ++i) {
            const float4 qq = q4[i], kk = k4[i], vv = v4[i];
            const float ke[4] = {kk.x, kk.y, kk.z, kk.w}, ve[4] = {vv.x, vv.y, vv.z, vv.w}, qe[4] = {qq.x, qq.y, qq.z, qq.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              col[4 * i + e] = fmaf(sa, col[4 * i + e], ke[e] * sbv);
              row[4 * i + e] = fmaf(sa, row[4 * i + e], ve[e] * sbk);
              num = fmaf(qe[e], col[4 * i + e], num);
            }
          }
        }
        num = group_sum<SPLIT>(num);
        nj = fmaf(sa, nj, sb * kj);
        const float qj = rows[0][tt][j], dhj = rows[3][tt][j];
        const float2 s = block_sum2<NW>(half == 0 ? make_float2(qj * nj, dhj * num) : make_float2(0.f, 0.f), red2,
                                        tt & 1, warp, lane);
        const float em = expf(-m);
        const float den = fmaxf(fabsf(s.x), em) + p.eps;
        const float dden = -s.y / (den * den);
        const bool qn_branch = fabsf(s.x) >= em;
        const float dqn = qn_branch ? (s.x > 0.f ? dden : (s.x < 0.f ? -dden : 0.f)) : 0.f;
        const float dm_read = qn_branch ? 0.f : -dden * em;
        if (half == 0) sdnum[tt & 1][j] = dhj / den;
        __syncthreads();
        float dqj = 0.f;
        {
          const float4* d4 = reinterpret_cast<const float4*>(&sdnum[tt & 1][i0]);
#pragma unroll
          for (int i = 0; i < L / 4; ++i) {
            const float4 dd = d4[i];
            dqj = fmaf(row[4 * i], dd.x, dqj);
            dqj = fmaf(row[4 * i + 1], dd.y, dqj);
            dqj = fmaf(row[4 * i + 2], dd.z, dqj);
            dqj = fmaf(row[4 * i + 3], dd.w, dqj);
          }
        }
        dqj = group_sum<SPLIT>(dqj);
        dqj = fmaf(dqn, nj, dqj);
        const size_t tok = (static_cast<size_t>(b) * p.T + t0 + tt) * p.H + h;
        if (half == 0) p.dq[tok * D + j] = dqj;
        const float gq = block_sum<NW>(half == 0 ? qj * dqj : 0.f, red, tt & 1, warp, lane);
        if (tid == 0) {
          float* a = aux + (static_cast<size_t>(t0 + tt) * p.H + h) * kAux;
          a[0] = den; a[1] = dqn; a[2] = dm_read; a[3] = gq; a[4] = m; a[5] = m_prev;
        }
      }
    }
    // G at the end of the sequence: <dC_T, C_T> + <dn_T, n_T>
    float part = 0.f;
    if (p.dc_last) {
#pragma unroll
      for (int i = 0; i < L; ++i) part = fmaf(p.dc_last[(static_cast<size_t>(bh) * D + i0 + i) * D + j], col[i], part);
    }
    if (p.dn_last && half == 0) part = fmaf(p.dn_last[static_cast<size_t>(bh) * D + j], nj, part);
    __syncthreads();
    g_init = block_sum<NW>(part, red, 0, warp, lane);
  }

  // ---- pass B: backward; col[i] = dC[i0 + i][j], row[i] = dC[j][i0 + i] ----
  float col[L], row[L];
#pragma unroll
  for (int i = 0; i < L; ++i) {
    col[i] = p.dc_last ? p.dc_last[(static_cast<size_t>(bh) * D + i0 + i) * D + j] : 0.f;
    row[i] = p.dc_last ? p.dc_last[(static_cast<size_t>(bh) * D + j) * D + i0 + i] : 0.f;
  }
  float dnj = p.dn_last ? p.dn_last[static_cast<size_t>(bh) * D + j] : 0.f;
  float dm = p.dm_last ? p.dm_last[bh] : 0.f;
  float G = g_init;
  const int nblocks = (p.T + kTS - 1) / kTS;
  for (int blk = nblocks - 1; blk >= 0; --blk) {
    const int t0 = blk * kTS;
    __syncthreads();
    stage_rows<D, NT, 4>(p, src, rows, sli, slf, sdone, b, h, t0, tid);
    __syncthreads();
    const int steps = min(kTS, p.T - t0);
    for (int tt = steps - 1; tt >= 0; --tt) {
      const float* a = aux + (static_cast<size_t>(t0 + tt) * p.H + h) * kAux;
      const float den = a[0], dqn = a[1], dm_read = a[2], gq = a[3], m_t = a[4], m_prev = a[5];
      const bool reset = sdone[tt] != 0;
      const float li = sli[tt], lf = slf[tt];
      const float m_dec = m_prev + lf;                 // -inf at a reset
      const float sa = reset ? 0.f : expf(m_dec - m_t), sb = expf(li - m_t);
      const float qj = rows[0][tt][j], kj = rows[1][tt][j], vj = rows[2][tt][j];
      const float dnum_j = rows[3][tt][j] / den;
      if (half == 0) sdnum[tt & 1][j] = dnum_j;
      __syncthreads();
      // cotangents of (C_t, n_t, m_t, G_t) including this step's read-out
      float dvj = 0.f, wj = 0.f;
      {
        const float4* q4 = reinterpret_cast<const float4*>(&rows[0][tt][i0]);
        const float4* k4 = reinterpret_cast<const float4*>(&rows[1][tt][i0]);
        const float4* v4 = reinterpret_cast<const float4*>(&rows[2][tt][i0]);
        const float4* d4 = reinterpret_cast<const float4*>(&sdnum[tt & 1][i0]);
#pragma unroll
        for (int i = 0; i < L / 4; ++i) {
          const float4 qq = q4[i], kk = k4[i], vv = v4[i], dd = d4[i];
          const float qe[4] = {qq.x, qq.y, qq.z, qq.w}, ke[4] = {kk.x, kk.y, kk.z, kk.w};
          const float ve[4] = {vv.x, vv.y, vv.z, vv.w}, de[4] = {dd.x, dd.y, dd.z, dd.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            col[4 * i + e] = fmaf(qe[e], dnum_j, col[4 * i + e]);
            row[4 * i + e] = fmaf(qj, de[e], row[4 * i + e]);
            dvj = fmaf(col[4 * i + e], ke[e], dvj);
            wj = fmaf(row[4 * i + e], ve[e], wj);
          }
        }
      }
      dvj = group_sum<SPLIT>(dvj);
      wj = group_sum<SPLIT>(wj);
      dnj = fmaf(dqn, qj, dnj);
      wj += dnj;
      dm += dm_read;
      G += gq;
      const size_t tok = (static_cast<size_t>(b) * p.T + t0 + tt) * p.H + h;
      if (half == 0) {
        p.dv[tok * D + j] = sb * dvj;
        p.dk[tok * D + j] = sb * wj;
      }
      const float sb_dsb = sb * block_sum<NW>(half == 0 ? kj * wj : 0.f, red, tt & 1, warp, lane);
      float d_li, d_lf;
      if (reset) {
        d_li = dm;
        d_lf = 0.f;
        dm = 0.f;
        G = 0.f;
        dnj = 0.f;
#pragma unroll
        for (int i = 0; i < L; ++i) { col[i] = 0.f; row[i] = 0.f; }
      } else {
        // sa = 0 (the past is more than e^-100 below this step's input gate, or the carry is initialize_carry's
        // m = -1e9): nothing flows to the past, exactly
        const float sa_dsa = sa == 0.f ? 0.f : G - sb_dsb;
        const float dm_t = dm - sa_dsa - sb_dsb;
        float d_mprev = sa_dsa;
        d_lf = sa_dsa;
        d_li = sb_dsb;
        if (m_dec >= li) { d_lf += dm_t; d_mprev += dm_t; }
        else d_li += dm_t;
        dm = d_mprev;
        G = sa_dsa;
        dnj *= sa;
#pragma unroll
        for (int i = 0; i < L; ++i) { col[i] *= sa; row[i] *= sa; }
      }
      if (tid == 0) {
        p.dlog_i[tok] = d_li;
        p.dlog_f[tok] = d_lf;
      }
    }
  }
  if (p.dc0) {
#pragma unroll
    for (int i = 0; i < L; ++i) p.dc0[(static_cast<size_t>(bh) * D + i0 + i) * D + j] = col[i];
  }
  if (p.dn0 && half == 0) p.dn0[static_cast<size_t>(bh) * D + j] = dnj;
  if (p.dm0 && tid == 0) p.dm0[bh] = dm;
}

template <typename K>
int launch(K kernel, const MlstmParams& p, int threads, mxk_stream_t stream) {
  kernel<<<p.B * p.H, threads, 0, static_cast<cudaStream_t>(stream)>>>(p);
  return launch_status();
}

int check(int B, int T, int H, int d) {
  if (B <= 0 || T <= 0 || H <= 0 || static_cast<long long>(B) * H > 0x7fffffffLL) return MXK_ERR_DIMS;
  if (d != 32 && d != 64 && d != 128) return MXK_ERR_UNSUPPORTED;
  return MXK_OK;
}

}  // namespace
}  // namespace mxk

extern "C" {

size_t mxk_mlstm_bwd_workspace_bytes(int B, int T, int H, int d) {
  if (mxk::check(B, T, H, d) != MXK_OK) return 0;
  return static_cast<size_t>(B) * T * H * mxk::kAux * sizeof(float);
}

int mxk_mlstm_f32_fwd(const float* q, const float* k, const float* v, const float* log_i, const float* log_f,
                      const float* c0, const float* n0, const float* m0, const float* f0, const uint8_t* done,
                      float* h, float* c_last, float* n_last, float* m_last, float* f_last, int B, int T, int H, int d,
                      float eps, mxk_stream_t stream) {
  using namespace mxk;
  if (!q || !k || !v || !log_i || !log_f || !h) return MXK_ERR_NULL;
  if (int st = check(B, T, H, d)) return st;
  MlstmParams p{};
  p.q = q; p.k = k; p.v = v; p.log_i = log_i; p.log_f = log_f;
  p.c0 = c0; p.n0 = n0; p.m0 = m0; p.f0 = f0; p.done = done;
  p.h = h; p.c_last = c_last; p.n_last = n_last; p.m_last = m_last; p.f_last = f_last;
  p.B = B; p.T = T; p.H = H; p.eps = eps;
  if (d == 32) return launch(mlstm_fwd_kernel<32, 1>, p, 32, stream);
  if (d == 64) return launch(mlstm_fwd_kernel<64, 1>, p, 64, stream);
  return launch(mlstm_fwd_kernel<128, 2>, p, 256, stream);
}

int mxk_mlstm_f32_bwd(const float* q, const float* k, const float* v, const float* log_i, const float* log_f,
                      const float* c0, const float* n0, const float* m0, const uint8_t* done, const float* dh,
                      const float* dc_last, const float* dn_last, const float* dm_last, float* dq, float* dk, float* dv,
                      float* dlog_i, float* dlog_f, float* dc0, float* dn0, float* dm0, void* workspace,
                      size_t workspace_bytes, int B, int T, int H, int d, float eps, mxk_stream_t stream) {
  using namespace mxk;
  if (!q || !k || !v || !log_i || !log_f || !dh || !dq || !dk || !dv || !dlog_i || !dlog_f) return MXK_ERR_NULL;
  if (int st = check(B, T, H, d)) return st;
  if (!workspace || workspace_bytes < mxk_mlstm_bwd_workspace_bytes(B, T, H, d)) return MXK_ERR_WORKSPACE;
  if (reinterpret_cast<uintptr_t>(workspace) & 3u) return MXK_ERR_ALIGN;
  MlstmParams p{};
  p.q = q; p.k = k; p.v = v; p.log_i = log_i; p.log_f = log_f;
  p.c0 = c0; p.n0 = n0; p.m0 = m0; p.done = done;
  p.dh = dh; p.dc_last = dc_last; p.dn_last = dn_last; p.dm_last = dm_last;
  p.dq = dq; p.dk = dk; p.dv = dv; p.dlog_i = dlog_i; p.dlog_f = dlog_f;
  p.dc0 = dc0; p.dn0 = dn0; p.dm0 = dm0;
  p.aux = static_cast<float*>(workspace);
  p.B = B; p.T = T; p.H = H; p.eps = eps;
  if (d == 32) return launch(mlstm_bwd_kernel<32, 1>, p, 32, stream);
  if (d == 64) return launch(mlstm_bwd_kernel<64, 1>, p, 64, stream);
  return launch(mlstm_bwd_kernel<128, 2>, p, 256, stream);
}

}  // extern "C"
