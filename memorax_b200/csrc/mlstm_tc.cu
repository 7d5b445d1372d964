// mLSTM (mlstm.py:163-240 under Memoroid.scan_fn's reset rule) in chunked form on the sm_100a tensor cores:
// bf16 q, k, v in, bf16 h out, fp32 gates and carried state.  Forward kernel.
//
// The stabilised recurrence  m_t = max(m_{t-1} + lf_t, li_t),
//   C_t = exp(m_{t-1} + lf_t - m_t) C_{t-1} + exp(li_t - m_t) k_t v_t^T,   n_t likewise with k_t,
//   h_t = q_t^T C_t / (max(|q_t . n_t|, exp(-m_t)) + eps)
// unrolls over a 64-token chunk with cumf_t = lf_0 + .. + lf_t (chunk-local) into
//   D_tj   = exp(li_j + cumf_t - cumf_j - m_t)          key j in [last reset <= t, t]       (<= 1)
//   w_t    = exp(m_in + cumf_t - m_t)                    rows with no reset up to t ("live") (<= 1)
//   kappa_j = exp(li_j + cumf_T - cumf_j - m_T)          keys after the chunk's last reset ("keep")
//   delta  = exp(m_in + cumf_T - m_T)                    0 if the chunk has a reset
//   [num | q.n]_t = w_t q_t [C_in | n_in] + sum_j D_tj (q_t . k_j) [v_j | 1]
//   [C | n]_out   = delta [C_in | n_in] + sum_j kappa_j k_j [v_j | 1]
// i.e. linear attention (linattn.cu) with a decay mask: the same operand formats, the same one CTA per
// (batch, head) with the fp32 state [C | n]^T resident in tensor memory, the same "1" column that makes the
// normaliser q.n column 64 of the output accumulator.  Per chunk:
//   MMA 1:       P = Q K^T                                  (lower TMEM lanes)
//   warp 1:      gate scans (cumulative sum, segmented running maximum) -> D, w, kappa, delta factors, under the tile wait
//   epilogue A:  lower rows P~ = D o P (bf16), q_t <- w_t q_t in place; upper rows scale the state by delta
//                in tensor memory; all threads kappa o [V | 1]
//   MMA 2:       O = (w o Q) S_in^T + P~ [V | 1];   S += K^T (kappa o [V | 1])
//   epilogue B:  lower rows divide by the denominator and stage the output tile; upper rows convert the
//                new state to the next chunk's bf16 operand.
#include <cuda_bf16.h>

#include <cstddef>

#include "mxk_common.cuh"
#include "linattn_common.cuh"
#include "mlstm_tc_common.cuh"
#include "tma.cuh"

namespace mxk {
namespace {

using namespace umma;
using namespace linattn;
using namespace mlstm_tc;

struct FwdParams {
  const float* log_i; const float* log_f;          // (B,T,H)
  const float* c0; const float* n0; const float* m0; const float* f0;   // (B,H,d,d) [key][value], (B,H,d), (B,H), (B,H)
  const uint8_t* done;
  float* c_last; float* n_last; float* m_last; float* f_last;
  float* m_steps;        // optional (B,T,H): the stabiliser after every step (residual of the backward pass)
  uint4* chunk_states;   // optional residual: bf16 [C | n]^T panels entering every chunk
  int* status;
  int B, T, H, d;
  float eps;
  CUtensorMap map_q, map_k, map_o;   // 64-token tiles as SW tiles
  CUtensorMap map_v;                 // 64-token tiles in panel order
};

struct FwdSmem {
  uint4 q[kPanels * kC];        // Q, then w o Q, SW tile
  uint4 k[kPanels * kC];        // K, SW tile
  uint4 p[kPanels * kC];        // P~ = D o (Q K^T), SW tile; then the staged output tile
  uint4 alt[kPanelsX * kC];     // kappa o [V | 1]             [v/8][j]
  uint4 v[kPanelsX * kC];       // V | 1                       [v/8][j]
  uint4 s[kPanelsX * kD];       // bf16 [C | n]^T entering the chunk, then leaving it   [v/8][k]
  ChunkGates gates;
  uint64_t bar[2];
  uint64_t bar_load;
  uint32_t tmem;
};
static_assert(sizeof(FwdSmem) <= 56 * 1024, "four CTAs per SM");
static_assert(offsetof(FwdSmem, k) % 1024 == 0 && offsetof(FwdSmem, p) % 1024 == 0, "SW tiles are 1024-byte aligned");

#ifdef MXK_TIMING
}  // namespace
__device__ unsigned long long g_mtc_phase_cycles[16];
namespace {
#define MXK_TM(i) do { if (tid == 0 && (blockIdx.x % 37) == 0) { const long long now_ = clock64(); atomicAdd(&g_mtc_phase_cycles[i], (unsigned long long)(now_ - t_prev_)); t_prev_ = now_; } } while (0)
#else
#define MXK_TM(i) do {} while (0)
#endif
constexpr uint32_t kTmemCols = 128;
constexpr uint32_t kUpper = 16u << 16;

__global__ void __launch_bounds__(kThreads, 4) mlstm_tc_fwd_kernel(const __grid_constant__ FwdParams p) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  FwdSmem& sm = *reinterpret_cast<FwdSmem*>(smem_raw);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int bh = blockIdx.x, b = bh / p.H, h = bh % p.H;
  const bool upper = lane >= 16;
  const int row = warp * 16 + (lane & 15);   // lower: query row t; upper: state row (key feature)
  const int nchunks = (p.T + kC - 1) / kC;
  const int hd = p.d;

  if (tid == 0) {
    mbar_init(&sm.bar[0], 1);
    mbar_init(&sm.bar[1], 1);
    mbar_init(&sm.bar_load, 1);
    mbar_init_fence();
  }
  if (warp == 0) tmem_alloc(&sm.tmem, kTmemCols);
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem = sm.tmem;
  const uint32_t lane_base = tmem + (static_cast<uint32_t>(warp * 32) << 16);

  auto issue_chunk_loads = [&](int cc) {
    fence_smem_to_async();   // earlier generic-proxy accesses to the buffers come first
    tma::expect_bytes(&sm.bar_load, 3 * kPanels * kC * 16);
    tma::load_plain_tile(sm.q, &p.map_q, &sm.bar_load, cc * kC, h, b);
    tma::load_plain_tile(sm.k, &p.map_k, &sm.bar_load, cc * kC, h, b);
    tma::load_panel_tile(sm.v, &p.map_v, &sm.bar_load, cc * kC, h, b);
    if (cc > 0 && cc + 1 < nchunks) {   // not while a sequence starts: the prefetch would queue in front of every CTA's first tiles
      tma::prefetch_plain_tile(&p.map_q, (cc + 1) * kC, h, b);
      tma::prefetch_plain_tile(&p.map_k, (cc + 1) * kC, h, b);
      tma::prefetch_panel_tile(&p.map_v, (cc + 1) * kC, h, b);
    }
  };
  if (tid == 0) issue_chunk_loads(0);

  // Carried state -> TMEM (fp32, upper lanes) and its bf16 operand copy.  Upper thread `row` owns
  // [C | n]^T... row k of C (all values v) and n_k: C is (d_k, d_v) row-major in memory.
  {
    const float* c0 = (p.c0 && row < hd) ? p.c0 + (static_cast<size_t>(bh) * hd + row) * hd : nullptr;
    float vals[kDX];
#pragma unroll
    for (int vcol = 0; vcol < kDX; ++vcol) {
      float x = 0.f;
      if (upper && row < hd) {
        if (vcol < kD) x = (c0 && vcol < hd) ? c0[vcol] : 0.f;
        else if (vcol == kD) x = p.n0 ? p.n0[static_cast<size_t>(bh) * hd + row] : 0.f;
      }
      vals[vcol] = x;
    }
#pragma unroll
    for (int pn = 0; pn < kPanelsX; ++pn) {
      tmem_st8(lane_base + pn * 8, vals + pn * 8);
      if (upper) sm.s[pn * kD + row] = pack8_bf16(vals + pn * 8);
    }
    tmem_st_wait();
  }
  // the ones column of V | 1 has seven more columns in its panel: zero once, TMA never writes them
  if (tid < kC) sm.v[kPanels * kC + tid] = make_uint4(0, 0, 0, 0);

  const uint8_t* drow = p.done ? p.done + static_cast<size_t>(b) * p.T : nullptr;
  const uint32_t idesc_p = idesc_bf16(kC, kC, false, false);
  const uint32_t idesc_o = idesc_bf16(kC, kDX, false, true);
  const uint32_t idesc_s = idesc_bf16(kD, kDX, true, true);
  bool timed_out = false;
  float m_in = p.m0 ? p.m0[bh] : -1e9f;       // initialize_carry's stabiliser (mlstm.py:231-240)
  float f_in = p.f0 ? p.f0[bh] : 0.f;
  DoneFlags done_flags = load_done_flags(drow, 0, p.T, lane);
  LaneGates lane_gates = load_lane_gates(p.log_i, p.log_f, b, h, 0, p.T, p.H, lane);   // used by warp 1
  // Warp 1 computes a chunk's gate factors at the top of the chunk, while the other warps wait for the tiles
  // (one chunk ahead, under the previous chunk's second MMA group, measured 3 % slower: the scan then delays
  // the output epilogue), stores the stabilisers and fetches the gates of the chunk after.
  auto scan_chunk = [&](int cc, uint64_t dmc) {
    chunk_gate_scan(sm.gates, lane_gates, dmc, m_in, f_in, lane, cc & 1);
    lane_gates = load_lane_gates(p.log_i, p.log_f, b, h, (cc + 1) * kC, p.T, p.H, lane);
    m_in = sm.gates.m_out;
    f_in = sm.gates.f_out;
    if (p.m_steps) {
      const int ta = cc * kC + 2 * lane;
      float* dst = p.m_steps + (static_cast<size_t>(b) * p.T + ta) * p.H + h;
      if (ta < p.T) dst[0] = sm.gates.m[2 * lane];
      if (ta + 1 < p.T) dst[p.H] = sm.gates.m[2 * lane + 1];
    }
  };
#ifdef MXK_TIMING
  long long t_prev_ = clock64();
#endif

  for (int c = 0; c < nchunks; ++c) {
    MXK_TM(0);
    const int t0 = c * kC;
    const int valid = min(kC, p.T - t0);
    const uint64_t dm = done_mask_from_flags(done_flags);
    done_flags = load_done_flags(drow, t0 + kC, p.T, lane);
    const bool has_reset = dm != 0ull;
    if (warp == 1) scan_chunk(c, dm);   // while the other warps wait for the tiles
    mbar_wait_flag(&sm.bar_load, c & 1, timed_out);
    MXK_TM(1);
    if (tid < kC) sm.v[kPanels * kC + tid].x = tid < valid ? kOneBf16 : 0u;
    if (tid == 0) tma::wait_group_read<0>();   // the previous output tile has left p
    fence_smem_to_async();
    fence_before_sync();
    __syncthreads();
    MXK_TM(2);

    if (warp == 0) {
      const bool leader = elect_one();
      fence_after_sync();
      const Operand aq = sw_operand(smem_u32(sm.q), false), bk = sw_operand(smem_u32(sm.k), false);
      gemm<kD / 16>(tmem, aq, bk, idesc_p, false, leader);                           // P -> lower lanes
      if (leader) commit(&sm.bar[0]);
      if (p.chunk_states && tid == 0) {   // residual for the backward pass: the state entering this chunk
        tma::store_bulk(p.chunk_states + (static_cast<size_t>(bh) * nchunks + c) * (kPanelsX * kD), sm.s, kPanelsX * kD * 16);
        tma::commit_group();
      }
    }
    mbar_wait_flag(&sm.bar[0], c & 1, timed_out);
    fence_after_sync();
    MXK_TM(3);
    const float delta = sm.gates.delta;

    // ---- epilogue A ----
    {
      float vals[kDX];
      tmem_ld_row<kDX>(lane_base, vals);
      if (!upper) {
        // P~_tj = P_tj 2^(rowterm2_t + lic2_j) on the keys of row t's segment
        const int lo = row_first_key(dm, row);
        const float rt = sm.gates.rowterm2[row];
        const float4* lic4 = reinterpret_cast<const float4*>(sm.gates.lic2);
#pragma unroll
        for (int pn = 0; pn < kPanels; ++pn) {
          const float4 c0 = lic4[2 * pn], c1 = lic4[2 * pn + 1];
          const float cj[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
          float f[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const int j = pn * 8 + e;
            f[e] = (j >= lo && j <= row) ? vals[j] * ex2_fast(rt + cj[e]) : 0.f;
          }
          sm.p[sw_idx(row, pn)] = pack8_bf16(f);
        }
      } else {
        // the same-numbered upper thread scales query row `row` by w_t in place and its state row by delta
        const float w = sm.gates.w[row];
#pragma unroll
        for (int pn = 0; pn < kPanels; ++pn) {
          float f[8];
          unpack8_bf16(sm.q[sw_idx(row, pn)], f);
#pragma unroll
          for (int e = 0; e < 8; ++e) f[e] *= w;
          sm.q[sw_idx(row, pn)] = pack8_bf16(f);
        }
#pragma unroll
        for (int i = 0; i < kDX; ++i) vals[i] *= delta;
      }
      // the state rows go back scaled by delta; the lower lanes of the same (warp-wide) store rewrite their
      // consumed P values, which the next product overwrites.  With a reset the state is replaced, not scaled.
      if (!has_reset) {
#pragma unroll
        for (int pn = 0; pn < kPanelsX; ++pn) tmem_st8(lane_base + pn * 8, vals + pn * 8);
        tmem_st_wait();
      }
    }
#pragma unroll
    for (int r = 0; r < 5; ++r) {   // kappa o [V | 1]: 576 vectors, vector (seg, j) at seg * kC + j
      const int vid = r * kThreads + tid;
      if (vid < kPanelsX * kC) {
        const float kap = sm.gates.kappa[vid & (kC - 1)];
        float f[8];
        unpack8_bf16(sm.v[vid], f);
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] *= kap;
        sm.alt[vid] = pack8_bf16(f);
      }
    }
    MXK_TM(4);
    if (tid == 0) tma::wait_group_read<0>();   // the residual copy has left s, which epilogue B rewrites
    fence_smem_to_async();
    fence_before_sync();
    __syncthreads();
    MXK_TM(5);

    if (warp == 0) {
      const bool leader = elect_one();
      fence_after_sync();
      const Operand aql = sw_operand(smem_u32(sm.q), false), bs{smem_u32(sm.s), kD, true};
      const Operand ap = sw_operand(smem_u32(sm.p), false), bv{smem_u32(sm.v), kC, true};
      const Operand ak = sw_operand(smem_u32(sm.k), true), balt{smem_u32(sm.alt), kC, true};
      gemm<kD / 16>(tmem, aql, bs, idesc_o, false, leader);                          // O  = (w o Q) S_in^T
      gemm<kC / 16>(tmem, ap, bv, idesc_o, true, leader);                            // O += P~ (V | 1)
      gemm<kC / 16>(tmem + kUpper, ak, balt, idesc_s, !has_reset, leader);           // S (+)= K^T (kappa o (V | 1))
      if (leader) commit(&sm.bar[1]);
    }
    mbar_wait_flag(&sm.bar[1], c & 1, timed_out);
    fence_after_sync();
    if (tid == 0 && c + 1 < nchunks) issue_chunk_loads(c + 1);
    MXK_TM(6);

    // ---- epilogue B ----
    {
      float orow[kDX];
      tmem_ld_row<kDX>(lane_base, orow);
      if (!upper) {
        const float inv = 1.f / (fmaxf(fabsf(orow[kD]), sm.gates.em[c & 1][row]) + p.eps);
#pragma unroll
        for (int pn = 0; pn < kPanels; ++pn) {
          float f[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) f[e] = orow[pn * 8 + e] * inv;
          sm.p[sw_idx(row, pn)] = pack8_bf16(f);
        }
      } else {
#pragma unroll
        for (int pn = 0; pn < kPanelsX; ++pn) sm.s[pn * kD + row] = pack8_bf16(orow + pn * 8);
        if (c == nchunks - 1 && row < hd) {
          if (p.c_last) {
            float* out = p.c_last + (static_cast<size_t>(bh) * hd + row) * hd;
#pragma unroll
            for (int vcol = 0; vcol < kD; ++vcol)
              if (vcol < hd) out[vcol] = orow[vcol];
          }
          if (p.n_last) p.n_last[static_cast<size_t>(bh) * hd + row] = orow[kD];
        }
      }
    }
    fence_smem_to_async();
    __syncthreads();
    if (tid == 0) {
      tma::store_plain_tile(&p.map_o, sm.p, t0, h, b);
      tma::commit_group();
    }
    MXK_TM(7);
  }

  if (tid == 0) {
    if (p.m_last) p.m_last[bh] = sm.gates.m_out;
    if (p.f_last) p.f_last[bh] = sm.gates.f_out;
    tma::wait_group_all();
  }
  if (timed_out && p.status) atomicExch(p.status, 1);
  fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, kTmemCols);
}

}  // namespace
}  // namespace mxk

#ifdef MXK_TIMING
extern "C" int mxk_debug_mtc_phase_cycles(unsigned long long* out, int reset) {
  if (reset) {
    unsigned long long z[16] = {};
    return (int)cudaMemcpyToSymbol(mxk::g_mtc_phase_cycles, z, sizeof(z));
  }
  return (int)cudaMemcpyFromSymbol(out, mxk::g_mtc_phase_cycles, 16 * sizeof(unsigned long long));
}
#endif

extern "C" {

size_t mxk_mlstm_bf16_chunk_states_bytes(int B, int T, int H, int d) {
  if (B <= 0 || T <= 0 || H <= 0 || d < 8 || d > mxk::linattn::kD || d % 8) return 0;
  const size_t nchunks = (static_cast<size_t>(T) + mxk::linattn::kC - 1) / mxk::linattn::kC;
  return static_cast<size_t>(B) * H * nchunks * (mxk::linattn::kPanelsX * mxk::linattn::kD) * sizeof(uint4);
}

int mxk_mlstm_bf16_fwd(const void* q, const void* k, const void* v, const float* log_i, const float* log_f,
                       const float* c0, const float* n0, const float* m0, const float* f0, const uint8_t* done,
                       void* h, float* c_last, float* n_last, float* m_last, float* f_last, float* m_steps,
                       void* chunk_states, int* status, int B, int T, int H, int d, float eps, mxk_stream_t stream) {
  using namespace mxk;
  if (!q || !k || !v || !log_i || !log_f || !h) return MXK_ERR_NULL;
  if (B <= 0 || T <= 0 || H <= 0 || static_cast<long long>(B) * H > 0x7fffffffLL) return MXK_ERR_DIMS;
  if (d < 8 || d > kD || d % 8) return MXK_ERR_UNSUPPORTED;
  for (const void* ptr : {q, k, v, (const void*)h, (const void*)chunk_states})
    if (ptr && !aligned16(ptr)) return MXK_ERR_ALIGN;
  for (const void* ptr : {(const void*)log_i, (const void*)log_f, (const void*)c0, (const void*)n0, (const void*)m0, (const void*)f0,
                          (const void*)c_last, (const void*)n_last, (const void*)m_last, (const void*)f_last, (const void*)m_steps})
    if (ptr && (reinterpret_cast<uintptr_t>(ptr) & 3u)) return MXK_ERR_ALIGN;
  FwdParams prm;
  prm.log_i = log_i; prm.log_f = log_f;
  prm.c0 = c0; prm.n0 = n0; prm.m0 = m0; prm.f0 = f0;
  prm.done = done;
  prm.c_last = c_last; prm.n_last = n_last; prm.m_last = m_last; prm.f_last = f_last;
  prm.m_steps = m_steps;
  prm.chunk_states = static_cast<uint4*>(chunk_states);
  prm.status = status;
  prm.B = B; prm.T = T; prm.H = H; prm.d = d;
  prm.eps = eps;
  if (!tma::make_sw_map(&prm.map_q, q, B, T, H, kC, d) || !tma::make_sw_map(&prm.map_k, k, B, T, H, kC, d) ||
      !tma::make_panel_map(&prm.map_v, v, B, T, H, d, kC, kPanels) || !tma::make_sw_map(&prm.map_o, h, B, T, H, kC, d))
    return MXK_ERR_UNSUPPORTED;
  cudaError_t e = cudaFuncSetAttribute(mlstm_tc_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(sizeof(FwdSmem)));
  if (e != cudaSuccess) return static_cast<int>(e);
  mlstm_tc_fwd_kernel<<<B * H, kThreads, sizeof(FwdSmem), static_cast<cudaStream_t>(stream)>>>(prm);
  return launch_status();
}

}  // extern "C"
