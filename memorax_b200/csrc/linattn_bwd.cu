// Backward of chunked causal linear attention on the sm_100a tensor cores.
//
// One CTA owns one (batch, head) sequence and walks its 64-token chunks right
// to left, carrying G^T = (dL/dS)^T with gz = dL/dz as one extra column in
// tensor memory (fp32).  The state entering each chunk comes from the forward
// call's residual (bf16, already in operand order).  Per chunk, with
// D_i = max(den_i, eps), c_i = [den_i > eps]:
//   phase 1 (independent MMAs):  P = phi(Q) phi(K)^T,  dA = dO V^T,  R = dO S_in
//   epilogue 1 (one thread per query row):
//     den_i  = sum_j M_ij P_ij + live_i phi(q_i).z_in
//     don_i  = sum_j M_ij P_ij dA_ij + live_i phi(q_i).R_i          (= do_i . num_i)
//     dden_i = -c_i don_i / D_i^2
//     Pn_ij  = M_ij P_ij / D_i          dP_ij = M_ij (dA_ij / D_i + dden_i)
//     dOs_i  = live_i [do_i / D_i | dden_i]
//   phase 2:  dphiQ = dP phi(K) + dOs [S_in | z_in]
//             dphiK = dP^T phi(Q) + keep [V | 1] [G | gz]^T
//             dV    = Pn^T dO + keep phi(K) G^T
//             [G|gz]^T = [no reset] [G|gz]^T + phi(Q)^T dOs
//   epilogue 2: dq = dphiQ * phi'(q), dk = dphiK * phi'(k), dv; refresh the
//   bf16 operand copy of G.
#include <cuda_bf16.h>

#include "linattn_common.cuh"
#include "mxk_common.cuh"

namespace mxk {
namespace {

using namespace umma;
using namespace linattn;

constexpr int kPanelsK = kPanels + 2;  // 80 columns: a K = 80 contraction needs whole K=16 steps

struct BwdParams {
  const __nv_bfloat16* q;
  const __nv_bfloat16* k;
  const __nv_bfloat16* v;
  const __nv_bfloat16* d_o;
  const uint4* chunk_states;
  const uint8_t* done;
  const float* ds_last;
  const float* dz_last;
  __nv_bfloat16* dq;
  __nv_bfloat16* dk;
  __nv_bfloat16* dv;
  float* ds0;
  float* dz0;
  int* status;
  int B, T, H;
  float eps;
  int feature_map;
};

struct BwdSmem {
  uint4 q[kPanels * kC];      // phi(Q)                 [k/8][i]
  uint4 k[kPanels * kC];      // phi(K)                 [k/8][j]
  uint4 kk[kPanels * kC];     // keep rows of phi(K)
  uint4 v[kPanels * kC];      // V                      [v/8][j]
  uint4 vk[kPanelsK * kC];    // keep rows of V | 1 | 0 [v/8][j]
  uint4 d_o[kPanels * kC];    // dO                     [v/8][i]
  uint4 dos[kPanelsK * kC];   // live rows of dO/D | dden | 0
  uint4 s[kPanelsK * kD];     // S_in^T | z_in | 0      [v/8][k]
  uint4 g[kPanelsK * kD];     // G^T | gz | 0           [v/8][k]
  uint4 pn[kPanels * kC];     // P / D                  [j/8][i]
  uint4 dp[kPanels * kC];     // dP                     [j/8][i]
  uint64_t bar[2];
  uint32_t tmem;
};

// 256 TMEM columns per CTA (two CTAs per SM).  M = 64 accumulators use 16 of a
// warp's 32 TMEM lanes, so lanes 0..15 ("lower" threads) and 16..31 ("upper"
// threads) hold different matrices in the same columns:
//   columns   0.. 63   first P (0..31) and dA (32..63), each issued as two N = 32 halves: keys
//                      0..31 in the lower lanes, keys 32..63 in the upper lanes, so that both
//                      half-warps own 32 keys of the same query row; later dphiQ (lower) and
//                      dphiK (upper)
//   columns  64..135   lower: dV                  upper: G^T | gz (persistent)
//   columns 136..167   R, state features 0..31 in the lower lanes, 32..63 in the upper lanes
#ifdef MXK_TIMING
}  // namespace
__device__ unsigned long long g_bwd_phase_cycles[8];
namespace {
#define MXK_TB(i) do { if (tid == 0 && (blockIdx.x % 37) == 0) { const long long now_ = clock64(); atomicAdd(&g_bwd_phase_cycles[i], (unsigned long long)(now_ - t_prev_)); t_prev_ = now_; } } while (0)
#else
#define MXK_TB(i) do {} while (0)
#endif
constexpr uint32_t kBwdTmemCols = 256;
constexpr uint32_t kUpper = 16u << 16;
constexpr uint32_t kColLo = 0, kColHi = 64, kColP = 0, kColA = 32, kColR = 136;

__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }

__global__ void __launch_bounds__(kThreads, 2) linattn_bwd_kernel(const BwdParams p) {
  extern __shared__ __align__(128) uint8_t smem_raw[];
  BwdSmem& sm = *reinterpret_cast<BwdSmem*>(smem_raw);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int bh = blockIdx.x, b = bh / p.H, h = bh % p.H;
  const bool upper = lane >= 16;
  const int row = warp * 16 + (lane & 15);
  const int nchunks = (p.T + kC - 1) / kC;
  const uint4 zero4 = make_uint4(0, 0, 0, 0);

  if (tid == 0) {
    mbar_init(&sm.bar[0], 1);
    mbar_init(&sm.bar[1], 1);
    mbar_init_fence();
  }
  if (warp == 0) tmem_alloc(&sm.tmem, kBwdTmemCols);
  // zero padding panels that never change (columns 72..79 of the 80-wide operands)
  if (tid < kC) {
    sm.vk[(kPanelsK - 1) * kC + tid] = zero4;
    sm.dos[(kPanelsK - 1) * kC + tid] = zero4;
    sm.s[(kPanelsK - 1) * kD + tid] = zero4;
    sm.g[(kPanelsK - 1) * kD + tid] = zero4;
  }
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem = sm.tmem;
  const uint32_t lane_base = tmem + (static_cast<uint32_t>(warp * 32) << 16);

  // Cotangent of the next carry -> TMEM (upper lanes) and its bf16 operand copy
  // (upper thread `row` owns G^T[row][.] = dS[.][row]).
  {
    const float* gs = p.ds_last ? p.ds_last + static_cast<size_t>(bh) * kD * kD : nullptr;
    const float* gz = p.dz_last ? p.dz_last + static_cast<size_t>(bh) * kD : nullptr;
    float vals[kDX];   // all loads first: the TMEM stores below are compiler memory barriers
#pragma unroll
    for (int vcol = 0; vcol < kDX; ++vcol) {
      float x = 0.f;
      if (upper) {
        if (vcol < kD) x = gs ? gs[vcol * kD + row] : 0.f;
        else if (vcol == kD) x = gz ? gz[row] : 0.f;
      }
      vals[vcol] = x;
    }
#pragma unroll
    for (int pn = 0; pn < kPanelsX; ++pn) {
      tmem_st8(lane_base + kColHi + pn * 8, vals + pn * 8);
      if (upper) sm.g[pn * kD + row] = pack8_bf16(vals + pn * 8);
    }
    tmem_st_wait();
  }

  const size_t stride_t = static_cast<size_t>(p.H) * kD;
  const size_t seq_base = (static_cast<size_t>(b) * p.T * p.H + h) * kD;
  const uint8_t* drow = p.done ? p.done + static_cast<size_t>(b) * p.T : nullptr;
  const uint32_t id_kk = idesc_bf16(kC, kC, false, false);   // A, B contract over columns
  const uint32_t id_km = idesc_bf16(kC, kC, false, true);    // B contracts over rows
  const uint32_t id_mm = idesc_bf16(kC, kC, true, true);
  const uint32_t id_g = idesc_bf16(kD, kDX, true, true);
  bool timed_out = false;

  // This thread's 16 vectors (q, k, v, dO of four tile positions) of chunk cc.
  uint4 pre[16];
  uint4 pre_s[5];   // this thread's share of the 576 vectors of S_in
  auto prefetch = [&](int cc) {
    const int base_t = cc * kC;
    {
      const uint4* src = p.chunk_states + (static_cast<size_t>(bh) * nchunks + cc) * (kPanelsX * kD);
#pragma unroll
      for (int i = 0; i < 5; ++i)
        if (i * kThreads + tid < kPanelsX * kD) pre_s[i] = __ldg(src + i * kThreads + tid);
    }
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      int trow, seg;
      tile_vec(r * kThreads + tid, trow, seg);
      const size_t g = seq_base + static_cast<size_t>(base_t + trow) * stride_t + seg * 8;
      const bool in = base_t + trow < p.T;
      pre[4 * r] = in ? __ldg(reinterpret_cast<const uint4*>(p.q + g)) : zero4;
      pre[4 * r + 1] = in ? __ldg(reinterpret_cast<const uint4*>(p.k + g)) : zero4;
      pre[4 * r + 2] = in ? __ldg(reinterpret_cast<const uint4*>(p.v + g)) : zero4;
      pre[4 * r + 3] = in ? __ldg(reinterpret_cast<const uint4*>(p.d_o + g)) : zero4;
    }
  };
  prefetch(nchunks - 1);
  uint32_t done_flags = load_done_flags(drow, (nchunks - 1) * kC, p.T, lane);
#ifdef MXK_TIMING
  long long t_prev_ = clock64();
#endif

  for (int it = 0; it < nchunks; ++it) {
    const int c = nchunks - 1 - it;
    const int t0 = c * kC;
    const int valid = min(kC, p.T - t0);
    const uint64_t dm = done_mask_from_flags(done_flags);
    done_flags = load_done_flags(drow, t0 - kC, p.T, lane);   // the next (earlier) chunk's flags
    const bool has_reset = dm != 0ull;
    MXK_TB(0);

    // ---- stage phi(Q), phi(K), V, dO (prefetched during the previous chunk), S_in ----
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      int trow, seg;
      tile_vec(r * kThreads + tid, trow, seg);
      uint4 qv = pre[4 * r], kv = pre[4 * r + 1];
      const uint4 vv = pre[4 * r + 2], gv = pre[4 * r + 3];
      if (p.feature_map && trow < valid) {
        qv = phi8(qv);
        kv = phi8(kv);
      }
      const int slot = seg * kC + trow;
      const bool keep = row_keep(dm, trow);
      sm.q[slot] = qv;
      sm.k[slot] = kv;
      sm.kk[slot] = keep ? kv : zero4;
      sm.v[slot] = vv;
      sm.vk[slot] = keep ? vv : zero4;
      sm.d_o[slot] = gv;
    }
    if (tid < kC) sm.vk[kPanels * kC + tid] = make_uint4((tid < valid && row_keep(dm, tid)) ? kOneBf16 : 0u, 0, 0, 0);
#pragma unroll
    for (int i = 0; i < 5; ++i)
      if (i * kThreads + tid < kPanelsX * kD) sm.s[i * kThreads + tid] = pre_s[i];
    fence_smem_to_async();
    fence_before_sync();
    MXK_TB(1);
    __syncthreads();

    if (tid == 0) {
      fence_after_sync();
      const Operand aq{smem_u32(sm.q), kC, false}, bk{smem_u32(sm.k), kC, false};
      const Operand ado{smem_u32(sm.d_o), kC, false}, bv{smem_u32(sm.v), kC, false};
      const Operand bs{smem_u32(sm.s), kD, false};
      const uint32_t id_half = idesc_bf16(kC, 32, false, false);
      const Operand bk_hi{smem_u32(sm.k) + 32 * 16, kC, false}, bv_hi{smem_u32(sm.v) + 32 * 16, kC, false};
      const Operand bs_hi{smem_u32(sm.s) + 32 * 16, kD, false};
      gemm(tmem + kColP, aq, bk, id_half, kD / 16, false);                 // P,  keys 0..31
      gemm(tmem + kUpper + kColP, aq, bk_hi, id_half, kD / 16, false);     // P,  keys 32..63
      gemm(tmem + kColA, ado, bv, id_half, kD / 16, false);                // dA, keys 0..31
      gemm(tmem + kUpper + kColA, ado, bv_hi, id_half, kD / 16, false);    // dA, keys 32..63
      gemm(tmem + kColR, ado, bs, id_half, kD / 16, false);                // R,  features 0..31
      gemm(tmem + kUpper + kColR, ado, bs_hi, id_half, kD / 16, false);    // R,  features 32..63
      commit(&sm.bar[0]);
    }
    if (!mbar_wait(&sm.bar[0], it & 1)) timed_out = true;
    fence_after_sync();
    MXK_TB(2);

    // ---- epilogue 1: both half-warps own the same query row; each covers 32 keys / features ----
    {
      const bool live = row_live(dm, row);
      const int lo = row_first_key(dm, row);
      const int j0 = upper ? 32 : 0, p0 = upper ? 4 : 0;
      float s_dot = 0.f, z_dot = 0.f;
      {
        float rr[32];
        tmem_ld_row<32>(lane_base + kColR, rr);
#pragma unroll
        for (int pp = 0; pp < 4; ++pp) {
          float fq[8];
          unpack8_bf16(sm.q[(p0 + pp) * kC + row], fq);
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const int kk = (p0 + pp) * 8 + e;
            s_dot = fmaf(fq[e], rr[pp * 8 + e], s_dot);
            z_dot = fmaf(fq[e], bf16_lo(sm.s[kPanels * kD + kk].x), z_dot);
          }
        }
      }
      float pv[32], av[32];
      tmem_ld_row<32>(lane_base + kColP, pv);
      tmem_ld_row<32>(lane_base + kColA, av);
      float den = live ? z_dot : 0.f, don = live ? s_dot : 0.f;
#pragma unroll
      for (int e = 0; e < 32; ++e) {
        const int j = j0 + e;
        const bool m = (j >= lo && j <= row);
        pv[e] = m ? pv[e] : 0.f;
        av[e] = m ? av[e] : 0.f;
        den += pv[e];
        don = fmaf(pv[e], av[e], don);
      }
      den += __shfl_xor_sync(0xffffffffu, den, 16);
      don += __shfl_xor_sync(0xffffffffu, don, 16);
      const float dcl = fmaxf(den, p.eps);
      const float inv = 1.f / dcl;
      const float dden = den > p.eps ? -don * inv * inv : 0.f;
#pragma unroll
      for (int jq = 0; jq < 4; ++jq) {
        float a[8], d8[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const int x = jq * 8 + e, j = j0 + x;
          a[e] = pv[x] * inv;
          d8[e] = (j >= lo && j <= row) ? fmaf(av[x], inv, dden) : 0.f;
        }
        sm.pn[(p0 + jq) * kC + row] = pack8_bf16(a);
        sm.dp[(p0 + jq) * kC + row] = pack8_bf16(d8);
      }
      // scaled dO rows: two panels per thread pair member (lower: panels 0..3, upper: 4..7 and the extra column)
      {
        const float sc = live ? inv : 0.f;
        const int p0 = upper ? 4 : 0;
#pragma unroll
        for (int pp = 0; pp < 4; ++pp) {
          float f[8];
          unpack8_bf16(sm.d_o[(p0 + pp) * kC + row], f);
#pragma unroll
          for (int e = 0; e < 8; ++e) f[e] *= sc;
          sm.dos[(p0 + pp) * kC + row] = pack8_bf16(f);
        }
        if (upper) sm.dos[kPanels * kC + row] = make_uint4(pack_bf16(live ? dden : 0.f, 0.f), 0, 0, 0);
      }
    }
    fence_smem_to_async();
    fence_before_sync();
    MXK_TB(3);
    __syncthreads();

    if (tid == 0) {
      fence_after_sync();
      // dphiQ = dP phi(K) + dOs [S|z]                      (lower, columns 0..63)
      gemm(tmem + kColLo, Operand{smem_u32(sm.dp), kC, false}, Operand{smem_u32(sm.k), kC, true}, id_km, kC / 16, false);
      gemm(tmem + kColLo, Operand{smem_u32(sm.dos), kC, false}, Operand{smem_u32(sm.s), kD, false}, id_kk, 5, true);
      // dphiK = dP^T phi(Q) + keep[V|1] [G|gz]^T           (upper, columns 0..63)
      gemm(tmem + kUpper + kColLo, Operand{smem_u32(sm.dp), kC, true}, Operand{smem_u32(sm.q), kC, true}, id_mm, kC / 16, false);
      gemm(tmem + kUpper + kColLo, Operand{smem_u32(sm.vk), kC, false}, Operand{smem_u32(sm.g), kD, false}, id_kk, 5, true);
      // dV = (P/D)^T dO + keep phi(K) G^T                  (lower, columns 64..127)
      gemm(tmem + kColHi, Operand{smem_u32(sm.pn), kC, true}, Operand{smem_u32(sm.d_o), kC, true}, id_mm, kC / 16, false);
      gemm(tmem + kColHi, Operand{smem_u32(sm.kk), kC, false}, Operand{smem_u32(sm.g), kD, true}, id_km, kD / 16, true);
      // [G|gz]^T = [no reset][G|gz]^T + phi(Q)^T dOs       (upper, columns 64..135)
      gemm(tmem + kUpper + kColHi, Operand{smem_u32(sm.q), kC, true}, Operand{smem_u32(sm.dos), kC, true}, id_g, kC / 16, !has_reset);
      commit(&sm.bar[1]);
    }
    if (c > 0) prefetch(c - 1);   // in flight while the MMAs and the output epilogue run
    if (!mbar_wait(&sm.bar[1], it & 1)) timed_out = true;
    fence_after_sync();
    MXK_TB(4);

    // ---- epilogue 2 ----
    {
      // one stream: lower chains dphiQ through phi'(q) into dq, upper dphiK through phi'(k) into dk.
      // Output rows leave through per-warp staging areas (buffers the finished MMAs no longer
      // need) so that every store instruction writes complete 128-byte rows.
      const int rows_valid = valid - warp * 16;
      __nv_bfloat16* const gq = p.dq + seq_base + static_cast<size_t>(t0 + warp * 16) * stride_t;
      __nv_bfloat16* const gk = p.dk + seq_base + static_cast<size_t>(t0 + warp * 16) * stride_t;
      __nv_bfloat16* const gv = p.dv + seq_base + static_cast<size_t>(t0 + warp * 16) * stride_t;
      {
        float acc[kD];
        tmem_ld_row<kD>(lane_base + kColLo, acc);
        const uint4* feat = upper ? &sm.k[row] : &sm.q[row];
        uint4 packed[kPanels];
#pragma unroll
        for (int pn = 0; pn < kPanels; ++pn) {
          float f[8];
          unpack8_bf16(feat[pn * kC], f);
#pragma unroll
          for (int e = 0; e < 8; ++e) f[e] = acc[pn * 8 + e] * ((p.feature_map && f[e] <= 1.f) ? f[e] : 1.f);
          packed[pn] = pack8_bf16(f);
        }
        store_rows_coalesced(sm.dos + warp * (16 * 9), packed, !upper, lane, gq, stride_t, rows_valid);
        store_rows_coalesced(sm.vk + warp * (16 * 9), packed, upper, lane, gk, stride_t, rows_valid);
      }
      // one stream: lower stores dV, upper refreshes the bf16 operand copy of G | gz
      {
        float acc[kDX];
        tmem_ld_row<kDX>(lane_base + kColHi, acc);
        uint4 packed[kPanelsX];
#pragma unroll
        for (int pn = 0; pn < kPanelsX; ++pn) packed[pn] = pack8_bf16(acc + pn * 8);
        if (upper) {
#pragma unroll
          for (int pn = 0; pn < kPanelsX; ++pn) sm.g[pn * kD + row] = packed[pn];
        }
        store_rows_coalesced(sm.pn + warp * (16 * 9), packed, !upper, lane, gv, stride_t, rows_valid);   // pn, dp: one 16 KB region
        if (upper && c == 0) {
          if (p.ds0) {
            float* out = p.ds0 + static_cast<size_t>(bh) * kD * kD;
#pragma unroll
            for (int vcol = 0; vcol < kD; ++vcol) out[vcol * kD + row] = acc[vcol];
          }
          if (p.dz0) p.dz0[static_cast<size_t>(bh) * kD + row] = acc[kD];
        }
      }
    }
    MXK_TB(5);
    __syncthreads();   // staging areas alias buffers that the next chunk refills
    MXK_TB(6);
  }

  if (timed_out && p.status) atomicExch(p.status, 1);
  fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, kBwdTmemCols);
}

}  // namespace
}  // namespace mxk

#ifdef MXK_TIMING
extern "C" int mxk_debug_bwd_phase_cycles(unsigned long long* out, int reset) {
  if (reset) {
    unsigned long long z[8] = {};
    return (int)cudaMemcpyToSymbol(mxk::g_bwd_phase_cycles, z, sizeof(z));
  }
  return (int)cudaMemcpyFromSymbol(out, mxk::g_bwd_phase_cycles, 8 * sizeof(unsigned long long));
}
#endif

extern "C" {

int mxk_linattn_bf16_bwd(const void* q, const void* k, const void* v, const void* d_o, const void* chunk_states,
                         const uint8_t* done, const float* ds_last, const float* dz_last, void* dq, void* dk,
                         void* dv, float* ds0, float* dz0, int* status, int B, int T, int H, int d, float eps,
                         int feature_map, mxk_stream_t stream) {
  using namespace mxk;
  using namespace mxk::linattn;
  if (!q || !k || !v || !d_o || !chunk_states || !dq || !dk || !dv) return MXK_ERR_NULL;
  if (B <= 0 || T <= 0 || H <= 0 || static_cast<long long>(B) * H > 0x7fffffffLL) return MXK_ERR_DIMS;
  if (d != kD) return MXK_ERR_UNSUPPORTED;
  for (const void* ptr : {q, k, v, d_o, chunk_states, (const void*)dq, (const void*)dk, (const void*)dv})
    if (!aligned16(ptr)) return MXK_ERR_ALIGN;
  for (const void* ptr : {(const void*)ds_last, (const void*)dz_last, (const void*)ds0, (const void*)dz0})
    if (ptr && (reinterpret_cast<uintptr_t>(ptr) & 3u)) return MXK_ERR_ALIGN;
  BwdParams prm;
  prm.q = static_cast<const __nv_bfloat16*>(q);
  prm.k = static_cast<const __nv_bfloat16*>(k);
  prm.v = static_cast<const __nv_bfloat16*>(v);
  prm.d_o = static_cast<const __nv_bfloat16*>(d_o);
  prm.chunk_states = static_cast<const uint4*>(chunk_states);
  prm.done = done;
  prm.ds_last = ds_last;
  prm.dz_last = dz_last;
  prm.dq = static_cast<__nv_bfloat16*>(dq);
  prm.dk = static_cast<__nv_bfloat16*>(dk);
  prm.dv = static_cast<__nv_bfloat16*>(dv);
  prm.ds0 = ds0;
  prm.dz0 = dz0;
  prm.status = status;
  prm.B = B; prm.T = T; prm.H = H;
  prm.eps = eps;
  prm.feature_map = feature_map;
  cudaError_t e = cudaFuncSetAttribute(linattn_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(sizeof(BwdSmem)));
  if (e != cudaSuccess) return static_cast<int>(e);
  linattn_bwd_kernel<<<B * H, kThreads, sizeof(BwdSmem), static_cast<cudaStream_t>(stream)>>>(prm);
  return launch_status();
}

}  // extern "C"
